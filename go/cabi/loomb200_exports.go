// C exports in the style of welvet/cabi for foreign callers that hold int64 handles: the B200 counterparts of
// LoomDispatchBitNetQuantizeActivation, LoomDispatchDenseBitNetTernaryQuantized and LoomDispatchBitNetGateProduct
// (welvet/cabi/acceleration_wgpu_exports.go:804-922).  Same argument order and the same JSON status strings
// ({"status": "ok"} / {"error": "..."}, freed by the caller with FreeLoomString, welvet/cabi/main.go:44-47); the network
// handle is replaced by a context handle, GPU buffer handles map to loomb200 buffers and the weight handle to a packed
// matrix, so weightScale and tileSize are accepted and ignored (the scale lives with the matrix, there is no tile knob).
//
// NOT COMPILED WHERE THIS LIBRARY IS BUILT (no Go toolchain in the build image).  Built with
// `go build -buildmode=c-shared` next to the other cabi files.
package main

/*
#include <stdlib.h>
*/
import "C"

import (
	"encoding/json"
	"sync"
	"unsafe"

	"github.com/openfluke/loom/go/loomb200"
)

var (
	b200Mu      sync.RWMutex
	b200NextID  int64 = 1
	b200Ctx           = map[int64]*loomb200.Context{}
	b200Buffers       = map[int64]*loomb200.Buffer{}
	b200Weights       = map[int64]*loomb200.Weight{}
)

func b200Err(msg string) *C.char {
	b, _ := json.Marshal(map[string]string{"error": msg})
	return C.CString(string(b))
}

func b200OK() *C.char { return C.CString(`{"status": "ok"}`) }

//export LoomB200Open
func LoomB200Open(device C.int) C.longlong {
	ctx, err := loomb200.Open(int(device))
	if err != nil {
		return -1
	}
	b200Mu.Lock()
	defer b200Mu.Unlock()
	id := b200NextID
	b200NextID++
	b200Ctx[id] = ctx
	return C.longlong(id)
}

//export LoomB200CreateBuffer
func LoomB200CreateBuffer(ctxHandle C.longlong, bytes C.longlong) C.longlong {
	b200Mu.Lock()
	defer b200Mu.Unlock()
	ctx, ok := b200Ctx[int64(ctxHandle)]
	if !ok {
		return -1
	}
	buf, err := ctx.Alloc(int(bytes))
	if err != nil {
		return -1
	}
	id := b200NextID
	b200NextID++
	b200Buffers[id] = buf
	return C.longlong(id)
}

func b200Lookup(ctxHandle int64, bufs ...int64) (*loomb200.Context, []*loomb200.Buffer, string) {
	b200Mu.RLock()
	defer b200Mu.RUnlock()
	ctx, ok := b200Ctx[ctxHandle]
	if !ok {
		return nil, nil, "invalid context handle"
	}
	out := make([]*loomb200.Buffer, len(bufs))
	for i, h := range bufs {
		if h == 0 {
			continue // optional buffer (bias)
		}
		b, ok := b200Buffers[h]
		if !ok {
			return nil, nil, "invalid buffer handle"
		}
		out[i] = b
	}
	return ctx, out, ""
}

//export LoomB200DispatchBitNetQuantizeActivation
func LoomB200DispatchBitNetQuantizeActivation(ctxHandle C.longlong, batchSize C.int, inputSize C.int, inputHandle C.longlong,
	qPackedHandle C.longlong, scaleHandle C.longlong) *C.char {
	ctx, b, msg := b200Lookup(int64(ctxHandle), int64(inputHandle), int64(qPackedHandle), int64(scaleHandle))
	if msg != "" {
		return b200Err(msg)
	}
	// the scale buffer receives amax (the CPU path's convention), not amax/127 as the WGSL kernel writes
	if err := ctx.QuantizeActivation(int(batchSize), int(inputSize), b[0], b[1], b[2]); err != nil {
		return b200Err(err.Error())
	}
	return b200OK()
}

//export LoomB200DispatchDenseBitNetTernaryQuantized
func LoomB200DispatchDenseBitNetTernaryQuantized(ctxHandle C.longlong, batchSize C.int, inputSize C.int, outputSize C.int,
	qPackedHandle C.longlong, scaleHandle C.longlong, weightHandle C.longlong, biasHandle C.longlong, outputHandle C.longlong,
	weightScale C.float, activation C.int, tileSize C.int) *C.char {
	ctx, b, msg := b200Lookup(int64(ctxHandle), int64(qPackedHandle), int64(scaleHandle), int64(biasHandle), int64(outputHandle))
	if msg != "" {
		return b200Err(msg)
	}
	b200Mu.RLock()
	w, ok := b200Weights[int64(weightHandle)]
	b200Mu.RUnlock()
	if !ok {
		return b200Err("invalid weight handle")
	}
	if w.Rows != int(outputSize) || w.Cols != int(inputSize) {
		return b200Err("weight shape does not match inputSize/outputSize")
	}
	_ = weightScale // the per-matrix scale was given at upload
	_ = tileSize    // no tile knob on this path
	if err := ctx.TernaryLinear(w, int(batchSize), b[0], b[1], b[2], nil, int(activation), b[3]); err != nil {
		return b200Err(err.Error())
	}
	return b200OK()
}

//export LoomB200DispatchBitNetGateProduct
func LoomB200DispatchBitNetGateProduct(ctxHandle C.longlong, batchSize C.int, hiddenSize C.int, activation C.int,
	gatePreHandle C.longlong, upPreHandle C.longlong, outputHandle C.longlong) *C.char {
	ctx, b, msg := b200Lookup(int64(ctxHandle), int64(gatePreHandle), int64(upPreHandle), int64(outputHandle))
	if msg != "" {
		return b200Err(msg)
	}
	if err := ctx.GateProduct(int(batchSize), int(hiddenSize), int(activation), b[0], b[1], b[2]); err != nil {
		return b200Err(err.Error())
	}
	return b200OK()
}

//export LoomB200UploadTernary
func LoomB200UploadTernary(ctxHandle C.longlong, words *C.uint, rows C.int, cols C.int, scale C.float) C.longlong {
	b200Mu.Lock()
	defer b200Mu.Unlock()
	ctx, ok := b200Ctx[int64(ctxHandle)]
	if !ok {
		return -1
	}
	n := int(rows) * ((int(cols) + 15) / 16)
	view := (*[1 << 30]uint32)(unsafe.Pointer(words))[:n:n]
	w, err := ctx.UploadTernary(view, int(rows), int(cols), float32(scale))
	if err != nil {
		return -1
	}
	id := b200NextID
	b200NextID++
	b200Weights[id] = w
	return C.longlong(id)
}
