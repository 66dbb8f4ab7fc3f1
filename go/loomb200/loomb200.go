// Package loomb200 binds libloom_b200.so (include/loom_b200.h) for Go hosts: the CUDA implementation of Loom's BitNet
// ternary x int8 linear path on B200.  It stands where poly reaches wgpu today: syncBitNetPackedMatrix
// (poly/bitnet_gpu.go:28-50), the three BitNet dispatchers (poly/wgpu_kernels.go:384-507), the packed-ternary layer
// forwards (poly/dense.go:66-101, poly/swiglu.go:270-322, poly/mha.go:204-371) and the ternary branches of
// ForwardTokenIDsWGPU (poly/wgpu_forward.go:31-596).
//
// NOT COMPILED WHERE THIS LIBRARY IS BUILT: the build image has no Go toolchain.  The file is the source a maintainer adds
// under poly/ (or vendors as a module); every call is a thin cgo forward, and the cgo pointer rule is honoured by the
// library itself (host slices are copied during the call, never retained).
package loomb200

/*
#cgo CFLAGS: -I${SRCDIR}/../../include
#cgo LDFLAGS: -L${SRCDIR}/../../loom_b200/lib -lloom_b200
#include <stdlib.h>
#include "loom_b200.h"
*/
import "C"

import (
	"fmt"
	"runtime"
	"unsafe"
)

// Activation codes (poly.ActivationType values; -1 = linear).
const (
	ActReLU      = 0
	ActSiLU      = 1
	ActGELU      = 2
	ActTanh      = 3
	ActSigmoid   = 4
	ActLeakyReLU = 5
	ActReLU2     = 6
	ActLinear    = -1
)

// Error carries the library's return code and message (loom_b200_last_error).
type Error struct {
	Code int
	Msg  string
}

func (e *Error) Error() string { return fmt.Sprintf("loom_b200 %d: %s", e.Code, e.Msg) }

// Context stands where *poly.WGPUContext stands: one device, one stream.  Not safe for concurrent use.
type Context struct{ c *C.loom_b200_ctx }

// Weight is a packed ternary matrix resident in HBM: what GPUWeights[key] + GPUScaleValues[key] hold today.
type Weight struct {
	w          *C.loom_b200_weight
	Rows, Cols int
}

// Buffer is a device allocation owned by the library until Free.
type Buffer struct {
	p     unsafe.Pointer
	Bytes int
}

func (ctx *Context) check(rc C.int) error {
	if rc == 0 {
		return nil
	}
	return &Error{int(rc), C.GoString(C.loom_b200_last_error(ctx.c))}
}

// APIVersion mirrors loom_accel_api_version (poly/accel/include/loom_accel.h:22).
func APIVersion() int { return int(C.loom_b200_api_version()) }

// DeviceCount is the number of sm_100 devices; 0 means the path is unavailable (there is no CPU fallback in the library).
func DeviceCount() int { return int(C.loom_b200_device_count()) }

// Open creates a context on `device` with a stream of its own.
func Open(device int) (*Context, error) {
	var c *C.loom_b200_ctx
	if rc := C.loom_b200_ctx_create(C.int(device), nil, &c); rc != 0 {
		return nil, &Error{int(rc), C.GoString(C.loom_b200_last_error(nil))}
	}
	ctx := &Context{c}
	runtime.SetFinalizer(ctx, func(x *Context) { x.Close() })
	return ctx, nil
}

func (ctx *Context) Close() {
	if ctx.c != nil {
		C.loom_b200_ctx_destroy(ctx.c)
		ctx.c = nil
	}
}

// Sync waits for the stream and reports a bounded device-side wait that ran out (LOOM_B200_ERR_TIMEOUT).
func (ctx *Context) Sync() error { return ctx.check(C.loom_b200_sync(ctx.c)) }

// SetOption sets a tuning knob (results never depend on them), e.g. "pdl", "prefill_gemm", "attn_cluster".
func (ctx *Context) SetOption(key string, value int) error {
	k := C.CString(key)
	defer C.free(unsafe.Pointer(k))
	return ctx.check(C.loom_b200_ctx_set_option(ctx.c, k, C.int(value)))
}

// ---- buffers (WGPUContext.CreatePersistentBuffer / ReadBuffer) ----

func (ctx *Context) Alloc(bytes int) (*Buffer, error) {
	var p unsafe.Pointer
	if err := ctx.check(C.loom_b200_buffer_alloc(ctx.c, C.size_t(bytes), &p)); err != nil {
		return nil, err
	}
	return &Buffer{p, bytes}, nil
}

func (ctx *Context) Free(b *Buffer) error {
	err := ctx.check(C.loom_b200_buffer_free(ctx.c, b.p))
	b.p = nil
	return err
}

func (ctx *Context) UploadF32(b *Buffer, src []float32) error {
	if len(src) == 0 {
		return nil
	}
	return ctx.check(C.loom_b200_buffer_upload(ctx.c, b.p, unsafe.Pointer(&src[0]), C.size_t(4*len(src))))
}

func (ctx *Context) DownloadF32(dst []float32, b *Buffer) error {
	if len(dst) == 0 {
		return nil
	}
	return ctx.check(C.loom_b200_buffer_download(ctx.c, unsafe.Pointer(&dst[0]), b.p, C.size_t(4*len(dst))))
}

// ---- weights: syncBitNetPackedMatrix, SetMicrosoftBitNetPackedMatrixBytes, entity blobs ----

func newWeight(w *C.loom_b200_weight) *Weight {
	var r, c C.int
	C.loom_b200_weight_info(w, &r, &c, nil, nil)
	return &Weight{w, int(r), int(c)}
}

// UploadTernary takes BitNetTernaryMatrix.Words / Rows / Cols / Scale (poly/bitnet_cpu.go:16-43).
func (ctx *Context) UploadTernary(words []uint32, rows, cols int, scale float32) (*Weight, error) {
	var w *C.loom_b200_weight
	rc := C.loom_b200_upload_ternary(ctx.c, (*C.uint32_t)(unsafe.Pointer(&words[0])), C.int(rows), C.int(cols),
		C.int((cols+15)/16), C.float(scale), &w)
	if err := ctx.check(rc); err != nil {
		return nil, err
	}
	return newWeight(w), nil
}

// PackTernaryF32 ternarises a float32 master that already sits in device memory (absmean, per matrix).
func (ctx *Context) PackTernaryF32(master *Buffer, rows, cols int) (*Weight, error) {
	var w *C.loom_b200_weight
	if err := ctx.check(C.loom_b200_pack_ternary_f32(ctx.c, (*C.float)(master.p), C.int(rows), C.int(cols), &w)); err != nil {
		return nil, err
	}
	return newWeight(w), nil
}

// UploadMicrosoftU8 takes the offline U8 layout of microsoft/bitnet checkpoints (4 rows per byte).
func (ctx *Context) UploadMicrosoftU8(packed []byte, rows, cols int, scale float32) (*Weight, error) {
	var w *C.loom_b200_weight
	rc := C.loom_b200_upload_microsoft_u8(ctx.c, (*C.uint8_t)(unsafe.Pointer(&packed[0])), C.int(rows), C.int(cols), C.float(scale), &w)
	if err := ctx.check(rc); err != nil {
		return nil, err
	}
	return newWeight(w), nil
}

// UploadEntityBlob takes a BITNET_TERNARY blob of an .entity checkpoint and returns the slab offset it is keyed by.
func (ctx *Context) UploadEntityBlob(blob []byte) (*Weight, int, error) {
	var w *C.loom_b200_weight
	var off C.int
	rc := C.loom_b200_upload_entity_blob(ctx.c, (*C.uint8_t)(unsafe.Pointer(&blob[0])), C.size_t(len(blob)), &off, &w)
	if err := ctx.check(rc); err != nil {
		return nil, 0, err
	}
	return newWeight(w), int(off), nil
}

func (ctx *Context) FreeWeight(w *Weight) {
	if w.w != nil {
		C.loom_b200_weight_free(ctx.c, w.w)
		w.w = nil
	}
}

// ---- the three dispatchers (device buffers in, device buffers out) ----

// QuantizeActivation = DispatchBitNetQuantizeActivation: x [batch,n] fp32 -> q [batch,n] int8, amax [batch] fp32.
func (ctx *Context) QuantizeActivation(batch, n int, x, q, amax *Buffer) error {
	return ctx.check(C.loom_b200_quantize_activation(ctx.c, C.int(batch), C.int(n), (*C.float)(x.p), (*C.int8_t)(q.p), (*C.float)(amax.p)))
}

// TernaryLinear = DispatchDenseBitNetTernaryQuantized with bias, activation and residual fused; bias and residual may be nil.
func (ctx *Context) TernaryLinear(w *Weight, batch int, q, amax, bias, residual *Buffer, act int, out *Buffer) error {
	var bp, rp *C.float
	if bias != nil {
		bp = (*C.float)(bias.p)
	}
	if residual != nil {
		rp = (*C.float)(residual.p)
	}
	return ctx.check(C.loom_b200_ternary_linear(ctx.c, w.w, C.int(batch), (*C.int8_t)(q.p), (*C.float)(amax.p), bp, rp, C.int(act),
		(*C.float)(out.p), nil))
}

// GateProduct = DispatchBitNetGateProduct.
func (ctx *Context) GateProduct(batch, hidden, act int, gate, up, out *Buffer) error {
	return ctx.check(C.loom_b200_gate_product(ctx.c, C.int(batch), C.int(hidden), C.int(act), (*C.float)(gate.p), (*C.float)(up.p), (*C.float)(out.p)))
}

// ---- layer forwards (host tensors in and out, like the *PackedTernaryCPU functions) ----

func f32ptr(s []float32) *C.float {
	if len(s) == 0 {
		return nil
	}
	return (*C.float)(unsafe.Pointer(&s[0]))
}

// DenseForward = DenseForwardPackedTernaryCPU: in [batch,cols] -> pre, post [batch,rows].
func (ctx *Context) DenseForward(w *Weight, act int, in []float32, batch int, pre, post []float32) error {
	return ctx.check(C.loom_b200_dense_forward(ctx.c, w.w, C.int(act), f32ptr(in), C.int(batch), f32ptr(pre), f32ptr(post)))
}

// SwiGLUForward = SwiGLUForwardPackedTernaryCPU.
func (ctx *Context) SwiGLUForward(gate, up, down *Weight, biasGate, biasUp, biasDown, innerNorm []float32, rmsEps float64, act int,
	in []float32, seq int, pre, post []float32) error {
	return ctx.check(C.loom_b200_swiglu_forward(ctx.c, gate.w, up.w, down.w, f32ptr(biasGate), f32ptr(biasUp), f32ptr(biasDown),
		f32ptr(innerNorm), C.int(len(innerNorm)), C.double(rmsEps), C.int(act), f32ptr(in), C.int(seq), f32ptr(pre), f32ptr(post)))
}

// MHA = the attention layer with its KV ring on the device (MHAForwardPackedTernaryCPU).
type MHA struct {
	ctx *Context
	m   *C.loom_b200_mha
}

type MHAConfig struct {
	DModel, NumHeads, NumKVHeads, HeadDim, MaxSeqLen int
	RoPETheta, RMSNormEps                            float64
	BQ, BK, BV, BO, QNorm, KNorm, InnerNorm           []float32
}

func (ctx *Context) NewMHA(cfg MHAConfig, wq, wk, wv, wo *Weight) (*MHA, error) {
	var m *C.loom_b200_mha
	rc := C.loom_b200_mha_create(ctx.c, C.int(cfg.DModel), C.int(cfg.NumHeads), C.int(cfg.NumKVHeads), C.int(cfg.HeadDim),
		C.int(cfg.MaxSeqLen), C.double(cfg.RoPETheta), C.double(cfg.RMSNormEps), wq.w, wk.w, wv.w, wo.w,
		f32ptr(cfg.BQ), f32ptr(cfg.BK), f32ptr(cfg.BV), f32ptr(cfg.BO), f32ptr(cfg.QNorm), C.int(len(cfg.QNorm)),
		f32ptr(cfg.KNorm), C.int(len(cfg.KNorm)), f32ptr(cfg.InnerNorm), C.int(len(cfg.InnerNorm)), &m)
	if err := ctx.check(rc); err != nil {
		return nil, err
	}
	return &MHA{ctx, m}, nil
}

func (m *MHA) Forward(in []float32, batch, seq int, pre, post []float32) error {
	return m.ctx.check(C.loom_b200_mha_forward(m.m, f32ptr(in), C.int(batch), C.int(seq), f32ptr(pre), f32ptr(post)))
}
func (m *MHA) Reset() error  { return m.ctx.check(C.loom_b200_mha_reset(m.m)) }
func (m *MHA) KVOffset() int { return int(C.loom_b200_mha_kv_offset(m.m)) }
func (m *MHA) Close() {
	if m.m != nil {
		C.loom_b200_mha_destroy(m.m)
		m.m = nil
	}
}

// ---- the decoder stack (InitHFDecoderBlocks + Transformer on this path) ----

type DecoderDims struct {
	NumLayers, Hidden, NumHeads, NumKVHeads, HeadDim, Intermediate, Vocab int
	RMSEps, RoPETheta                                                      float64
	Activation, MaxSeqLen                                                   int
}

type Decoder struct {
	ctx  *Context
	d    *C.loom_b200_decoder
	dims DecoderDims
}

func (ctx *Context) NewDecoder(dims DecoderDims) (*Decoder, error) {
	cd := C.loom_b200_decoder_dims{
		num_layers: C.int(dims.NumLayers), hidden: C.int(dims.Hidden), num_heads: C.int(dims.NumHeads),
		num_kv_heads: C.int(dims.NumKVHeads), head_dim: C.int(dims.HeadDim), intermediate: C.int(dims.Intermediate),
		vocab: C.int(dims.Vocab), rms_eps: C.double(dims.RMSEps), rope_theta: C.double(dims.RoPETheta),
		activation: C.int(dims.Activation), max_seq_len: C.int(dims.MaxSeqLen),
	}
	var d *C.loom_b200_decoder
	if err := ctx.check(C.loom_b200_decoder_create(ctx.c, &cd, &d)); err != nil {
		return nil, err
	}
	return &Decoder{ctx, d, dims}, nil
}

// SetBlock installs one decoder block: gains (nil = ones), the seven projections in slab order q, k, v, o, gate, up, down,
// and the inner-norm vectors (nil = none).
func (dec *Decoder) SetBlock(block int, norm1, norm2 []float32, w [7]*Weight, attnInner, ffnInner []float32) error {
	var arr [7]*C.loom_b200_weight
	for i := range w {
		arr[i] = w[i].w
	}
	// the array of handles is C memory for the duration of the call (cgo forbids Go pointers to Go pointers)
	cw := (**C.loom_b200_weight)(C.malloc(C.size_t(7 * unsafe.Sizeof(arr[0]))))
	defer C.free(unsafe.Pointer(cw))
	copy((*[7]*C.loom_b200_weight)(unsafe.Pointer(cw))[:], arr[:])
	return dec.ctx.check(C.loom_b200_decoder_set_block(dec.d, C.int(block), f32ptr(norm1), f32ptr(norm2), cw,
		f32ptr(attnInner), C.int(len(attnInner)), f32ptr(ffnInner), C.int(len(ffnInner))))
}

// SetEmbeddings takes the tied fp32 embedding / LM head in device memory and the final norm gain.
func (dec *Decoder) SetEmbeddings(emb *Buffer, finalGain []float32) error {
	return dec.ctx.check(C.loom_b200_decoder_set_embeddings(dec.d, (*C.float)(emb.p), f32ptr(finalGain)))
}

// Forward = ForwardTokenIDsWGPU(tokens, nil, true, true): logits of the last token (nil to skip the read-back).
func (dec *Decoder) Forward(tokens []int32, logits []float32) error {
	return dec.ctx.check(C.loom_b200_decoder_forward(dec.d, (*C.int32_t)(unsafe.Pointer(&tokens[0])), C.int(len(tokens)), f32ptr(logits)))
}

// Generate = Transformer.Generate with greedy sampling; the loop runs on the device.
func (dec *Decoder) Generate(prompt []int32, maxNew int) ([]int32, error) {
	out := make([]int32, maxNew+1)
	rc := C.loom_b200_decoder_generate(dec.d, (*C.int32_t)(unsafe.Pointer(&prompt[0])), C.int(len(prompt)), C.int(maxNew),
		(*C.int32_t)(unsafe.Pointer(&out[0])), nil)
	return out[:maxNew], dec.ctx.check(rc)
}

// Continue runs `steps` greedy steps on the device without waiting (the body of Generate's loop); ReadTokens returns the
// last n tokens the loop fed to a forward.
func (dec *Decoder) Continue(steps int) error {
	return dec.ctx.check(C.loom_b200_decoder_continue(dec.d, C.int(steps)))
}

func (dec *Decoder) ReadTokens(n int) ([]int32, error) {
	out := make([]int32, n)
	rc := C.loom_b200_decoder_read_tokens(dec.d, (*C.int32_t)(unsafe.Pointer(&out[0])), C.int(n))
	return out, dec.ctx.check(rc)
}

// SetLMHeadTernary installs an untied LM head given as a packed ternary matrix [vocab, hidden]
// (poly/transformer.go:721-755); nil returns to the tied fp32 head.
func (dec *Decoder) SetLMHeadTernary(head *Weight) error {
	var w *C.loom_b200_weight
	if head != nil {
		w = head.w
	}
	return dec.ctx.check(C.loom_b200_decoder_set_lm_head_ternary(dec.d, w))
}

// SetKVOffset cuts the selected sequence back to an earlier position (the rings are not cleared).
func (dec *Decoder) SetKVOffset(kvOffset int) error {
	return dec.ctx.check(C.loom_b200_decoder_set_kv_offset(dec.d, C.int(kvOffset)))
}

// UploadCache restores the first kvOffset rows of a block's KV rings from host memory (position-major, like the cache
// the CPU path keeps, poly/mha.go:269-270).
func (dec *Decoder) UploadCache(block, kvOffset int, k, v []float32) error {
	return dec.ctx.check(C.loom_b200_decoder_upload_cache(dec.d, C.int(block), C.int(kvOffset), f32ptr(k), f32ptr(v)))
}

// ---- independent sequences on one decoder (the reference shares one KV ring across a batch, poly/mha.go:258-270) ----

// SetBatch gives the decoder `batch` sequences with KV rings of their own; call it before the first SetBlock.
func (dec *Decoder) SetBatch(batch int) error {
	return dec.ctx.check(C.loom_b200_decoder_set_batch(dec.d, C.int(batch)))
}

// Select picks the sequence the single-sequence calls (Forward for its prompt, KVOffset, Reset ...) act on.
func (dec *Decoder) Select(seq int) error {
	return dec.ctx.check(C.loom_b200_decoder_select(dec.d, C.int(seq)))
}

// StepBatch forwards one token per sequence (nil: continue greedily) and returns the logits [batch*vocab] (nil to skip).
func (dec *Decoder) StepBatch(tokens []int32, logits []float32) error {
	var t *C.int32_t
	if len(tokens) > 0 {
		t = (*C.int32_t)(unsafe.Pointer(&tokens[0]))
	}
	return dec.ctx.check(C.loom_b200_decoder_step_batch(dec.d, t, f32ptr(logits)))
}

// ContinueBatch runs `steps` greedy steps for all sequences on the device without waiting.
func (dec *Decoder) ContinueBatch(steps int) error {
	return dec.ctx.check(C.loom_b200_decoder_continue_batch(dec.d, C.int(steps)))
}

// ReadTokensBatch returns the last n tokens every sequence fed to a forward, [batch][n] flattened.
func (dec *Decoder) ReadTokensBatch(batch, n int) ([]int32, error) {
	out := make([]int32, batch*n)
	rc := C.loom_b200_decoder_read_tokens_batch(dec.d, (*C.int32_t)(unsafe.Pointer(&out[0])), C.int(n))
	return out, dec.ctx.check(rc)
}

func (dec *Decoder) Reset() error  { return dec.ctx.check(C.loom_b200_decoder_reset(dec.d)) }
func (dec *Decoder) KVOffset() int { return int(C.loom_b200_decoder_kv_offset(dec.d)) }
func (dec *Decoder) Close() {
	if dec.d != nil {
		C.loom_b200_decoder_destroy(dec.d)
		dec.d = nil
	}
}

// ---- tensor parallelism: one process (or one pinned goroutine + context) per GPU ----

// TPUniqueID is created by rank 0 and handed to every rank by any transport.
func TPUniqueID() ([128]byte, error) {
	var id [128]byte
	if rc := C.loom_b200_tp_unique_id((*C.uint8_t)(unsafe.Pointer(&id[0]))); rc != 0 {
		return id, &Error{int(rc), C.GoString(C.loom_b200_last_error(nil))}
	}
	return id, nil
}

func (ctx *Context) TPInit(rank, world int, id [128]byte) error {
	return ctx.check(C.loom_b200_tp_init(ctx.c, C.int(rank), C.int(world), (*C.uint8_t)(unsafe.Pointer(&id[0]))))
}
