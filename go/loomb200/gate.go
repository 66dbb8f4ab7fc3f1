// The routing gate of the B200 path, the counterpart of usePackedTernaryCPU (poly/bitnet_cpu.go:277-284).
//
// NOT COMPILED WHERE THIS LIBRARY IS BUILT (no Go toolchain in the build image).
package loomb200

// LayerState is what the gate looks at: the fields of poly.VolumetricLayer and poly.Network it needs, passed by value so
// that this package does not import poly.
type LayerState struct {
	UseExactDType  bool // Network.UseExactDType
	UseGPU         bool // Network.UseGPU
	IsTernary      bool // layer.DType == DTypeTernary
	HasWeightStore bool // layer.WeightStore != nil
}

// UsePackedTernaryB200 says whether a layer forward should go to this library.  It is the reference's gate with the GPU
// condition inverted: the CPU path runs when UseGPU is false (poly/bitnet_cpu.go:277-284), this one when it is true and a
// B200 context was opened.  There is no fallback inside the library: if this returns true and a call fails, the caller
// gets the error (and may decide to route the layer to the CPU path itself, as transformer.go:390-405 does today).
func UsePackedTernaryB200(s LayerState, ctx *Context) bool {
	return ctx != nil && ctx.c != nil && s.UseExactDType && s.UseGPU && s.IsTernary && s.HasWeightStore
}
