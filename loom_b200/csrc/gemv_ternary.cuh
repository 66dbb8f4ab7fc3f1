// gemv_ternary.cuh -- parameter block of the packed-ternary decode GEMV (shared with the decoder).
#pragma once
#include "common.cuh"

// What the kernel does with the activations before the integer dot products.
enum LbPrologue : int {
    LB_PRO_Q8 = 0,          // x = int8 [M,K] already quantized, amax_in [M]
    LB_PRO_F32 = 1,         // x = fp32 [M,K]: absmax-quantize            (Dense; poly/dense.go:85-88)
    LB_PRO_BLOCKNORM = 2,   // x = fp32: RMSNorm with gain (x/rms*g), then quantize   (poly/norm.go:102-138)
    LB_PRO_INNERNORM = 3,   // x = fp32: inner norm (x*sc*w), then quantize           (poly/bitnet_cpu.go:893-913)
    LB_PRO_INNERNORM64 = 4, // x = fp64: inner norm in fp64, quantize from fp64       (poly/bitnet_cpu.go:868-887)
};

// What happens to a finished row sum.
enum LbOutKind : int {
    LB_OUT_F32 = 0,    // float(y + bias) -> Activate -> (+ residual)
    LB_OUT_F64 = 1,    // y + bias kept in fp64 (the MHA query)
    LB_OUT_SWIGLU = 2, // segments 0/1 are gate/up, interleaved strip by strip: float(gateProduct(yg+bg, yu+bu))
    LB_OUT_ACC = 3,    // raw int32 accumulators only
};

struct LbGemvSeg {
    const uint32_t* tiles;  // tiled weights of this matrix
    const float* bias;      // [rows] or null
    void* out;              // [M, rows] (float or double by kind); null = discard
    float* pre_out;         // optional [M, rows] value before Activate (LB_OUT_F32)
    int32_t* acc_out;       // optional [M, rows] raw accumulators
    int rows;               // real rows
    int strips;             // padded rows / 16
    int vstrip0;            // first virtual strip (concatenated order)
    float scale;
    int kind;
};

struct LbGemvParams {
    LbGemvSeg seg[3];
    int nseg;
    int interleave2;  // 1: virtual strip v -> segment v&1, strip v>>1 (gate/up pairs)
    int group;        // strips per epilogue group (2 for gate/up pairs, else 1)
    int K, kblocks, M;
    int total_tiles;  // virtual strips * kblocks
    int max_local_strips;
    // prologue
    int pro;
    const void* x;
    const float* amax_in;
    const float* norm_w;  // gain / inner-norm weights or null
    int norm_w_len;
    double eps;
    int8_t* q_out;     // optional side outputs, written by CTA 0
    float* amax_out;
    void* norm_out;    // normalised row (float for 2/3, double for 4)
    // epilogue
    int act;
    const float* residual;  // [M, rows of segment 0] or null
    // stream-K fix-up scratch (zero between launches)
    int32_t* fix_acc;
    unsigned int* fix_cnt;
    int* status;
    int debug;  // timing experiments only: 1 = skip the arithmetic, 2 = skip the weight copies
};

// Launches the GEMV on ctx->stream (programmatic dependent launch unless disabled).
int lb_launch_gemv(loom_b200_ctx* ctx, const LbGemvParams& p);
// Fills in the derived fields (vstrip0, total_tiles, max_local_strips) and checks shapes.
int lb_gemv_finalize_params(loom_b200_ctx* ctx, LbGemvParams& p);
