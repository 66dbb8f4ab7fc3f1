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

// Compile-time epilogue families (one kernel instantiation each).
enum LbEpi : int {
    LB_EPI_GENERIC = 0,  // per-segment LbOutKind, any activation, bias, residual, pre/acc side outputs
    LB_EPI_QKV = 1,      // segment 0 -> fp64 (query), segments 1,2 -> fp32 rows of the KV ring (poly/mha.go:274-283)
    LB_EPI_RESID = 2,    // float(y + bias) + residual (O and down projections; poly/mha.go:365, poly/swiglu.go:317)
    LB_EPI_SWIGLU = 3,   // gate/up pair -> float(gateProduct) (poly/swiglu.go:306-310)
    LB_EPI_TPSUM = 4,    // row-parallel shard: the partial sums of every rank meet through the peer mailboxes, then float(y + bias) + residual
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
    int ring_hd;            // with out_ring: the ring is head-major [rows/ring_hd][out_ring][ring_hd] (0 = position-major rows)
    int out_ring;  // > 0: token n goes to row (*pos_ptr + n) % out_ring of `out` (the KV ring), else row n
    // > 0: the tokens are independent sequences: token n writes row pos_ptr[n] % out_ring of the ring that starts
    // seq_stride elements after the ring of token n - 1
    long long seq_stride;
};

// Tokens one pass can carry for K input columns: the int8 activations of all tokens sit in shared memory beside a
// weight ring of at least two stages.  8 for every K up to ~19,000; 5 for K = 28,672.
int lb_gemv_max_tokens(int K);

struct LbGemvParams {
    LbGemvSeg seg[3];
    int nseg;
    int interleave2;  // 1: virtual strip v -> segment v&1, strip v>>1 (gate/up pairs)
    int group;        // strips per epilogue group (2 for gate/up pairs, else 1)
    int K, kblocks, M;
    int total_tiles;  // virtual strips * kblocks
    int max_local_strips;
    int stages;       // ring stages per warp (1..3)
    int stage_bytes;  // shared staging for the fp32/fp64 prologues (0 = use the slow generic prologue)
    int gain_bytes;   // shared copy of norm_w, made before the dependency wait (0 = read norm_w from global memory)
    int aligned;  // 1: CTAs own whole strip groups; 0: stream-K with the int32 fix-up
    // aligned partition without divisions in the kernel: CTA b owns groups [b*part_q + min(b, part_r), +part_q (+1 if b < part_r));
    // kb_magic = ceil(2^32 / kblocks) turns an offset below 65536 tiles into (strip, k-block) with one multiply
    int part_q, part_r;
    unsigned kb_magic;
    // prologue
    int pro;
    const void* x;
    const float* amax_in;
    const float* norm_w;  // gain / inner-norm weights or null
    int norm_w_len;
    double eps;
    const double* given_ss;   // optional [M]: sum of squares over the full vector (tensor-parallel row shards)
    const float* given_amax;  // optional [M]: absmax of the normalised full vector
    int norm_count;           // elements the mean runs over (0 = K)
    // Tensor-parallel row shard with LB_EPI_TPSUM: the epilogue exchanges the partial sums with the other ranks through
    // the peer mailboxes.  xchg_ctr[2] is the exchange's sequence number, xchg_ctr[4] counts the CTAs that are done; the
    // last one moves the sequence on.
    void* const* xchg_peers;
    int xchg_rank, xchg_world;
    unsigned int* xchg_ctr;
    int8_t* q_out;     // optional side outputs, written by CTA 0
    float* amax_out;
    float* norm_out;   // normalised row as float32 (what the layers report as preAct)
    // epilogue
    int epi;             // LbEpi
    const int* pos_ptr;  // device scalar: position of token 0 (KV ring rows), or null
    int act;
    const float* residual;  // [M, rows of segment 0] or null
    // stream-K fix-up scratch (zero between launches)
    int32_t* fix_acc;
    unsigned int* fix_cnt;
    int* status;
    unsigned long long* trace;  // optional row of 8 phase timestamps (ns) written by CTA 0, or null
};

// Launches the GEMV on ctx->stream (programmatic dependent launch unless disabled).
int lb_launch_gemv(loom_b200_ctx* ctx, const LbGemvParams& p);
// Fills in the derived fields (vstrip0, total_tiles, max_local_strips) and checks shapes.
int lb_gemv_finalize_params(loom_b200_ctx* ctx, LbGemvParams& p);

// The value a prologue hands to the quantizer for input x: block RMSNorm (x / rms) * g rounded to float32
// (poly/norm.go:102-138), inner RMSNorm (x * (1/rms)) * w rounded to float32 (poly/bitnet_cpu.go:893-913) or,
// on the float64 attention output, x * ((1/rms) * w) kept in float64 (poly/bitnet_cpu.go:868-887); plain rows pass through.
template <int PRO>
__device__ __forceinline__ double lb_pro_value(double x, double root, double rr, double w) {
    if (PRO == LB_PRO_BLOCKNORM) return (double)(float)__dmul_rn(lb_div_by(x, root, rr), w);
    if (PRO == LB_PRO_INNERNORM64) return __dmul_rn(x, __dmul_rn(rr, w));
    if (PRO == LB_PRO_INNERNORM) return (double)(float)__dmul_rn(__dmul_rn(x, rr), w);
    return x;
}

// Inputs at least this wide are normalised and quantized by one stand-alone launch (lb_launch_norm_quantize)
// instead of inside every CTA of the GEMV.
constexpr int kSplitQuantK = 8192;
constexpr int kSplitQuantTokens = 3;  // ... and so are passes of at least this many tokens
int lb_launch_norm_quantize(loom_b200_ctx* ctx, const LbGemvParams& p, int8_t* q, float* amax);
