// layers.cuh -- device-side building blocks of the packed-ternary Dense / SwiGLU / MHA layers, shared by the
// host-buffer layer calls (layers.cu) and the decoder loop (decoder.cu).
#pragma once
#include "gemv_ternary.cuh"
#include "glue.cuh"

constexpr int kChunkTokens = 8;  // tokens one GEMV pass carries in its N dimension

// SwiGLUForwardPackedTernaryCPU on device buffers for M <= 8 tokens.
struct LbSwigluArgs {
    const loom_b200_weight *gate, *up, *down;
    const float *bias_gate, *bias_up, *bias_down;  // device or null
    const float* inner_w;                          // device or null (InnerNormWeight)
    int inner_w_len;
    double inner_eps;  // <= 0 -> 1e-5
    int act;
    // input: either a plain row (pro_mode LB_PRO_F32) or the block input with the RMSNorm fused in
    int pro_mode;
    const float* x;       // [M, hidden]
    const float* gain;    // block norm gain (LB_PRO_BLOCKNORM)
    double block_eps;
    float* prod;          // [M, inter] scratch: gate product before the inner norm
    float* pre_out;       // optional [M, inter]: normalised product (the layer's preAct)
    float* out;           // [M, hidden]
    const float* residual;  // optional [M, hidden], may alias out
    int M;
    // tensor parallelism: > 0 when gate/up hold a slice of the rows and down the matching slice of the columns;
    // the value is the unsharded intermediate size.  tp_stats: 2*M doubles, tp_acc: M*hidden int32 (device scratch).
    int inter_global = 0;
    double* tp_stats = nullptr;
    int32_t* tp_acc = nullptr;
};
int lb_swiglu_dev(loom_b200_ctx* ctx, const LbSwigluArgs& a);

// The MHA layer state (VolumetricLayer fields used by MHAForwardPackedTernaryCPU, poly/mha.go:204-371).
struct loom_b200_mha {
    loom_b200_ctx* ctx = nullptr;
    int d_model = 0, heads = 0, kv_heads = 0, head_dim = 0, q_dim = 0, kv_dim = 0, msl = 0;
    double theta = 10000.0, rms_eps = 0.0;
    const loom_b200_weight *wq = nullptr, *wk = nullptr, *wv = nullptr, *wo = nullptr;  // borrowed
    float *bq = nullptr, *bk = nullptr, *bv = nullptr, *bo = nullptr;                     // device, owned
    float *q_norm = nullptr, *k_norm = nullptr, *inner = nullptr;
    int q_norm_len = 0, k_norm_len = 0, inner_len = 0;
    float *cache_k = nullptr, *cache_v = nullptr;  // ring of the selected sequence: [kv_heads, msl, head_dim]
    float *cache_k_base = nullptr, *cache_v_base = nullptr;  // the allocation: `lanes` rings of ring_elems floats each
    int lanes = 1;                                 // independent sequences (one ring each)
    size_t ring_elems = 0;
    double* rope_div = nullptr;                    // [head_dim/2]
    int kv_offset = 0;                             // host mirror of KVOffset
    bool cache_live = false;
    // scratch for one chunk
    double *q = nullptr, *attn = nullptr, *part = nullptr;
    unsigned int* cnt = nullptr;
    int* pos_dev = nullptr;
    int splits = 1, max_total = 0;
    float* k_new = nullptr;                        // [kv_dim] the newest K row before RoPE (one-token steps with RoPE folded into attention)
    int attn_cluster = -1;                         // CTAs per KV head of the cluster attention (0 = not usable, -1 = not decided yet)
    int attn_cluster_lanes = -1;                   // the same for a pass of several sequences (clusters may run in waves)
    const float *next_k = nullptr, *next_v = nullptr;  // KV rings of the decoder block that follows (L2 prefetch), or null
    // tensor parallelism: > 0 when this object holds heads/world heads (wq/wk/wv row slices, wo a column slice);
    // the value is the unsharded heads*head_dim.  Scratch as for the SwiGLU arguments, borrowed from the decoder.
    int q_dim_global = 0;
    double* tp_stats = nullptr;
    int32_t* tp_acc = nullptr;
};

struct LbMhaStepArgs {
    int pro_mode;         // LB_PRO_F32 (layer call) or LB_PRO_BLOCKNORM (decoder: block norm fused)
    const float* x;       // [M, d_model]
    const float* gain;
    double block_eps;
    float* pre_out;       // optional [M, d_model]: normalised attention rows
    float* out;           // [M, d_model]
    const float* residual;  // optional, may alias out
    int M;
    int splits;           // attention splits along positions
    bool fold_rope;       // one-token step: let the attention kernel rotate q and the newest K row (no q/k norm only)
    // lanes_pos != null: the M tokens are independent sequences lane0 .. lane0+M-1, token n at position lanes_pos[n] of
    // its own ring (RoPE as a launch of its own, attention per (sequence, head))
    const int* lanes_pos = nullptr;
    int lane0 = 0;
};
// One chunk (M <= 8 tokens at positions *pos_dev ...): QKV -> q/k norm + RoPE -> attention -> inner norm -> O.
// Does not advance pos_dev.
int lb_mha_step_dev(loom_b200_mha* m, const LbMhaStepArgs& a);
// its three parts: the QKV projection, q/k norm + RoPE + attention, inner norm + output projection
int lb_mha_qkv_dev(loom_b200_mha* m, const LbMhaStepArgs& a);
int lb_mha_attn_dev(loom_b200_mha* m, const LbMhaStepArgs& a);
int lb_mha_o_dev(loom_b200_mha* m, const LbMhaStepArgs& a);
int lb_mha_alloc(loom_b200_ctx* ctx, loom_b200_mha* m, int max_splits, int lanes = 1);
void lb_mha_release(loom_b200_mha* m);

// ---- tensor parallelism (tp.cu) -------------------------------------------------------------------------
// NCCL data types and reductions by their ABI values (the library is loaded at run time)
constexpr int kTpInt32 = 2, kTpFloat32 = 7, kTpFloat64 = 8, kTpSum = 0, kTpMax = 2;
int lb_tp_allreduce(loom_b200_ctx* ctx, void* buf, size_t count, int dtype, int op);
int lb_tp_allgather_f32(loom_b200_ctx* ctx, const float* send, float* recv, size_t count_per_rank);
// Row-parallel projection of a token block (prompts under a tensor-parallel group), the pieces around the GEMM:
// per-token statistics of the whole row from this rank's slice x [M, Kl] (partial sum of squares -> all-reduce ->
// partial absmax of the normalised slice -> all-reduce), and the float epilogue after the int32 all-reduce of the
// accumulators: out = float(acc * os + bias) + residual.
int lb_tp_block_stats(loom_b200_ctx* ctx, bool x_is_f64, const void* x, int M, int Kl, int K_global, double eps, const float* inner_w,
                      int inner_w_len, double* ss, float* amax);
int lb_tp_block_finalize(loom_b200_ctx* ctx, int32_t* acc, int M, int rows, float scale, const float* amax, const float* bias,
                         const float* residual, float* out);
// Row-sharded ternary linear whose inner RMSNorm spans the sharded dimension: x_local [M, w->cols] (float or double)
// -> out [M, w->rows] (+ residual), identical on every rank.  stats: 2*M doubles of scratch; acc: M*w->rows int32.
int lb_tp_rowsharded_linear(loom_b200_ctx* ctx, const loom_b200_weight* w, bool x_is_f64, const void* x, int M, int K_global,
                            const float* inner_w, int inner_w_len, double eps, const float* bias, const float* residual,
                            float* out, double* stats, int32_t* acc);

// ---- token blocks on the tensor cores (gemm_ternary_i8.cu) ------------------------------------------------
// A block of tokens is quantized once (optionally through a block or inner RMSNorm, LbPrologue) into the
// context's GEMM scratch, then any number of projections run against those int8 rows.
struct LbGemmQuant {
    int pro;              // LbPrologue: LB_PRO_F32, LB_PRO_BLOCKNORM, LB_PRO_INNERNORM, LB_PRO_INNERNORM64
    const void* x;        // [tokens, K] float32 (float64 for LB_PRO_INNERNORM64)
    int K, tokens;
    const float* norm_w;  // gain / inner-norm weight or null
    int norm_w_len;
    double eps;
    float* norm_out;      // optional [tokens, K]: the normalised rows as float32
    // tensor-parallel row shard (x is this rank's slice): statistics of the whole row, agreed between the ranks
    const double* given_ss;   // [tokens] sum of squares over the whole row, or null
    const float* given_amax;  // [tokens] absmax of the normalised whole row, or null
    int norm_count;           // elements the mean runs over (0 = K)
};
struct LbGemmOut {
    const float* bias;      // [rows] or null
    const float* residual;  // [tokens, rows] or null, may alias out
    int act;
    float* out;             // [tokens, rows] float32 or null
    double* out_f64;        // [tokens, rows] float64 (before rounding and activation) or null
    float* pre_out;         // [tokens, rows] value before the activation or null
    int32_t* acc_out;       // [tokens, rows] raw accumulators or null
    // kv_hd > 0: `out` is a head-major KV ring [rows/kv_hd][kv_msl][kv_hd] and token t is written at position kv_pos0 + t
    int kv_hd, kv_msl, kv_pos0;
};
int lb_gemm_quantize(loom_b200_ctx* ctx, const LbGemmQuant& a);
int lb_gemm_run(loom_b200_ctx* ctx, const loom_b200_weight* w, int tokens, const LbGemmOut& o);
// gate and up projections fused with the gate product (needs the pre-expanded codes; LOOM_B200_ERR_UNSUPPORTED otherwise)
int lb_gemm_run_swiglu(loom_b200_ctx* ctx, const loom_b200_weight* gate, const loom_b200_weight* up, int tokens, const float* bias_g,
                       const float* bias_u, int act, float* prod);
// gate product from the raw accumulators of the gate and up projections of the block quantized last (K columns)
int lb_gemm_gate_product(loom_b200_ctx* ctx, const int32_t* acc_g, const int32_t* acc_u, int tokens, int inter, int K, float scale_g,
                         float scale_u, const float* bias_g, const float* bias_u, int act, float* prod);
constexpr int kGemmMinTokens = 32;  // from this many tokens on a projection runs on the tensor cores
