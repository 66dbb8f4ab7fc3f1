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
    float *cache_k = nullptr, *cache_v = nullptr;  // [msl, kv_dim]
    double* rope_div = nullptr;                    // [head_dim/2]
    int kv_offset = 0;                             // host mirror of KVOffset
    bool cache_live = false;
    // scratch for one chunk
    double *q = nullptr, *attn = nullptr, *part = nullptr;
    unsigned int* cnt = nullptr;
    int* pos_dev = nullptr;
    int splits = 1, max_total = 0;
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
};
// One chunk (M <= 8 tokens at positions *pos_dev ...): QKV -> q/k norm + RoPE -> attention -> inner norm -> O.
// Does not advance pos_dev.
int lb_mha_step_dev(loom_b200_mha* m, const LbMhaStepArgs& a);
int lb_mha_alloc(loom_b200_ctx* ctx, loom_b200_mha* m, int max_splits);
void lb_mha_release(loom_b200_mha* m);
