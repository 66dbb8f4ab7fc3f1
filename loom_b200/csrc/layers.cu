// layers.cu -- packed-ternary Dense / SwiGLU / MHA layer forwards behind the C ABI.
// Reference: DenseForwardPackedTernaryCPU (poly/dense.go:66-101), SwiGLUForwardPackedTernaryCPU
// (poly/swiglu.go:270-322), MHAForwardPackedTernaryCPU (poly/mha.go:204-371).
#include "layers.cuh"

#include <cmath>
#include <vector>

int lb_ternary_gemm(loom_b200_ctx* ctx, const loom_b200_weight* w, int tokens, const float* x, const float* bias,
                    const float* residual, int activation, float* out, float* pre_out, int32_t* acc_out, float* amax_out);

namespace {

void fill_seg(LbGemvSeg& s, const loom_b200_weight* w, const float* bias, void* out) {
    s = LbGemvSeg{};
    s.tiles = w->tiles;
    s.rows = w->rows;
    s.scale = w->scale;
    s.bias = bias;
    s.out = out;
}

}  // namespace

int lb_swiglu_dev(loom_b200_ctx* ctx, const LbSwigluArgs& a) {
    const int H = a.gate->cols, I = a.gate->rows;
    LB_REQUIRE(ctx, a.up->cols == H && a.up->rows == I && a.down->cols == I && a.down->rows == H,
               "swiglu: gate %dx%d, up %dx%d, down %dx%d do not fit together", a.gate->rows, a.gate->cols, a.up->rows,
               a.up->cols, a.down->rows, a.down->cols);
    // gate + up, one quantization shared by both, gate product in the epilogue
    LbGemvParams p = {};
    p.nseg = 2;
    fill_seg(p.seg[0], a.gate, a.bias_gate, a.prod);
    fill_seg(p.seg[1], a.up, a.bias_up, nullptr);
    p.K = H;
    p.M = a.M;
    p.pro = a.pro_mode;
    p.x = a.x;
    p.norm_w = a.gain;
    p.norm_w_len = a.gain ? H : 0;
    p.eps = a.block_eps;
    p.epi = LB_EPI_SWIGLU;
    p.act = a.act;
    if (int rc = lb_gemv_finalize_params(ctx, p)) return rc;
    if (int rc = lb_launch_gemv(ctx, p)) return rc;
    if (a.inter_global > 0 && ctx->tp_world > 1) {
        LB_REQUIRE(ctx, a.pre_out == nullptr && a.tp_stats && a.tp_acc, "swiglu: sharded down projection without scratch");
        return lb_tp_rowsharded_linear(ctx, a.down, false, a.prod, a.M, a.inter_global, a.inner_w, a.inner_w_len,
                                       a.inner_eps > 0 ? a.inner_eps : 1e-5, a.bias_down, a.residual, a.out, a.tp_stats, a.tp_acc);
    }
    // inner RMSNorm (always applied) + requantize + down projection (+ bias, + residual)
    LbGemvParams d = {};
    d.nseg = 1;
    fill_seg(d.seg[0], a.down, a.bias_down, a.out);
    d.K = I;
    d.M = a.M;
    d.pro = LB_PRO_INNERNORM;
    d.x = a.prod;
    d.norm_w = a.inner_w;
    d.norm_w_len = a.inner_w ? a.inner_w_len : 0;
    d.eps = a.inner_eps > 0 ? a.inner_eps : 1e-5;
    d.norm_out = a.pre_out;
    d.epi = LB_EPI_RESID;
    d.residual = a.residual;
    d.act = LOOM_B200_ACT_LINEAR;
    if (int rc = lb_gemv_finalize_params(ctx, d)) return rc;
    return lb_launch_gemv(ctx, d);
}

int lb_mha_alloc(loom_b200_ctx* ctx, loom_b200_mha* m, int max_splits, int lanes) {
    m->ctx = ctx;
    m->lanes = lanes < 1 ? 1 : lanes;
    m->ring_elems = (size_t)m->msl * m->kv_dim;
    const size_t cache = m->ring_elems * sizeof(float) * m->lanes;
    LB_CUDA(ctx, cudaMalloc(&m->cache_k_base, cache));
    LB_CUDA(ctx, cudaMalloc(&m->cache_v_base, cache));
    LB_CUDA(ctx, cudaMemsetAsync(m->cache_k_base, 0, cache, ctx->stream));
    LB_CUDA(ctx, cudaMemsetAsync(m->cache_v_base, 0, cache, ctx->stream));
    m->cache_k = m->cache_k_base;
    m->cache_v = m->cache_v_base;
    LB_CUDA(ctx, cudaMalloc(&m->q, (size_t)kChunkTokens * m->q_dim * sizeof(double)));
    LB_CUDA(ctx, cudaMalloc(&m->attn, (size_t)kChunkTokens * m->q_dim * sizeof(double)));
    LB_CUDA(ctx, cudaMalloc(&m->part, lb_attn_part_elems(kChunkTokens, m->heads, m->head_dim, max_splits) * sizeof(double)));
    LB_CUDA(ctx, cudaMalloc(&m->cnt, (size_t)kChunkTokens * m->heads * sizeof(unsigned int)));
    LB_CUDA(ctx, cudaMemsetAsync(m->cnt, 0, (size_t)kChunkTokens * m->heads * sizeof(unsigned int), ctx->stream));
    LB_CUDA(ctx, cudaMalloc(&m->k_new, (size_t)kChunkTokens * m->kv_dim * sizeof(float)));
    LB_CUDA(ctx, cudaMalloc(&m->pos_dev, sizeof(int)));
    LB_CUDA(ctx, cudaMemsetAsync(m->pos_dev, 0, sizeof(int), ctx->stream));
    // pow(theta, 2d/hd) in double on the host: the same libm call the CPU path makes once per use
    const int half = m->head_dim / 2;
    std::vector<double> div(half);
    for (int d = 0; d < half; ++d) div[d] = std::pow(m->theta, (double)(2 * d) / (double)m->head_dim);
    LB_CUDA(ctx, cudaMalloc(&m->rope_div, half * sizeof(double)));
    LB_CUDA(ctx, cudaMemcpyAsync(m->rope_div, div.data(), half * sizeof(double), cudaMemcpyHostToDevice, ctx->stream));
    LB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    m->splits = max_splits;
    return 0;
}

void lb_mha_release(loom_b200_mha* m) {
    void* ptrs[] = {m->bq, m->bk, m->bv, m->bo, m->q_norm, m->k_norm, m->inner, m->cache_k_base, m->cache_v_base,
                    m->rope_div, m->q, m->attn, m->part, m->cnt, m->pos_dev, m->k_new};
    for (void* p : ptrs)
        if (p) cudaFree(p);
}

// CTAs per KV head of the cluster attention for this layer's shape (0 = not usable); decided once
static int mha_cluster_size(loom_b200_mha* m, bool lanes = false) {
    int& slot = lanes ? m->attn_cluster_lanes : m->attn_cluster;
    if (slot < 0) {
        LbAttnParams t = {};
        t.M = 1;
        t.heads = m->heads;
        t.kv_heads = m->kv_heads;
        t.hd = m->head_dim;
        t.msl = m->msl;
        t.rope_div = m->rope_div;
        t.k_new = m->k_new;
        t.cache_k_w = m->cache_k;
        slot = m->ctx->opt_attn_cluster ? lb_attention_cluster_size(m->ctx, t, !lanes) : 0;
    }
    return slot;
}

// A pass of M sequences: the streaming kernel (one CTA per sequence and KV head) when that many CTAs fill a good part of
// the device or nothing else takes the shape; with few of them (tensor-parallel slices, few sequences) the cluster kernel's
// sixteen CTAs per (sequence, KV head) are faster (measured at the 8B shape: 64 CTAs 15.4 against 15.7 ms per step on one
// GPU, 32 CTAs 14.4 against 11.6 ms on two).
static bool mha_lanes_stream(loom_b200_mha* m, int M) {
    LbAttnParams t = {};
    t.heads = m->heads;
    t.kv_heads = m->kv_heads;
    t.hd = m->head_dim;
    if (!lb_attention_stream_supported(m->ctx, t)) return false;
    return m->kv_heads * M >= 48 || mha_cluster_size(m, true) == 0;
}

static bool mha_folds_rope(loom_b200_mha* m, const LbMhaStepArgs& a) {
    // one token of one sequence: RoPE goes into the attention kernel; one token of each of several sequences: only the
    // cluster kernel knows that layout, otherwise RoPE runs as a launch of its own
    if (!a.fold_rope || m->q_norm || m->k_norm || !m->ctx->opt_fold_rope || m->head_dim % 8 != 0) return false;
    if (a.lanes_pos) {
        // several sequences: the streaming kernel takes rotated queries and a complete ring (RoPE as a launch of its own)
        if (mha_lanes_stream(m, a.M)) return false;
        return mha_cluster_size(m, true) > 0;
    }
    return a.M == 1;
}

int lb_mha_qkv_dev(loom_b200_mha* m, const LbMhaStepArgs& a) {
    loom_b200_ctx* ctx = m->ctx;
    // Q (fp64), K and V (fp32, written straight into the ring rows of these positions)
    LbGemvParams p = {};
    p.nseg = 3;
    fill_seg(p.seg[0], m->wq, m->bq, m->q);
    fill_seg(p.seg[1], m->wk, m->bk, m->cache_k);
    fill_seg(p.seg[2], m->wv, m->bv, m->cache_v);
    const bool fold_rope = mha_folds_rope(m, a);
    p.seg[1].out_ring = m->msl;
    p.seg[2].out_ring = m->msl;
    p.seg[1].ring_hd = m->head_dim;
    p.seg[2].ring_hd = m->head_dim;
    if (a.lanes_pos) {  // one ring and one position per token
        p.seg[1].out = m->cache_k_base + (size_t)a.lane0 * m->ring_elems;
        p.seg[2].out = m->cache_v_base + (size_t)a.lane0 * m->ring_elems;
        p.seg[1].seq_stride = p.seg[2].seq_stride = (long long)m->ring_elems;
    }
    if (fold_rope) {  // the unrotated K row goes to a side buffer ([token][kv_dim]); the attention kernel rotates it into the ring
        p.seg[1].out = m->k_new;
        p.seg[1].out_ring = 0;
        p.seg[1].seq_stride = 0;
    }
    p.K = m->d_model;
    p.M = a.M;
    p.pro = a.pro_mode;
    p.x = a.x;
    p.norm_w = a.gain;
    p.norm_w_len = a.gain ? m->d_model : 0;
    p.eps = a.block_eps;
    p.epi = LB_EPI_QKV;
    p.pos_ptr = a.lanes_pos ? a.lanes_pos : m->pos_dev;
    p.act = LOOM_B200_ACT_LINEAR;
    if (int rc = lb_gemv_finalize_params(ctx, p)) return rc;
    return lb_launch_gemv(ctx, p);
}

int lb_mha_attn_dev(loom_b200_mha* m, const LbMhaStepArgs& a) {
    loom_b200_ctx* ctx = m->ctx;
    const bool fold_rope = mha_folds_rope(m, a);
    LbRopeParams r = {};
    r.q = m->q;
    r.cache_k = m->cache_k;
    r.pos_ptr = m->pos_dev;
    r.rope_div = m->rope_div;
    r.q_norm = m->q_norm;
    r.q_norm_len = m->q_norm_len;
    r.k_norm = m->k_norm;
    r.k_norm_len = m->k_norm_len;
    r.qk_eps = m->rms_eps > 0 ? m->rms_eps : 1e-6;
    r.M = a.M;
    r.heads = m->heads;
    r.kv_heads = m->kv_heads;
    r.hd = m->head_dim;
    r.msl = m->msl;
    if (a.lanes_pos) {
        r.cache_k = m->cache_k_base + (size_t)a.lane0 * m->ring_elems;
        r.pos_ptr = a.lanes_pos;
        r.seq_stride = (long long)m->ring_elems;
    }
    if (!fold_rope)
        if (int rc = lb_launch_rope(ctx, r)) return rc;

    LbAttnParams t = {};
    t.q = m->q;
    t.cache_k = m->cache_k;
    t.cache_v = m->cache_v;
    t.pos_ptr = m->pos_dev;
    t.out = m->attn;
    t.part = m->part;
    t.cnt = m->cnt;
    t.M = a.M;
    t.heads = m->heads;
    t.kv_heads = m->kv_heads;
    t.hd = m->head_dim;
    t.msl = m->msl;
    t.splits = a.splits < 1 ? 1 : (a.splits > m->splits ? m->splits : a.splits);
    t.max_chunk = (m->msl + t.splits - 1) / t.splits;
    if (a.lanes_pos) {
        t.cache_k = m->cache_k_base + (size_t)a.lane0 * m->ring_elems;
        t.cache_v = m->cache_v_base + (size_t)a.lane0 * m->ring_elems;
        t.pos_ptr = a.lanes_pos;
        t.seq_stride = (long long)m->ring_elems;
    }
    if (fold_rope) {
        t.rope_div = m->rope_div;
        t.k_new = m->k_new;
        t.cache_k_w = a.lanes_pos ? m->cache_k_base + (size_t)a.lane0 * m->ring_elems : m->cache_k;
        if (mha_cluster_size(m, a.lanes_pos != nullptr) > 0) {
            t.next_k = a.lanes_pos ? nullptr : m->next_k;  // (the prefetch follows one sequence's rings)
            t.next_v = a.lanes_pos ? nullptr : m->next_v;
            return lb_launch_attention_cluster(ctx, t, mha_cluster_size(m, a.lanes_pos != nullptr));
        }
    }
    if (a.lanes_pos && !fold_rope && mha_lanes_stream(m, a.M)) return lb_launch_attention_stream(ctx, t);
    return lb_launch_attention(ctx, t);
}

int lb_mha_o_dev(loom_b200_mha* m, const LbMhaStepArgs& a) {
    loom_b200_ctx* ctx = m->ctx;
    if (m->q_dim_global > 0 && ctx->tp_world > 1) {
        LB_REQUIRE(ctx, a.pre_out == nullptr && m->tp_stats && m->tp_acc, "mha: sharded output projection without scratch");
        return lb_tp_rowsharded_linear(ctx, m->wo, true, m->attn, a.M, m->q_dim_global, m->inner, m->inner_len,
                                       m->rms_eps > 0 ? m->rms_eps : 1e-5, m->bo, a.residual, a.out, m->tp_stats, m->tp_acc);
    }
    LbGemvParams o = {};
    o.nseg = 1;
    fill_seg(o.seg[0], m->wo, m->bo, a.out);
    o.K = m->q_dim;
    o.M = a.M;
    o.pro = LB_PRO_INNERNORM64;
    o.x = m->attn;
    o.norm_w = m->inner;
    o.norm_w_len = m->inner ? m->inner_len : 0;
    o.eps = m->rms_eps > 0 ? m->rms_eps : 1e-5;
    o.norm_out = a.pre_out;
    o.epi = LB_EPI_RESID;
    o.residual = a.residual;
    o.act = LOOM_B200_ACT_LINEAR;
    if (int rc = lb_gemv_finalize_params(ctx, o)) return rc;
    return lb_launch_gemv(ctx, o);
}

int lb_mha_step_dev(loom_b200_mha* m, const LbMhaStepArgs& a) {
    if (int rc = lb_mha_qkv_dev(m, a)) return rc;
    if (int rc = lb_mha_attn_dev(m, a)) return rc;
    return lb_mha_o_dev(m, a);
}

// ---- host-buffer layer calls (the C ABI) -------------------------------------------------------------

namespace {

// bump allocator over the context scratch buffer
struct Arena {
    char* base;
    size_t off = 0;
    explicit Arena(void* b) : base((char*)b) {}
    template <typename T>
    T* take(size_t n) {
        off = (off + 255) & ~(size_t)255;
        T* p = (T*)(base + off);
        off += n * sizeof(T);
        return p;
    }
};

size_t align256(size_t n) { return (n + 255) & ~(size_t)255; }

int upload_opt(loom_b200_ctx* ctx, const float* host, size_t n, float** dev) {
    *dev = nullptr;
    if (!host || n == 0) return 0;
    LB_CUDA(ctx, cudaMalloc(dev, n * sizeof(float)));
    LB_CUDA(ctx, cudaMemcpyAsync(*dev, host, n * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    LB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return 0;
}

}  // namespace

extern "C" {

int loom_b200_dense_forward(loom_b200_ctx* ctx, const loom_b200_weight* w, int activation, const float* in_host,
                            int batch, float* pre_host, float* post_host) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "dense_forward: ctx is NULL");
    LB_REQUIRE(ctx, w != nullptr, "dense_forward: weight is NULL");
    LB_REQUIRE(ctx, batch >= 0, "dense_forward: batch=%d", batch);
    if (batch == 0) return 0;
    LB_REQUIRE(ctx, in_host && (pre_host || post_host), "dense_forward: NULL buffer");
    if (ctx->capturing) return lb_fail(ctx, LOOM_B200_ERR_INVALID, "dense_forward takes host buffers and cannot be recorded");
    if (int rc = lb_set_device(ctx)) return rc;
    const int K = w->cols, N = w->rows;
    size_t need = align256((size_t)batch * K * 4) + 2 * align256((size_t)batch * N * 4) + 1024;
    if (int rc = lb_ensure_scratch(ctx, need)) return rc;
    Arena ar(ctx->scratch);
    float* x = ar.take<float>((size_t)batch * K);
    float* pre = ar.take<float>((size_t)batch * N);
    float* post = ar.take<float>((size_t)batch * N);
    LB_CUDA(ctx, cudaMemcpyAsync(x, in_host, (size_t)batch * K * 4, cudaMemcpyHostToDevice, ctx->stream));
    const int chunk = lb_gemv_max_tokens(K) < kChunkTokens ? lb_gemv_max_tokens(K) : kChunkTokens;
    // a block of tokens is a dense contraction: tensor cores (tcgen05) from kGemmMinTokens on, the GEMV below it
    if (batch >= kGemmMinTokens) {
        if (int rc = lb_ternary_gemm(ctx, w, batch, x, nullptr, nullptr, activation, post, pre, nullptr, nullptr)) return rc;
    } else
    for (int b0 = 0; b0 < batch; b0 += chunk) {
        LbGemvParams p = {};
        p.nseg = 1;
        fill_seg(p.seg[0], w, nullptr, post + (size_t)b0 * N);
        p.seg[0].pre_out = pre + (size_t)b0 * N;
        p.seg[0].kind = LB_OUT_F32;
        p.K = K;
        p.M = batch - b0 < chunk ? batch - b0 : chunk;
        p.pro = LB_PRO_F32;
        p.x = x + (size_t)b0 * K;
        p.epi = LB_EPI_GENERIC;
        p.act = activation;
        if (int rc = lb_gemv_finalize_params(ctx, p)) return rc;
        if (int rc = lb_launch_gemv(ctx, p)) return rc;
    }
    if (pre_host) LB_CUDA(ctx, cudaMemcpyAsync(pre_host, pre, (size_t)batch * N * 4, cudaMemcpyDeviceToHost, ctx->stream));
    if (post_host) LB_CUDA(ctx, cudaMemcpyAsync(post_host, post, (size_t)batch * N * 4, cudaMemcpyDeviceToHost, ctx->stream));
    LB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return 0;
}

int loom_b200_swiglu_forward(loom_b200_ctx* ctx, const loom_b200_weight* gate, const loom_b200_weight* up,
                             const loom_b200_weight* down, const float* bias_gate, const float* bias_up,
                             const float* bias_down, const float* inner_norm_w, int inner_norm_len, double rms_eps,
                             int activation, const float* in_host, int seq, float* pre_host, float* post_host) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "swiglu_forward: ctx is NULL");
    LB_REQUIRE(ctx, gate && up && down, "swiglu_forward: weight is NULL");
    LB_REQUIRE(ctx, seq >= 0, "swiglu_forward: seq=%d", seq);
    if (seq == 0) return 0;
    LB_REQUIRE(ctx, in_host && (pre_host || post_host), "swiglu_forward: NULL buffer");
    LB_REQUIRE(ctx, inner_norm_len >= 0 && (inner_norm_w || inner_norm_len == 0), "swiglu_forward: inner norm length without weights");
    if (ctx->capturing) return lb_fail(ctx, LOOM_B200_ERR_INVALID, "swiglu_forward takes host buffers and cannot be recorded");
    if (int rc = lb_set_device(ctx)) return rc;
    const int H = gate->cols, I = gate->rows;
    size_t need = 2 * align256((size_t)seq * H * 4) + 2 * align256((size_t)seq * I * 4) + 3 * align256((size_t)I * 4) +
                  align256((size_t)H * 4) + 4096;
    if (int rc = lb_ensure_scratch(ctx, need)) return rc;
    Arena ar(ctx->scratch);
    float* x = ar.take<float>((size_t)seq * H);
    float* out = ar.take<float>((size_t)seq * H);
    float* prod = ar.take<float>((size_t)seq * I);
    float* pre = ar.take<float>((size_t)seq * I);
    float* bg = bias_gate ? ar.take<float>(I) : nullptr;
    float* bu = bias_up ? ar.take<float>(I) : nullptr;
    float* iw = inner_norm_len > 0 ? ar.take<float>(inner_norm_len) : nullptr;
    float* bd = bias_down ? ar.take<float>(H) : nullptr;
    auto h2d = [&](float* d, const float* h, size_t n) {
        return d ? cudaMemcpyAsync(d, h, n * 4, cudaMemcpyHostToDevice, ctx->stream) : cudaSuccess;
    };
    LB_CUDA(ctx, h2d(x, in_host, (size_t)seq * H));
    LB_CUDA(ctx, h2d(bg, bias_gate, I));
    LB_CUDA(ctx, h2d(bu, bias_up, I));
    LB_CUDA(ctx, h2d(bd, bias_down, H));
    LB_CUDA(ctx, h2d(iw, inner_norm_w, inner_norm_len));
    const int sw_chunk = lb_gemv_max_tokens(I > H ? I : H) < kChunkTokens ? lb_gemv_max_tokens(I > H ? I : H) : kChunkTokens;
    for (int s0 = 0; s0 < seq; s0 += sw_chunk) {
        LbSwigluArgs a = {};
        a.gate = gate;
        a.up = up;
        a.down = down;
        a.bias_gate = bg;
        a.bias_up = bu;
        a.bias_down = bd;
        a.inner_w = iw;
        a.inner_w_len = inner_norm_len;
        a.inner_eps = rms_eps;
        a.act = activation;
        a.pro_mode = LB_PRO_F32;
        a.x = x + (size_t)s0 * H;
        a.prod = prod + (size_t)s0 * I;
        a.pre_out = pre + (size_t)s0 * I;
        a.out = out + (size_t)s0 * H;
        a.M = seq - s0 < sw_chunk ? seq - s0 : sw_chunk;
        if (int rc = lb_swiglu_dev(ctx, a)) return rc;
    }
    if (pre_host) LB_CUDA(ctx, cudaMemcpyAsync(pre_host, pre, (size_t)seq * I * 4, cudaMemcpyDeviceToHost, ctx->stream));
    if (post_host) LB_CUDA(ctx, cudaMemcpyAsync(post_host, out, (size_t)seq * H * 4, cudaMemcpyDeviceToHost, ctx->stream));
    LB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return 0;
}

int loom_b200_mha_create(loom_b200_ctx* ctx, int d_model, int num_heads, int num_kv_heads, int head_dim,
                         int max_seq_len, double rope_theta, double rms_eps, const loom_b200_weight* wq,
                         const loom_b200_weight* wk, const loom_b200_weight* wv, const loom_b200_weight* wo,
                         const float* bq, const float* bk, const float* bv, const float* bo, const float* q_norm_w,
                         int q_norm_len, const float* k_norm_w, int k_norm_len, const float* inner_norm_w,
                         int inner_norm_len, loom_b200_mha** out) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "mha_create: ctx is NULL");
    LB_REQUIRE(ctx, out != nullptr, "mha_create: out is NULL");
    *out = nullptr;
    LB_REQUIRE(ctx, wq && wk && wv && wo, "mha_create: weight is NULL");
    LB_REQUIRE(ctx, d_model > 0 && num_heads > 0 && head_dim > 0 && head_dim % 2 == 0, "mha_create: bad dimensions (head_dim must be even: RoPE rotates pairs)");
    if (num_kv_heads == 0) num_kv_heads = num_heads;
    LB_REQUIRE(ctx, num_heads % num_kv_heads == 0, "mha_create: %d heads over %d kv heads", num_heads, num_kv_heads);
    const int qd = num_heads * head_dim, kvd = num_kv_heads * head_dim;
    LB_REQUIRE(ctx, wq->rows == qd && wq->cols == d_model && wk->rows == kvd && wk->cols == d_model &&
                        wv->rows == kvd && wv->cols == d_model && wo->rows == d_model && wo->cols == qd,
               "mha_create: projection shapes do not match the layer dimensions");
    LB_REQUIRE(ctx, qd == d_model, "mha_create: query width %d != d_model %d is not supported", qd, d_model);
    if (ctx->capturing) return lb_fail(ctx, LOOM_B200_ERR_INVALID, "mha_create cannot be recorded");
    if (int rc = lb_set_device(ctx)) return rc;
    auto* m = new loom_b200_mha();
    m->d_model = d_model;
    m->heads = num_heads;
    m->kv_heads = num_kv_heads;
    m->head_dim = head_dim;
    m->q_dim = qd;
    m->kv_dim = kvd;
    m->msl = max_seq_len == 0 ? 512 : max_seq_len;  // poly/mha.go:217-220
    m->theta = rope_theta > 0 ? rope_theta : 10000.0;
    m->rms_eps = rms_eps;
    m->wq = wq;
    m->wk = wk;
    m->wv = wv;
    m->wo = wo;
    m->q_norm_len = q_norm_w ? q_norm_len : 0;
    m->k_norm_len = k_norm_w ? k_norm_len : 0;
    m->inner_len = inner_norm_w ? inner_norm_len : 0;
    int rc = lb_mha_alloc(ctx, m, 16);
    if (!rc) rc = upload_opt(ctx, bq, qd, &m->bq);
    if (!rc) rc = upload_opt(ctx, bk, kvd, &m->bk);
    if (!rc) rc = upload_opt(ctx, bv, kvd, &m->bv);
    if (!rc) rc = upload_opt(ctx, bo, d_model, &m->bo);
    if (!rc) rc = upload_opt(ctx, q_norm_w, m->q_norm_len, &m->q_norm);
    if (!rc) rc = upload_opt(ctx, k_norm_w, m->k_norm_len, &m->k_norm);
    if (!rc) rc = upload_opt(ctx, inner_norm_w, m->inner_len, &m->inner);
    if (rc) {
        lb_mha_release(m);
        delete m;
        return rc;
    }
    *out = m;
    return 0;
}

void loom_b200_mha_destroy(loom_b200_mha* m) {
    if (!m) return;
    if (m->ctx) {
        cudaSetDevice(m->ctx->device);
        cudaStreamSynchronize(m->ctx->stream);
    }
    lb_mha_release(m);
    delete m;
}

int loom_b200_mha_reset(loom_b200_mha* m) {
    if (!m) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "mha_reset: layer is NULL");
    m->kv_offset = 0;
    return 0;
}

int loom_b200_mha_kv_offset(const loom_b200_mha* m) { return m ? m->kv_offset : -1; }

int loom_b200_mha_forward(loom_b200_mha* m, const float* in_host, int batch, int seq, float* pre_host, float* post_host) {
    if (!m) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "mha_forward: layer is NULL");
    loom_b200_ctx* ctx = m->ctx;
    LB_REQUIRE(ctx, batch > 0 && seq > 0, "mha_forward: batch=%d seq=%d", batch, seq);
    LB_REQUIRE(ctx, in_host && (pre_host || post_host), "mha_forward: NULL buffer");
    if (ctx->capturing) return lb_fail(ctx, LOOM_B200_ERR_INVALID, "mha_forward takes host buffers and cannot be recorded");
    if (int rc = lb_set_device(ctx)) return rc;
    // mhaPrepareKVForForward, poly/mha_layout.go:62-70: the ring keeps its contents only for a one-token step
    const bool incremental = batch == 1 && seq == 1 && m->cache_live && m->kv_offset > 0;
    if (!incremental) {
        const size_t cache = (size_t)m->msl * m->kv_dim * sizeof(float);
        LB_CUDA(ctx, cudaMemsetAsync(m->cache_k, 0, cache, ctx->stream));
        LB_CUDA(ctx, cudaMemsetAsync(m->cache_v, 0, cache, ctx->stream));
        m->cache_live = true;
        m->kv_offset = 0;
    }
    const int total = batch * seq, D = m->d_model;
    LB_REQUIRE(ctx, m->kv_offset + total <= m->msl, "mha_forward: %d positions exceed MaxSeqLen %d (the reference's ring would wrap)", m->kv_offset + total, m->msl);
    size_t need = 3 * align256((size_t)total * D * 4) + 1024;
    if (int rc = lb_ensure_scratch(ctx, need)) return rc;
    Arena ar(ctx->scratch);
    float* x = ar.take<float>((size_t)total * D);
    float* pre = ar.take<float>((size_t)total * D);
    float* post = ar.take<float>((size_t)total * D);
    LB_CUDA(ctx, cudaMemcpyAsync(x, in_host, (size_t)total * D * 4, cudaMemcpyHostToDevice, ctx->stream));
    LB_CUDA(ctx, cudaMemcpyAsync(m->pos_dev, &m->kv_offset, sizeof(int), cudaMemcpyHostToDevice, ctx->stream));
    LB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    const int widest = m->q_dim > D ? m->q_dim : D;
    const int mh_chunk = lb_gemv_max_tokens(widest) < kChunkTokens ? lb_gemv_max_tokens(widest) : kChunkTokens;
    for (int s0 = 0; s0 < total; s0 += mh_chunk) {
        LbMhaStepArgs a = {};
        a.pro_mode = LB_PRO_F32;
        a.x = x + (size_t)s0 * D;
        a.pre_out = pre + (size_t)s0 * D;
        a.out = post + (size_t)s0 * D;
        a.M = total - s0 < mh_chunk ? total - s0 : mh_chunk;
        a.splits = a.M == 1 ? 8 : 1;
        if (int rc = lb_mha_step_dev(m, a)) return rc;
        if (int rc = lb_launch_add_scalar(ctx, m->pos_dev, a.M)) return rc;
    }
    m->kv_offset += total;
    if (pre_host) LB_CUDA(ctx, cudaMemcpyAsync(pre_host, pre, (size_t)total * D * 4, cudaMemcpyDeviceToHost, ctx->stream));
    if (post_host) LB_CUDA(ctx, cudaMemcpyAsync(post_host, post, (size_t)total * D * 4, cudaMemcpyDeviceToHost, ctx->stream));
    LB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return 0;
}

int loom_b200_mha_download_cache(loom_b200_mha* m, float* k_host, float* v_host) {
    if (!m) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "mha_download_cache: layer is NULL");
    loom_b200_ctx* ctx = m->ctx;
    if (int rc = lb_set_device(ctx)) return rc;
    // the device ring is head-major [kv head][position][hd]; the caller gets the reference's [position][kv head * hd]
    const size_t elems = (size_t)m->msl * m->kv_dim;
    std::vector<float> tmp(elems);
    for (int which = 0; which < 2; ++which) {
        float* host = which == 0 ? k_host : v_host;
        if (!host) continue;
        LB_CUDA(ctx, cudaMemcpyAsync(tmp.data(), which == 0 ? m->cache_k : m->cache_v, elems * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
        LB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        for (int h = 0; h < m->kv_heads; ++h)
            for (int pos = 0; pos < m->msl; ++pos)
                memcpy(host + (size_t)pos * m->kv_dim + (size_t)h * m->head_dim, tmp.data() + ((size_t)h * m->msl + pos) * m->head_dim,
                       (size_t)m->head_dim * sizeof(float));
    }
    LB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return 0;
}

}  // extern "C"
