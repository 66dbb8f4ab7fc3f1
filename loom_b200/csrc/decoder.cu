// decoder.cu -- the decoder block loop on the GPU: the ternary branches of ForwardTokenIDsWGPU
// (poly/wgpu_forward.go:31-596) with the CPU path's arithmetic (forwardOnCPUNormal,
// poly/transformer_forward.go:220-253) and Generate's greedy loop (poly/transformer.go:341-485).
//
// One decode step is a single recorded frame (CUDA graph) of six launches per block -- QKV GEMV with the block
// RMSNorm fused in, q/k norm + RoPE, attention, O GEMV (+ inner norm, + residual), gate/up GEMV (+ block norm,
// + SwiGLU product), down GEMV (+ inner norm, + residual) -- followed by the fp32 LM head.  Positions, the
// current token and the output cursor live in device memory, so the same frame replays for every token and
// the greedy loop never waits for the host.
#include "layers.cuh"

#include <chrono>
#include <vector>

struct loom_b200_graph;  // defined in abi.cu

struct LbDecBlock {
    loom_b200_mha mha;
    const loom_b200_weight *gate = nullptr, *up = nullptr, *down = nullptr;
    float *g1 = nullptr, *g2 = nullptr;  // block RMSNorm gains [hidden]
    float* ffn_inner = nullptr;
    int ffn_inner_len = 0;
    bool ready = false;
};

struct loom_b200_decoder {
    loom_b200_ctx* ctx = nullptr;
    loom_b200_decoder_dims d{};
    std::vector<LbDecBlock> blocks;
    const float* emb = nullptr;  // borrowed device pointer [vocab, hidden]
    const loom_b200_weight* head_tern = nullptr;  // untied LM head as a packed ternary matrix [vocab, hidden] (borrowed), or null
    float* final_gain = nullptr;
    float *x = nullptr, *prod = nullptr, *logits = nullptr, *hidden = nullptr;
    int *tok = nullptr, *pos = nullptr, *step = nullptr, *out_tokens = nullptr;
    int out_cap = 0;
    int kv_offset = 0;
    int* h_tok = nullptr;       // pinned
    float* h_logits = nullptr;  // pinned [vocab]
    loom_b200_graph* step_graph = nullptr;
    int decode_splits = 16;
    // tensor parallelism: this rank's part of the stack (world 1 = everything)
    int tp_world = 1, tp_rank = 0;
    int heads_l = 0, kv_heads_l = 0, inter_l = 0;  // local heads, KV heads and intermediate units
    bool head_sharded = false;                     // LM head computed in vocabulary slices and gathered
    double* tp_stats = nullptr;
    int32_t* tp_acc = nullptr;
    // prompt blocks on the tensor cores: residual stream, queries, attention output, gate product and the raw
    // gate/up accumulators of up to pf_cap tokens
    int pf_cap = 0;
    int* pf_tok = nullptr;
    float *pf_x = nullptr, *pf_prod = nullptr;
    double *pf_q = nullptr, *pf_attn = nullptr;
    int32_t *pf_accg = nullptr, *pf_accu = nullptr;
    double* pf_ss = nullptr;  // tensor-parallel prompts: agreed per-token statistics
    float* pf_amax = nullptr;
    const float* last_resid = nullptr;  // residual stream of the last pass (x or pf_x) and its rows
    int last_resid_rows = 0;
    int step_launches = 0;              // kernels of one recorded decode step (without the argmax)
    // greedy step folded into the LM head's tail (one GPU, streaming head): the head's last CTA publishes the next token,
    // appends it to the output ring, advances the position and gathers the next embedding row, so a step is
    // {blocks, head} and needs no argmax, position or embedding launch
    bool fused_tail = false;
    // independent sequences ("lanes"): `batch` KV rings per block and one position, current token, output ring and logits
    // row per sequence.  The single-sequence calls act on the selected lane: pos, step, out_tokens, logits and cur_tok
    // point into the arrays below at that lane.
    int batch = 1, lane = 0;
    int *pos_all = nullptr, *step_all = nullptr, *tok_all = nullptr, *out_tokens_all = nullptr;
    float* logits_all = nullptr;
    int* cur_tok = nullptr;             // the current token of the selected lane (tok when there is one sequence)
    std::vector<int> kv_offsets;        // host mirror of every lane's position
    int* h_tok_all = nullptr;           // pinned [batch]
};

namespace {

constexpr int kPrefillBlock = 1024;  // prompt tokens per pass of the tensor-core path

void dec_free_prefill(loom_b200_decoder* dec) {
    void* ptrs[] = {dec->pf_tok, dec->pf_x, dec->pf_prod, dec->pf_q, dec->pf_attn, dec->pf_accg, dec->pf_accu, dec->pf_ss, dec->pf_amax};
    for (void* p : ptrs)
        if (p) cudaFree(p);
    dec->pf_tok = nullptr;
    dec->pf_x = dec->pf_prod = nullptr;
    dec->pf_q = dec->pf_attn = nullptr;
    dec->pf_accg = dec->pf_accu = nullptr;
    dec->pf_ss = nullptr;
    dec->pf_amax = nullptr;
    dec->pf_cap = 0;
}

int dec_ensure_prefill(loom_b200_decoder* dec, int tokens) {
    loom_b200_ctx* ctx = dec->ctx;
    if (tokens <= dec->pf_cap) return 0;
    LB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    dec_free_prefill(dec);
    const loom_b200_decoder_dims& d = dec->d;
    const size_t T = (size_t)tokens, qd = (size_t)d.num_heads * d.head_dim;  // (under a tensor-parallel group the slices need less)
    LB_CUDA(ctx, cudaMalloc(&dec->pf_tok, T * sizeof(int)));
    LB_CUDA(ctx, cudaMalloc(&dec->pf_x, T * d.hidden * sizeof(float)));
    LB_CUDA(ctx, cudaMalloc(&dec->pf_prod, T * d.intermediate * sizeof(float)));
    LB_CUDA(ctx, cudaMalloc(&dec->pf_q, T * qd * sizeof(double)));
    LB_CUDA(ctx, cudaMalloc(&dec->pf_attn, T * qd * sizeof(double)));
    LB_CUDA(ctx, cudaMalloc(&dec->pf_accg, T * d.intermediate * sizeof(int32_t)));
    LB_CUDA(ctx, cudaMalloc(&dec->pf_accu, T * d.intermediate * sizeof(int32_t)));
    if (dec->tp_world > 1) {  // agreed per-token statistics of the row-parallel projections; pf_accg doubles as their accumulator plane
        LB_REQUIRE(ctx, d.intermediate >= d.hidden, "decoder: prompts under a tensor-parallel group need intermediate >= hidden");
        LB_CUDA(ctx, cudaMalloc(&dec->pf_ss, T * sizeof(double)));
        LB_CUDA(ctx, cudaMalloc(&dec->pf_amax, T * sizeof(float)));
    }
    dec->pf_cap = tokens;
    return 0;
}

// Points the single-sequence state (position, output ring, logits row, current token, KV rings) at one lane.
void dec_point_at_lane(loom_b200_decoder* dec, int lane) {
    dec->lane = lane;
    dec->pos = dec->pos_all + lane;
    dec->step = dec->step_all + lane;
    dec->out_tokens = dec->out_tokens_all + (size_t)lane * dec->out_cap;
    dec->logits = dec->logits_all + (size_t)lane * dec->d.vocab;
    dec->cur_tok = dec->batch > 1 ? dec->tok_all + lane : dec->tok;
    dec->kv_offset = dec->kv_offsets.empty() ? 0 : dec->kv_offsets[lane];
    for (size_t i = 0; i < dec->blocks.size(); ++i) {
        LbDecBlock& b = dec->blocks[i];
        if (!b.ready) continue;
        loom_b200_mha& m = b.mha;
        m.cache_k = m.cache_k_base + (size_t)lane * m.ring_elems;
        m.cache_v = m.cache_v_base + (size_t)lane * m.ring_elems;
        m.pos_dev = dec->pos;
    }
    for (size_t i = 0; i + 1 < dec->blocks.size(); ++i) {  // the attention of a block prefetches the KV rows of the block after it
        if (dec->blocks[i].ready && dec->blocks[i + 1].ready) {
            dec->blocks[i].mha.next_k = dec->blocks[i + 1].mha.cache_k;
            dec->blocks[i].mha.next_v = dec->blocks[i + 1].mha.cache_v;
        }
    }
}

// Untied ternarised LM head (applyPackedTernaryLMHead, poly/transformer.go:736-755): the final RMSNorm is the GEMV's
// prologue, the logits are float32(packed matvec of the quantized normalised row).
int dec_head_ternary(loom_b200_decoder* dec, const float* x_row) {
    loom_b200_ctx* ctx = dec->ctx;
    LbGemvParams p = {};
    p.nseg = 1;
    p.seg[0].tiles = dec->head_tern->tiles;
    p.seg[0].rows = dec->head_tern->rows;
    p.seg[0].scale = dec->head_tern->scale;
    p.seg[0].out = dec->logits;
    p.seg[0].kind = LB_OUT_F32;
    p.K = dec->d.hidden;
    p.M = 1;
    p.pro = LB_PRO_BLOCKNORM;
    p.x = x_row;
    p.norm_w = dec->final_gain;
    p.norm_w_len = dec->d.hidden;
    p.eps = dec->d.rms_eps > 0 ? dec->d.rms_eps : 1e-6;
    p.norm_out = dec->hidden;
    p.epi = LB_EPI_GENERIC;
    p.act = LOOM_B200_ACT_LINEAR;
    if (int rc = lb_gemv_finalize_params(ctx, p)) return rc;
    return lb_launch_gemv(ctx, p);
}

// The greedy tail of a head launch that ends a pass of M tokens.
void dec_fill_tail(loom_b200_decoder* dec, LbLmHeadParams& h, int M) {
    h.tok_out = dec->cur_tok;
    h.out_tokens = dec->out_tokens;
    h.out_cap = dec->out_cap;
    h.step = dec->step;
    h.pos = dec->pos;
    h.pos_delta = M;
    h.emb = dec->emb;
    h.emb_vocab = dec->d.vocab;
    h.x_next = dec->x;
}

// Whether the fp32 head can carry the greedy step in its tail: the streaming kernel takes the table, and either one GPU
// or a vocabulary-sharded head whose ranks can exchange their (maximum, index) pairs through the peer mailboxes.
bool dec_tail_possible(const loom_b200_decoder* dec, const float* emb) {
    const loom_b200_ctx* ctx = dec->ctx;
    if (!lb_lm_head_streams(ctx, emb, dec->d.hidden)) return false;
    if (dec->tp_world == 1) return true;
    return dec->head_sharded && ctx->tp_peer && ctx->opt_tp_peer;
}

// this rank's vocabulary slice of the head and the mailbox exchange of its tail
void dec_shard_head(loom_b200_decoder* dec, LbLmHeadParams& h, float* logits_row) {
    loom_b200_ctx* ctx = dec->ctx;
    const int vl = dec->d.vocab / dec->tp_world;
    h.head = dec->emb + (size_t)dec->tp_rank * vl * dec->d.hidden;
    h.vocab = vl;
    h.logits = logits_row + (size_t)dec->tp_rank * vl;
    if (dec->fused_tail) {
        h.xchg_peers = (void* const*)ctx->peer_xbuf_dev;
        h.xchg_rank = dec->tp_rank;
        h.xchg_world = dec->tp_world;
        h.vocab_offset = dec->tp_rank * vl;
        h.xchg_ctr = ctx->x_ctr;
    }
}

// with the greedy step in the tail of a sharded head nothing in the step needs the whole row of logits: gather it only
// for a caller that reads it (every rank makes the same calls, so every rank gets here together)
int dec_gather_logits(loom_b200_decoder* dec, float* logits_row) {
    if (!(dec->head_sharded && dec->fused_tail)) return 0;
    const int vl = dec->d.vocab / dec->tp_world;
    return lb_tp_allgather_f32(dec->ctx, logits_row + (size_t)dec->tp_rank * vl, logits_row, (size_t)vl);
}

// A block of M prompt tokens (already in pf_tok) at positions pos0..pos0+M-1 through the whole stack, every
// projection as a token-block GEMM on the tensor cores.  Same arithmetic as dec_forward_chunk: the quantizer applies
// the same norms, the GEMM accumulates the same int32 sums, the epilogues rescale in float64.
int dec_prefill_block(loom_b200_decoder* dec, int M, int pos0, bool head) {
    loom_b200_ctx* ctx = dec->ctx;
    const loom_b200_decoder_dims& d = dec->d;
    const int H = d.hidden, I = dec->tp_world > 1 ? dec->inter_l : d.intermediate;
    const bool tp = dec->tp_world > 1;
    const double block_eps = d.rms_eps > 0 ? d.rms_eps : 1e-6;
    // Row-parallel projection of the block under a tensor-parallel group: statistics of the whole row agreed by two small
    // all-reduces, this rank's slice quantized with them, the GEMM writing raw int32 sums, one all-reduce of those, then
    // the float epilogue (same arithmetic as one GPU: integer sums are exact in any order).
    auto row_parallel = [&](const loom_b200_weight* w, bool f64, const void* x, int K_global, const float* inner_w, int inner_len,
                            double eps, const float* bias) -> int {
        if (int rc = lb_tp_block_stats(ctx, f64, x, M, w->cols, K_global, eps, inner_w, inner_len, dec->pf_ss, dec->pf_amax)) return rc;
        LbGemmQuant q = {};
        q.pro = f64 ? LB_PRO_INNERNORM64 : LB_PRO_INNERNORM;
        q.x = x;
        q.K = w->cols;
        q.tokens = M;
        q.norm_w = inner_w;
        q.norm_w_len = inner_w ? inner_len : 0;
        q.eps = eps;
        q.given_ss = dec->pf_ss;
        q.given_amax = dec->pf_amax;
        q.norm_count = K_global;
        if (int rc = lb_gemm_quantize(ctx, q)) return rc;
        LbGemmOut go = {};
        go.act = LOOM_B200_ACT_LINEAR;
        go.acc_out = dec->pf_accg;
        if (int rc = lb_gemm_run(ctx, w, M, go)) return rc;
        return lb_tp_block_finalize(ctx, dec->pf_accg, M, H, w->scale, dec->pf_amax, bias, dec->pf_x, dec->pf_x);
    };
    if (int rc = lb_launch_embed(ctx, dec->emb, d.vocab, H, dec->pf_tok, M, dec->pf_x)) return rc;
    for (auto& b : dec->blocks) {
        loom_b200_mha& m = b.mha;
        LbGemmQuant qa = {};
        qa.pro = LB_PRO_BLOCKNORM;
        qa.x = dec->pf_x;
        qa.K = H;
        qa.tokens = M;
        qa.norm_w = b.g1;
        qa.norm_w_len = H;
        qa.eps = block_eps;
        if (int rc = lb_gemm_quantize(ctx, qa)) return rc;
        LbGemmOut o = {};
        o.act = LOOM_B200_ACT_LINEAR;
        o.bias = m.bq;
        o.out_f64 = dec->pf_q;
        if (int rc = lb_gemm_run(ctx, m.wq, M, o)) return rc;
        o = LbGemmOut{};
        o.act = LOOM_B200_ACT_LINEAR;
        o.bias = m.bk;
        o.out = m.cache_k;  // head-major ring: token t of the block goes to position pos0 + t of every KV head (a prompt never wraps)
        o.kv_hd = m.head_dim;
        o.kv_msl = m.msl;
        o.kv_pos0 = pos0;
        if (int rc = lb_gemm_run(ctx, m.wk, M, o)) return rc;
        o.bias = m.bv;
        o.out = m.cache_v;
        if (int rc = lb_gemm_run(ctx, m.wv, M, o)) return rc;

        LbRopeParams r = {};
        r.q = dec->pf_q;
        r.cache_k = m.cache_k;
        r.pos_ptr = m.pos_dev;
        r.rope_div = m.rope_div;
        r.q_norm = m.q_norm;
        r.q_norm_len = m.q_norm_len;
        r.k_norm = m.k_norm;
        r.k_norm_len = m.k_norm_len;
        r.qk_eps = m.rms_eps > 0 ? m.rms_eps : 1e-6;
        r.M = M;
        r.heads = m.heads;
        r.kv_heads = m.kv_heads;
        r.hd = m.head_dim;
        r.msl = m.msl;
        if (int rc = lb_launch_rope(ctx, r)) return rc;

        LbAttnParams t = {};
        t.q = dec->pf_q;
        t.cache_k = m.cache_k;
        t.cache_v = m.cache_v;
        t.pos_ptr = m.pos_dev;
        t.out = dec->pf_attn;
        t.part = m.part;
        t.cnt = m.cnt;
        t.M = M;
        t.heads = m.heads;
        t.kv_heads = m.kv_heads;
        t.hd = m.head_dim;
        t.msl = m.msl;
        t.splits = 1;
        t.max_chunk = pos0 + M;
        if (lb_attention_prefill_supported(t)) {
            if (int rc = lb_launch_attention_prefill(ctx, t)) return rc;
        } else if (int rc = lb_launch_attention(ctx, t)) {
            return rc;
        }

        if (tp) {
            if (int rc = row_parallel(m.wo, true, dec->pf_attn, m.q_dim_global, m.inner, m.inner_len, m.rms_eps > 0 ? m.rms_eps : 1e-5, m.bo)) return rc;
        } else {
            qa = LbGemmQuant{};
            qa.pro = LB_PRO_INNERNORM64;
            qa.x = dec->pf_attn;
            qa.K = m.q_dim;
            qa.tokens = M;
            qa.norm_w = m.inner;
            qa.norm_w_len = m.inner ? m.inner_len : 0;
            qa.eps = m.rms_eps > 0 ? m.rms_eps : 1e-5;
            if (int rc = lb_gemm_quantize(ctx, qa)) return rc;
            o = LbGemmOut{};
            o.act = LOOM_B200_ACT_LINEAR;
            o.bias = m.bo;
            o.out = dec->pf_x;
            o.residual = dec->pf_x;
            if (int rc = lb_gemm_run(ctx, m.wo, M, o)) return rc;
        }

        qa = LbGemmQuant{};
        qa.pro = LB_PRO_BLOCKNORM;
        qa.x = dec->pf_x;
        qa.K = H;
        qa.tokens = M;
        qa.norm_w = b.g2;
        qa.norm_w_len = H;
        qa.eps = block_eps;
        if (int rc = lb_gemm_quantize(ctx, qa)) return rc;
        // gate and up as one GEMM with two accumulators and the gate product in its epilogue; without the pre-expanded
        // codes: two GEMMs that write raw accumulators, then the gate-product kernel
        int frc = lb_gemm_run_swiglu(ctx, b.gate, b.up, M, nullptr, nullptr, d.activation, dec->pf_prod);
        if (frc == LOOM_B200_ERR_UNSUPPORTED) {
            o = LbGemmOut{};
            o.act = LOOM_B200_ACT_LINEAR;
            o.acc_out = dec->pf_accg;
            if (int rc = lb_gemm_run(ctx, b.gate, M, o)) return rc;
            o.acc_out = dec->pf_accu;
            if (int rc = lb_gemm_run(ctx, b.up, M, o)) return rc;
            if (int rc = lb_gemm_gate_product(ctx, dec->pf_accg, dec->pf_accu, M, I, H, b.gate->scale, b.up->scale, nullptr, nullptr,
                                              d.activation, dec->pf_prod))
                return rc;
        } else if (frc) {
            return frc;
        }

        if (tp) {
            if (int rc = row_parallel(b.down, false, dec->pf_prod, d.intermediate, b.ffn_inner, b.ffn_inner_len, 1e-5, nullptr)) return rc;
            continue;
        }
        qa = LbGemmQuant{};
        qa.pro = LB_PRO_INNERNORM;
        qa.x = dec->pf_prod;
        qa.K = I;
        qa.tokens = M;
        qa.norm_w = b.ffn_inner;
        qa.norm_w_len = b.ffn_inner ? b.ffn_inner_len : 0;
        qa.eps = 1e-5;  // the decoder builder never sets RMSNormEps on the SwiGLU layer
        if (int rc = lb_gemm_quantize(ctx, qa)) return rc;
        o = LbGemmOut{};
        o.act = LOOM_B200_ACT_LINEAR;
        o.out = dec->pf_x;
        o.residual = dec->pf_x;
        if (int rc = lb_gemm_run(ctx, b.down, M, o)) return rc;
    }
    if (head && dec->head_tern) {
        if (int rc = dec_head_ternary(dec, dec->pf_x + (size_t)(M - 1) * H)) return rc;
    } else if (head) {
        LbLmHeadParams h = {};
        h.x = dec->pf_x + (size_t)(M - 1) * H;
        h.gain = dec->final_gain;
        h.eps = block_eps;
        h.head = dec->emb;
        h.vocab = d.vocab;
        h.hidden = H;
        h.logits = dec->logits;
        h.hidden_out = dec->hidden;
        if (dec->head_sharded) dec_shard_head(dec, h, dec->logits);
        if (dec->fused_tail) dec_fill_tail(dec, h, M);
        if (int rc = lb_launch_lm_head(ctx, h)) return rc;
        if (dec->head_sharded && !dec->fused_tail)
            if (int rc = lb_tp_allgather_f32(ctx, h.logits, dec->logits, (size_t)h.vocab)) return rc;
    }
    dec->last_resid = dec->pf_x;
    dec->last_resid_rows = M;
    if (head && dec->fused_tail) return 0;  // the head's tail advanced the position
    return lb_launch_add_scalar(ctx, dec->pos, M);
}

// linears_only: just the ternary projections of the step, on the step's own buffers (a measurement frame: the
// attention, the embedding, the head and the position update are left out, so nothing of the sequence state moves)
// embed: gather the rows of tok[0..M) first (false when the previous head's tail already left the row in x)
// tok_src: where the M token ids are (null = the staging buffer the host paths fill)
int dec_forward_chunk(loom_b200_decoder* dec, int M, int splits, bool head, int head_row, bool linears_only = false, bool embed = true,
                      const int* tok_src = nullptr) {
    loom_b200_ctx* ctx = dec->ctx;
    const loom_b200_decoder_dims& d = dec->d;
    if (!linears_only && embed)
        if (int rc = lb_launch_embed(ctx, dec->emb, d.vocab, d.hidden, tok_src ? tok_src : dec->tok, M, dec->x)) return rc;
    for (auto& b : dec->blocks) {
        LbMhaStepArgs a = {};
        a.pro_mode = LB_PRO_BLOCKNORM;
        a.x = dec->x;
        a.gain = b.g1;
        a.block_eps = d.rms_eps > 0 ? d.rms_eps : 1e-6;
        a.out = dec->x;
        a.residual = dec->x;
        a.M = M;
        a.splits = splits;
        a.fold_rope = M == 1;
        if (int rc = lb_mha_qkv_dev(&b.mha, a)) return rc;
        if (!linears_only)
            if (int rc = lb_mha_attn_dev(&b.mha, a)) return rc;
        if (int rc = lb_mha_o_dev(&b.mha, a)) return rc;
        LbSwigluArgs s = {};
        s.gate = b.gate;
        s.up = b.up;
        s.down = b.down;
        s.inner_w = b.ffn_inner;
        s.inner_w_len = b.ffn_inner_len;
        s.inner_eps = 0.0;  // the decoder builder never sets RMSNormEps on the SwiGLU layer: default 1e-5
        s.act = d.activation;
        s.pro_mode = LB_PRO_BLOCKNORM;
        s.x = dec->x;
        s.gain = b.g2;
        s.block_eps = d.rms_eps > 0 ? d.rms_eps : 1e-6;
        s.prod = dec->prod;
        s.out = dec->x;
        s.residual = dec->x;
        s.M = M;
        if (dec->tp_world > 1) {
            s.inter_global = d.intermediate;
            s.tp_stats = dec->tp_stats;
            s.tp_acc = dec->tp_acc;
        }
        if (int rc = lb_swiglu_dev(ctx, s)) return rc;
    }
    if (linears_only) return 0;
    if (head && dec->head_tern) {
        if (int rc = dec_head_ternary(dec, dec->x + (size_t)head_row * d.hidden)) return rc;
    } else if (head) {
        LbLmHeadParams h = {};
        h.x = dec->x + (size_t)head_row * d.hidden;
        h.gain = dec->final_gain;
        h.eps = d.rms_eps > 0 ? d.rms_eps : 1e-6;
        h.head = dec->emb;
        h.vocab = d.vocab;
        h.hidden = d.hidden;
        h.logits = dec->logits;
        h.hidden_out = dec->hidden;
        if (dec->head_sharded) dec_shard_head(dec, h, dec->logits);
        if (dec->fused_tail) dec_fill_tail(dec, h, M);
        if (int rc = lb_launch_lm_head(ctx, h)) return rc;
        if (dec->head_sharded && !dec->fused_tail)
            if (int rc = lb_tp_allgather_f32(ctx, h.logits, dec->logits, (size_t)h.vocab)) return rc;
    }
    dec->last_resid = dec->x;
    dec->last_resid_rows = M;
    if (head && dec->fused_tail) return 0;  // the head's tail advanced the position
    return lb_launch_add_scalar(ctx, dec->pos, M);
}

// One token for each of the sequences lane0 .. lane0+M-1 (M <= 8), every sequence at its own position of its own KV
// rings: the projections carry the M tokens in one pass over the weights (the same GEMV launches as an M-token chunk of
// one sequence), RoPE and attention run per (sequence, head), and the head serves several hidden rows per pass over the
// table.  Its tail publishes every sequence's next token and advances its position.
int dec_forward_lanes(loom_b200_decoder* dec, int lane0, int M) {
    loom_b200_ctx* ctx = dec->ctx;
    const loom_b200_decoder_dims& d = dec->d;
    const int H = d.hidden;
    if (int rc = lb_launch_embed(ctx, dec->emb, d.vocab, H, dec->tok_all + lane0, M, dec->x)) return rc;
    for (auto& b : dec->blocks) {
        LbMhaStepArgs a = {};
        a.pro_mode = LB_PRO_BLOCKNORM;
        a.x = dec->x;
        a.gain = b.g1;
        a.block_eps = d.rms_eps > 0 ? d.rms_eps : 1e-6;
        a.out = dec->x;
        a.residual = dec->x;
        a.M = M;
        a.splits = 4;
        a.fold_rope = true;
        a.lanes_pos = dec->pos_all + lane0;
        a.lane0 = lane0;
        if (int rc = lb_mha_step_dev(&b.mha, a)) return rc;
        LbSwigluArgs s = {};
        s.gate = b.gate;
        s.up = b.up;
        s.down = b.down;
        s.inner_w = b.ffn_inner;
        s.inner_w_len = b.ffn_inner_len;
        s.inner_eps = 0.0;
        s.act = d.activation;
        s.pro_mode = LB_PRO_BLOCKNORM;
        s.x = dec->x;
        s.gain = b.g2;
        s.block_eps = d.rms_eps > 0 ? d.rms_eps : 1e-6;
        s.prod = dec->prod;
        s.out = dec->x;
        s.residual = dec->x;
        s.M = M;
        if (dec->tp_world > 1) {
            s.inter_global = d.intermediate;
            s.tp_stats = dec->tp_stats;
            s.tp_acc = dec->tp_acc;
        }
        if (int rc = lb_swiglu_dev(ctx, s)) return rc;
    }
    const int rpp = lb_lm_head_rows_per_pass(ctx, dec->emb, H);
    LB_REQUIRE(ctx, rpp >= 1, "decoder: sequences in parallel need the streaming LM head");
    for (int r0 = 0; r0 < M; r0 += rpp) {
        LbLmHeadParams h = {};
        h.nb = M - r0 < rpp ? M - r0 : rpp;
        h.x = dec->x + (size_t)r0 * H;
        h.x_stride = H;
        h.gain = dec->final_gain;
        h.eps = d.rms_eps > 0 ? d.rms_eps : 1e-6;
        h.head = dec->emb;
        h.vocab = d.vocab;
        h.hidden = H;
        h.logits = dec->logits_all + (size_t)(lane0 + r0) * d.vocab;
        if (dec->head_sharded) dec_shard_head(dec, h, dec->logits_all + (size_t)(lane0 + r0) * d.vocab);
        h.logits_stride = d.vocab;
        h.tok_out = dec->tok_all + lane0 + r0;
        h.out_tokens = dec->out_tokens_all + (size_t)(lane0 + r0) * dec->out_cap;
        h.out_tokens_stride = dec->out_cap;
        h.out_cap = dec->out_cap;
        h.step = dec->step_all + lane0 + r0;
        h.pos = dec->pos_all + lane0 + r0;
        h.pos_delta = 1;
        if (int rc = lb_launch_lm_head(ctx, h)) return rc;
    }
    return 0;
}

int dec_check_ready(loom_b200_decoder* dec) {
    loom_b200_ctx* ctx = dec->ctx;
    LB_REQUIRE(ctx, dec->emb != nullptr, "decoder: embeddings are not set");
    for (size_t i = 0; i < dec->blocks.size(); ++i)
        LB_REQUIRE(ctx, dec->blocks[i].ready, "decoder: block %zu has no weights", i);
    return 0;
}

void dec_drop_graph(loom_b200_decoder* dec) {
    if (dec->step_graph) {
        loom_b200_graph_free(dec->ctx, dec->step_graph);
        dec->step_graph = nullptr;
    }
}

// One token at position *pos: eager the first time (sizes every scratch buffer), recorded after.  The token is tok[0];
// with the greedy tail folded into the head its embedding row is already in x unless the token came from the host
// (host_token), in which case it is gathered by a launch of its own in front of the recorded frame.
int dec_step(loom_b200_decoder* dec, bool host_token) {
    loom_b200_ctx* ctx = dec->ctx;
    const loom_b200_decoder_dims& d = dec->d;
    const bool in_frame = !dec->fused_tail;  // without the fused tail the gather is the first launch of the frame
    if (dec->fused_tail && host_token)
        if (int rc = lb_launch_embed(ctx, dec->emb, d.vocab, d.hidden, dec->cur_tok, 1, dec->x)) return rc;
    if (dec->step_graph) return loom_b200_graph_launch(ctx, dec->step_graph);
    if (dec->tp_world > 1 && !ctx->opt_tp_graph) return dec_forward_chunk(dec, 1, dec->decode_splits, true, 0, false, in_frame, dec->cur_tok);
    if (int rc = dec_forward_chunk(dec, 1, dec->decode_splits, true, 0, false, in_frame, dec->cur_tok)) return rc;  // warm-up run, counts as the step
    // record the same step for all later tokens
    if (int rc = loom_b200_graph_begin(ctx)) return rc;
    const uint64_t l0 = ctx->launches;
    int rc = dec_forward_chunk(dec, 1, dec->decode_splits, true, 0, false, in_frame, dec->cur_tok);
    dec->step_launches = (int)(ctx->launches - l0);
    loom_b200_graph* g = nullptr;
    int rc2 = loom_b200_graph_end(ctx, &g);
    if (rc) {
        if (g) loom_b200_graph_free(ctx, g);
        return rc;
    }
    if (rc2) return rc2;
    dec->step_graph = g;
    return 0;
}

}  // namespace

extern "C" {

int loom_b200_decoder_create(loom_b200_ctx* ctx, const loom_b200_decoder_dims* dims, loom_b200_decoder** out) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "decoder_create: ctx is NULL");
    LB_REQUIRE(ctx, dims && out, "decoder_create: NULL argument");
    *out = nullptr;
    const loom_b200_decoder_dims& d = *dims;
    LB_REQUIRE(ctx, d.num_layers > 0 && d.hidden > 0 && d.num_heads > 0 && d.head_dim > 0 && d.intermediate > 0 && d.vocab > 0,
               "decoder_create: bad dimensions");
    LB_REQUIRE(ctx, d.num_heads * d.head_dim == d.hidden, "decoder_create: heads*head_dim must equal hidden");
    LB_REQUIRE(ctx, d.head_dim % 2 == 0, "decoder_create: head_dim %d must be even (RoPE rotates pairs)", d.head_dim);
    if (ctx->capturing) return lb_fail(ctx, LOOM_B200_ERR_INVALID, "decoder_create cannot be recorded");
    if (int rc = lb_set_device(ctx)) return rc;
    const int W = ctx->tp_world, kvh = d.num_kv_heads == 0 ? d.num_heads : d.num_kv_heads;
    LB_REQUIRE(ctx, d.num_heads % W == 0 && kvh % W == 0 && d.intermediate % W == 0,
               "decoder_create: heads %d, kv heads %d and intermediate %d must be multiples of the group size %d", d.num_heads, kvh,
               d.intermediate, W);
    LB_REQUIRE(ctx, W == 1 || (d.intermediate / W) % 4 == 0, "decoder_create: intermediate slice %d must be a multiple of 4", d.intermediate / W);
    auto* dec = new loom_b200_decoder();
    dec->ctx = ctx;
    dec->d = d;
    if (dec->d.num_kv_heads == 0) dec->d.num_kv_heads = d.num_heads;
    if (dec->d.max_seq_len <= 0) dec->d.max_seq_len = 2048;  // NewTransformer default, poly/transformer.go:111-113
    dec->blocks.resize(d.num_layers);
    dec->tp_world = ctx->tp_world;
    dec->tp_rank = ctx->tp_rank;
    dec->heads_l = d.num_heads / W;
    dec->kv_heads_l = dec->d.num_kv_heads / W;
    dec->inter_l = d.intermediate / W;
    dec->head_sharded = W > 1 && d.vocab % W == 0;
    // attention splits for one-token steps: heads x splits CTAs should be resident together (two per SM)
    dec->decode_splits = (2 * ctx->sm_count) / dec->heads_l;
    if (dec->decode_splits > 16) dec->decode_splits = 16;
    if (dec->decode_splits < 1) dec->decode_splits = 1;
    if (ctx->opt_decode_splits > 0) dec->decode_splits = ctx->opt_decode_splits;  // read when the decoder is created
    dec->out_cap = dec->d.max_seq_len;
    cudaError_t e = cudaSuccess;
    auto A = [&](void** p, size_t bytes) {
        if (e == cudaSuccess) e = cudaMalloc(p, bytes);
        if (e == cudaSuccess) e = cudaMemsetAsync(*p, 0, bytes, ctx->stream);
    };
    A((void**)&dec->x, (size_t)kChunkTokens * d.hidden * 4);
    A((void**)&dec->prod, (size_t)kChunkTokens * dec->inter_l * 4);
    A((void**)&dec->logits_all, (size_t)d.vocab * 4);
    A((void**)&dec->hidden, (size_t)d.hidden * 4);
    A((void**)&dec->tok, kChunkTokens * sizeof(int));
    A((void**)&dec->pos_all, sizeof(int));
    A((void**)&dec->step_all, sizeof(int));
    A((void**)&dec->tok_all, sizeof(int));
    A((void**)&dec->out_tokens_all, (size_t)dec->out_cap * sizeof(int));
    dec->kv_offsets.assign(1, 0);
    dec_point_at_lane(dec, 0);
    if (W > 1) {
        A((void**)&dec->tp_stats, 2 * kChunkTokens * sizeof(double));
        A((void**)&dec->tp_acc, (size_t)kChunkTokens * d.hidden * sizeof(int32_t));
    }
    if (e == cudaSuccess) e = cudaMallocHost((void**)&dec->h_tok, kChunkTokens * sizeof(int));
    if (e == cudaSuccess) e = cudaMallocHost((void**)&dec->h_logits, (size_t)d.vocab * 4);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        loom_b200_decoder_destroy(dec);
        return lb_fail(ctx, LOOM_B200_ERR_CUDA, "decoder_create: %s", cudaGetErrorString(e));
    }
    *out = dec;
    return 0;
}

void loom_b200_decoder_destroy(loom_b200_decoder* dec) {
    if (!dec) return;
    if (dec->ctx) {
        cudaSetDevice(dec->ctx->device);
        cudaStreamSynchronize(dec->ctx->stream);
    }
    dec_drop_graph(dec);
    for (auto& b : dec->blocks) {
        if (b.ready) {
            b.mha.pos_dev = nullptr;  // shared with the decoder
            lb_mha_release(&b.mha);
        }
        if (b.g1) cudaFree(b.g1);
        if (b.g2) cudaFree(b.g2);
        if (b.ffn_inner) cudaFree(b.ffn_inner);
    }
    dec_free_prefill(dec);
    void* ptrs[] = {dec->final_gain, dec->x, dec->prod, dec->logits_all, dec->hidden, dec->tok, dec->pos_all, dec->step_all,
                    dec->tok_all, dec->out_tokens_all, dec->tp_stats, dec->tp_acc};
    for (void* p : ptrs)
        if (p) cudaFree(p);
    if (dec->h_tok) cudaFreeHost(dec->h_tok);
    if (dec->h_tok_all) cudaFreeHost(dec->h_tok_all);
    if (dec->h_logits) cudaFreeHost(dec->h_logits);
    delete dec;
}

int loom_b200_decoder_set_block(loom_b200_decoder* dec, int block, const float* norm1_gain, const float* norm2_gain,
                                const loom_b200_weight* const* w7, const float* attn_inner_norm, int attn_inner_len,
                                const float* ffn_inner_norm, int ffn_inner_len) {
    if (!dec) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "decoder_set_block: decoder is NULL");
    loom_b200_ctx* ctx = dec->ctx;
    const loom_b200_decoder_dims& d = dec->d;
    LB_REQUIRE(ctx, block >= 0 && block < d.num_layers, "decoder_set_block: block %d out of range", block);
    LB_REQUIRE(ctx, w7 != nullptr, "decoder_set_block: weights are NULL");
    for (int i = 0; i < 7; ++i) LB_REQUIRE(ctx, w7[i] != nullptr, "decoder_set_block: weight %d is NULL", i);
    if (ctx->capturing) return lb_fail(ctx, LOOM_B200_ERR_INVALID, "decoder_set_block cannot be recorded");
    if (int rc = lb_set_device(ctx)) return rc;
    // with a group of W ranks these are the slice shapes: heads/W heads, kv_heads/W KV heads, intermediate/W units
    const int H = d.hidden, I = dec->inter_l, qd = dec->heads_l * d.head_dim, kvd = dec->kv_heads_l * d.head_dim;
    const int rows[7] = {qd, kvd, kvd, H, I, I, H}, cols[7] = {H, H, H, qd, H, H, I};
    for (int i = 0; i < 7; ++i)
        LB_REQUIRE(ctx, w7[i]->rows == rows[i] && w7[i]->cols == cols[i], "decoder_set_block: weight %d is %dx%d, expected %dx%d", i,
                   w7[i]->rows, w7[i]->cols, rows[i], cols[i]);
    LbDecBlock& b = dec->blocks[block];
    LB_REQUIRE(ctx, !b.ready, "decoder_set_block: block %d is already set", block);
    dec_drop_graph(dec);
    loom_b200_mha& m = b.mha;
    m.d_model = H;
    m.heads = dec->heads_l;
    m.kv_heads = dec->kv_heads_l;
    if (dec->tp_world > 1) {
        m.q_dim_global = d.num_heads * d.head_dim;
        m.tp_stats = dec->tp_stats;
        m.tp_acc = dec->tp_acc;
    }
    m.head_dim = d.head_dim;
    m.q_dim = qd;
    m.kv_dim = kvd;
    m.msl = d.max_seq_len;
    m.theta = d.rope_theta > 0 ? d.rope_theta : 10000.0;
    m.rms_eps = d.rms_eps;  // SetRMSNormEps reaches the MHA layers, poly/transformer.go:162-175
    m.wq = w7[0];
    m.wk = w7[1];
    m.wv = w7[2];
    m.wo = w7[3];
    if (int rc = lb_mha_alloc(ctx, &m, 32, dec->batch)) return rc;
    cudaFree(m.pos_dev);
    m.pos_dev = dec->pos;
    b.gate = w7[4];
    b.up = w7[5];
    b.down = w7[6];
    std::vector<float> ones(H, 1.0f);
    LB_CUDA(ctx, cudaMalloc(&b.g1, (size_t)H * 4));
    LB_CUDA(ctx, cudaMalloc(&b.g2, (size_t)H * 4));
    LB_CUDA(ctx, cudaMemcpyAsync(b.g1, norm1_gain ? norm1_gain : ones.data(), (size_t)H * 4, cudaMemcpyHostToDevice, ctx->stream));
    LB_CUDA(ctx, cudaMemcpyAsync(b.g2, norm2_gain ? norm2_gain : ones.data(), (size_t)H * 4, cudaMemcpyHostToDevice, ctx->stream));
    if (attn_inner_norm && attn_inner_len > 0) {
        LB_CUDA(ctx, cudaMalloc(&m.inner, (size_t)attn_inner_len * 4));
        LB_CUDA(ctx, cudaMemcpyAsync(m.inner, attn_inner_norm, (size_t)attn_inner_len * 4, cudaMemcpyHostToDevice, ctx->stream));
        m.inner_len = attn_inner_len;
    }
    if (ffn_inner_norm && ffn_inner_len > 0) {
        LB_CUDA(ctx, cudaMalloc(&b.ffn_inner, (size_t)ffn_inner_len * 4));
        LB_CUDA(ctx, cudaMemcpyAsync(b.ffn_inner, ffn_inner_norm, (size_t)ffn_inner_len * 4, cudaMemcpyHostToDevice, ctx->stream));
        b.ffn_inner_len = ffn_inner_len;
    }
    LB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    b.ready = true;
    dec_point_at_lane(dec, dec->lane);
    return 0;
}

int loom_b200_decoder_set_embeddings(loom_b200_decoder* dec, const float* emb_dev, const float* final_gain) {
    if (!dec) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "decoder_set_embeddings: decoder is NULL");
    loom_b200_ctx* ctx = dec->ctx;
    LB_REQUIRE(ctx, emb_dev != nullptr, "decoder_set_embeddings: embeddings are NULL");
    if (ctx->capturing) return lb_fail(ctx, LOOM_B200_ERR_INVALID, "decoder_set_embeddings cannot be recorded");
    if (int rc = lb_set_device(ctx)) return rc;
    dec_drop_graph(dec);
    dec->emb = emb_dev;
    dec->fused_tail = dec_tail_possible(dec, emb_dev);
    const int H = dec->d.hidden;
    std::vector<float> ones(H, 1.0f);
    if (!dec->final_gain) LB_CUDA(ctx, cudaMalloc(&dec->final_gain, (size_t)H * 4));
    LB_CUDA(ctx, cudaMemcpyAsync(dec->final_gain, final_gain ? final_gain : ones.data(), (size_t)H * 4, cudaMemcpyHostToDevice, ctx->stream));
    LB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return 0;
}

int loom_b200_decoder_set_lm_head_ternary(loom_b200_decoder* dec, const loom_b200_weight* head) {
    if (!dec) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "decoder_set_lm_head_ternary: decoder is NULL");
    loom_b200_ctx* ctx = dec->ctx;
    if (ctx->capturing) return lb_fail(ctx, LOOM_B200_ERR_INVALID, "decoder_set_lm_head_ternary cannot be recorded");
    LB_REQUIRE(ctx, dec->emb != nullptr, "decoder_set_lm_head_ternary: set the embeddings first");
    LB_REQUIRE(ctx, dec->tp_world == 1 && dec->batch == 1, "decoder_set_lm_head_ternary: one GPU, one sequence");
    if (head) {
        LB_REQUIRE(ctx, head->rows == dec->d.vocab && head->cols == dec->d.hidden, "decoder_set_lm_head_ternary: head is %dx%d, expected %dx%d",
                   head->rows, head->cols, dec->d.vocab, dec->d.hidden);
        LB_REQUIRE(ctx, head->device == ctx->device, "decoder_set_lm_head_ternary: head lives on device %d", head->device);
    }
    dec_drop_graph(dec);
    dec->head_tern = head;
    // the greedy step folded into the fp32 head's tail does not exist for this head: argmax, position and embedding are launches again
    dec->fused_tail = head == nullptr && dec_tail_possible(dec, dec->emb);
    return 0;
}

int loom_b200_decoder_reset(loom_b200_decoder* dec) {
    if (!dec) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "decoder_reset: decoder is NULL");
    loom_b200_ctx* ctx = dec->ctx;
    if (ctx->capturing) return lb_fail(ctx, LOOM_B200_ERR_INVALID, "decoder_reset cannot be recorded");
    if (int rc = lb_set_device(ctx)) return rc;
    dec->kv_offset = 0;
    LB_CUDA(ctx, cudaMemsetAsync(dec->pos, 0, sizeof(int), ctx->stream));
    LB_CUDA(ctx, cudaMemsetAsync(dec->step, 0, sizeof(int), ctx->stream));
    return 0;
}

int loom_b200_decoder_kv_offset(const loom_b200_decoder* dec) { return dec ? dec->kv_offset : -1; }

int loom_b200_decoder_forward(loom_b200_decoder* dec, const int32_t* tokens, int n, float* logits_host) {
    if (!dec) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "decoder_forward: decoder is NULL");
    loom_b200_ctx* ctx = dec->ctx;
    LB_REQUIRE(ctx, tokens && n > 0, "decoder_forward: no tokens");
    if (ctx->capturing) return lb_fail(ctx, LOOM_B200_ERR_INVALID, "decoder_forward takes host buffers and cannot be recorded");
    if (int rc = dec_check_ready(dec)) return rc;
    if (int rc = lb_set_device(ctx)) return rc;
    // A multi-token call restarts the KV ring like the CPU path does (poly/mha_layout.go:62-70);
    // a one-token call continues it when there is something to continue.
    const bool incremental = n == 1 && dec->kv_offset > 0;
    if (!incremental) {
        if (int rc = loom_b200_decoder_reset(dec)) return rc;
    }
    LB_REQUIRE(ctx, dec->kv_offset + n <= dec->d.max_seq_len, "decoder_forward: %d positions exceed MaxSeqLen %d", dec->kv_offset + n, dec->d.max_seq_len);
    if (n == 1) {
        dec->h_tok[0] = tokens[0];
        LB_CUDA(ctx, cudaMemcpyAsync(dec->cur_tok, dec->h_tok, sizeof(int), cudaMemcpyHostToDevice, ctx->stream));
        if (int rc = dec_step(dec, true)) return rc;
    } else if (n >= kGemmMinTokens && ctx->opt_prefill_gemm) {
        const int cap = n < kPrefillBlock ? n : kPrefillBlock;
        if (int rc = dec_ensure_prefill(dec, cap)) return rc;
        for (int s0 = 0; s0 < n; s0 += cap) {
            const int M = n - s0 < cap ? n - s0 : cap;
            LB_CUDA(ctx, cudaMemcpyAsync(dec->pf_tok, tokens + s0, (size_t)M * sizeof(int), cudaMemcpyHostToDevice, ctx->stream));
            if (int rc = dec_prefill_block(dec, M, dec->kv_offset + s0, s0 + M == n)) return rc;
        }
    } else {
        // tokens per pass: what the widest input row (hidden, or this rank's slice of the intermediate) leaves room for
        const int widest = dec->inter_l > dec->d.hidden ? dec->inter_l : dec->d.hidden;
        const int chunk = lb_gemv_max_tokens(widest) < kChunkTokens ? lb_gemv_max_tokens(widest) : kChunkTokens;
        for (int s0 = 0; s0 < n; s0 += chunk) {
            const int M = n - s0 < chunk ? n - s0 : chunk;
            LB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));  // h_tok is reused
            for (int i = 0; i < M; ++i) dec->h_tok[i] = tokens[s0 + i];
            LB_CUDA(ctx, cudaMemcpyAsync(dec->tok, dec->h_tok, M * sizeof(int), cudaMemcpyHostToDevice, ctx->stream));
            const bool last = s0 + M == n;
            if (int rc = dec_forward_chunk(dec, M, 1, last, M - 1)) return rc;
        }
    }
    dec->kv_offset += n;
    if (logits_host) {
        if (int rc = dec_gather_logits(dec, dec->logits)) return rc;
        LB_CUDA(ctx, cudaMemcpyAsync(dec->h_logits, dec->logits, (size_t)dec->d.vocab * 4, cudaMemcpyDeviceToHost, ctx->stream));
        if (int rc = lb_sync_checked(ctx)) return rc;
        memcpy(logits_host, dec->h_logits, (size_t)dec->d.vocab * 4);
    }
    return 0;
}

int loom_b200_decoder_last_hidden(loom_b200_decoder* dec, float* hidden_host) {
    if (!dec) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "decoder_last_hidden: decoder is NULL");
    loom_b200_ctx* ctx = dec->ctx;
    LB_REQUIRE(ctx, hidden_host != nullptr, "decoder_last_hidden: NULL buffer");
    if (int rc = lb_set_device(ctx)) return rc;
    LB_CUDA(ctx, cudaMemcpyAsync(hidden_host, dec->hidden, (size_t)dec->d.hidden * 4, cudaMemcpyDeviceToHost, ctx->stream));
    LB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return 0;
}

int loom_b200_decoder_continue(loom_b200_decoder* dec, int steps) {
    if (!dec) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "decoder_continue: decoder is NULL");
    loom_b200_ctx* ctx = dec->ctx;
    LB_REQUIRE(ctx, steps >= 0, "decoder_continue: steps=%d", steps);
    LB_REQUIRE(ctx, dec->kv_offset > 0, "decoder_continue: nothing to continue (run a prompt first)");
    LB_REQUIRE(ctx, dec->kv_offset + steps <= dec->d.max_seq_len, "decoder_continue: %d positions exceed MaxSeqLen %d", dec->kv_offset + steps, dec->d.max_seq_len);
    if (ctx->capturing) return lb_fail(ctx, LOOM_B200_ERR_INVALID, "decoder_continue cannot be recorded");
    if (int rc = lb_set_device(ctx)) return rc;
    for (int i = 0; i < steps; ++i) {
        if (!dec->fused_tail)
            if (int rc = lb_launch_argmax_advance(ctx, dec->logits, dec->d.vocab, dec->tok, dec->out_tokens, dec->out_cap, dec->step, nullptr)) return rc;
        if (int rc = dec_step(dec, false)) return rc;
    }
    dec->kv_offset += steps;
    return 0;
}

int loom_b200_decoder_download_cache(loom_b200_decoder* dec, int block, float* k_host, float* v_host) {
    if (!dec) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "decoder_download_cache: decoder is NULL");
    loom_b200_ctx* ctx = dec->ctx;
    LB_REQUIRE(ctx, block >= 0 && block < (int)dec->blocks.size() && dec->blocks[block].ready, "decoder_download_cache: block %d is not set", block);
    return loom_b200_mha_download_cache(&dec->blocks[block].mha, k_host, v_host);
}

int loom_b200_decoder_set_batch(loom_b200_decoder* dec, int batch) {
    if (!dec) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "decoder_set_batch: decoder is NULL");
    loom_b200_ctx* ctx = dec->ctx;
    LB_REQUIRE(ctx, batch >= 1 && batch <= 256, "decoder_set_batch: %d sequences (1..256)", batch);
    LB_REQUIRE(ctx, dec->tp_world == 1 || (ctx->tp_peer && ctx->opt_tp_peer && dec->head_sharded),
               "decoder_set_batch: under a tensor-parallel group sequences in parallel need the peer-memory exchange (tp_attach_peers) and a vocabulary that divides by the group");
    for (auto& b : dec->blocks) LB_REQUIRE(ctx, !b.ready, "decoder_set_batch must be called before decoder_set_block");
    if (ctx->capturing) return lb_fail(ctx, LOOM_B200_ERR_INVALID, "decoder_set_batch cannot be recorded");
    if (int rc = lb_set_device(ctx)) return rc;
    LB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    void* old[] = {dec->logits_all, dec->pos_all, dec->step_all, dec->tok_all, dec->out_tokens_all};
    for (void* p : old)
        if (p) cudaFree(p);
    dec->logits_all = nullptr;
    dec->pos_all = dec->step_all = dec->tok_all = dec->out_tokens_all = nullptr;
    if (dec->h_tok_all) cudaFreeHost(dec->h_tok_all);
    dec->h_tok_all = nullptr;
    const size_t B = (size_t)batch;
    cudaError_t e = cudaSuccess;
    auto A = [&](void** p, size_t bytes) {
        if (e == cudaSuccess) e = cudaMalloc(p, bytes);
        if (e == cudaSuccess) e = cudaMemsetAsync(*p, 0, bytes, ctx->stream);
    };
    A((void**)&dec->logits_all, B * dec->d.vocab * 4);
    A((void**)&dec->pos_all, B * sizeof(int));
    A((void**)&dec->step_all, B * sizeof(int));
    A((void**)&dec->tok_all, B * sizeof(int));
    A((void**)&dec->out_tokens_all, B * dec->out_cap * sizeof(int));
    if (e == cudaSuccess) e = cudaMallocHost((void**)&dec->h_tok_all, B * sizeof(int));
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) return lb_fail(ctx, LOOM_B200_ERR_CUDA, "decoder_set_batch: %s", cudaGetErrorString(e));
    dec->batch = batch;
    dec->kv_offsets.assign(B, 0);
    dec_drop_graph(dec);
    dec_point_at_lane(dec, 0);
    return 0;
}

int loom_b200_decoder_batch(const loom_b200_decoder* dec) { return dec ? dec->batch : -1; }

int loom_b200_decoder_select(loom_b200_decoder* dec, int seq) {
    if (!dec) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "decoder_select: decoder is NULL");
    loom_b200_ctx* ctx = dec->ctx;
    LB_REQUIRE(ctx, seq >= 0 && seq < dec->batch, "decoder_select: sequence %d of %d", seq, dec->batch);
    if (ctx->capturing) return lb_fail(ctx, LOOM_B200_ERR_INVALID, "decoder_select cannot be recorded");
    if (seq == dec->lane) return 0;
    dec->kv_offsets[dec->lane] = dec->kv_offset;
    dec_drop_graph(dec);  // the recorded step holds the previous sequence's ring pointers
    dec_point_at_lane(dec, seq);
    return 0;
}

// host bookkeeping shared by the two batch calls: every sequence must have a prompt behind it and room for `steps` more
static int dec_batch_ready(loom_b200_decoder* dec, int steps, const char* who) {
    loom_b200_ctx* ctx = dec->ctx;
    if (int rc = dec_check_ready(dec)) return rc;
    LB_REQUIRE(ctx, dec->fused_tail, "%s: sequences in parallel need the streaming LM head (a hidden size it has room for; under a tensor-parallel group the peer-memory exchange)", who);
    dec->kv_offsets[dec->lane] = dec->kv_offset;
    for (int i = 0; i < dec->batch; ++i) {
        LB_REQUIRE(ctx, dec->kv_offsets[i] > 0, "%s: sequence %d has no prompt behind it (select it and run decoder_forward first)", who, i);
        LB_REQUIRE(ctx, dec->kv_offsets[i] + steps <= dec->d.max_seq_len, "%s: sequence %d would exceed MaxSeqLen %d", who, i, dec->d.max_seq_len);
    }
    return 0;
}

int loom_b200_decoder_step_batch(loom_b200_decoder* dec, const int32_t* tokens, float* logits_host) {
    if (!dec) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "decoder_step_batch: decoder is NULL");
    loom_b200_ctx* ctx = dec->ctx;
    if (ctx->capturing) return lb_fail(ctx, LOOM_B200_ERR_INVALID, "decoder_step_batch cannot be recorded");
    if (int rc = lb_set_device(ctx)) return rc;
    if (int rc = dec_batch_ready(dec, 1, "decoder_step_batch")) return rc;
    const int B = dec->batch;
    if (tokens) {
        LB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));  // the pinned staging buffer is reused
        for (int i = 0; i < B; ++i) dec->h_tok_all[i] = tokens[i];
        LB_CUDA(ctx, cudaMemcpyAsync(dec->tok_all, dec->h_tok_all, (size_t)B * sizeof(int), cudaMemcpyHostToDevice, ctx->stream));
    }
    for (int l0 = 0; l0 < B; l0 += kChunkTokens) {
        const int M = B - l0 < kChunkTokens ? B - l0 : kChunkTokens;
        if (int rc = dec_forward_lanes(dec, l0, M)) return rc;
    }
    for (int i = 0; i < B; ++i) dec->kv_offsets[i] += 1;
    dec->kv_offset = dec->kv_offsets[dec->lane];
    if (logits_host) {
        for (int i = 0; i < B; ++i)
            if (int rc = dec_gather_logits(dec, dec->logits_all + (size_t)i * dec->d.vocab)) return rc;
        LB_CUDA(ctx, cudaMemcpyAsync(logits_host, dec->logits_all, (size_t)B * dec->d.vocab * 4, cudaMemcpyDeviceToHost, ctx->stream));
        if (int rc = lb_sync_checked(ctx)) return rc;
    }
    return 0;
}

int loom_b200_decoder_continue_batch(loom_b200_decoder* dec, int steps) {
    if (!dec) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "decoder_continue_batch: decoder is NULL");
    loom_b200_ctx* ctx = dec->ctx;
    LB_REQUIRE(ctx, steps >= 0, "decoder_continue_batch: steps=%d", steps);
    if (ctx->capturing) return lb_fail(ctx, LOOM_B200_ERR_INVALID, "decoder_continue_batch cannot be recorded");
    if (int rc = lb_set_device(ctx)) return rc;
    if (int rc = dec_batch_ready(dec, steps, "decoder_continue_batch")) return rc;
    const int B = dec->batch;
    for (int s = 0; s < steps; ++s)
        for (int l0 = 0; l0 < B; l0 += kChunkTokens) {
            const int M = B - l0 < kChunkTokens ? B - l0 : kChunkTokens;
            if (int rc = dec_forward_lanes(dec, l0, M)) return rc;
        }
    for (int i = 0; i < B; ++i) dec->kv_offsets[i] += steps;
    dec->kv_offset = dec->kv_offsets[dec->lane];
    return 0;
}

int loom_b200_decoder_read_tokens_batch(loom_b200_decoder* dec, int32_t* tokens_host, int n) {
    if (!dec) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "decoder_read_tokens_batch: decoder is NULL");
    loom_b200_ctx* ctx = dec->ctx;
    LB_REQUIRE(ctx, tokens_host && n > 0, "decoder_read_tokens_batch: bad arguments");
    if (ctx->capturing) return lb_fail(ctx, LOOM_B200_ERR_INVALID, "decoder_read_tokens_batch takes host buffers and cannot be recorded");
    if (int rc = lb_set_device(ctx)) return rc;
    if (int rc = lb_sync_checked(ctx)) return rc;
    std::vector<int> steps(dec->batch);
    LB_CUDA(ctx, cudaMemcpy(steps.data(), dec->step_all, (size_t)dec->batch * sizeof(int), cudaMemcpyDeviceToHost));
    for (int i = 0; i < dec->batch; ++i) {
        const int consumed = steps[i] - 1;  // the newest entry is the token the next step will consume
        LB_REQUIRE(ctx, n <= consumed && steps[i] <= dec->out_cap, "decoder_read_tokens_batch: sequence %d: %d tokens asked, %d consumed (ring of %d)", i, n, consumed, dec->out_cap);
        LB_CUDA(ctx, cudaMemcpy(tokens_host + (size_t)i * n, dec->out_tokens_all + (size_t)i * dec->out_cap + (consumed - n), (size_t)n * sizeof(int), cudaMemcpyDeviceToHost));
    }
    return 0;
}

int loom_b200_decoder_set_kv_offset(loom_b200_decoder* dec, int kv_offset) {
    if (!dec) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "decoder_set_kv_offset: decoder is NULL");
    loom_b200_ctx* ctx = dec->ctx;
    LB_REQUIRE(ctx, kv_offset > 0 && kv_offset <= dec->kv_offset, "decoder_set_kv_offset: %d outside (0, %d]: a sequence can only be cut back", kv_offset, dec->kv_offset);
    if (ctx->capturing) return lb_fail(ctx, LOOM_B200_ERR_INVALID, "decoder_set_kv_offset cannot be recorded");
    if (int rc = lb_set_device(ctx)) return rc;
    LB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    LB_CUDA(ctx, cudaMemcpy(dec->pos, &kv_offset, sizeof(int), cudaMemcpyHostToDevice));
    dec->kv_offset = kv_offset;
    return 0;
}

int loom_b200_decoder_step_launches(const loom_b200_decoder* dec) { return dec ? dec->step_launches + (dec->fused_tail ? 0 : 1) : -1; }

int loom_b200_decoder_linears_frame(loom_b200_decoder* dec) {
    if (!dec) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "decoder_linears_frame: decoder is NULL");
    loom_b200_ctx* ctx = dec->ctx;
    if (int rc = dec_check_ready(dec)) return rc;
    LB_REQUIRE(ctx, dec->tp_world == 1, "decoder_linears_frame: not available under a tensor-parallel group");
    if (int rc = lb_set_device(ctx)) return rc;
    return dec_forward_chunk(dec, 1, dec->decode_splits, false, 0, true);
}

int loom_b200_decoder_read_tokens(loom_b200_decoder* dec, int32_t* tokens_host, int n) {
    if (!dec) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "decoder_read_tokens: decoder is NULL");
    loom_b200_ctx* ctx = dec->ctx;
    LB_REQUIRE(ctx, tokens_host && n > 0, "decoder_read_tokens: bad arguments");
    if (ctx->capturing) return lb_fail(ctx, LOOM_B200_ERR_INVALID, "decoder_read_tokens takes host buffers and cannot be recorded");
    if (int rc = lb_set_device(ctx)) return rc;
    if (int rc = lb_sync_checked(ctx)) return rc;
    int step = 0;
    LB_CUDA(ctx, cudaMemcpy(&step, dec->step, sizeof(int), cudaMemcpyDeviceToHost));
    // with the greedy tail folded into the head, the newest entry of the ring is the token the NEXT step will consume
    const int consumed = dec->fused_tail ? step - 1 : step;
    LB_REQUIRE(ctx, n <= consumed && step <= dec->out_cap, "decoder_read_tokens: %d tokens asked, %d consumed since the last reset (ring of %d)", n, consumed, dec->out_cap);
    LB_CUDA(ctx, cudaMemcpy(tokens_host, dec->out_tokens + (consumed - n), (size_t)n * sizeof(int), cudaMemcpyDeviceToHost));
    return 0;
}

int loom_b200_decoder_upload_cache(loom_b200_decoder* dec, int block, int kv_offset, const float* k_host, const float* v_host) {
    if (!dec) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "decoder_upload_cache: decoder is NULL");
    loom_b200_ctx* ctx = dec->ctx;
    LB_REQUIRE(ctx, block >= 0 && block < (int)dec->blocks.size() && dec->blocks[block].ready, "decoder_upload_cache: block %d is not set", block);
    LB_REQUIRE(ctx, k_host && v_host, "decoder_upload_cache: NULL buffer");
    LB_REQUIRE(ctx, kv_offset > 0 && kv_offset < dec->d.max_seq_len, "decoder_upload_cache: kv_offset %d outside (0, MaxSeqLen %d)", kv_offset, dec->d.max_seq_len);
    if (ctx->capturing) return lb_fail(ctx, LOOM_B200_ERR_INVALID, "decoder_upload_cache takes host buffers and cannot be recorded");
    if (int rc = lb_set_device(ctx)) return rc;
    loom_b200_mha& m = dec->blocks[block].mha;
    // host rows are position-major [position][kv head * hd]; the device ring is head-major [kv head][position][hd]
    std::vector<float> tmp((size_t)kv_offset * m.head_dim);
    LB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    for (int which = 0; which < 2; ++which) {
        const float* host = which == 0 ? k_host : v_host;
        float* ring = which == 0 ? m.cache_k : m.cache_v;
        for (int h = 0; h < m.kv_heads; ++h) {
            for (int pos = 0; pos < kv_offset; ++pos)
                memcpy(tmp.data() + (size_t)pos * m.head_dim, host + (size_t)pos * m.kv_dim + (size_t)h * m.head_dim, (size_t)m.head_dim * sizeof(float));
            LB_CUDA(ctx, cudaMemcpy(ring + (size_t)h * m.msl * m.head_dim, tmp.data(), tmp.size() * sizeof(float), cudaMemcpyHostToDevice));
        }
    }
    dec->kv_offset = kv_offset;
    LB_CUDA(ctx, cudaMemcpy(dec->pos, &kv_offset, sizeof(int), cudaMemcpyHostToDevice));
    return 0;
}

int loom_b200_decoder_last_residual(loom_b200_decoder* dec, float* rows_host, int max_rows, int* rows_out) {
    if (!dec) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "decoder_last_residual: decoder is NULL");
    loom_b200_ctx* ctx = dec->ctx;
    LB_REQUIRE(ctx, rows_host && max_rows > 0, "decoder_last_residual: NULL buffer");
    LB_REQUIRE(ctx, dec->last_resid && dec->last_resid_rows > 0, "decoder_last_residual: nothing has been forwarded yet");
    if (ctx->capturing) return lb_fail(ctx, LOOM_B200_ERR_INVALID, "decoder_last_residual takes host buffers and cannot be recorded");
    if (int rc = lb_set_device(ctx)) return rc;
    const int rows = dec->last_resid_rows < max_rows ? dec->last_resid_rows : max_rows;
    LB_CUDA(ctx, cudaMemcpyAsync(rows_host, dec->last_resid, (size_t)rows * dec->d.hidden * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
    if (int rc = lb_sync_checked(ctx)) return rc;
    if (rows_out) *rows_out = rows;
    return 0;
}

int loom_b200_decoder_generate(loom_b200_decoder* dec, const int32_t* prompt, int n_prompt, int max_new,
                               int32_t* out_tokens, loom_b200_gen_metrics* metrics) {
    if (!dec) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "decoder_generate: decoder is NULL");
    loom_b200_ctx* ctx = dec->ctx;
    LB_REQUIRE(ctx, prompt && n_prompt > 0 && max_new >= 0 && (out_tokens || max_new == 0), "decoder_generate: bad arguments");
    LB_REQUIRE(ctx, max_new <= dec->out_cap, "decoder_generate: %d new tokens exceed the output ring of %d", max_new, dec->out_cap);
    LB_REQUIRE(ctx, n_prompt + max_new <= dec->d.max_seq_len, "decoder_generate: %d positions exceed MaxSeqLen %d", n_prompt + max_new, dec->d.max_seq_len);
    if (int rc = dec_check_ready(dec)) return rc;
    using clk = std::chrono::steady_clock;
    dec->kv_offset = 0;  // Generate starts with Transformer.Reset
    auto t0 = clk::now();
    // prefill: a one-token prompt still starts a fresh sequence
    if (n_prompt == 1) {
        if (int rc = loom_b200_decoder_reset(dec)) return rc;
        dec->h_tok[0] = prompt[0];
        LB_CUDA(ctx, cudaMemcpyAsync(dec->cur_tok, dec->h_tok, sizeof(int), cudaMemcpyHostToDevice, ctx->stream));
        if (int rc = dec_step(dec, true)) return rc;
        dec->kv_offset = 1;
    } else {
        if (int rc = loom_b200_decoder_forward(dec, prompt, n_prompt, nullptr)) return rc;
    }
    LB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    auto t1 = clk::now();
    const uint64_t launches0 = ctx->launches;
    cudaEvent_t e0, e1;
    LB_CUDA(ctx, cudaEventCreate(&e0));
    LB_CUDA(ctx, cudaEventCreate(&e1));
    LB_CUDA(ctx, cudaEventRecord(e0, ctx->stream));
    // every sampled token is followed by a forward, the last one included (as Generate does)
    for (int i = 0; i < max_new; ++i) {
        if (!dec->fused_tail)
            if (int rc = lb_launch_argmax_advance(ctx, dec->logits, dec->d.vocab, dec->tok, dec->out_tokens, dec->out_cap, dec->step, nullptr)) return rc;
        if (int rc = dec_step(dec, false)) return rc;
    }
    LB_CUDA(ctx, cudaEventRecord(e1, ctx->stream));
    if (max_new > 0)
        LB_CUDA(ctx, cudaMemcpyAsync(out_tokens, dec->out_tokens, (size_t)max_new * sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    if (int rc = lb_sync_checked(ctx)) return rc;
    auto t2 = clk::now();
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    dec->kv_offset += max_new;
    if (metrics) {
        metrics->prefill_seconds = std::chrono::duration<double>(t1 - t0).count();
        metrics->decode_seconds = std::chrono::duration<double>(t2 - t1).count();
        metrics->decode_device_seconds = ms * 1e-3;
        metrics->prefill_tokens = n_prompt;
        metrics->generated_tokens = max_new;
        // per block: QKV, (RoPE unless folded into attention), attention, O, gate/up, down; + head (+ argmax, embed, position
        // when the greedy tail is not folded into the head)
        metrics->launches_per_token = max_new > 0 ? (double)(dec->step_launches + (dec->fused_tail ? 0 : 1)) : 0.0;
        (void)launches0;
    }
    return 0;
}

}  // extern "C"
