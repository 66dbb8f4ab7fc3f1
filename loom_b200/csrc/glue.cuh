// glue.cuh -- the steps either side of the ternary projections inside the decoder block loop:
// embedding gather, q/k norm + RoPE, causal GQA attention over the fp32 KV ring, the fp32 tied LM head
// with the final RMSNorm fused in, and greedy argmax.  Launch wrappers only; kernels are in glue.cu.
#pragma once
#include "common.cuh"

// x[n,:] = emb[tok[n],:]; token ids outside [0,vocab) give a zero row (poly/transformer.go:551-577)
int lb_launch_embed(loom_b200_ctx* ctx, const float* emb, int vocab, int hidden, const int* tok_dev, int n, float* x);

struct LbRopeParams {
    double* q;          // [M, heads*hd] fp64, rotated in place
    float* cache_k;     // [kv_heads, msl, hd] fp32 ring (head-major); rows (pos0+n)%msl of every head rotated in place
    const int* pos_ptr; // device scalar: position of token 0
    const double* rope_div;  // [hd/2] = pow(theta, 2d/hd), computed on the host in double
    const float* q_norm;     // per-head RMSNorm gains or null (poly/mha.go:285-290)
    int q_norm_len;
    const float* k_norm;
    int k_norm_len;
    double qk_eps;
    int M, heads, kv_heads, hd, msl;
    long long seq_stride;  // > 0: the M tokens are independent sequences: token n is at position pos_ptr[n] of the ring n * seq_stride elements on
    unsigned long long* trace;
};
int lb_launch_rope(loom_b200_ctx* ctx, const LbRopeParams& p);

struct LbAttnParams {
    const double* q;       // [M, heads*hd] after RoPE
    const float* cache_k;  // [kv_heads, msl, hd]: head-major, so the positions of one head are contiguous
    const float* cache_v;
    const int* pos_ptr;
    double* out;           // [M, heads*hd] fp64 attention output (before the inner norm)
    double* part;          // split scratch [M*heads*splits*(hd+2)]
    unsigned int* cnt;     // [M*heads], zero between launches
    int M, heads, kv_heads, hd, msl, splits;
    long long seq_stride;  // > 0: the M tokens are independent sequences (see LbRopeParams)
    int max_chunk;         // positions one CTA may hold scores for (shared memory sizing)
    int tile;              // positions per shared-memory tile (set by the launcher)
    // One-token steps without q/k norm can fold RoPE in (one launch less per block): q arrives unrotated, the newest K
    // row arrives unrotated in k_new [kv_heads*hd] instead of the ring, and the kernel rotates both (same arithmetic as
    // lb_rope_kernel) and stores the rotated K row into the ring for later steps.  rope_div == null: plain attention.
    const double* rope_div;
    const float* k_new;
    float* cache_k_w;
    // cluster kernel only: the K and V rings of the decoder block that runs next (same layout), prefetched into L2; or null
    const float* next_k;
    const float* next_v;
    unsigned long long* trace;
    int* status;           // device status word for bounded waits
};
int lb_launch_attention(loom_b200_ctx* ctx, const LbAttnParams& p);
// One-token steps with RoPE folded in: the cluster kernel (attention_decode.cu).  lb_attention_cluster_size returns the
// cluster size to use (CTAs per KV head), or 0 when the shape or the device does not allow it; the launch takes that size.
int lb_attention_cluster_size(loom_b200_ctx* ctx, const LbAttnParams& p, bool one_wave);
int lb_launch_attention_cluster(loom_b200_ctx* ctx, const LbAttnParams& p, int cluster);
// A pass of several sequences (seq_stride > 0), plain attention: one CTA per (sequence, KV head) streams the context through
// tiles with a running softmax (attention_decode.cu).
bool lb_attention_stream_supported(const loom_b200_ctx* ctx, const LbAttnParams& p);
int lb_launch_attention_stream(loom_b200_ctx* ctx, const LbAttnParams& p);
size_t lb_attn_part_elems(int M, int heads, int hd, int splits);
// The same attention for a block of M prompt tokens at once (splits, part and cnt are not used): K/V tiles are shared
// by the heads of a GQA group and by 64/group consecutive query tokens.  Needs head_dim % 16 == 0, head_dim <= 128
// and a group size that divides 64; lb_attention_prefill_supported says whether a shape qualifies.
bool lb_attention_prefill_supported(const LbAttnParams& p);
int lb_launch_attention_prefill(loom_b200_ctx* ctx, const LbAttnParams& p);

struct LbLmHeadParams {
    // nb hidden rows (independent sequences) share one pass over the table: row b is x + b * x_stride, its logits go to
    // logits + b * logits_stride and its greedy tail to tok_out[b], out_tokens + b * out_tokens_stride, step[b], pos[b]
    int nb;                // 0 or 1 = a single row
    long long x_stride, logits_stride, out_tokens_stride;
    const float* x;        // [hidden] last hidden row (before the final norm)
    const float* gain;     // final RMSNorm gain [hidden] or null (= 1)
    double eps;
    const float* head;     // [vocab, hidden] fp32 (tied embedding)
    int vocab, hidden;
    float* logits;         // [vocab]
    float* hidden_out;     // optional [hidden]: the normalised row
    unsigned long long* trace;
    // Greedy tail (tok_out == null: none).  The CTA that finishes last takes the first maximum of the logits
    // (poly/sampling.go:45-55), publishes it as the next token, appends it to the output ring (out_tokens[*step], then
    // *step += 1), advances *pos by pos_delta (pos may be null) and gathers the token's embedding row into x_next
    // (may be null): what lb_argmax_advance_kernel, lb_add_scalar_kernel and lb_embed_kernel did as three more launches.
    int* tok_out;
    int* out_tokens;
    int out_cap;
    int* step;
    int* pos;
    int pos_delta;
    const float* emb;      // [emb_vocab, hidden] embedding table of the next token (the head itself when tied)
    int emb_vocab;
    float* x_next;
    // Vocabulary-sharded head under a tensor-parallel group with peer mailboxes: `head` is this rank's slice (rows
    // vocab_offset ...), and the tail exchanges every rank's (maximum, index) pair instead of gathering the logits: the
    // first maximum over the slices in rank order is the first maximum of the whole row.  xchg_ctr[5] is the sequence number.
    void* const* xchg_peers;
    int xchg_rank, xchg_world, vocab_offset;
    unsigned int* xchg_ctr;
    // scratch of the tail, set by the launcher: per-CTA (value, index) and the arrival counter (zero between launches)
    float* part_val;
    int* part_idx;
    unsigned int* cnt;
    int* status;
};
int lb_launch_lm_head(loom_b200_ctx* ctx, const LbLmHeadParams& p);
// whether the streaming head (the one that can carry the greedy tail) takes this table
bool lb_lm_head_streams(const loom_b200_ctx* ctx, const float* head, int hidden);
// hidden rows the streaming head serves in one pass over the table (0 = the streaming head does not take this table)
int lb_lm_head_rows_per_pass(const loom_b200_ctx* ctx, const float* head, int hidden);

// Greedy step: first index of the maximum (poly/sampling.go:45-55) -> tok[0]; appends it to
// out_tokens[*step]; then *step += 1 and *pos += 1 so that a recorded frame can be replayed as is.
int lb_launch_argmax_advance(loom_b200_ctx* ctx, const float* logits, int vocab, int* tok, int* out_tokens,
                             int out_cap, int* step, int* pos);
// *pos += delta (after a prefill chunk)
int lb_launch_add_scalar(loom_b200_ctx* ctx, int* pos, int delta);
