// lm_head.cu -- the fp32 tied LM head as a streaming kernel: logits[v] = float(sum_d float64(h_d) * float64(W_vd)) over the
// final-normalised hidden row (applyFP32LMHeadRows, poly/transformer.go:659-719; final RMSNorm poly/norm.go:102-138),
// with the greedy step folded into its tail (poly/sampling.go:45-55, poly/transformer.go:434-485).
//
// The head is 63 % of the bytes of a BitNet-2B decode step (1.31 GB), so this kernel is a pure HBM stream: one CTA per
// SM, every warp owns a contiguous range of vocabulary rows and pulls them through a private two-stage shared-memory
// ring with one bulk async copy (TMA engine) per row, first two rows requested before the dependency wait.  The
// normalised hidden row sits in shared memory as float64 in the order the lanes read it (conflict-free 16-byte loads).
// The CTA that finishes last reduces the per-CTA maxima to the next token, appends it to the output ring, advances the
// position and gathers the token's embedding row for the next step: no argmax, position or embedding launch.
#include "glue.cuh"
#include "tp_xchg.cuh"

namespace {

constexpr int kHeadMaxRows = 4;  // hidden rows (independent sequences) one pass of the table serves at most

__device__ __forceinline__ void argmax_merge(float& best, int& idx, float ov, int oi) {
    if (ov > best || (ov == best && oi < idx)) {
        best = ov;
        idx = oi;
    }
}

// NB = hidden rows (independent sequences) one pass of the table serves; p.nb <= NB of them are real
template <int NW, int NB>
__global__ void __launch_bounds__(NW * 32, 1) lb_lm_head_stream_kernel(const LbLmHeadParams p) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ double red[32];
    __shared__ float sv[NB][NW];
    __shared__ int si[NB][NW];
    __shared__ int s_last, s_tok;
    constexpr int T = NW * 32;
    const int H = p.hidden, H4 = H >> 2, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kiter = (H4 + 31) >> 5;                       // float4 columns per lane
    const int nb = p.nb < 1 ? 1 : (p.nb > NB ? NB : p.nb);
    double* sh = reinterpret_cast<double*>(smem_raw);      // [NB][kiter][2][32][2] doubles: every row in lane order, zero padded
    const size_t sh_row = (size_t)kiter * 128;
    const size_t sh_bytes = (size_t)NB * sh_row * sizeof(double);
    float* ring = reinterpret_cast<float*>(smem_raw + sh_bytes) + (size_t)warp * 2 * H;  // this warp's two stages of one row
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + sh_bytes + (size_t)NW * 2 * H * sizeof(float)) + warp * 2;
    // rows of this CTA and of this warp: contiguous slices
    const int r0 = (int)((long long)p.vocab * blockIdx.x / gridDim.x), r1 = (int)((long long)p.vocab * (blockIdx.x + 1) / gridDim.x);
    const int w0 = r0 + (r1 - r0) * warp / NW, w1 = r0 + (r1 - r0) * (warp + 1) / NW;
    const uint32_t row_bytes = (uint32_t)H * 4;
    const uint64_t stream_policy = lb_policy_evict_first();  // 1.3 GB read once per token: do not let it own the L2
    if (lane == 0) {
        lb_mbar_init(&bars[0], 1);
        lb_mbar_init(&bars[1], 1);
        lb_fence_mbar_init();
    }
    __syncwarp();
    lb_pdl_launch_dependents();
    // the head is a weight: its first rows are requested while the last block is still running
    if (lane == 0) {
        for (int s = 0; s < 2 && w0 + s < w1; ++s) {
            lb_mbar_expect_tx(&bars[s], row_bytes);
            lb_bulk_g2s_stream(ring + (size_t)s * H, p.head + (size_t)(w0 + s) * H, row_bytes, &bars[s], stream_policy);
        }
    }
    lb_pdl_wait();
    lb_trace(p.trace, 2);
    // final RMSNorm of every hidden row (float64 like the reference), rounded to float32 and kept as float64
    for (int b = 0; b < NB; ++b) {
        const float* xb = p.x + (size_t)(b < nb ? b : 0) * p.x_stride;
        double ss = 0.0;
        for (int i = tid; i < H; i += T) {
            const double v = (double)xb[i];
            ss = __dadd_rn(ss, __dmul_rn(v, v));
        }
        ss = lb_warp_sum(ss);
        __syncthreads();
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        ss = 0.0;
        for (int i = 0; i < NW; ++i) ss += red[i];
        const double rms = sqrt(__dadd_rn(__ddiv_rn(ss, (double)H), p.eps));
        const double rrms = __ddiv_rn(1.0, rms);
        for (int i = tid; i < kiter * 128; i += T) {
            // slot i holds column 4 * (k * 32 + l) + 2 * half + j
            const int j = i & 1, l = (i >> 1) & 31, half = (i >> 6) & 1, k = i >> 7;
            const int col = 4 * (k * 32 + l) + 2 * half + j;
            double y = 0.0;
            if (col < H && b < nb) {
                const double g = p.gain ? (double)p.gain[col] : 1.0;
                const float yf = (float)__dmul_rn(lb_div_by((double)xb[col], rms, rrms), g);
                y = (double)yf;
                if (blockIdx.x == 0 && p.hidden_out && b == 0) p.hidden_out[col] = yf;
            }
            sh[(size_t)b * sh_row + i] = y;
        }
    }
    __syncthreads();
    lb_trace(p.trace, 3);

    float best[NB];
    int bidx[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) {
        best[b] = -INFINITY;
        bidx[b] = 0x7fffffff;
    }
    bool failed = false;
    for (int r = w0; r < w1; ++r) {
        const int st = (r - w0) & 1;
        const uint32_t parity = (uint32_t)(((r - w0) >> 1) & 1);
        if (!failed && !lb_mbar_wait_bounded(&bars[st], parity)) {
            failed = true;
            if (lane == 0) atomicExch(p.status, 1);
        }
        const float4* row = reinterpret_cast<const float4*>(ring + (size_t)st * H);
        double a[NB][4];
#pragma unroll
        for (int b = 0; b < NB; ++b) a[b][0] = a[b][1] = a[b][2] = a[b][3] = 0.0;
        if (!failed) {
#pragma unroll 2
            for (int k = 0; k < kiter; ++k) {
                const int c4 = k * 32 + lane;
                float4 w = make_float4(0.f, 0.f, 0.f, 0.f);
                if (c4 < H4) w = row[c4];
                const double w0d = (double)w.x, w1d = (double)w.y, w2d = (double)w.z, w3d = (double)w.w;  // converted once, used by every row
#pragma unroll
                for (int b = 0; b < NB; ++b) {
                    const double* shb = sh + (size_t)b * sh_row;
                    const double2 s01 = *reinterpret_cast<const double2*>(shb + ((size_t)(k * 2 + 0) * 32 + lane) * 2);
                    const double2 s23 = *reinterpret_cast<const double2*>(shb + ((size_t)(k * 2 + 1) * 32 + lane) * 2);
                    a[b][0] = fma(w0d, s01.x, a[b][0]);
                    a[b][1] = fma(w1d, s01.y, a[b][1]);
                    a[b][2] = fma(w2d, s23.x, a[b][2]);
                    a[b][3] = fma(w3d, s23.y, a[b][3]);
                }
            }
        }
        __syncwarp();
        if (lane == 0 && r + 2 < w1) {  // the stage is free again: request the row after next
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            lb_mbar_expect_tx(&bars[st], row_bytes);
            lb_bulk_g2s_stream(ring + (size_t)st * H, p.head + (size_t)(r + 2) * H, row_bytes, &bars[st], stream_policy);
        }
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            const double acc = lb_warp_sum((a[b][0] + a[b][1]) + (a[b][2] + a[b][3]));
            const float lg = (float)acc;
            if (lane == 0 && b < nb) p.logits[(size_t)b * p.logits_stride + r] = lg;
            argmax_merge(best[b], bidx[b], lg, r);  // rows ascend: a later equal value never replaces an earlier one
        }
    }
    lb_trace(p.trace, 4);
    if (!p.tok_out) return;

    // ---- greedy tail, once per hidden row ----
    if (lane == 0) {
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            sv[b][warp] = best[b];
            si[b][warp] = bidx[b];
        }
    }
    __syncthreads();
    if (tid < nb) {
        float bv = sv[tid][0];
        int bi = si[tid][0];
        for (int w = 1; w < NW; ++w) argmax_merge(bv, bi, sv[tid][w], si[tid][w]);
        p.part_val[(size_t)tid * gridDim.x + blockIdx.x] = bv;
        p.part_idx[(size_t)tid * gridDim.x + blockIdx.x] = bi;
    }
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        const unsigned old = atomicAdd(p.cnt, 1u);
        s_last = old + 1 == gridDim.x;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (warp < nb) {  // warp b reduces row b
        const int b = warp;
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int i = lane; i < (int)gridDim.x; i += 32) argmax_merge(bv, bi, __ldcg(p.part_val + (size_t)b * gridDim.x + i), __ldcg(p.part_idx + (size_t)b * gridDim.x + i));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            argmax_merge(bv, bi, ov, oi);
        }
        if (lane == 0 && p.xchg_peers) {
            // every rank's (maximum, index) of row b to every other rank, then the merge in rank order
            const uint32_t seq = p.xchg_ctr[5];
            const size_t half = (size_t)(seq & 1);
            const int W = p.xchg_world, me = p.xchg_rank;
            const float mv = bv;
            const int mi = bi == 0x7fffffff ? bi : bi + p.vocab_offset;
            for (int q = 0; q < W; ++q) {
                if (q == me) continue;
                char* dst = (char*)p.xchg_peers[q] + kXRegionD + (((half * kXMaxRanks + me) * 8 + b) * 2) * 8;
                ll_store(dst, __float_as_uint(mv), seq);
                ll_store(dst + 8, (uint32_t)mi, seq);
            }
            bv = -INFINITY;
            bi = 0x7fffffff;
            bool ok = true;
            for (int q = 0; q < W; ++q) {
                uint32_t dv = __float_as_uint(mv), di = (uint32_t)mi;
                if (q != me) {
                    const char* src = (const char*)p.xchg_peers[me] + kXRegionD + (((half * kXMaxRanks + q) * 8 + b) * 2) * 8;
                    ok = ll_wait(src, seq, &dv) && ok;
                    ok = ll_wait(src + 8, seq, &di) && ok;
                }
                argmax_merge(bv, bi, __uint_as_float(dv), (int)di);
            }
            if (!ok) atomicExch(p.status, 5);
        }
        if (lane == 0) {
            if (bi == 0x7fffffff) bi = 0;  // only NaNs: the reference keeps index 0
            if (b == 0) s_tok = bi;
            p.tok_out[b] = bi;
            if (p.out_tokens && p.step) {
                const int s = p.step[b];
                if (s < p.out_cap) p.out_tokens[(size_t)b * p.out_tokens_stride + s] = bi;
                p.step[b] = s + 1;
            }
            if (p.pos) p.pos[b] += p.pos_delta;
        }
    }
    __syncthreads();
    if (tid == 0) {
        *p.cnt = 0;
        if (p.xchg_peers) p.xchg_ctr[5] += 1;  // every warp of this CTA has read the old value (barrier above)
    }
    if (p.x_next && p.emb) {  // the embedding row of the new token, for the step that follows (poly/transformer.go:551-577)
        const int t = s_tok;
        const bool ok = t >= 0 && t < p.emb_vocab;
        const float* src = p.emb + (size_t)(ok ? t : 0) * H;
        for (int i = tid; i < H; i += T) p.x_next[i] = ok ? src[i] : 0.0f;
    }
    lb_trace(p.trace, 5);
}

template <int NW, int NB = 1>
size_t head_smem(int H) {
    const int kiter = ((H >> 2) + 31) >> 5;
    return (size_t)NB * kiter * 128 * sizeof(double) + (size_t)NW * 2 * H * sizeof(float) + (size_t)NW * 2 * sizeof(uint64_t);
}

template <int NW, int NB>
int launch_stream(loom_b200_ctx* ctx, const LbLmHeadParams& p, unsigned attr_bit) {
    auto kern = lb_lm_head_stream_kernel<NW, NB>;
    const size_t smem = head_smem<NW, NB>(p.hidden);
    if (!(ctx->func_attr_mask2 & attr_bit)) {
        LB_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
        ctx->func_attr_mask2 |= attr_bit;
    }
    int grid = ctx->sm_count;
    if (grid > p.vocab / NW) grid = p.vocab / NW > 0 ? p.vocab / NW : 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(NW * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->opt_pdl ? 1 : 0;
    LB_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, p));
    ctx->launches++;
    return 0;
}

}  // namespace

int lb_launch_lm_head_legacy(loom_b200_ctx* ctx, const LbLmHeadParams& p);

bool lb_lm_head_streams(const loom_b200_ctx* ctx, const float* head, int hidden) {
    return ctx->opt_head_stream && (hidden & 3) == 0 && (((uintptr_t)head) & 15) == 0 && head_smem<4>(hidden) <= 220 * 1024;
}

int lb_launch_lm_head(loom_b200_ctx* ctx, const LbLmHeadParams& pin) {
    LbLmHeadParams p = pin;
    p.status = ctx->status_dev;
    const bool fits8 = head_smem<8>(p.hidden) <= 220 * 1024;
    if (!lb_lm_head_streams(ctx, p.head, p.hidden)) {
        if (p.tok_out) return lb_fail(ctx, LOOM_B200_ERR_UNSUPPORTED, "lm_head: the greedy tail needs the streaming kernel (hidden %d)", p.hidden);
        return lb_launch_lm_head_legacy(ctx, p);
    }
    if (p.nb < 1) p.nb = 1;
    if (p.nb > kHeadMaxRows) return lb_fail(ctx, LOOM_B200_ERR_INVALID, "lm_head: %d hidden rows in one pass (at most %d)", p.nb, kHeadMaxRows);
    if (p.tok_out) {
        if (!ctx->head_scratch) {
            if (ctx->capturing) return lb_fail(ctx, LOOM_B200_ERR_INVALID, "lm_head scratch would be allocated while recording a graph");
            const size_t bytes = (size_t)kHeadMaxRows * ctx->sm_count * 8 + 64;
            LB_CUDA(ctx, cudaMalloc(&ctx->head_scratch, bytes));
            LB_CUDA(ctx, cudaMemsetAsync(ctx->head_scratch, 0, bytes, ctx->stream));
        }
        p.part_val = reinterpret_cast<float*>(ctx->head_scratch);
        p.part_idx = reinterpret_cast<int*>(p.part_val + (size_t)kHeadMaxRows * ctx->sm_count);
        p.cnt = reinterpret_cast<unsigned int*>(p.part_idx + (size_t)kHeadMaxRows * ctx->sm_count);
    }
    p.trace = lb_trace_row(ctx, "lm_head");
    // several rows per pass when they fit beside the ring: four with six warps, two with eight
    if (p.nb > 2 && head_smem<6, 4>(p.hidden) <= 220 * 1024) return launch_stream<6, 4>(ctx, p, 1u << 10);
    if (p.nb > 1) {
        if (p.nb > 2) return lb_fail(ctx, LOOM_B200_ERR_UNSUPPORTED, "lm_head: %d rows of %d columns do not fit in one pass", p.nb, p.hidden);
        if (head_smem<8, 2>(p.hidden) <= 220 * 1024) return launch_stream<8, 2>(ctx, p, 1u << 11);
        if (head_smem<4, 2>(p.hidden) <= 220 * 1024) return launch_stream<4, 2>(ctx, p, 1u << 12);
        return lb_fail(ctx, LOOM_B200_ERR_UNSUPPORTED, "lm_head: two rows of %d columns do not fit in one pass", p.hidden);
    }
    return fits8 ? launch_stream<8, 1>(ctx, p, 1u << 8) : launch_stream<4, 1>(ctx, p, 1u << 9);
}

int lb_lm_head_rows_per_pass(const loom_b200_ctx* ctx, const float* head, int hidden) {
    if (!lb_lm_head_streams(ctx, head, hidden)) return 0;
    if (head_smem<6, 4>(hidden) <= 220 * 1024) return 4;
    if (head_smem<8, 2>(hidden) <= 220 * 1024 || head_smem<4, 2>(hidden) <= 220 * 1024) return 2;
    return 1;
}
