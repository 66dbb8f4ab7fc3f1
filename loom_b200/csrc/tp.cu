// tp.cu -- tensor parallelism across the GPUs of one box: NCCL plumbing and the small kernels a row-sharded
// ternary linear needs around its partial dot products.
//
// The reference has no multi-device code; this is the sharding the integer arithmetic allows without changing a
// bit of the result: output rows are independent (column-parallel Q/K/V/gate/up) and the K reduction is an exact
// int32 sum (row-parallel O/down).  A row-sharded projection therefore all-reduces
//   (1) one float64 partial sum of squares per token  (the inner RMSNorm runs over the sharded dimension),
//   (2) one float32 partial absmax per token of the normalised values (max is exact),
//   (3) the int32 partial accumulators [tokens, rows] (exact),
// and only then applies the float64 rescale, bias and residual -- identically on every rank.
// NCCL is loaded at run time (dlopen of libnccl.so.2): single-GPU users need no NCCL at all.
#include "layers.cuh"
#include "tp_xchg.cuh"

#include <dlfcn.h>

// ncclUniqueId: 128 opaque bytes passed by value
struct UniqueId128 {
    char internal[128];
};

namespace {

struct NcclApi {
    void* handle = nullptr;
    int (*GetUniqueId)(void*) = nullptr;
    int (*CommInitRank)(void**, int, UniqueId128, int) = nullptr;
    int (*CommDestroy)(void*) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
};

NcclApi g_nccl;

constexpr int kNcclInt32 = kTpInt32, kNcclFloat32 = kTpFloat32, kNcclFloat64 = kTpFloat64, kNcclSum = kTpSum, kNcclMax = kTpMax;

int load_nccl(loom_b200_ctx* ctx) {
    if (g_nccl.handle) return 0;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return lb_fail(ctx, LOOM_B200_ERR_COMM, "cannot load libnccl.so.2: %s", dlerror());
    g_nccl.GetUniqueId = (int (*)(void*))dlsym(h, "ncclGetUniqueId");
    g_nccl.CommInitRank = (int (*)(void**, int, UniqueId128, int))dlsym(h, "ncclCommInitRank");
    g_nccl.CommDestroy = (int (*)(void*))dlsym(h, "ncclCommDestroy");
    g_nccl.AllReduce = (int (*)(const void*, void*, size_t, int, int, void*, cudaStream_t))dlsym(h, "ncclAllReduce");
    g_nccl.AllGather = (int (*)(const void*, void*, size_t, int, void*, cudaStream_t))dlsym(h, "ncclAllGather");
    g_nccl.GetErrorString = (const char* (*)(int))dlsym(h, "ncclGetErrorString");
    if (!g_nccl.GetUniqueId || !g_nccl.CommInitRank || !g_nccl.CommDestroy || !g_nccl.AllReduce || !g_nccl.AllGather)
        return lb_fail(ctx, LOOM_B200_ERR_COMM, "libnccl.so.2 lacks an expected symbol");
    g_nccl.handle = h;
    return 0;
}

int nccl_fail(loom_b200_ctx* ctx, const char* what, int rc) {
    return lb_fail(ctx, LOOM_B200_ERR_COMM, "%s failed: %s", what, g_nccl.GetErrorString ? g_nccl.GetErrorString(rc) : "?");
}

// per-token sum of squares of a local slice (float64 accumulation), T = float or double
template <typename T>
__global__ void __launch_bounds__(256) lb_sumsq_kernel(const T* __restrict__ x, int n, double* __restrict__ out) {
    __shared__ double red[8];
    lb_pdl_launch_dependents();
    lb_pdl_wait();
    const T* row = x + (size_t)blockIdx.x * n;
    double ss = 0.0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const double v = (double)row[i];
        ss = __dadd_rn(ss, __dmul_rn(v, v));
    }
    ss = lb_warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int i = 0; i < 8; ++i) t += red[i];
        out[blockIdx.x] = t;
    }
}

// per-token absmax of the inner-normalised local slice, computed exactly as the GEMV prologue computes the values
template <typename T>
__global__ void __launch_bounds__(256) lb_scaled_absmax_kernel(const T* __restrict__ x, int n, const double* __restrict__ ss,
                                                               int norm_count, double eps, const float* __restrict__ w, int wlen,
                                                               float* __restrict__ out) {
    __shared__ float red[8];
    lb_pdl_launch_dependents();
    lb_pdl_wait();
    const T* row = x + (size_t)blockIdx.x * n;
    const double sc = __ddiv_rn(1.0, sqrt(__dadd_rn(__ddiv_rn(ss[blockIdx.x], (double)norm_count), eps)));
    float m = 0.0f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const double wi = (w && i < wlen) ? (double)w[i] : 1.0;
        double y;
        if (sizeof(T) == 8) y = __dmul_rn((double)row[i], __dmul_rn(sc, wi));
        else y = (double)(float)__dmul_rn(__dmul_rn((double)row[i], sc), wi);
        m = fmaxf(m, (float)fabs(y));
    }
    m = lb_warp_max(m);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 0; i < 8; ++i) m = fmaxf(m, red[i]);
        out[blockIdx.x] = m < 1e-5f ? 1e-5f : m;  // the quantizer's floor (poly/bitnet_cpu.go:53-55), so that the rescale sees it too
    }
}

// out[n,r] = float(acc[n,r] * os[n] + bias[r]) + residual[n,r]   (O and down projections after the all-reduce)
__global__ void lb_tp_finalize_kernel(const int32_t* __restrict__ acc, int M, int rows, float scale, const float* __restrict__ amax,
                                      const float* __restrict__ bias, const float* residual, float* out) {
    lb_pdl_launch_dependents();
    lb_pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)M * rows) return;
    const int n = (int)(i / rows), r = (int)(i % rows);
    double y = __dmul_rn((double)acc[i], lb_output_scale(scale, amax[n]));
    if (bias) y = __dadd_rn(y, (double)bias[r]);
    float f = (float)y;
    if (residual) f = __fadd_rn(f, residual[i]);
    out[i] = f;
}

// ---- exchange through peer memory (layout and store / poll pair: tp_xchg.cuh) -----------------------------------
// the kernel's last block moves the exchange counter on: a block that starts late still reads the old value
__device__ __forceinline__ void x_finish(unsigned int* ctr, unsigned int* done, uint32_t seq) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned int t = atomicAdd(done, 1u);
        if (t == gridDim.x - 1) {
            *done = 0;
            __threadfence();
            *ctr = seq + 1;
        }
    }
}

// Per token (one CTA of 1024 threads): partial sum of squares -> exchange -> scale -> partial absmax of the normalised
// slice -> exchange -> quantize the slice.  Writes ss[n], amax[n] (whole-vector absmax, floored) and the int8 slice
// q[n, :], which the GEMV then takes as it is: the same per-element operations as the single-GPU prologue
// (lb_pro_value, lb_quant_i8), so the same bytes.
constexpr int kStatThreads = 1024;

template <typename T>
__global__ void __launch_bounds__(kStatThreads) lb_tp_stats_peer_kernel(const T* __restrict__ x, int n_local, int norm_count, double eps,
                                                                        const float* __restrict__ w, int wlen, void* const* peers,
                                                                        int rank, int world, unsigned int* ctr, double* __restrict__ ss_out,
                                                                        float* __restrict__ amax_out, int8_t* __restrict__ q_out,
                                                                        int* status) {
    constexpr int PRO = sizeof(T) == 8 ? LB_PRO_INNERNORM64 : LB_PRO_INNERNORM;
    __shared__ double red[32];
    __shared__ float redf[32];
    __shared__ uint32_t s_part[kXMaxRanks * 2];
    __shared__ uint32_t s_seq;
    __shared__ double s_ss;
    __shared__ float s_amax;
    __shared__ int s_bad;
    lb_pdl_launch_dependents();
    lb_pdl_wait();
    const int n = blockIdx.x, tid = threadIdx.x;
    if (tid == 0) {
        s_seq = ctr[0];
        s_bad = 0;
    }
    const T* row = x + (size_t)n * n_local;
    double ss = 0.0;
    for (int i = tid; i < n_local; i += kStatThreads) {
        const double v = (double)row[i];
        ss = __dadd_rn(ss, __dmul_rn(v, v));
    }
    ss = lb_warp_sum(ss);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    const uint32_t seq = s_seq;
    const size_t half = (size_t)(seq & 1);
    if (tid == 0) {
        double t = 0.0;
        for (int i = 0; i < 32; ++i) t += red[i];
        s_ss = t;
    }
    __syncthreads();
    if (tid < world * 2) {  // my partial to every rank (own mailbox included), low and high word
        const int peer = tid >> 1, hw = tid & 1;
        const unsigned long long bits = (unsigned long long)__double_as_longlong(s_ss);
        char* dst = (char*)peers[peer] + kXRegionA + ((((half * kXMaxRanks + rank) * 8 + n) * 2 + hw) * 8);
        ll_store(dst, (uint32_t)(bits >> (32 * hw)), seq);
    }
    if (tid < world * 2) {  // every rank's partial from my mailbox
        const int r = tid >> 1, hw = tid & 1;
        const char* src = (const char*)peers[rank] + kXRegionA + ((((half * kXMaxRanks + r) * 8 + n) * 2 + hw) * 8);
        if (!ll_wait(src, seq, &s_part[tid])) s_bad = 1;
    }
    __syncthreads();
    if (tid == 0) {
        double t = 0.0;
        for (int r = 0; r < world; ++r)  // rank order on every rank: identical bits everywhere
            t = __dadd_rn(t, __longlong_as_double((long long)(((unsigned long long)s_part[2 * r + 1] << 32) | s_part[2 * r])));
        s_ss = t;
        ss_out[n] = t;
    }
    __syncthreads();
    const double root = sqrt(__dadd_rn(__ddiv_rn(s_ss, (double)norm_count), eps));
    const double rr = __ddiv_rn(1.0, root);
    float m = 0.0f;
    for (int i = tid; i < n_local; i += kStatThreads) {
        const double wi = (w && i < wlen) ? (double)w[i] : 1.0;
        m = fmaxf(m, (float)fabs(lb_pro_value<PRO>((double)row[i], root, rr, wi)));
    }
    m = lb_warp_max(m);
    if ((tid & 31) == 0) redf[tid >> 5] = m;
    __syncthreads();
    if (tid < world) {
        float t = 0.0f;
        for (int i = 0; i < 32; ++i) t = fmaxf(t, redf[i]);
        char* dst = (char*)peers[tid] + kXRegionB + (((half * kXMaxRanks + rank) * 8 + n) * 8);
        ll_store(dst, __float_as_uint(t), seq);
    }
    if (tid < world) {
        const char* src = (const char*)peers[rank] + kXRegionB + (((half * kXMaxRanks + tid) * 8 + n) * 8);
        if (!ll_wait(src, seq, &s_part[tid])) s_bad = 1;
    }
    __syncthreads();
    if (tid == 0) {
        float t = 0.0f;
        for (int r = 0; r < world; ++r) t = fmaxf(t, __uint_as_float(s_part[r]));
        t = t < 1e-5f ? 1e-5f : t;  // the quantizer's floor (poly/bitnet_cpu.go:53-55)
        s_amax = t;
        amax_out[n] = t;
        if (s_bad) atomicExch(status, 5);
    }
    __syncthreads();
    const double qs = __ddiv_rn(127.0, (double)s_amax);
    uint32_t* qrow = reinterpret_cast<uint32_t*>(q_out + (size_t)n * n_local);
    for (int u = tid; u < (n_local >> 2); u += kStatThreads) {
        uint32_t packed = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int i = 4 * u + k;
            const double wi = (w && i < wlen) ? (double)w[i] : 1.0;
            packed |= (uint32_t)(lb_quant_i8(lb_pro_value<PRO>((double)row[i], root, rr, wi), qs) & 0xff) << (8 * k);
        }
        qrow[u] = packed;
    }
    x_finish(ctr, ctr + 1, seq);
}

// out[n,r] = float(sum over ranks of acc[n,r] * os[n] + bias[r]) + residual[n,r]: every thread sends its partial
// accumulator to every rank, then adds up what the ranks sent it, in rank order.
__global__ void __launch_bounds__(256) lb_tp_finalize_peer_kernel(const int32_t* __restrict__ acc, int M, int rows, float scale,
                                                                  const float* __restrict__ amax, const float* __restrict__ bias,
                                                                  const float* residual, float* out, void* const* peers, int rank,
                                                                  int world, unsigned int* ctr, int* status) {
    __shared__ uint32_t s_seq;
    lb_pdl_launch_dependents();
    lb_pdl_wait();
    if (threadIdx.x == 0) s_seq = ctr[0];
    __syncthreads();
    const uint32_t seq = s_seq;
    const size_t half = (size_t)(seq & 1);
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < (size_t)M * rows) {
        const uint32_t mine = (uint32_t)acc[i];
        for (int r = 0; r < world; ++r)
            ll_store((char*)peers[r] + kXRegionC + ((half * kXMaxRanks + rank) * kXMaxAcc + i) * 8, mine, seq);
        int sum = 0;
        bool ok = true;
        for (int r = 0; r < world; ++r) {
            uint32_t d;
            ok = ll_wait((const char*)peers[rank] + kXRegionC + ((half * kXMaxRanks + r) * kXMaxAcc + i) * 8, seq, &d) && ok;
            sum += (int)d;
        }
        if (!ok) atomicExch(status, 5);
        const int n = (int)(i / rows), r = (int)(i % rows);
        double y = __dmul_rn((double)sum, lb_output_scale(scale, amax[n]));
        if (bias) y = __dadd_rn(y, (double)bias[r]);
        float f = (float)y;
        if (residual) f = __fadd_rn(f, residual[i]);
        out[i] = f;
    }
    x_finish(ctr, ctr + 1, seq);
}

}  // namespace

int lb_tp_allreduce(loom_b200_ctx* ctx, void* buf, size_t count, int dtype, int op) {
    if (ctx->tp_world <= 1) return 0;
    int rc = g_nccl.AllReduce(buf, buf, count, dtype, op, ctx->nccl_comm, ctx->stream);
    if (rc != 0) return nccl_fail(ctx, "ncclAllReduce", rc);
    return 0;
}

int lb_tp_allgather_f32(loom_b200_ctx* ctx, const float* send, float* recv, size_t count_per_rank) {
    if (ctx->tp_world <= 1) return 0;
    int rc = g_nccl.AllGather(send, recv, count_per_rank, kNcclFloat32, ctx->nccl_comm, ctx->stream);
    if (rc != 0) return nccl_fail(ctx, "ncclAllGather", rc);
    return 0;
}

// Row-sharded ternary linear with the inner RMSNorm over the sharded dimension:
//   x_local [M, K_local] (float or double) -> out [M, rows] (+ residual), identical on every rank.
// stats: device scratch of at least 2*M doubles; acc: device scratch of M*rows int32.
int lb_tp_rowsharded_linear(loom_b200_ctx* ctx, const loom_b200_weight* w, bool x_is_f64, const void* x, int M, int K_global,
                            const float* inner_w, int inner_w_len, double eps, const float* bias, const float* residual,
                            float* out, double* stats, int32_t* acc) {
    const int Kl = w->cols;
    double* ss = stats;
    float* amax = reinterpret_cast<float*>(stats + M);
    const bool peer = ctx->tp_peer && ctx->opt_tp_peer && ctx->tp_world > 1 && (size_t)M * w->rows <= (size_t)kXMaxAcc && M <= 8;
    // Two launches: the statistics kernel, then the GEMV that takes its int8 slice and exchanges the partial sums in its
    // own epilogue.  Option "tp_fused" = 0 keeps the three-launch form (statistics, GEMV, finalize).  Moving the
    // statistics exchange into the GEMV's prologue as well (one launch) was built and measured 2.3x slower -- every CTA
    // repeats two NVLink round trips and the staged prologue cannot be used -- and is not kept.
    const bool fused = peer && ctx->opt_tp_fused && (Kl & 3) == 0 && out != nullptr;
    int8_t* q8 = nullptr;
    if (peer) {
        LB_REQUIRE(ctx, (Kl & 3) == 0, "tensor-parallel shard width %d must be a multiple of 4", Kl);
        if (int rc = lb_ensure_quant_scratch(ctx, (size_t)kChunkTokens * Kl + 256)) return rc;
        q8 = reinterpret_cast<int8_t*>(ctx->quant_scratch);
        void* const* peers = (void* const*)ctx->peer_xbuf_dev;
        if (x_is_f64)
            lb_tp_stats_peer_kernel<double><<<M, kStatThreads, 0, ctx->stream>>>((const double*)x, Kl, K_global, eps, inner_w, inner_w ? inner_w_len : 0,
                                                                                 peers, ctx->tp_rank, ctx->tp_world, ctx->x_ctr, ss, amax, q8,
                                                                                 ctx->status_dev);
        else
            lb_tp_stats_peer_kernel<float><<<M, kStatThreads, 0, ctx->stream>>>((const float*)x, Kl, K_global, eps, inner_w, inner_w ? inner_w_len : 0,
                                                                                peers, ctx->tp_rank, ctx->tp_world, ctx->x_ctr, ss, amax, q8,
                                                                                ctx->status_dev);
        LB_CHECK_LAUNCH(ctx, "lb_tp_stats_peer_kernel");
        ctx->launches++;
    } else {
    if (x_is_f64) lb_sumsq_kernel<double><<<M, 256, 0, ctx->stream>>>((const double*)x, Kl, ss);
    else lb_sumsq_kernel<float><<<M, 256, 0, ctx->stream>>>((const float*)x, Kl, ss);
    LB_CHECK_LAUNCH(ctx, "lb_sumsq_kernel");
    if (int rc = lb_tp_allreduce(ctx, ss, (size_t)M, kNcclFloat64, kNcclSum)) return rc;
    if (x_is_f64)
        lb_scaled_absmax_kernel<double><<<M, 256, 0, ctx->stream>>>((const double*)x, Kl, ss, K_global, eps, inner_w, inner_w_len, amax);
    else
        lb_scaled_absmax_kernel<float><<<M, 256, 0, ctx->stream>>>((const float*)x, Kl, ss, K_global, eps, inner_w, inner_w_len, amax);
    LB_CHECK_LAUNCH(ctx, "lb_scaled_absmax_kernel");
    if (int rc = lb_tp_allreduce(ctx, amax, (size_t)M, kNcclFloat32, kNcclMax)) return rc;
    }
    LbGemvParams p = {};
    p.nseg = 1;
    p.seg[0].tiles = w->tiles;
    p.seg[0].rows = w->rows;
    p.seg[0].scale = w->scale;
    p.seg[0].acc_out = acc;
    p.seg[0].kind = LB_OUT_ACC;
    p.K = Kl;
    p.M = M;
    if (peer) {  // the statistics kernel already quantized the slice
        p.pro = LB_PRO_Q8;
        p.x = q8;
        p.amax_in = amax;
    } else {
        p.pro = x_is_f64 ? LB_PRO_INNERNORM64 : LB_PRO_INNERNORM;
        p.x = x;
        p.norm_w = inner_w;
        p.norm_w_len = inner_w ? inner_w_len : 0;
        p.eps = eps;
        p.given_ss = ss;
        p.given_amax = amax;
        p.norm_count = K_global;
    }
    p.epi = LB_EPI_GENERIC;
    p.act = LOOM_B200_ACT_LINEAR;
    if (fused) {
        p.epi = LB_EPI_TPSUM;
        p.seg[0].acc_out = nullptr;
        p.seg[0].kind = LB_OUT_F32;
        p.seg[0].out = out;
        p.seg[0].bias = bias;
        p.residual = residual;
        p.xchg_peers = (void* const*)ctx->peer_xbuf_dev;
        p.xchg_rank = ctx->tp_rank;
        p.xchg_world = ctx->tp_world;
        p.xchg_ctr = ctx->x_ctr;
    }
    LB_REQUIRE(ctx, (Kl & 3) == 0, "tensor-parallel shard width %d must be a multiple of 4", Kl);
    if (int rc = lb_gemv_finalize_params(ctx, p)) return rc;
    if (int rc = lb_launch_gemv(ctx, p)) return rc;
    const size_t n = (size_t)M * w->rows;
    if (fused) return 0;
    if (peer) {
        lb_tp_finalize_peer_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(acc, M, w->rows, w->scale, amax, bias, residual, out,
                                                                                          (void* const*)ctx->peer_xbuf_dev, ctx->tp_rank,
                                                                                          ctx->tp_world, ctx->x_ctr + 2, ctx->status_dev);
        LB_CHECK_LAUNCH(ctx, "lb_tp_finalize_peer_kernel");
        ctx->launches++;
        return 0;
    }
    if (int rc = lb_tp_allreduce(ctx, acc, (size_t)M * w->rows, kNcclInt32, kNcclSum)) return rc;
    lb_tp_finalize_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(acc, M, w->rows, w->scale, amax, bias, residual, out);
    LB_CHECK_LAUNCH(ctx, "lb_tp_finalize_kernel");
    return 0;
}

int lb_tp_block_stats(loom_b200_ctx* ctx, bool x_is_f64, const void* x, int M, int Kl, int K_global, double eps, const float* inner_w,
                      int inner_w_len, double* ss, float* amax) {
    if (x_is_f64) lb_sumsq_kernel<double><<<M, 256, 0, ctx->stream>>>((const double*)x, Kl, ss);
    else lb_sumsq_kernel<float><<<M, 256, 0, ctx->stream>>>((const float*)x, Kl, ss);
    LB_CHECK_LAUNCH(ctx, "lb_sumsq_kernel");
    if (int rc = lb_tp_allreduce(ctx, ss, (size_t)M, kNcclFloat64, kNcclSum)) return rc;
    if (x_is_f64)
        lb_scaled_absmax_kernel<double><<<M, 256, 0, ctx->stream>>>((const double*)x, Kl, ss, K_global, eps, inner_w, inner_w ? inner_w_len : 0, amax);
    else
        lb_scaled_absmax_kernel<float><<<M, 256, 0, ctx->stream>>>((const float*)x, Kl, ss, K_global, eps, inner_w, inner_w ? inner_w_len : 0, amax);
    LB_CHECK_LAUNCH(ctx, "lb_scaled_absmax_kernel");
    ctx->launches += 2;
    return lb_tp_allreduce(ctx, amax, (size_t)M, kNcclFloat32, kNcclMax);
}

int lb_tp_block_finalize(loom_b200_ctx* ctx, int32_t* acc, int M, int rows, float scale, const float* amax, const float* bias,
                         const float* residual, float* out) {
    if (int rc = lb_tp_allreduce(ctx, acc, (size_t)M * rows, kNcclInt32, kNcclSum)) return rc;
    const size_t n = (size_t)M * rows;
    lb_tp_finalize_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(acc, M, rows, scale, amax, bias, residual, out);
    LB_CHECK_LAUNCH(ctx, "lb_tp_finalize_kernel");
    ctx->launches++;
    return 0;
}

extern "C" {

int loom_b200_tp_unique_id(uint8_t* id128) {
    if (!id128) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "tp_unique_id: NULL buffer");
    if (int rc = load_nccl(nullptr)) return rc;
    UniqueId128 id;
    int rc = g_nccl.GetUniqueId(&id);
    if (rc != 0) return nccl_fail(nullptr, "ncclGetUniqueId", rc);
    memcpy(id128, id.internal, 128);
    return 0;
}

int loom_b200_tp_init(loom_b200_ctx* ctx, int rank, int world, const uint8_t* id128) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "tp_init: ctx is NULL");
    LB_REQUIRE(ctx, world >= 1 && rank >= 0 && rank < world && id128, "tp_init: rank %d of %d", rank, world);
    LB_REQUIRE(ctx, ctx->nccl_comm == nullptr, "tp_init: the context already has a communicator");
    if (world == 1) {
        ctx->tp_rank = 0;
        ctx->tp_world = 1;
        return 0;
    }
    if (int rc = load_nccl(ctx)) return rc;
    if (int rc = lb_set_device(ctx)) return rc;
    UniqueId128 id;
    memcpy(id.internal, id128, 128);
    void* comm = nullptr;
    int rc = g_nccl.CommInitRank(&comm, world, id, rank);
    if (rc != 0) return nccl_fail(ctx, "ncclCommInitRank", rc);
    ctx->nccl_comm = comm;
    ctx->tp_rank = rank;
    ctx->tp_world = world;
    return 0;
}

int loom_b200_tp_peer_handle(loom_b200_ctx* ctx, uint8_t* handle64) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "tp_peer_handle: ctx is NULL");
    LB_REQUIRE(ctx, handle64 != nullptr, "tp_peer_handle: NULL buffer");
    LB_REQUIRE(ctx, ctx->tp_world > 1 && ctx->tp_world <= kXMaxRanks, "tp_peer_handle: needs a group of 2..%d ranks (tp_init first)", kXMaxRanks);
    if (ctx->capturing) return lb_fail(ctx, LOOM_B200_ERR_INVALID, "tp_peer_handle cannot be recorded");
    if (int rc = lb_set_device(ctx)) return rc;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the C ABI passes IPC handles as 64 bytes");
    if (!ctx->xbuf) {
        LB_CUDA(ctx, cudaMalloc(&ctx->xbuf, kXBytes));
        LB_CUDA(ctx, cudaMemset(ctx->xbuf, 0, kXBytes));
        LB_CUDA(ctx, cudaMalloc(&ctx->x_ctr, 8 * sizeof(unsigned int)));
        // {statistics sequence, arrivals, accumulator sequence, arrivals, arrivals of the GEMV that carries both exchanges};
        // sequence numbers start at 1: a zeroed mailbox never matches
        const unsigned int init[8] = {1u, 0u, 1u, 0u, 0u, 1u, 0u, 0u};  // [5]: sequence of the sharded head's (max, index) exchange
        LB_CUDA(ctx, cudaMemcpy(ctx->x_ctr, init, sizeof(init), cudaMemcpyHostToDevice));
    }
    cudaIpcMemHandle_t h;
    LB_CUDA(ctx, cudaIpcGetMemHandle(&h, ctx->xbuf));
    memcpy(handle64, &h, 64);
    return 0;
}

int loom_b200_tp_attach_peers(loom_b200_ctx* ctx, const uint8_t* handles) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "tp_attach_peers: ctx is NULL");
    LB_REQUIRE(ctx, handles != nullptr, "tp_attach_peers: NULL handles");
    LB_REQUIRE(ctx, ctx->xbuf != nullptr, "tp_attach_peers: call tp_peer_handle first");
    LB_REQUIRE(ctx, !ctx->tp_peer, "tp_attach_peers: peers are already attached");
    if (ctx->capturing) return lb_fail(ctx, LOOM_B200_ERR_INVALID, "tp_attach_peers cannot be recorded");
    if (int rc = lb_set_device(ctx)) return rc;
    for (int r = 0; r < ctx->tp_world; ++r) {
        if (r == ctx->tp_rank) {
            ctx->peer_xbuf_host[r] = ctx->xbuf;
            continue;
        }
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + (size_t)r * 64, 64);
        void* p = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            cudaGetLastError();
            for (int q = 0; q < r; ++q)
                if (q != ctx->tp_rank && ctx->peer_xbuf_host[q]) cudaIpcCloseMemHandle(ctx->peer_xbuf_host[q]);
            memset(ctx->peer_xbuf_host, 0, sizeof(ctx->peer_xbuf_host));
            return lb_fail(ctx, LOOM_B200_ERR_COMM, "cudaIpcOpenMemHandle for rank %d: %s", r, cudaGetErrorString(e));
        }
        ctx->peer_xbuf_host[r] = p;
    }
    LB_CUDA(ctx, cudaMalloc(&ctx->peer_xbuf_dev, kXMaxRanks * sizeof(void*)));
    LB_CUDA(ctx, cudaMemcpy(ctx->peer_xbuf_dev, ctx->peer_xbuf_host, kXMaxRanks * sizeof(void*), cudaMemcpyHostToDevice));
    ctx->tp_peer = true;
    return 0;
}

void loom_b200_tp_finalize(loom_b200_ctx* ctx) {
    if (!ctx) return;
    if (ctx->xbuf || ctx->nccl_comm) {
        cudaSetDevice(ctx->device);
        cudaStreamSynchronize(ctx->stream);
    }
    if (ctx->tp_peer) {
        for (int r = 0; r < ctx->tp_world; ++r)
            if (r != ctx->tp_rank && ctx->peer_xbuf_host[r]) cudaIpcCloseMemHandle(ctx->peer_xbuf_host[r]);
        ctx->tp_peer = false;
    }
    memset(ctx->peer_xbuf_host, 0, sizeof(ctx->peer_xbuf_host));
    if (ctx->peer_xbuf_dev) cudaFree(ctx->peer_xbuf_dev);
    if (ctx->x_ctr) cudaFree(ctx->x_ctr);
    if (ctx->xbuf) cudaFree(ctx->xbuf);
    ctx->peer_xbuf_dev = nullptr;
    ctx->x_ctr = nullptr;
    ctx->xbuf = nullptr;
    if (ctx->nccl_comm) {
        g_nccl.CommDestroy(ctx->nccl_comm);
        ctx->nccl_comm = nullptr;
    }
    ctx->tp_world = 1;
    ctx->tp_rank = 0;
}

int loom_b200_tp_allreduce_i32(loom_b200_ctx* ctx, int32_t* buf, size_t n) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "tp_allreduce_i32: ctx is NULL");
    LB_REQUIRE(ctx, buf || n == 0, "tp_allreduce_i32: NULL buffer");
    if (int rc = lb_set_device(ctx)) return rc;
    return lb_tp_allreduce(ctx, buf, n, kNcclInt32, kNcclSum);
}

int loom_b200_tp_rank(const loom_b200_ctx* ctx) { return ctx ? ctx->tp_rank : -1; }
int loom_b200_tp_world(const loom_b200_ctx* ctx) { return ctx ? ctx->tp_world : -1; }

int loom_b200_tp_rowsharded_linear(loom_b200_ctx* ctx, const loom_b200_weight* w, int batch, const float* x_local,
                                   int cols_global, const float* inner_w_local, int inner_w_len, double eps,
                                   const float* bias, const float* residual, float* out) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "tp_rowsharded_linear: ctx is NULL");
    LB_REQUIRE(ctx, w && x_local && out, "tp_rowsharded_linear: NULL argument");
    LB_REQUIRE(ctx, batch >= 1 && batch <= kChunkTokens, "tp_rowsharded_linear: batch %d outside 1..%d", batch, kChunkTokens);
    LB_REQUIRE(ctx, cols_global >= w->cols, "tp_rowsharded_linear: cols_global %d below the slice width %d", cols_global, w->cols);
    LB_REQUIRE(ctx, inner_w_len >= 0 && (inner_w_local || inner_w_len == 0), "tp_rowsharded_linear: inner norm length without weights");
    if (ctx->capturing) return lb_fail(ctx, LOOM_B200_ERR_INVALID, "tp_rowsharded_linear uses the context scratch and cannot be recorded");
    if (int rc = lb_set_device(ctx)) return rc;
    const size_t stats_bytes = 2 * (size_t)batch * sizeof(double), acc_bytes = (size_t)batch * w->rows * sizeof(int32_t);
    if (int rc = lb_ensure_scratch(ctx, 256 + stats_bytes + acc_bytes)) return rc;
    double* stats = reinterpret_cast<double*>(ctx->scratch);
    int32_t* acc = reinterpret_cast<int32_t*>((char*)ctx->scratch + ((stats_bytes + 255) & ~(size_t)255));
    return lb_tp_rowsharded_linear(ctx, w, false, x_local, batch, cols_global, inner_w_local, inner_w_len, eps > 0 ? eps : 1e-5, bias,
                                   residual, out, stats, acc);
}

}  // extern "C"
