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
    LbGemvParams p = {};
    p.nseg = 1;
    p.seg[0].tiles = w->tiles;
    p.seg[0].rows = w->rows;
    p.seg[0].scale = w->scale;
    p.seg[0].acc_out = acc;
    p.seg[0].kind = LB_OUT_ACC;
    p.K = Kl;
    p.M = M;
    p.pro = x_is_f64 ? LB_PRO_INNERNORM64 : LB_PRO_INNERNORM;
    p.x = x;
    p.norm_w = inner_w;
    p.norm_w_len = inner_w ? inner_w_len : 0;
    p.eps = eps;
    p.given_ss = ss;
    p.given_amax = amax;
    p.norm_count = K_global;
    p.epi = LB_EPI_GENERIC;
    p.act = LOOM_B200_ACT_LINEAR;
    LB_REQUIRE(ctx, (Kl & 3) == 0, "tensor-parallel shard width %d must be a multiple of 4", Kl);
    if (int rc = lb_gemv_finalize_params(ctx, p)) return rc;
    if (int rc = lb_launch_gemv(ctx, p)) return rc;
    if (int rc = lb_tp_allreduce(ctx, acc, (size_t)M * w->rows, kNcclInt32, kNcclSum)) return rc;
    const size_t n = (size_t)M * w->rows;
    lb_tp_finalize_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(acc, M, w->rows, w->scale, amax, bias, residual, out);
    LB_CHECK_LAUNCH(ctx, "lb_tp_finalize_kernel");
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

void loom_b200_tp_finalize(loom_b200_ctx* ctx) {
    if (!ctx || !ctx->nccl_comm) return;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    g_nccl.CommDestroy(ctx->nccl_comm);
    ctx->nccl_comm = nullptr;
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
