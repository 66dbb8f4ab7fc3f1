// quantize.cu -- per-token absmax int8 activation quantization, the SwiGLU gate product and the
// BitNet inner RMSNorm as stand-alone dispatches (the decode path fuses them into the GEMV instead).
#include "gemv_ternary.cuh"

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float block_max(float v, float* red) {
    v = lb_warp_max(v);
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();  // red may still be read by a previous call
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = red[0];
    for (int i = 1; i < (int)(blockDim.x >> 5); ++i) r = fmaxf(r, red[i]);
    return r;
}

__device__ __forceinline__ double block_sum(double v, double* red) {
    v = lb_warp_sum(v);
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    double r = 0.0;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) r += red[i];  // fixed order: every thread gets the same bits
    return r;
}

// One CTA per token.  T = float or double.
template <typename T>
__global__ void __launch_bounds__(kThreads) lb_quantize_kernel(const T* __restrict__ x, int n, int8_t* __restrict__ q,
                                                               float* __restrict__ amax_out) {
    __shared__ float red[32];
    const T* row = x + (size_t)blockIdx.x * n;
    int8_t* qrow = q + (size_t)blockIdx.x * n;
    float m = 0.0f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) m = fmaxf(m, (float)fabs((double)row[i]));
    m = block_max(m, red);
    if (m < 1e-5f) m = 1e-5f;
    double s = __ddiv_rn(127.0, (double)m);
    if ((n & 3) == 0 && ((uintptr_t)qrow & 3) == 0) {
        uint32_t* q4 = reinterpret_cast<uint32_t*>(qrow);
        for (int i = threadIdx.x; i < n / 4; i += blockDim.x) {
            uint32_t p = 0;
#pragma unroll
            for (int k = 0; k < 4; ++k) p |= (uint32_t)(lb_quant_i8((double)row[4 * i + k], s) & 0xff) << (8 * k);
            q4[i] = p;
        }
    } else {
        for (int i = threadIdx.x; i < n; i += blockDim.x) qrow[i] = (int8_t)lb_quant_i8((double)row[i], s);
    }
    if (threadIdx.x == 0) amax_out[blockIdx.x] = m;
}

__global__ void lb_gate_product_kernel(const float* __restrict__ gate, const float* __restrict__ up, size_t n, int act,
                                       float* __restrict__ out) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = (float)lb_gate_product((double)gate[i], (double)up[i], act);
}

__global__ void __launch_bounds__(kThreads) lb_inner_rmsnorm_kernel(float* __restrict__ x, int n,
                                                                    const float* __restrict__ weight, int wlen,
                                                                    double eps) {
    __shared__ double red[32];
    float* row = x + (size_t)blockIdx.x * n;
    double ss = 0.0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        double f = (double)row[i];
        ss = __dadd_rn(ss, __dmul_rn(f, f));
    }
    ss = block_sum(ss, red);
    double sc = __ddiv_rn(1.0, sqrt(__dadd_rn(__ddiv_rn(ss, (double)n), eps)));
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        double w = (weight && i < wlen) ? (double)weight[i] : 1.0;
        row[i] = (float)__dmul_rn(__dmul_rn((double)row[i], sc), w);
    }
}

// ---- stand-alone prologue of the GEMV for wide inputs ---------------------------------------------------------
// The GEMV normally normalises and quantizes its input row inside every CTA (nothing to launch, nothing to
// write).  That costs time proportional to K in each CTA; from kSplitQuantK columns on it is cheaper to do it
// once, here, with one 1024-thread CTA per token, and let the GEMV load the int8 row.  Same operations in the
// same order per element as stage_row_fast, so the int8 values and the absmax are the same bits.
constexpr int kNqThreads = 1024;

template <int PRO>
__global__ void __launch_bounds__(kNqThreads) lb_norm_quantize_kernel(const LbGemvParams p, int8_t* __restrict__ q,
                                                                      float* __restrict__ amax_out) {
    __shared__ double red_d[32];
    __shared__ float red_f[32];
    constexpr bool f64 = PRO == LB_PRO_INNERNORM64;
    const int n = blockIdx.x, tid = threadIdx.x, K = p.K, units = K >> 2;
    lb_pdl_launch_dependents();
    lb_pdl_wait();
    const void* row = f64 ? (const void*)((const double*)p.x + (size_t)n * K) : (const void*)((const float*)p.x + (size_t)n * K);
    auto load4 = [&](int idx, double* v) {
        if (f64) {
            const double2 a = reinterpret_cast<const double2*>(row)[2 * idx], b = reinterpret_cast<const double2*>(row)[2 * idx + 1];
            v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
        } else {
            const float4 a = reinterpret_cast<const float4*>(row)[idx];
            v[0] = (double)a.x; v[1] = (double)a.y; v[2] = (double)a.z; v[3] = (double)a.w;
        }
    };
    const bool have_w = PRO != LB_PRO_F32 && p.norm_w != nullptr;
    auto weights4 = [&](int idx, double* w) {
        w[0] = w[1] = w[2] = w[3] = 1.0;
        if (!have_w) return;
        if (4 * idx + 4 <= p.norm_w_len) {
            const float4 g = reinterpret_cast<const float4*>(p.norm_w)[idx];
            w[0] = (double)g.x; w[1] = (double)g.y; w[2] = (double)g.z; w[3] = (double)g.w;
        } else {
            for (int k = 0; k < 4; ++k)
                if (4 * idx + k < p.norm_w_len) w[k] = (double)p.norm_w[4 * idx + k];
        }
    };
    double root = 1.0, rr = 1.0;
    if (PRO >= LB_PRO_BLOCKNORM) {
        double ss = 0.0;
        if (p.given_ss) {
            ss = p.given_ss[n];
        } else {
#pragma unroll 2
            for (int idx = tid; idx < units; idx += kNqThreads) {
                double v[4];
                load4(idx, v);
#pragma unroll
                for (int k = 0; k < 4; ++k) ss = __dadd_rn(ss, __dmul_rn(v[k], v[k]));
            }
            ss = block_sum(ss, red_d);
        }
        const double mean = __dadd_rn(__ddiv_rn(ss, (double)(p.norm_count > 0 ? p.norm_count : K)), p.eps);
        root = sqrt(mean);
        rr = __ddiv_rn(1.0, root);
    }
    float m = 0.0f;
    if (p.given_amax) {
        m = p.given_amax[n];
    } else {
#pragma unroll 2
        for (int idx = tid; idx < units; idx += kNqThreads) {
            double v[4], w[4];
            load4(idx, v);
            weights4(idx, w);
#pragma unroll
            for (int k = 0; k < 4; ++k) m = fmaxf(m, (float)fabs(lb_pro_value<PRO>(v[k], root, rr, w[k])));
        }
        m = block_max(m, red_f);
    }
    const float amax = m < 1e-5f ? 1e-5f : m;
    const double s = __ddiv_rn(127.0, (double)amax);
#pragma unroll 2
    for (int idx = tid; idx < units; idx += kNqThreads) {
        double v[4], w[4];
        load4(idx, v);
        weights4(idx, w);
        uint32_t packed = 0;
        float y4[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const double y = lb_pro_value<PRO>(v[k], root, rr, w[k]);
            y4[k] = (float)y;
            packed |= (uint32_t)(lb_quant_i8(y, s) & 0xff) << (8 * k);
        }
        reinterpret_cast<uint32_t*>(q + (size_t)n * K)[idx] = packed;
        if (p.norm_out) reinterpret_cast<float4*>(p.norm_out + (size_t)n * K)[idx] = make_float4(y4[0], y4[1], y4[2], y4[3]);
    }
    if (tid == 0) amax_out[n] = amax;
}

}  // namespace

int lb_launch_norm_quantize(loom_b200_ctx* ctx, const LbGemvParams& p, int8_t* q, float* amax) {
    using Kern = void (*)(const LbGemvParams, int8_t*, float*);
    Kern kern = nullptr;
    switch (p.pro) {
        case LB_PRO_F32: kern = lb_norm_quantize_kernel<LB_PRO_F32>; break;
        case LB_PRO_BLOCKNORM: kern = lb_norm_quantize_kernel<LB_PRO_BLOCKNORM>; break;
        case LB_PRO_INNERNORM: kern = lb_norm_quantize_kernel<LB_PRO_INNERNORM>; break;
        case LB_PRO_INNERNORM64: kern = lb_norm_quantize_kernel<LB_PRO_INNERNORM64>; break;
        default: return lb_fail(ctx, LOOM_B200_ERR_INVALID, "norm_quantize: prologue %d has nothing to quantize", p.pro);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.M);
    cfg.blockDim = dim3(kNqThreads);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->opt_pdl ? 1 : 0;
    LB_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, p, q, amax));
    ctx->launches++;
    return 0;
}

extern "C" {

int loom_b200_quantize_activation(loom_b200_ctx* ctx, int batch, int in, const float* x, int8_t* q, float* amax) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "quantize_activation: ctx is NULL");
    LB_REQUIRE(ctx, batch >= 0 && in > 0, "quantize_activation: bad shape batch=%d in=%d", batch, in);
    if (batch == 0) return 0;
    LB_REQUIRE(ctx, x && q && amax, "quantize_activation: NULL buffer");
    if (int rc = lb_set_device(ctx)) return rc;
    // wide rows: the 1024-thread kernel with vector loads (same operations per element, same bytes out)
    if (in >= 2048 && (in & 3) == 0 && (((uintptr_t)x) & 15) == 0 && (((uintptr_t)q) & 3) == 0) {
        LbGemvParams p = {};
        p.pro = LB_PRO_F32;
        p.x = x;
        p.K = in;
        p.M = batch;
        return lb_launch_norm_quantize(ctx, p, q, amax);
    }
    lb_quantize_kernel<float><<<batch, kThreads, 0, ctx->stream>>>(x, in, q, amax);
    LB_CHECK_LAUNCH(ctx, "lb_quantize_kernel<float>");
    return 0;
}

int loom_b200_quantize_activation_f64(loom_b200_ctx* ctx, int batch, int in, const double* x, int8_t* q, float* amax) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "quantize_activation_f64: ctx is NULL");
    LB_REQUIRE(ctx, batch >= 0 && in > 0, "quantize_activation_f64: bad shape batch=%d in=%d", batch, in);
    if (batch == 0) return 0;
    LB_REQUIRE(ctx, x && q && amax, "quantize_activation_f64: NULL buffer");
    if (int rc = lb_set_device(ctx)) return rc;
    lb_quantize_kernel<double><<<batch, kThreads, 0, ctx->stream>>>(x, in, q, amax);
    LB_CHECK_LAUNCH(ctx, "lb_quantize_kernel<double>");
    return 0;
}

int loom_b200_gate_product(loom_b200_ctx* ctx, int batch, int hidden, int activation, const float* gate, const float* up,
                           float* out) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "gate_product: ctx is NULL");
    LB_REQUIRE(ctx, batch >= 0 && hidden > 0, "gate_product: bad shape batch=%d hidden=%d", batch, hidden);
    if (batch == 0) return 0;
    LB_REQUIRE(ctx, gate && up && out, "gate_product: NULL buffer");
    if (int rc = lb_set_device(ctx)) return rc;
    size_t n = (size_t)batch * hidden;
    lb_gate_product_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(gate, up, n, activation, out);
    LB_CHECK_LAUNCH(ctx, "lb_gate_product_kernel");
    return 0;
}

int loom_b200_inner_rmsnorm(loom_b200_ctx* ctx, int batch, int n, float* x, const float* weight, int weight_len,
                            double eps) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "inner_rmsnorm: ctx is NULL");
    LB_REQUIRE(ctx, batch >= 0 && n > 0, "inner_rmsnorm: bad shape batch=%d n=%d", batch, n);
    if (batch == 0) return 0;
    LB_REQUIRE(ctx, x != nullptr, "inner_rmsnorm: NULL buffer");
    LB_REQUIRE(ctx, weight_len >= 0 && (weight || weight_len == 0), "inner_rmsnorm: weight_len %d without weights", weight_len);
    if (int rc = lb_set_device(ctx)) return rc;
    if (eps <= 0) eps = 1e-5;
    lb_inner_rmsnorm_kernel<<<batch, kThreads, 0, ctx->stream>>>(x, n, weight, weight_len, eps);
    LB_CHECK_LAUNCH(ctx, "lb_inner_rmsnorm_kernel");
    return 0;
}

}  // extern "C"
