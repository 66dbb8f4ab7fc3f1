// quantize.cu -- per-token absmax int8 activation quantization, the SwiGLU gate product and the
// BitNet inner RMSNorm as stand-alone dispatches (the decode path fuses them into the GEMV instead).
#include "common.cuh"

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

}  // namespace

extern "C" {

int loom_b200_quantize_activation(loom_b200_ctx* ctx, int batch, int in, const float* x, int8_t* q, float* amax) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "quantize_activation: ctx is NULL");
    LB_REQUIRE(ctx, batch >= 0 && in > 0, "quantize_activation: bad shape batch=%d in=%d", batch, in);
    if (batch == 0) return 0;
    LB_REQUIRE(ctx, x && q && amax, "quantize_activation: NULL buffer");
    if (int rc = lb_set_device(ctx)) return rc;
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
