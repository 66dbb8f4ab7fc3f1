// no_alloc.cu -- the ternary linear for callers that must not allocate device memory.
//
// The regular entry point (loom_b200_ternary_linear) keeps the scratch of its stream-K fix-up -- int32 partial
// sums and arrival counters -- in buffers that the context grows with cudaMalloc the first time a larger shape
// comes along.  Some hosts cannot accept that on their inference path: an embedder that gives the process a
// fixed device-memory budget and has already spent it, a frame loop that promised its caller "no allocation
// after load", or code that runs where entering the CUDA allocator is forbidden.  For them this file offers the
// same computation with the scratch in a fixed array that is part of the library image: every GPU that loads
// the library holds these 1.02 MiB until the process exits, and nothing is ever allocated or freed here.
//
// Bounded device-side waits inside the kernel report through the context's own status word (it exists since
// ctx_create, so using it allocates nothing): a wait that runs out inside this call reaches loom_b200_sync like
// one inside the regular call does.
#include "gemv_ternary.cuh"

#include <atomic>

namespace {

constexpr int kCntInts = 4096;        // one arrival counter per 16-row strip  -> at most 65,536 rows
constexpr int kAccInts = 262144;      // partial sums: 16 * strips * tokens-per-pass ints (1 MiB)
constexpr int kPadInts = 64;          // keeps the partial sums 256-byte aligned behind the counters
constexpr int kScratchInts = kCntInts + kPadInts + kAccInts;

// The scratch itself.  In host code this name is only a handle for cudaGetSymbolAddress: it is not a device
// address and must never be handed to a kernel as one.
static __device__ __align__(256) int32_t g_no_alloc_scratch[kScratchInts];

constexpr int kMaxDevices = 64;
// Device address of the array on each device, looked up once.  Contexts of different devices may be driven from
// different threads, so the table is atomic; two threads that race on the same device store the same value.
std::atomic<int32_t*> g_scratch_ptr[kMaxDevices];

// First call on a device: resolve the array's device address with that device current.
int scratch_for_device(loom_b200_ctx* ctx, int32_t** out) {
    const int dev = ctx->device;
    if (dev < 0 || dev >= kMaxDevices) return lb_fail(ctx, LOOM_B200_ERR_UNSUPPORTED, "ternary_linear_no_alloc: device index %d is above %d", dev, kMaxDevices - 1);
    int32_t* p = g_scratch_ptr[dev].load(std::memory_order_acquire);
    if (!p) {
        void* sym = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&sym, g_no_alloc_scratch);  // ctx->device is current (lb_set_device)
        if (e != cudaSuccess || !sym)
            return lb_fail(ctx, LOOM_B200_ERR_CUDA, "ternary_linear_no_alloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        p = static_cast<int32_t*>(sym);
        g_scratch_ptr[dev].store(p, std::memory_order_release);
    }
    *out = p;
    return 0;
}

}  // namespace

extern "C" int loom_b200_ternary_linear_no_alloc(loom_b200_ctx* ctx, const loom_b200_weight* w, int batch, const int8_t* q,
                                                 const float* amax, const float* bias, const float* residual,
                                                 int activation, float* out) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "ternary_linear_no_alloc: ctx is NULL");
    LB_REQUIRE(ctx, w != nullptr, "ternary_linear_no_alloc: weight is NULL");
    LB_REQUIRE(ctx, batch >= 0, "ternary_linear_no_alloc: batch=%d", batch);
    if (batch == 0) return 0;
    LB_REQUIRE(ctx, q && amax && out, "ternary_linear_no_alloc: NULL buffer");
    LB_REQUIRE(ctx, w->device == ctx->device, "ternary_linear_no_alloc: weight lives on device %d, context on %d", w->device, ctx->device);
    // tokens one pass carries: the same rule as the regular entry point (8, fewer for very wide inputs)
    const int pass = lb_gemv_max_tokens(w->cols);
    const int per_pass = batch < pass ? batch : pass;
    // the fixed scratch bounds the shapes this entry point takes
    if (w->strips > kCntInts || (long long)w->strips * 16 * per_pass > kAccInts)
        return lb_fail(ctx, LOOM_B200_ERR_UNSUPPORTED,
                       "ternary_linear_no_alloc: %d rows x %d tokens per pass exceed the built-in scratch "
                       "(rows <= %d and 16*ceil(rows/16)*tokens_per_pass <= %d); use loom_b200_ternary_linear",
                       w->rows, per_pass, kCntInts * 16, kAccInts);
    if (int rc = lb_set_device(ctx)) return rc;
    int32_t* base = nullptr;
    if (int rc = scratch_for_device(ctx, &base)) return rc;
    unsigned int* cnt = reinterpret_cast<unsigned int*>(base);
    int32_t* acc = base + kCntInts + kPadInts;
    // The array keeps whatever the previous call (of any context) left behind: start from zero.
    LB_CUDA(ctx, cudaMemsetAsync(cnt, 0, (size_t)w->strips * sizeof(unsigned int), ctx->stream));
    LB_CUDA(ctx, cudaMemsetAsync(acc, 0, (size_t)w->strips * 16 * per_pass * sizeof(int32_t), ctx->stream));
    // Point the launcher at the built-in scratch for the duration of this call; calls on one context are
    // serialised by contract, so nobody else sees the swap.  Sizes are set to the fixed capacity so that the
    // launcher has nothing to grow.  The status word stays the context's own.
    int32_t* save_acc = ctx->fix_acc;
    unsigned int* save_cnt = ctx->fix_cnt;
    size_t save_acc_n = ctx->fix_acc_elems, save_cnt_n = ctx->fix_cnt_elems;
    int save_part = ctx->opt_gemv_partition;
    ctx->fix_acc = acc;
    ctx->fix_cnt = cnt;
    ctx->fix_acc_elems = kAccInts;
    ctx->fix_cnt_elems = kCntInts;
    ctx->opt_gemv_partition = 1;  // stream-K over tiles: the variant whose partial sums go through the scratch
    int rc = 0;
    for (int b0 = 0; b0 < batch && !rc; b0 += pass) {
        LbGemvParams p = {};
        p.nseg = 1;
        p.seg[0].tiles = w->tiles;
        p.seg[0].rows = w->rows;
        p.seg[0].scale = w->scale;
        p.seg[0].bias = bias;
        p.seg[0].out = out + (size_t)b0 * w->rows;
        p.seg[0].kind = LB_OUT_F32;
        p.K = w->cols;
        p.M = batch - b0 < pass ? batch - b0 : pass;
        p.pro = LB_PRO_Q8;
        p.x = q + (size_t)b0 * w->cols;
        p.amax_in = amax + b0;
        p.epi = LB_EPI_GENERIC;
        p.act = activation;
        p.residual = residual ? residual + (size_t)b0 * w->rows : nullptr;
        rc = lb_gemv_finalize_params(ctx, p);
        if (!rc) rc = lb_launch_gemv(ctx, p);
    }
    ctx->fix_acc = save_acc;
    ctx->fix_cnt = save_cnt;
    ctx->fix_acc_elems = save_acc_n;
    ctx->fix_cnt_elems = save_cnt_n;
    ctx->opt_gemv_partition = save_part;
    if (rc == LOOM_B200_ERR_UNSUPPORTED)  // e.g. a shared-memory limit of the launcher: say where the caller can go instead
        ctx->last_error += " (loom_b200_ternary_linear_no_alloc; loom_b200_ternary_linear takes the same shapes)";
    return rc;
}
