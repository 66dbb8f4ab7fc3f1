// abi.cu -- context, device buffers and packed-weight management behind the C ABI.
#include "common.cuh"

#include <cstdlib>
#include <mutex>
#include <vector>

namespace {

std::mutex g_err_mu;
std::string g_global_error;  // errors raised without a context (ctx_create)

}  // namespace

int lb_fail(loom_b200_ctx* ctx, int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    if (ctx) {
        ctx->last_error = buf;
    } else {
        std::lock_guard<std::mutex> lk(g_err_mu);
        g_global_error = buf;
    }
    return code;
}

const char* lb_global_error() { return g_global_error.c_str(); }

struct loom_b200_graph {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
};

#define LB_NO_CAPTURE(ctx, what)                                                                               \
    do {                                                                                                       \
        if ((ctx)->capturing)                                                                                  \
            return lb_fail((ctx), LOOM_B200_ERR_INVALID, "%s is not allowed between graph_begin and graph_end", what); \
    } while (0)

int lb_ensure_fixup(loom_b200_ctx* ctx, size_t acc_elems, size_t cnt_elems) {
    if ((acc_elems > ctx->fix_acc_elems || cnt_elems > ctx->fix_cnt_elems) && ctx->capturing)
        return lb_fail(ctx, LOOM_B200_ERR_INVALID, "scratch would grow while recording a graph: run the same calls once before graph_begin");
    if (acc_elems > ctx->fix_acc_elems) {
        // growing happens between launches on this stream; wait for users of the old buffer first
        LB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        if (ctx->fix_acc) cudaFree(ctx->fix_acc);
        ctx->fix_acc = nullptr;
        size_t n = acc_elems + acc_elems / 2;
        LB_CUDA(ctx, cudaMalloc(&ctx->fix_acc, n * sizeof(int32_t)));
        LB_CUDA(ctx, cudaMemsetAsync(ctx->fix_acc, 0, n * sizeof(int32_t), ctx->stream));
        ctx->fix_acc_elems = n;
    }
    if (cnt_elems > ctx->fix_cnt_elems) {
        LB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        if (ctx->fix_cnt) cudaFree(ctx->fix_cnt);
        ctx->fix_cnt = nullptr;
        size_t n = cnt_elems + cnt_elems / 2;
        LB_CUDA(ctx, cudaMalloc(&ctx->fix_cnt, n * sizeof(unsigned int)));
        LB_CUDA(ctx, cudaMemsetAsync(ctx->fix_cnt, 0, n * sizeof(unsigned int), ctx->stream));
        ctx->fix_cnt_elems = n;
    }
    return 0;
}

int lb_ensure_scratch(loom_b200_ctx* ctx, size_t bytes) {
    if (bytes <= ctx->scratch_bytes) return 0;
    LB_NO_CAPTURE(ctx, "growing the scratch buffer");
    LB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (ctx->scratch) cudaFree(ctx->scratch);
    ctx->scratch = nullptr;
    ctx->scratch_bytes = 0;
    size_t n = bytes + bytes / 4 + 4096;
    LB_CUDA(ctx, cudaMalloc(&ctx->scratch, n));
    ctx->scratch_bytes = n;
    return 0;
}

int lb_sync_checked(loom_b200_ctx* ctx) {
    LB_CUDA(ctx, cudaMemcpyAsync(ctx->status_host, ctx->status_dev, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    LB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    const int code = *ctx->status_host;
    if (code == 0) return 0;
    *ctx->status_host = 0;
    LB_CUDA(ctx, cudaMemsetAsync(ctx->status_dev, 0, sizeof(int), ctx->stream));
    static const char* what[] = {"", "a shared-memory tile copy did not complete", "",
                                 "the tensor-core pipeline of the GEMM stalled", "", "a tensor-parallel peer did not answer",
                                 "self-test: a flag that nothing sets"};
    return lb_fail(ctx, LOOM_B200_ERR_TIMEOUT, "a bounded device-side wait ran out (%d: %s); results of the calls since the last sync are invalid",
                   code, code >= 1 && code <= 6 ? what[code] : "unknown");
}

int lb_ensure_quant_scratch(loom_b200_ctx* ctx, size_t bytes) {
    if (bytes <= ctx->quant_scratch_bytes) return 0;
    LB_NO_CAPTURE(ctx, "growing the quantization scratch buffer");
    LB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (ctx->quant_scratch) cudaFree(ctx->quant_scratch);
    ctx->quant_scratch = nullptr;
    ctx->quant_scratch_bytes = 0;
    // sized for a full pass of kMaxM tokens at this width, so that later calls with more tokens find it large enough
    size_t n = bytes * 2 + 4096;
    LB_CUDA(ctx, cudaMalloc(&ctx->quant_scratch, n));
    ctx->quant_scratch_bytes = n;
    return 0;
}

// ---- re-tiling kernels -------------------------------------------------------------------------

// One thread per output u32 of the tiled layout.
__global__ void lb_retile_kernel(const uint32_t* __restrict__ words, int rows, int cols, int row_words, int strips,
                                 int kblocks, uint32_t* __restrict__ tiles) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t total = (size_t)strips * kblocks * kTileWords;
    if (idx >= total) return;
    int slot = (int)(idx & 3);
    int lane = (int)((idx >> 2) & 31);
    size_t tile = idx >> 7;
    int kb = (int)(tile % kblocks);
    int strip = (int)(tile / kblocks);
    int g = lane >> 2, t = lane & 3;
    int row = strip * kTileRows + g + 8 * (slot & 1);
    int wi = kb * 8 + t + 4 * (slot >> 1);
    uint32_t v = 0x55555555u;  // sixteen codes of 1 = weight 0
    if (row < rows && wi < row_words) {
        v = words[(size_t)row * row_words + wi];
        int first_pad = cols - wi * 16;  // columns of this word that are real
        if (first_pad < 16) {
            uint32_t keep = first_pad <= 0 ? 0u : ((1u << (2 * first_pad)) - 1u);
            v = (v & keep) | (0x55555555u & ~keep);
        }
    }
    tiles[idx] = v;
}

// Inverse: one thread per u32 of the reference layout; padding bits come back as zero.
__global__ void lb_untile_kernel(const uint32_t* __restrict__ tiles, int rows, int cols, int row_words, int kblocks,
                                 uint32_t* __restrict__ words) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)rows * row_words) return;
    int row = (int)(idx / row_words), wi = (int)(idx % row_words);
    int strip = row / kTileRows, r = row % kTileRows;
    int kb = wi / 8, w8 = wi % 8;
    int g = r & 7, t = w8 & 3;
    int slot = (r >> 3) | ((w8 >> 2) << 1);
    uint32_t v = tiles[((size_t)strip * kblocks + kb) * kTileWords + (size_t)(g * 4 + t) * 4 + slot];
    int real = cols - wi * 16;
    if (real < 16) v &= real <= 0 ? 0u : ((1u << (2 * real)) - 1u);
    words[idx] = v;
}

// ---- device-side ternarizer (absmean) --------------------------------------------------------------

constexpr int kAbsBlocks = 1024;

__global__ void lb_abs_sum_kernel(const float* __restrict__ w, size_t n, double* __restrict__ partial,
                                  int* __restrict__ all_ternary) {
    __shared__ double red[32];
    __shared__ int tern[32];
    size_t per = (n + gridDim.x - 1) / gridDim.x;
    size_t s = (size_t)blockIdx.x * per, e = s + per < n ? s + per : n;
    double acc = 0.0;
    int ok = 1;
    for (size_t i = s + threadIdx.x; i < e; i += blockDim.x) {
        float v = w[i];
        acc += fabs((double)v);
        bool t = fabs((double)v) < 1e-6 || fabs((double)__fsub_rn(v, 1.0f)) < 1e-6 ||
                 fabs((double)__fadd_rn(v, 1.0f)) < 1e-6;
        if (!t) ok = 0;
    }
    acc = lb_warp_sum(acc);
    ok = __all_sync(0xffffffffu, ok);
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) {
        red[warp] = acc;
        tern[warp] = ok;
    }
    __syncthreads();
    if (warp == 0) {
        int nw = blockDim.x >> 5;
        double v = lane < nw ? red[lane] : 0.0;
        int o = lane < nw ? tern[lane] : 1;
        v = lb_warp_sum(v);
        o = __all_sync(0xffffffffu, o);
        if (lane == 0) {
            partial[blockIdx.x] = v;
            if (!o) atomicAnd(all_ternary, 0);
        }
    }
}

// out[0] = scale (float), out[1] = all-ternary flag
__global__ void lb_abs_finish_kernel(const double* __restrict__ partial, int nparts, size_t n,
                                     const int* __restrict__ all_ternary, float* __restrict__ out) {
    __shared__ double red[32];
    double acc = 0.0;
    for (int i = threadIdx.x; i < nparts; i += blockDim.x) acc += partial[i];
    acc = lb_warp_sum(acc);
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) red[warp] = acc;
    __syncthreads();
    if (warp == 0) {
        int nw = blockDim.x >> 5;
        double v = lane < nw ? red[lane] : 0.0;
        v = lb_warp_sum(v);
        if (lane == 0) {
            float s = (float)__ddiv_rn(v, (double)n);
            if (s == 0.0f) s = 1.0f;
            int tern = *all_ternary;
            out[0] = tern ? 1.0f : s;
            out[1] = tern ? 1.0f : 0.0f;
        }
    }
}

__device__ __forceinline__ uint32_t lb_tern_code(float v, float scale) {
    float ratio = __fdiv_rn(v, scale);  // float32 division, then round half away in double
    double r = round((double)ratio);
    int q = r > 1.0 ? 1 : (r < -1.0 ? -1 : (int)r);
    return (uint32_t)(q + 1);
}

__global__ void lb_pack_tiles_kernel(const float* __restrict__ w, int rows, int cols, int strips, int kblocks,
                                     const float* __restrict__ scale_ptr, uint32_t* __restrict__ tiles) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t total = (size_t)strips * kblocks * kTileWords;
    if (idx >= total) return;
    float scale = scale_ptr[0];
    int slot = (int)(idx & 3);
    int lane = (int)((idx >> 2) & 31);
    size_t tile = idx >> 7;
    int kb = (int)(tile % kblocks);
    int strip = (int)(tile / kblocks);
    int g = lane >> 2, t = lane & 3;
    int row = strip * kTileRows + g + 8 * (slot & 1);
    int col0 = (kb * 8 + t + 4 * (slot >> 1)) * 16;
    uint32_t v = 0;
    for (int i = 0; i < 16; ++i) {
        int c = col0 + i;
        uint32_t code = 1u;
        if (row < rows && c < cols) code = lb_tern_code(w[(size_t)row * cols + c], scale);
        v |= code << (2 * i);
    }
    tiles[idx] = v;
}

namespace {

int alloc_weight(loom_b200_ctx* ctx, int rows, int cols, loom_b200_weight** out) {
    auto* w = new loom_b200_weight();
    w->rows = rows;
    w->cols = cols;
    w->row_words = (cols + 15) / 16;
    w->strips = (rows + kTileRows - 1) / kTileRows;
    w->kblocks = (cols + kTileCols - 1) / kTileCols;
    w->device = ctx->device;
    cudaError_t e = cudaMalloc(&w->tiles, w->tile_bytes());
    if (e != cudaSuccess) {
        size_t want = w->tile_bytes();
        delete w;
        return lb_fail(ctx, LOOM_B200_ERR_CUDA, "cudaMalloc(%zu) for packed weights: %s", want, cudaGetErrorString(e));
    }
    *out = w;
    return 0;
}

}  // namespace

extern "C" {

int loom_b200_api_version(void) { return LOOM_B200_API_VERSION; }

int loom_b200_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    int ok = 0;
    for (int i = 0; i < n; ++i) {
        int major = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, i) == cudaSuccess && major == 10) ++ok;
    }
    return ok;
}

const char* loom_b200_last_error(const loom_b200_ctx* ctx) { return ctx ? ctx->last_error.c_str() : lb_global_error(); }

int loom_b200_ctx_create(int device, void* stream, loom_b200_ctx** out) {
    if (!out) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "ctx_create: out is NULL");
    *out = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) {
        cudaGetLastError();
        return lb_fail(nullptr, LOOM_B200_ERR_NO_DEVICE,
                       "no CUDA device: this library has no CPU fallback (cudaGetDeviceCount: %s)",
                       cudaGetErrorString(e));
    }
    if (device < 0 || device >= n) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "device %d out of range [0,%d)", device, n);
    int major = 0;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
    if (major != 10)
        return lb_fail(nullptr, LOOM_B200_ERR_NO_DEVICE, "device %d has compute capability %d.x; the kernels are built for sm_100a only", device, major);
    auto* ctx = new loom_b200_ctx();
    ctx->device = device;
    if ((e = cudaSetDevice(device)) != cudaSuccess) {
        delete ctx;
        return lb_fail(nullptr, LOOM_B200_ERR_CUDA, "cudaSetDevice(%d): %s", device, cudaGetErrorString(e));
    }
    cudaDeviceGetAttribute(&ctx->sm_count, cudaDevAttrMultiProcessorCount, device);
    if (stream) {
        ctx->stream = (cudaStream_t)stream;
    } else {
        if ((e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking)) != cudaSuccess) {
            delete ctx;
            return lb_fail(nullptr, LOOM_B200_ERR_CUDA, "cudaStreamCreate: %s", cudaGetErrorString(e));
        }
        ctx->owns_stream = true;
    }
    if ((e = cudaMalloc(&ctx->status_dev, sizeof(int))) != cudaSuccess ||
        (e = cudaMemset(ctx->status_dev, 0, sizeof(int))) != cudaSuccess) {
        delete ctx;
        return lb_fail(nullptr, LOOM_B200_ERR_CUDA, "status word: %s", cudaGetErrorString(e));
    }
    if ((e = cudaMallocHost(&ctx->status_host, sizeof(int))) != cudaSuccess) {
        cudaFree(ctx->status_dev);
        delete ctx;
        return lb_fail(nullptr, LOOM_B200_ERR_CUDA, "status word: %s", cudaGetErrorString(e));
    }
    *ctx->status_host = 0;
    if (const char* v = getenv("LOOM_B200_GEMV_VARIANT")) ctx->opt_gemv_variant = atoi(v) == 1 ? 1 : 0;
    if (const char* v = getenv("LOOM_B200_GEMV_CTAS_PER_SM")) ctx->opt_gemv_ctas_per_sm = atoi(v) > 0 ? atoi(v) : 2;
    if (const char* v = getenv("LOOM_B200_PDL")) ctx->opt_pdl = atoi(v) != 0;
    *out = ctx;
    return 0;
}

int loom_b200_ctx_set_option(loom_b200_ctx* ctx, const char* key, int value) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "ctx_set_option: ctx is NULL");
    LB_REQUIRE(ctx, key != nullptr, "ctx_set_option: key is NULL");
    if (!strcmp(key, "gemv_variant")) {
        LB_REQUIRE(ctx, value == 0 || value == 1, "ctx_set_option: gemv_variant must be 0 (mma) or 1 (dp4a)");
        ctx->opt_gemv_variant = value;
    } else if (!strcmp(key, "gemv_ctas_per_sm")) {
        LB_REQUIRE(ctx, value >= 1 && value <= 8, "ctx_set_option: gemv_ctas_per_sm must be in [1,8]");
        ctx->opt_gemv_ctas_per_sm = value;
    } else if (!strcmp(key, "gemv_partition")) {
        LB_REQUIRE(ctx, value >= 0 && value <= 2, "ctx_set_option: gemv_partition must be 0 (auto), 1 (stream-K) or 2 (whole strips)");
        ctx->opt_gemv_partition = value;
    } else if (!strcmp(key, "trace")) {
        LB_NO_CAPTURE(ctx, "switching the trace");
        if (int rc = lb_set_device(ctx)) return rc;
        LB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        ctx->trace_seq = 0;
        if (value && !ctx->trace_dev) {
            LB_CUDA(ctx, cudaMalloc(&ctx->trace_dev, (size_t)kTraceSlots * 8 * sizeof(unsigned long long)));
            LB_CUDA(ctx, cudaMemset(ctx->trace_dev, 0, (size_t)kTraceSlots * 8 * sizeof(unsigned long long)));
        } else if (!value && ctx->trace_dev) {
            cudaFree(ctx->trace_dev);
            ctx->trace_dev = nullptr;
        }
    } else if (!strcmp(key, "head_stream")) {
        ctx->opt_head_stream = value != 0;
    } else if (!strcmp(key, "attn_cluster")) {
        ctx->opt_attn_cluster = value < 0 ? 0 : value;
    } else if (!strcmp(key, "pdl")) {
        ctx->opt_pdl = value != 0;
    } else if (!strcmp(key, "fold_rope")) {
        ctx->opt_fold_rope = value != 0;
    } else if (!strcmp(key, "decode_splits")) {
        if (value < 0 || value > 32) return lb_fail(ctx, LOOM_B200_ERR_INVALID, "ctx_set_option: decode_splits is 0..32");
        ctx->opt_decode_splits = value;
    } else if (!strcmp(key, "gemm_splitk")) {
        ctx->opt_gemm_splitk = value != 0;
    } else if (!strcmp(key, "gemm_tile")) {
        if (value != 0 && value != 128 && value != 256) return lb_fail(ctx, LOOM_B200_ERR_INVALID, "ctx_set_option: gemm_tile is 0, 128 or 256");
        ctx->opt_gemm_tile = value;
    } else if (!strcmp(key, "attn_stream")) {
        ctx->opt_attn_stream = value != 0;
    } else if (!strcmp(key, "gemv_lean")) {
        ctx->opt_gemv_lean = value != 0;
    } else if (!strcmp(key, "tp_fused")) {
        ctx->opt_tp_fused = value != 0;
    } else if (!strcmp(key, "quant_regs")) {
        ctx->opt_quant_regs = value != 0;
    } else if (!strcmp(key, "gemm_stream")) {
        ctx->opt_gemm_stream = value != 0;
    } else if (!strcmp(key, "gemm_cache")) {
        ctx->opt_gemm_cache = value != 0;
    } else if (!strcmp(key, "prefill_gemm")) {
        ctx->opt_prefill_gemm = value != 0;
    } else if (!strcmp(key, "tp_peer")) {
        ctx->opt_tp_peer = value != 0;
    } else if (!strcmp(key, "tp_graph")) {
        ctx->opt_tp_graph = value != 0;
    } else {
        return lb_fail(ctx, LOOM_B200_ERR_INVALID, "ctx_set_option: unknown key '%s'", key);
    }
    return 0;
}

void loom_b200_ctx_destroy(loom_b200_ctx* ctx) {
    if (!ctx) return;
    loom_b200_tp_finalize(ctx);
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->fix_acc) cudaFree(ctx->fix_acc);
    if (ctx->fix_cnt) cudaFree(ctx->fix_cnt);
    if (ctx->scratch) cudaFree(ctx->scratch);
    if (ctx->status_dev) cudaFree(ctx->status_dev);
    if (ctx->status_host) cudaFreeHost(ctx->status_host);
    if (ctx->trace_dev) cudaFree(ctx->trace_dev);
    if (ctx->argmax_scratch) cudaFree(ctx->argmax_scratch);
    if (ctx->head_scratch) cudaFree(ctx->head_scratch);
    if (ctx->gemm_scratch) cudaFree(ctx->gemm_scratch);
    if (ctx->quant_scratch) cudaFree(ctx->quant_scratch);
    if (ctx->owns_stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
}

int loom_b200_sync(loom_b200_ctx* ctx) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "sync: ctx is NULL");
    LB_NO_CAPTURE(ctx, "sync");
    if (int rc = lb_set_device(ctx)) return rc;
    return lb_sync_checked(ctx);
}

__global__ void lb_selftest_wait_kernel(const volatile int* flag, unsigned int polls, int* status) {
    for (unsigned int i = 0; i < polls; ++i)
        if (*flag != 0) return;
    atomicExch(status, 6);  // nothing set the flag: report instead of waiting on
}

int loom_b200_selftest_wait_timeout(loom_b200_ctx* ctx, unsigned int polls) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "selftest_wait_timeout: ctx is NULL");
    LB_REQUIRE(ctx, polls >= 1 && polls <= 10000000u, "selftest_wait_timeout: %u polls (1..10,000,000)", polls);
    LB_NO_CAPTURE(ctx, "selftest_wait_timeout");
    if (int rc = lb_set_device(ctx)) return rc;
    if (int rc = lb_ensure_scratch(ctx, 256)) return rc;
    LB_CUDA(ctx, cudaMemsetAsync(ctx->scratch, 0, sizeof(int), ctx->stream));
    lb_selftest_wait_kernel<<<1, 1, 0, ctx->stream>>>((const volatile int*)ctx->scratch, polls, ctx->status_dev);
    LB_CHECK_LAUNCH(ctx, "lb_selftest_wait_kernel");
    return lb_sync_checked(ctx);
}

int loom_b200_graph_begin(loom_b200_ctx* ctx) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "graph_begin: ctx is NULL");
    LB_NO_CAPTURE(ctx, "graph_begin");
    if (int rc = lb_set_device(ctx)) return rc;
    LB_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
    ctx->capturing = true;
    return 0;
}

int loom_b200_graph_end(loom_b200_ctx* ctx, loom_b200_graph** out) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "graph_end: ctx is NULL");
    LB_REQUIRE(ctx, out != nullptr, "graph_end: out is NULL");
    LB_REQUIRE(ctx, ctx->capturing, "graph_end without graph_begin");
    *out = nullptr;
    ctx->capturing = false;
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamEndCapture(ctx->stream, &g);
    if (e != cudaSuccess || !g) {
        cudaGetLastError();
        return lb_fail(ctx, LOOM_B200_ERR_CUDA, "cudaStreamEndCapture: %s", cudaGetErrorString(e));
    }
    auto* gr = new loom_b200_graph();
    gr->graph = g;
    e = cudaGraphInstantiate(&gr->exec, g, 0);
    if (e != cudaSuccess) {
        cudaGraphDestroy(g);
        delete gr;
        return lb_fail(ctx, LOOM_B200_ERR_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(e));
    }
    *out = gr;
    return 0;
}

int loom_b200_graph_launch(loom_b200_ctx* ctx, loom_b200_graph* graph) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "graph_launch: ctx is NULL");
    LB_REQUIRE(ctx, graph && graph->exec, "graph_launch: graph is NULL");
    LB_NO_CAPTURE(ctx, "graph_launch");
    if (int rc = lb_set_device(ctx)) return rc;
    LB_CUDA(ctx, cudaGraphLaunch(graph->exec, ctx->stream));
    return 0;
}

void loom_b200_graph_free(loom_b200_ctx* ctx, loom_b200_graph* graph) {
    if (!graph) return;
    if (ctx) {
        cudaSetDevice(ctx->device);
        cudaStreamSynchronize(ctx->stream);
    }
    if (graph->exec) cudaGraphExecDestroy(graph->exec);
    if (graph->graph) cudaGraphDestroy(graph->graph);
    delete graph;
}

const char* loom_b200_trace_label(const loom_b200_ctx* ctx, int slot) {
    if (!ctx || slot < 0 || slot >= kTraceSlots || !ctx->trace_label[slot]) return "";
    return ctx->trace_label[slot];
}

int loom_b200_trace_read(loom_b200_ctx* ctx, uint64_t* host, int ctas) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "trace_read: ctx is NULL");
    LB_REQUIRE(ctx, host && ctas > 0 && ctas <= kTraceSlots, "trace_read: bad arguments");
    LB_REQUIRE(ctx, ctx->trace_dev != nullptr, "trace_read: tracing is off (set option \"trace\" to 1)");
    LB_NO_CAPTURE(ctx, "trace_read");
    if (int rc = lb_set_device(ctx)) return rc;
    LB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    LB_CUDA(ctx, cudaMemcpy(host, ctx->trace_dev, (size_t)ctas * 8 * sizeof(uint64_t), cudaMemcpyDeviceToHost));
    return 0;
}

void* loom_b200_ctx_stream(loom_b200_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }
uint64_t loom_b200_launch_count(const loom_b200_ctx* ctx) { return ctx ? ctx->launches : 0; }

int loom_b200_buffer_alloc(loom_b200_ctx* ctx, size_t bytes, void** dptr) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "buffer_alloc: ctx is NULL");
    LB_REQUIRE(ctx, dptr != nullptr, "buffer_alloc: dptr is NULL");
    LB_NO_CAPTURE(ctx, "buffer_alloc");
    if (int rc = lb_set_device(ctx)) return rc;
    *dptr = nullptr;
    LB_CUDA(ctx, cudaMalloc(dptr, bytes ? bytes : 1));
    return 0;
}

int loom_b200_buffer_free(loom_b200_ctx* ctx, void* dptr) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "buffer_free: ctx is NULL");
    if (!dptr) return 0;
    LB_NO_CAPTURE(ctx, "buffer_free");
    if (int rc = lb_set_device(ctx)) return rc;
    LB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    LB_CUDA(ctx, cudaFree(dptr));
    return 0;
}

int loom_b200_buffer_upload(loom_b200_ctx* ctx, void* dst, const void* src, size_t bytes) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "buffer_upload: ctx is NULL");
    LB_REQUIRE(ctx, (dst && src) || bytes == 0, "buffer_upload: NULL pointer");
    if (bytes == 0) return 0;
    LB_NO_CAPTURE(ctx, "buffer_upload");
    if (int rc = lb_set_device(ctx)) return rc;
    // The caller's memory may be pageable and may be reused after return: finish the copy here.
    LB_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    LB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return 0;
}

int loom_b200_buffer_download(loom_b200_ctx* ctx, void* dst, const void* src, size_t bytes) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "buffer_download: ctx is NULL");
    LB_REQUIRE(ctx, (dst && src) || bytes == 0, "buffer_download: NULL pointer");
    if (bytes == 0) return 0;
    LB_NO_CAPTURE(ctx, "buffer_download");
    if (int rc = lb_set_device(ctx)) return rc;
    LB_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    LB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return 0;
}

int loom_b200_buffer_zero(loom_b200_ctx* ctx, void* dst, size_t bytes) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "buffer_zero: ctx is NULL");
    LB_REQUIRE(ctx, dst || bytes == 0, "buffer_zero: NULL pointer");
    if (bytes == 0) return 0;
    if (int rc = lb_set_device(ctx)) return rc;
    LB_CUDA(ctx, cudaMemsetAsync(dst, 0, bytes, ctx->stream));
    return 0;
}

int loom_b200_upload_ternary(loom_b200_ctx* ctx, const uint32_t* words, int rows, int cols, int row_words, float scale,
                             loom_b200_weight** out) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "upload_ternary: ctx is NULL");
    LB_REQUIRE(ctx, out != nullptr, "upload_ternary: out is NULL");
    *out = nullptr;
    LB_REQUIRE(ctx, words != nullptr, "upload_ternary: words is NULL");
    LB_REQUIRE(ctx, rows > 0 && cols > 0, "upload_ternary: bad shape %dx%d", rows, cols);
    LB_REQUIRE(ctx, row_words == (cols + 15) / 16, "upload_ternary: row_words %d != ceil(%d/16)", row_words, cols);
    if (int rc = lb_set_device(ctx)) return rc;
    loom_b200_weight* w = nullptr;
    if (int rc = alloc_weight(ctx, rows, cols, &w)) return rc;
    w->scale = scale == 0.0f ? 1.0f : scale;
    size_t nwords = (size_t)rows * row_words;
    uint32_t* tmp = nullptr;
    cudaError_t e = cudaMalloc(&tmp, nwords * sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMemcpyAsync(tmp, words, nwords * sizeof(uint32_t), cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) {
        size_t total = (size_t)w->strips * w->kblocks * kTileWords;
        lb_retile_kernel<<<(unsigned)((total + 255) / 256), 256, 0, ctx->stream>>>(tmp, rows, cols, row_words, w->strips,
                                                                                   w->kblocks, w->tiles);
        e = cudaGetLastError();
        ctx->launches++;
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (tmp) cudaFree(tmp);
    if (e != cudaSuccess) {
        loom_b200_weight_free(ctx, w);
        return lb_fail(ctx, LOOM_B200_ERR_CUDA, "upload_ternary: %s", cudaGetErrorString(e));
    }
    *out = w;
    return 0;
}

int loom_b200_pack_ternary_f32(loom_b200_ctx* ctx, const float* master_dev, int rows, int cols, loom_b200_weight** out) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "pack_ternary_f32: ctx is NULL");
    LB_REQUIRE(ctx, out != nullptr, "pack_ternary_f32: out is NULL");
    *out = nullptr;
    LB_REQUIRE(ctx, master_dev != nullptr, "pack_ternary_f32: master is NULL");
    LB_REQUIRE(ctx, rows > 0 && cols > 0, "pack_ternary_f32: bad shape %dx%d", rows, cols);
    if (int rc = lb_set_device(ctx)) return rc;
    loom_b200_weight* w = nullptr;
    if (int rc = alloc_weight(ctx, rows, cols, &w)) return rc;
    size_t n = (size_t)rows * cols;
    size_t need = kAbsBlocks * sizeof(double) + 64;
    if (int rc = lb_ensure_scratch(ctx, need)) {
        loom_b200_weight_free(ctx, w);
        return rc;
    }
    double* partial = (double*)ctx->scratch;
    int* flag = (int*)((char*)ctx->scratch + kAbsBlocks * sizeof(double));
    float* res = (float*)(flag + 4);
    int one = 1;
    cudaError_t e = cudaMemcpyAsync(flag, &one, sizeof(int), cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) {
        lb_abs_sum_kernel<<<kAbsBlocks, 256, 0, ctx->stream>>>(master_dev, n, partial, flag);
        lb_abs_finish_kernel<<<1, 256, 0, ctx->stream>>>(partial, kAbsBlocks, n, flag, res);
        size_t total = (size_t)w->strips * w->kblocks * kTileWords;
        lb_pack_tiles_kernel<<<(unsigned)((total + 255) / 256), 256, 0, ctx->stream>>>(master_dev, rows, cols, w->strips,
                                                                                       w->kblocks, res, w->tiles);
        e = cudaGetLastError();
        ctx->launches += 3;
    }
    float host_res[2] = {1.0f, 0.0f};
    if (e == cudaSuccess) e = cudaMemcpyAsync(host_res, res, sizeof(host_res), cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        loom_b200_weight_free(ctx, w);
        return lb_fail(ctx, LOOM_B200_ERR_CUDA, "pack_ternary_f32: %s", cudaGetErrorString(e));
    }
    w->scale = host_res[0];
    *out = w;
    return 0;
}

int loom_b200_upload_entity_blob(loom_b200_ctx* ctx, const uint8_t* blob, size_t len, int* offset_out, loom_b200_weight** out) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "upload_entity_blob: ctx is NULL");
    LB_REQUIRE(ctx, out != nullptr, "upload_entity_blob: out is NULL");
    *out = nullptr;
    LB_REQUIRE(ctx, blob != nullptr, "upload_entity_blob: blob is NULL");
    LB_REQUIRE(ctx, len >= 24, "upload_entity_blob: blob of %zu bytes is shorter than its 24-byte header", len);
    auto le32 = [&](size_t at) { return (uint32_t)blob[at] | ((uint32_t)blob[at + 1] << 8) | ((uint32_t)blob[at + 2] << 16) | ((uint32_t)blob[at + 3] << 24); };
    const uint32_t rows = le32(0), cols = le32(4), offset = le32(8), scale_bits = le32(12), n_words = le32(20);
    uint32_t row_words = le32(16);
    if (row_words == 0) row_words = (cols + 15) / 16;  // decodeEntityBitNetTernaryBlob's default
    LB_REQUIRE(ctx, rows > 0 && cols > 0 && rows < (1u << 24) && cols < (1u << 24), "upload_entity_blob: header says %u x %u", rows, cols);
    LB_REQUIRE(ctx, len >= 24 + (size_t)n_words * 4, "upload_entity_blob: truncated: have %zu bytes, need %zu", len, 24 + (size_t)n_words * 4);
    LB_REQUIRE(ctx, row_words >= (cols + 15) / 16 && (size_t)n_words >= (size_t)rows * row_words,
               "upload_entity_blob: %u words do not cover %u rows of %u words", n_words, rows, row_words);
    float scale;
    memcpy(&scale, &scale_bits, 4);
    std::vector<uint32_t> words((size_t)rows * row_words);
    for (size_t i = 0; i < words.size(); ++i) words[i] = le32(24 + 4 * i);  // little-endian on any host
    if (offset_out) *offset_out = (int)offset;
    return loom_b200_upload_ternary(ctx, words.data(), (int)rows, (int)cols, (int)row_words, scale, out);
}

int loom_b200_upload_microsoft_u8(loom_b200_ctx* ctx, const uint8_t* packed, int rows, int cols, float scale,
                                  loom_b200_weight** out) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "upload_microsoft_u8: ctx is NULL");
    LB_REQUIRE(ctx, out != nullptr, "upload_microsoft_u8: out is NULL");
    *out = nullptr;
    LB_REQUIRE(ctx, packed != nullptr, "upload_microsoft_u8: packed is NULL");
    LB_REQUIRE(ctx, rows > 0 && cols > 0 && rows % 4 == 0, "upload_microsoft_u8: rows %d must be a positive multiple of 4 (cols %d)", rows, cols);
    // Decode on the host into the reference's word layout (load-time work, like the reference's loader),
    // then take the common upload path.
    int rw = (cols + 15) / 16, pr_n = rows / 4;
    std::vector<uint32_t> words((size_t)rows * rw, 0u);
    for (int pr = 0; pr < pr_n; ++pr)
        for (int c = 0; c < cols; ++c) {
            uint8_t b = packed[(size_t)pr * cols + c];
            for (int lane = 0; lane < 4; ++lane) {
                uint32_t code = (b >> (2 * lane)) & 3u;
                if (code > 2) code = 1;
                words[(size_t)(lane * pr_n + pr) * rw + c / 16] |= code << (2 * (c % 16));
            }
        }
    return loom_b200_upload_ternary(ctx, words.data(), rows, cols, rw, scale, out);
}

int loom_b200_weight_info(const loom_b200_weight* w, int* rows, int* cols, int* row_words, float* scale) {
    if (!w) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "weight_info: weight is NULL");
    if (rows) *rows = w->rows;
    if (cols) *cols = w->cols;
    if (row_words) *row_words = w->row_words;
    if (scale) *scale = w->scale;
    return 0;
}

int loom_b200_weight_set_scale(loom_b200_weight* w, float scale) {
    if (!w) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "weight_set_scale: weight is NULL");
    w->scale = scale == 0.0f ? 1.0f : scale;
    return 0;
}

int loom_b200_weight_download_words(loom_b200_ctx* ctx, const loom_b200_weight* w, uint32_t* words_host) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "weight_download_words: ctx is NULL");
    LB_REQUIRE(ctx, w && words_host, "weight_download_words: NULL pointer");
    if (int rc = lb_set_device(ctx)) return rc;
    size_t nwords = (size_t)w->rows * w->row_words;
    uint32_t* tmp = nullptr;
    LB_CUDA(ctx, cudaMalloc(&tmp, nwords * sizeof(uint32_t)));
    lb_untile_kernel<<<(unsigned)((nwords + 255) / 256), 256, 0, ctx->stream>>>(w->tiles, w->rows, w->cols, w->row_words,
                                                                                w->kblocks, tmp);
    cudaError_t e = cudaGetLastError();
    ctx->launches++;
    if (e == cudaSuccess) e = cudaMemcpyAsync(words_host, tmp, nwords * sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    cudaFree(tmp);
    if (e != cudaSuccess) return lb_fail(ctx, LOOM_B200_ERR_CUDA, "weight_download_words: %s", cudaGetErrorString(e));
    return 0;
}

void loom_b200_weight_free(loom_b200_ctx* ctx, loom_b200_weight* w) {
    if (!w) return;
    if (ctx) {
        cudaSetDevice(ctx->device);
        cudaStreamSynchronize(ctx->stream);
    }
    if (w->tiles) cudaFree(w->tiles);
    if (w->codes8) cudaFree(w->codes8);
    delete w;
}

}  // extern "C"
