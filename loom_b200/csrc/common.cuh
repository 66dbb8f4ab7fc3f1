// common.cuh -- shared declarations of the loom_b200 CUDA library (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <string>

#include "../../include/loom_b200.h"

// ---- device layout of a packed ternary matrix -------------------------------------------------
//
// The reference keeps a matrix row-major, 16 two-bit codes per u32 (code = weight + 1).  On upload
// it is re-tiled into 512-byte tiles of 16 rows x 128 columns.  Inside a tile, lane L = g*4 + t
// (g = 0..7, t = 0..3) owns 16 contiguous bytes holding four of the reference's words:
//     [ word(row g, t), word(row g+8, t), word(row g, 4+t), word(row g+8, 4+t) ]
// where word(r, i) is the i-th u32 (columns 16i..16i+15) of row r inside the tile's 128-column block.
// A warp therefore reads a tile with one fully coalesced 16-byte access per lane, and the four words a
// lane holds are exactly the rows/columns that lane feeds to an m16n8k32 integer MMA (or four dp4a
// pairs).  Tiles are stored strip-major: tile index = strip * kblocks + kblock, strip = row / 16.
// Rows are padded to a multiple of 16 and columns to a multiple of 128 with code 1 (weight 0), so the
// hot loop never masks a tail.
constexpr int kTileRows = 16;
constexpr int kTileCols = 128;
constexpr int kTileBytes = 512;
constexpr int kTileWords = 128;
constexpr int kTraceSlots = 1024;  // launches remembered by the phase trace

struct loom_b200_weight {
    int rows = 0, cols = 0, row_words = 0;
    int strips = 0, kblocks = 0;  // padded rows / 16, padded cols / 128
    float scale = 1.0f;
    uint32_t* tiles = nullptr;  // strips * kblocks * 128 u32
    // Prefill cache, built the first time the matrix meets the token-block GEMM (context option "gemm_cache"): the codes
    // as one byte per weight, already in the shared-memory image the tensor core reads, [row block of 128][k-slice of
    // 128 columns][16 KB].  The device twin of ensureBitNetCodes (poly/bitnet_cpu.go:700-729): 4x the packed bytes.
    uint8_t* codes8 = nullptr;
    int device = 0;
    size_t tile_bytes() const { return (size_t)strips * kblocks * kTileBytes; }
};

struct loom_b200_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    bool owns_stream = false;
    int sm_count = 148;
    std::string last_error;
    uint64_t launches = 0;
    // scratch of the stream-K fix-up: int32 partial sums and arrival counters.  Both are zero
    // whenever no kernel is in flight (the last arriver of every group clears what it used).
    int32_t* fix_acc = nullptr;
    unsigned int* fix_cnt = nullptr;
    size_t fix_acc_elems = 0, fix_cnt_elems = 0;
    // small device scratch reused by the layer-level calls
    void* scratch = nullptr;
    size_t scratch_bytes = 0;
    // device status word written by kernels with bounded waits (0 = ok)
    int* status_dev = nullptr;
    int* status_host = nullptr;    // pinned mirror, refreshed by lb_sync_checked
    void* quant_scratch = nullptr;   // int8 row and absmax of the stand-alone GEMV prologue (wide inputs)
    size_t quant_scratch_bytes = 0;
    void* gemm_scratch = nullptr;    // int8 activations, amax and sums of the tensor-core GEMM path
    size_t gemm_scratch_bytes = 0;
    void* argmax_scratch = nullptr;  // per-CTA partial maxima of the greedy argmax
    void* head_scratch = nullptr;    // per-CTA partial maxima and arrival counter of the LM head's greedy tail
    unsigned func_attr_mask = 0;  // kernels whose shared-memory limit was raised on this device
    unsigned func_attr_mask2 = 0; // the same for the cluster attention instantiations
    int opt_head_stream = 1;      // the LM head streams its rows through shared memory with bulk copies (0 = warp-per-row loads)
    int opt_attn_cluster = 1;     // one-token decoder steps run the attention as a thread-block cluster per KV head (0: off, 1: the largest cluster that fits, 2..16: at most that many CTAs)
    // tuning knobs (loom_b200_ctx_set_option; initial values from LOOM_B200_* environment variables)
    int opt_gemv_variant = 0;      // 0 = integer-MMA inner loop, 1 = dp4a inner loop (batch 1 only)
    int opt_gemv_ctas_per_sm = 2;  // grid = SMs * this
    int opt_pdl = 1;               // programmatic dependent launch on/off
    int opt_gemv_partition = 0;    // 0 = choose, 1 = always stream-K, 2 = always whole strip groups
    unsigned long long* trace_dev = nullptr;  // [kTraceSlots][8] phase timestamps, one row per launch
    int trace_seq = 0;                          // next row
    const char* trace_label[kTraceSlots] = {};  // kernel that wrote each row
    bool capturing = false;        // between graph_begin and graph_end
    // tensor parallelism (tp.cu): rank and world size of this context's group; the NCCL communicator or null
    int tp_rank = 0, tp_world = 1;
    int opt_fold_rope = 1;         // one-token decoder steps rotate q and the newest K row inside the attention kernel
    int opt_decode_splits = 0;     // position splits of the one-token attention (0 = choose from the SM count)
    int opt_gemm_splitk = 1;       // split the K range of the GEMM over several CTAs when there are few output tiles
    int opt_gemm_tile = 0;         // tokens per CTA of the GEMM: 0 = choose, 128 or 256 = force
    int opt_prefill_gemm = 1;      // prompts of 32+ tokens run their projections as token-block GEMMs
    bool gemm_codes_fresh = false;  // a matrix's pre-expanded codes were built since the last GEMM launch
    int opt_attn_stream = 1;       // a pass of several sequences runs the attention as one streaming CTA per (sequence, KV head)
    int opt_gemv_lean = 1;         // decode-step launches use the GEMV instantiations without the stream-K and general-prologue code
    int opt_tp_fused = 1;          // row-parallel projections under a peer-memory group: the GEMV's epilogue exchanges the partial sums (0: a finalize kernel does)
    int opt_quant_regs = 1;        // the GEMM's quantizer keeps a token's row in registers (0: staged in shared memory)
    int opt_gemm_stream = 1;       // over pre-expanded codes the GEMM runs as a persistent kernel with two accumulator buffers (0: the one-shot kernel)
    int opt_gemm_cache = 1;        // the token-block GEMM reads pre-expanded int8 codes (built per matrix on first use) instead of expanding the 2-bit tiles in the kernel
    int opt_tp_graph = 1;          // record the sharded decode step (collectives included) as a graph
    void* nccl_comm = nullptr;
    // peer mailboxes (tp.cu): this rank's exchange buffer, the device table of every rank's buffer (own included) as
    // mapped into this process, and the device counters of the exchange sequence
    void* xbuf = nullptr;
    void** peer_xbuf_dev = nullptr;
    void* peer_xbuf_host[8] = {};
    unsigned int* x_ctr = nullptr;
    bool tp_peer = false;          // peers attached: row-parallel projections exchange through the mailboxes
    int opt_tp_peer = 1;           // 0 = keep the NCCL exchange even when peers are attached
};

int lb_fail(loom_b200_ctx* ctx, int code, const char* fmt, ...);
const char* lb_global_error();
int lb_ensure_fixup(loom_b200_ctx* ctx, size_t acc_elems, size_t cnt_elems);
int lb_ensure_scratch(loom_b200_ctx* ctx, size_t bytes);
// Waits for the context's stream and reads the device status word with it: a bounded device-side wait that ran out
// (a copy that never landed, a peer that never answered) comes back as LOOM_B200_ERR_TIMEOUT, and the word is cleared.
int lb_sync_checked(loom_b200_ctx* ctx);
int lb_ensure_quant_scratch(loom_b200_ctx* ctx, size_t bytes);

#define LB_CUDA(ctx, expr)                                                                          \
    do {                                                                                            \
        cudaError_t _e = (expr);                                                                    \
        if (_e != cudaSuccess)                                                                      \
            return lb_fail((ctx), LOOM_B200_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,             \
                           cudaGetErrorString(_e), __FILE__, __LINE__);                             \
    } while (0)

#define LB_CHECK_LAUNCH(ctx, name)                                                                  \
    do {                                                                                            \
        cudaError_t _e = cudaGetLastError();                                                        \
        if (_e != cudaSuccess)                                                                      \
            return lb_fail((ctx), LOOM_B200_ERR_CUDA, "launch of %s failed: %s", (name),          \
                           cudaGetErrorString(_e));                                                 \
        (ctx)->launches++;                                                                          \
    } while (0)

#define LB_REQUIRE(ctx, cond, ...)                                                                  \
    do {                                                                                            \
        if (!(cond)) return lb_fail((ctx), LOOM_B200_ERR_INVALID, __VA_ARGS__);                     \
    } while (0)

static inline unsigned long long* lb_trace_row(loom_b200_ctx* ctx, const char* label) {
    if (!ctx->trace_dev) return nullptr;
    int slot = ctx->trace_seq++ % kTraceSlots;
    ctx->trace_label[slot] = label;
    return ctx->trace_dev + (size_t)slot * 8;
}

static inline int lb_set_device(loom_b200_ctx* ctx) {
    cudaError_t e = cudaSetDevice(ctx->device);
    if (e != cudaSuccess) return lb_fail(ctx, LOOM_B200_ERR_CUDA, "cudaSetDevice(%d): %s", ctx->device, cudaGetErrorString(e));
    return 0;
}

// ---- arithmetic helpers (device) ----------------------------------------------------------------
// The CPU contract is IEEE double without fused multiply-add; the intrinsics below pin the rounding
// of every step so that the compiler cannot contract them.

__device__ __forceinline__ float lb_abs_to_f32(float v) { return fabsf(v); }

// Round half away from zero, exactly (Go's math.Round): trunc(x), then one step away when the discarded
// fraction is at least one half.  x - trunc(x) is exact, so no double rounding can occur (the library
// round() gives the same result but costs a long dependent sequence).
__device__ __forceinline__ double lb_round_half_away(double x) {
    const double t = trunc(x);
    const double d = __dsub_rn(x, t);
    return fabs(d) >= 0.5 ? __dadd_rn(t, copysign(1.0, x)) : t;
}

// bitNetQuantizedActivation: int8(clamp(Round(float64(v) * (127/float64(amax))), -128, 127)), Round = half away from
// zero = sign(r) * floor(|r| + 0.5).  Only full-rate instructions: float64 compares, min/max, rounding and conversions
// issue at a quarter of the rate of add/multiply on this GPU (16 against 64 lanes per clock per SM, measured), so the
// sign is handled on the bit pattern and the rounding by two additions.
__device__ __forceinline__ int lb_quant_i8(double v, double s) {
    const double r = __dmul_rn(v, s);
    const int sgn = __double2hiint(r) & 0x80000000;
    // copysign(0.5, r) and copysign(2^52, r).  Both additions round toward zero: |r| + 0.5 then never crosses an
    // integer upwards (floor of the rounded sum = floor of the exact sum, because the floor itself is representable),
    // and adding 2^52 leaves exactly floor(|r| + 0.5) = Round(|r|) in the low mantissa word, whatever the sign.
    const double u = __dadd_rz(__dadd_rz(r, __hiloint2double(sgn | 0x3fe00000, 0)), __hiloint2double(sgn | 0x43300000, 0));
    int n = __double2loint(u);  // |r| <= 127 (1 + 2^-52) by construction of s; anything larger saturates
    const int lim = sgn ? 128 : 127;
    n = (unsigned)n < (unsigned)lim ? n : lim;
    return sgn ? -n : n;
}

// max(m, |y|) for float64 values kept as bit patterns: for non-negative doubles the integer order is the numeric order
__device__ __forceinline__ unsigned long long lb_absmax_bits(unsigned long long m, double y) {
    const unsigned long long b = (unsigned long long)__double_as_longlong(y) & 0x7fffffffffffffffull;
    return b > m ? b : m;
}

// a / b with the reciprocal r = RN(1/b) computed once by the caller: q0 = RN(a*r), the exact remainder
// e = a - b*q0 (one FMA), q1 = RN(q0 + e*r).  With a correctly rounded reciprocal this is the correctly
// rounded quotient (Markstein), i.e. the same bits as an IEEE division, without its long latency.
__device__ __forceinline__ double lb_div_by(double a, double b, double r) {
    const double q0 = __dmul_rn(a, r);
    const double e = fma(-b, q0, a);
    return fma(e, r, q0);
}

// outputScale = float64(scale) * float64(amax) / 127, zero -> 1
__device__ __forceinline__ double lb_output_scale(float scale, float amax) {
    double os = __ddiv_rn(__dmul_rn((double)scale, (double)amax), 127.0);
    return os == 0.0 ? 1.0 : os;
}

__device__ __forceinline__ double lb_gate_product(double g, double u, int act) {
    if (act == LOOM_B200_ACT_RELU2) {
        if (g < 0) g = 0;
        return __dmul_rn(__dmul_rn(g, g), u);
    }
    double sig = __ddiv_rn(1.0, __dadd_rn(1.0, exp(-g)));
    return __dmul_rn(__dmul_rn(g, sig), u);
}

// Activate[float32], poly/poly.go:167-200
__device__ __forceinline__ float lb_activate(float v, int act) {
    switch (act) {
        case LOOM_B200_ACT_RELU: return v < 0.f ? 0.f : v;
        case LOOM_B200_ACT_SILU: return __fmul_rn(v, (float)__ddiv_rn(1.0, __dadd_rn(1.0, exp(-(double)v))));
        case LOOM_B200_ACT_GELU: {
            double x = (double)v;
            double inner = __dmul_rn(sqrt(2.0 / 3.14159265358979323846),
                                     __dadd_rn(x, __dmul_rn(0.044715, pow(x, 3.0))));
            return (float)__dmul_rn(__dmul_rn(0.5, x), __dadd_rn(1.0, tanh(inner)));
        }
        case LOOM_B200_ACT_TANH: return (float)tanh((double)v);
        case LOOM_B200_ACT_SIGMOID: return (float)__ddiv_rn(1.0, __dadd_rn(1.0, exp(-(double)v)));
        case LOOM_B200_ACT_LEAKY_RELU: return v < 0.f ? (float)__dmul_rn((double)v, 0.01) : v;
        case LOOM_B200_ACT_RELU2: return v < 0.f ? 0.f : __fmul_rn(v, v);
        default: return v;
    }
}

__device__ __forceinline__ float lb_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ double lb_warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ int lb_warp_sum_i(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Phase trace: when tracing is on, every launch gets a row of eight 64-bit slots and CTA 0 writes the GPU
// global timer (ns) into slot k at phase k.  Rows are assigned at launch (or recording) time.
__device__ __forceinline__ unsigned long long lb_gtime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void lb_trace(unsigned long long* row, int k) {
    if (row && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0) row[k] = lb_gtime();
}

// ---- sm_100a plumbing: mbarrier, bulk async copy (TMA engine), programmatic dependent launch ------

__device__ __forceinline__ uint32_t lb_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void lb_mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(lb_smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void lb_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(lb_smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool lb_mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(lb_smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limit` polls and returns false (callers set an error flag and leave).
__device__ __forceinline__ bool lb_mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint32_t limit = 4000000u) {
    for (uint32_t i = 0; i < limit; ++i)
        if (lb_mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void lb_fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// 1-D bulk copy global -> shared through the TMA engine; dst/src 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void lb_bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     lb_smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(lb_smem_u32(bar))
                 : "memory");
}
// The same copy for data that is read once per step (packed weights, the fp32 head, KV rows): the lines are marked
// evict-first in L2, so that a step's 2 GB of streams do not push out what IS reused from step to step -- the
// activations, the norm gains and the kernels' own instructions.
__device__ __forceinline__ uint64_t lb_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void lb_bulk_g2s_stream(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
                     lb_smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(lb_smem_u32(bar)), "l"(policy)
                 : "memory");
}
// Programmatic dependent launch: wait for the kernels this one depends on / release dependents.
__device__ __forceinline__ void lb_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void lb_pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
