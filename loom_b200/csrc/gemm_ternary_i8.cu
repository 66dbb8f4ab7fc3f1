// gemm_ternary_i8.cu -- batched-prefill ternary x int8 GEMM on the 5th-generation tensor cores (tcgen05, kind::i8).
//
// For a block of tokens the projection really is a dense contraction, so it runs on tcgen05.mma with the int32
// accumulator in tensor memory.  Replaces the per-token re-read of the weight row that
// ShaderTiledDenseBitNetTernaryQuantizedReduce does for prompts (poly/wgpu_shaders.go:512-642, dispatched once
// per (row, token) by poly/wgpu_kernels.go:416-475); arithmetic contract poly/bitnet_cpu.go:536-546,752-776.
//
//   D[128 weight rows, N tokens] (int32, TMEM) += A[128, 32] (u8 codes 0/1/2, shared) * B[N tokens, 32]^T (s8, shared)
//   N = 128 or 256 tokens per CTA.
//
// Warp roles (320 threads):
//   * load warp: ONE bulk async copy (TMA engine, mbarrier complete_tx) per 128-column k-slice brings the CTA's
//     activations.  The quantizer that feeds this kernel stores the int8 activations as the shared-memory image the
//     tensor core wants -- per (256-token tile, k-slice) a contiguous 32 KB block in K-major no-swizzle core-matrix
//     order [token/8][16-byte K chunk][token%8][16 B] (LBO = 128 B along K, SBO = 1024 B per eight tokens) -- because
//     the TMA engine is slow on many small copies (forty 0.5-1 KB copies per slice took 1.3 us).
//   * eight expansion warps (one 16-row strip each) read their packed tile (512 B per warp and slice) straight from
//     global memory, two slices ahead in registers, and expand 2-bit codes -> one byte per weight with
//     (word >> 2j) & 0x03030303 for j = 0..3 -- no transpose: byte b of result j is the code of column 4b+j, and the
//     quantizer stores the activation bytes of every 16-column group in the same order, so the K permutation cancels
//     in the dot product.  Codes stay unsigned (kind::i8 takes u8 x s8): sum(code*x) - sum(x) = sum(w*x), the same
//     correction as the GEMV, applied in the epilogue from the per-token sum the quantizer produced.
//   * MMA warp: one elected thread issues four K=32 MMAs per slice and commits them to the stage's "empty" mbarrier;
//     the last commit releases the epilogue.
//   * Epilogue: the expansion warps read their 32 TMEM lanes (= weight rows) with tcgen05.ld and apply the float64
//     rescale, bias, activation and residual exactly like the GEMV epilogue.
// Every mbarrier wait is bounded; on expiry the kernel raises the context's status word, frees its tensor memory
// and returns.
#include "layers.cuh"

namespace {

constexpr int kRowsPerCta = 128;   // weight rows = TMEM lanes = MMA M
constexpr int kSliceK = 128;       // K columns (= bytes) per pipeline stage
constexpr int kExpandThreads = 256;  // eight warps: one 16-row strip each; also the epilogue warps
constexpr int kMmaWarp = kExpandThreads / 32, kLoadWarp = kMmaWarp + 1;
constexpr int kGemmThreads = kExpandThreads + 64;
constexpr int kSliceBytesA = kRowsPerCta * kSliceK;  // 16 KB
constexpr int kMaxStages = 6;
constexpr uint32_t kWaitLimit = 20000000u;

// How the A operand reaches shared memory
enum GemmMode : int {
    GEMM_EXPAND = 0,  // eight warps expand the 2-bit tiles to bytes inside the kernel
    GEMM_CACHED = 1,  // one bulk copy per stage brings 16 KB of pre-expanded codes (loom_b200_weight::codes8)
};

struct GemmParams {
    const uint32_t* tiles;   // packed weights, tiled layout
    const uint8_t* codes8;   // pre-expanded codes of the (gate) matrix, or null
    const uint8_t* codes8_up;  // gate/up pair: pre-expanded codes of the up matrix
    float scale_up;
    const float* bias_up;
    int rows, strips, kblocks;
    float scale;
    const int8_t* q;         // int8 activations in core-matrix order (see lb_quantize_gemm_kernel), padded to whole CTA tiles
    const float* amax;       // [tokens]
    const int* xsum;         // [tokens]
    int tokens, Kp;
    const float* bias;       // [rows] or null
    const float* residual;   // [tokens, rows] or null
    int act;
    float* out;              // [tokens, rows] or null
    double* out_f64;         // [tokens, rows] float64 value before rounding (the attention query), or null
    float* pre_out;          // [tokens, rows] value before the activation, or null
    int32_t* acc_out;        // [tokens, rows] or null
    int kv_hd, kv_msl, kv_pos0;  // kv_hd > 0: `out` is a head-major KV ring [rows/kv_hd][kv_msl][kv_hd], token t goes to position kv_pos0 + t
    int* status;
    int32_t* part_acc;       // split-K: [tokens, rows] partial sums, zero between launches
    unsigned int* part_cnt;  // split-K: arrivals per (row tile, token tile), zero between launches
    unsigned long long* trace;  // optional: row 0 = kernel phases, row 1+i = ring phases of k-slice i (CTA 0 only)
};

__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    // K-major, no swizzle: start address, LBO = 128 B (next 16-byte K chunk), SBO = 1024 B (next 8 rows), version 1
    return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)(128 >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46);
}

__device__ __forceinline__ void mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}

__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(lb_smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(lb_smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool wait_bounded(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < kWaitLimit; ++i)
        if (lb_mbar_try_wait(bar, parity)) return true;
    return false;
}

// Float epilogue of sixteen tokens (columns c0 .. c0+15 of the CTA's tile) of weight row r: raw[j] = sum(code * x).
// int32 -> float64 by the exponent trick (2^52 + 2^31 + a as a bit pattern, minus the constant: exact, and a full-rate
// addition where the conversion instruction runs at quarter rate).
__device__ __forceinline__ double gemm_i2d(int a) {
    return __dadd_rn(__hiloint2double(0x43300000, (int)((unsigned)a ^ 0x80000000u)), -4503601774854144.0);
}

__device__ __forceinline__ void gemm_emit16(const GemmParams& p, int r, bool row_ok, bool failed, int tok0, int c0, const int* raw,
                                    const double* s_os, const int* s_xsum, double bias, bool has_bias) {
    int acc[16];
    double y[16];
    float f[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        acc[j] = raw[j] - s_xsum[c0 + j];
        const double t = __dmul_rn(gemm_i2d(acc[j]), s_os[c0 + j]);
        y[j] = has_bias ? __dadd_rn(t, bias) : t;
        f[j] = (float)y[j];
    }
    if (row_ok && !failed) {
        const int ntok = p.tokens - (tok0 + c0);  // columns of this step that are real tokens
        size_t o0 = (size_t)(tok0 + c0) * p.rows + r, ostride = (size_t)p.rows;
        if (p.kv_hd > 0) {
            o0 = ((size_t)(r / p.kv_hd) * p.kv_msl + p.kv_pos0 + tok0 + c0) * p.kv_hd + r % p.kv_hd;
            ostride = (size_t)p.kv_hd;
        }
        if (p.acc_out) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (j < ntok) p.acc_out[o0 + j * ostride] = acc[j];
        }
        if (p.out_f64) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (j < ntok) p.out_f64[o0 + j * ostride] = y[j];
        }
        if (p.out) {
            if (p.pre_out) {
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    if (j < ntok) p.pre_out[o0 + j * ostride] = f[j];
            }
            if (p.act != LOOM_B200_ACT_LINEAR) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    if (p.act == LOOM_B200_ACT_RELU) f[j] = f[j] < 0.f ? 0.f : f[j];
                    else if (p.act == LOOM_B200_ACT_RELU2) f[j] = f[j] < 0.f ? 0.f : __fmul_rn(f[j], f[j]);
                    else f[j] = lb_activate(f[j], p.act);
                }
            }
            if (p.residual) {
                float rs[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) rs[j] = j < ntok ? p.residual[o0 + j * ostride] : 0.f;
#pragma unroll
                for (int j = 0; j < 16; ++j) f[j] = __fadd_rn(f[j], rs[j]);
            }
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (j < ntok) p.out[o0 + j * ostride] = f[j];
        }
    }
}

// stages that fit beside 1 KB of alignment slack
template <int NTOK, int MODE>
struct GemmCfg {
    static constexpr int kSliceBytesB = NTOK * kSliceK;
    static constexpr int kStageBytesA = kSliceBytesA;
    static constexpr int kStageBytes = kStageBytesA + kSliceBytesB;
    static constexpr int kStages = (200 * 1024) / kStageBytes > kMaxStages ? kMaxStages : (200 * 1024) / kStageBytes;
    static constexpr size_t kSmem = (size_t)kStages * kStageBytes + 1024;
};

template <int NTOK, int MODE>
__global__ void __launch_bounds__(kGemmThreads, 1) lb_gemm_ternary_i8_kernel(const GemmParams p) {
    using Cfg = GemmCfg<NTOK, MODE>;
    constexpr int kStages = Cfg::kStages;
    constexpr int kTmemCols = NTOK;
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ __align__(8) uint64_t load_bar[kMaxStages], a_bar[kMaxStages], empty_bar[kMaxStages], done_bar;
    __shared__ uint32_t tmem_base_s;
    __shared__ double s_os[NTOK];
    __shared__ int s_xsum[NTOK];
    __shared__ int s_failed;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row0 = blockIdx.x * kRowsPerCta, tok0 = blockIdx.y * NTOK;
    uint8_t* a_ring = smem;
    uint8_t* b_ring = smem + kStages * Cfg::kStageBytesA;
    // one 128-column k-block per stage; with split-K (gridDim.z > 1) this CTA covers k-blocks [kbase, kbase + nslices)
    const int ktot = p.kblocks;
    const int kbase = (int)((long long)ktot * blockIdx.z / gridDim.z);
    const int nslices = (int)((long long)ktot * (blockIdx.z + 1) / gridDim.z) - kbase;
    const int strip0 = blockIdx.x * (kRowsPerCta / kTileRows);
    const int nstrips = p.strips - strip0 < kRowsPerCta / kTileRows ? p.strips - strip0 : kRowsPerCta / kTileRows;
    unsigned long long* tr = (p.trace && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) ? p.trace : nullptr;
    if (tr && tid == 0) tr[0] = lb_gtime();

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            lb_mbar_init(&load_bar[s], 1);
            lb_mbar_init(&a_bar[s], kExpandThreads / 32);  // one arrival per expansion warp
            lb_mbar_init(&empty_bar[s], 1);
        }
        lb_mbar_init(&done_bar, 1);
        lb_fence_mbar_init();
        s_failed = 0;
    }
    if (warp == kMmaWarp) {  // the MMA warp owns the tensor-memory allocation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(lb_smem_u32(&tmem_base_s)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;

    if (warp == kLoadWarp) {
        // ---------------- loads: packed weight tiles and activation groups of every k-slice ----------------
        bool failed = false;
        // activations of (256-token tile T, slice ks): 32 KB at ((T * nslices) + ks) * 32 KB; a 128-token CTA takes one half
        const int8_t* qbase = p.q + ((size_t)(tok0 >> 8) * ktot + kbase) * 32768 + (size_t)((tok0 & 255) >> 3) * 1024;
        for (int ks = 0; ks < nslices; ++ks) {
            const int s = ks % kStages;
            if (ks >= kStages && !failed && !wait_bounded(&empty_bar[s], (uint32_t)((ks / kStages - 1) & 1))) failed = true;
            if (failed) break;
            if (lane == 0) {
                lb_mbar_expect_tx(&load_bar[s], (uint32_t)(Cfg::kSliceBytesB + (MODE != GEMM_EXPAND ? Cfg::kStageBytesA : 0)));
                lb_bulk_g2s(b_ring + (size_t)s * Cfg::kSliceBytesB, qbase + (size_t)ks * 32768, (uint32_t)Cfg::kSliceBytesB, &load_bar[s]);
                if (MODE != GEMM_EXPAND) {  // the weights of this (row block, k-slice): 16 KB per matrix, already in the tensor core's layout
                    const size_t blk = ((size_t)blockIdx.x * ktot + kbase + ks) * kSliceBytesA;
                    lb_bulk_g2s(a_ring + (size_t)s * Cfg::kStageBytesA, p.codes8 + blk, (uint32_t)kSliceBytesA, &load_bar[s]);
                }
                if (tr) tr[(1 + ks) * 8 + 0] = lb_gtime();
            }
            __syncwarp();
        }
        if (failed && lane == 0) atomicExch(&s_failed, 1);
    } else if (warp < kMmaWarp) {
        // ---------------- expansion warps ----------------
        for (int i = tid; i < NTOK; i += kExpandThreads) {
            const int tok = tok0 + i;
            s_os[i] = tok < p.tokens ? lb_output_scale(p.scale, p.amax[tok]) : 0.0;
            s_xsum[i] = tok < p.tokens ? p.xsum[tok] : 0;
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");  // the per-token scales are read by other expansion warps later
        if (tr && tid == 0) tr[1] = lb_gtime();
        const int g = lane >> 2, t = lane & 3;
        bool failed = false;
        const bool have_strip = warp < nstrips;
        // packed tile of (this warp's strip, slice ks): 512 contiguous bytes, 16 per lane; rows past the matrix: weight 0
        const uint4 pad = make_uint4(0x55555555u, 0x55555555u, 0x55555555u, 0x55555555u);
        const uint4* tile0 = reinterpret_cast<const uint4*>(p.tiles + (size_t)(strip0 + (have_strip ? warp : 0)) * p.kblocks * kTileWords) + lane;
        auto fetch = [&](int ks) { return (have_strip && ks < nslices) ? __ldg(tile0 + (size_t)(kbase + ks) * (kTileWords / 4)) : pad; };
        uint4 w0 = MODE == GEMM_EXPAND ? fetch(0) : pad, w1 = MODE == GEMM_EXPAND ? fetch(1) : pad;
        for (int ks = 0; ks < (MODE == GEMM_EXPAND ? nslices : 0); ++ks) {
            const int s = ks % kStages;
            const uint4 w = w0;
            w0 = w1;
            w1 = fetch(ks + 2);
            // the stage's previous occupant must have been consumed by the tensor core
            if (ks >= kStages && !failed && !wait_bounded(&empty_bar[s], (uint32_t)((ks / kStages - 1) & 1))) failed = true;
            if (tr && tid == 0) tr[(1 + ks) * 8 + 2] = lb_gtime();
            uint8_t* a_dst = a_ring + (size_t)s * kSliceBytesA;
            // lane (g,t) holds [row g, word t] [row g+8, word t] [row g, word 4+t] [row g+8, word 4+t]
            const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int row = warp * 16 + g + 8 * (k & 1);  // row inside the 128-row block
                const int kc = t + 4 * (k >> 1);              // 16-byte K chunk inside the slice
                const uint32_t x = words[k];
                const uint4 e = make_uint4(x & 0x03030303u, (x >> 2) & 0x03030303u, (x >> 4) & 0x03030303u, (x >> 6) & 0x03030303u);
                *reinterpret_cast<uint4*>(a_dst + (row >> 3) * 1024 + kc * 128 + (row & 7) * 16) = e;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the MMA
            __syncwarp();  // every lane's writes and fence are ordered before the warp's single arrival
            if (lane == 0) mbar_arrive(&a_bar[s]);
            if (tr && tid == 0) tr[(1 + ks) * 8 + 3] = lb_gtime();
        }
        // ---------------- epilogue ----------------
        if (tr && tid == 0) tr[2] = lb_gtime();
        if (!failed && !wait_bounded(&done_bar, 0)) failed = true;
        if (tr && tid == 0) tr[3] = lb_gtime();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (failed) atomicExch(&s_failed, 1);
        // a warp may only touch the 32 TMEM lanes of its quarter (warp % 4); the two warps of a quarter split the columns
        const int quarter = warp & 3, chalf = warp >> 2;
        const int r = row0 + quarter * 32 + lane;
        const bool row_ok = r < p.rows;
        const double bias = (row_ok && p.bias) ? (double)p.bias[r] : 0.0;
        // Sixteen columns per step in a rolled loop.  The values of a step are first all computed in straight-line code
        // (sixteen independent int -> float64 -> float32 chains in flight: with two warps per scheduler the epilogue is
        // bound by instruction latency, not throughput), then stored under the per-output conditions.
        const bool has_bias = row_ok && p.bias != nullptr;
        auto emit = [&](int c0, const int* raw) { gemm_emit16(p, r, row_ok, failed, tok0, c0, raw, s_os, s_xsum, bias, has_bias); };
        const bool split = gridDim.z > 1;
#pragma unroll 1
        for (int c0 = chalf * (NTOK / 2); c0 < (chalf + 1) * (NTOK / 2); c0 += 16) {
            uint32_t v[16];
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0;
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                         : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                           "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                         : "r"(taddr)
                         : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (tr && tid == 0 && c0 == 0) tr[5] = lb_gtime();
            if (!split) {
                int raw[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) raw[j] = (int)v[j];
                emit(c0, raw);
            } else if (row_ok && !failed) {  // split-K: add this CTA's part to the tile's sums (integer addition: any order, same bits)
                const int ntok = p.tokens - (tok0 + c0);
                int32_t* dst = p.part_acc + (size_t)(tok0 + c0) * p.rows + r;
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    if (j < ntok) atomicAdd(dst + (size_t)j * p.rows, (int)v[j]);
            }
            if (tr && tid == 0 && c0 == 0) tr[6] = lb_gtime();
        }
        if (split) {
            // the CTA that completes the tile's sums runs the float epilogue on them and clears them for the next launch
            __shared__ int s_last;
            __threadfence();
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (tid == 0) s_last = atomicAdd(&p.part_cnt[blockIdx.y * gridDim.x + blockIdx.x], 1u) == gridDim.z - 1 ? 1 : 0;
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (s_last) {
                __threadfence();
#pragma unroll 1
                for (int c0 = chalf * (NTOK / 2); c0 < (chalf + 1) * (NTOK / 2); c0 += 16) {
                    int raw[16];
                    const int ntok = p.tokens - (tok0 + c0);
                    int32_t* src = p.part_acc + (size_t)(tok0 + c0) * p.rows + r;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        raw[j] = 0;
                        if (row_ok && j < ntok) {
                            raw[j] = __ldcg(src + (size_t)j * p.rows);
                            src[(size_t)j * p.rows] = 0;
                        }
                    }
                    emit(c0, raw);
                }
                if (tid == 0) p.part_cnt[blockIdx.y * gridDim.x + blockIdx.x] = 0;
            }
        }
        if (tr && tid == 0) tr[7] = lb_gtime();
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    } else {
        // ---------------- MMA issuer ----------------
        // instruction descriptor: D = S32, A = U8, B = S8, both K-major, N tokens, M = 128
        const uint32_t idesc = (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(NTOK >> 3) << 17) | ((uint32_t)(kRowsPerCta >> 4) << 24);
        bool failed = false;
        for (int ks = 0; ks < nslices; ++ks) {
            const int s = ks % kStages;
            if (MODE == GEMM_EXPAND && !failed && !wait_bounded(&a_bar[s], (uint32_t)((ks / kStages) & 1))) failed = true;
            if (!failed && !wait_bounded(&load_bar[s], (uint32_t)((ks / kStages) & 1))) failed = true;  // the activations (and the cached codes)
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (tr && lane == 0) tr[(1 + ks) * 8 + 4] = lb_gtime();
            if (lane == 0 && !failed) {
                const uint32_t a_addr = lb_smem_u32(a_ring + (size_t)s * Cfg::kStageBytesA);
                const uint32_t b_addr = lb_smem_u32(b_ring + (size_t)s * Cfg::kSliceBytesB);
#pragma unroll
                for (int k = 0; k < kSliceK / 32; ++k)  // K = 32 per instruction = two 16-byte chunks = 256 B further
                    mma_i8(tmem_base, smem_desc(a_addr + k * 256), smem_desc(b_addr + k * 256), idesc, (ks > 0 || k > 0) ? 1u : 0u);
                mma_commit(&empty_bar[s]);  // arrives when the MMAs that read this stage are done
                if (tr) tr[(1 + ks) * 8 + 5] = lb_gtime();
            }
            __syncwarp();
        }
        if (lane == 0) {
            if (failed) atomicExch(&s_failed, 1);
            mma_commit(&done_bar);
        }
        __syncwarp();
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncthreads();
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
    if (tid == 0 && s_failed) atomicExch(p.status, 3);
    if (tr && tid == 0) tr[4] = lb_gtime();
}

// ------------------------------------------------------------------------------------------------------------------
// Persistent variant over pre-expanded codes.  One CTA per SM walks output tiles (row tile fastest, so the CTAs that run
// together share a token tile's activations in L2); the shared-memory ring runs on across tile boundaries, and tensor
// memory holds TWO accumulator buffers, so the eight epilogue warps drain tile i (tcgen05.ld, float64 rescale, stores)
// while the MMA warp already accumulates tile i+1.  In the one-shot kernel above the epilogue of a 128 x 256 tile costs
// about as long as its twenty k-slices of MMAs, and two co-resident CTAs ran in lockstep instead of overlapping.
// DUAL: a gate / up pair that shares the activations -- both code blocks ride in one stage, two accumulators per buffer
// (gate at column 0, up at column NTOK), and the epilogue writes float32(gateProduct(yg + bg, yu + bu)) only
// (poly/swiglu.go:299-310): the two int32 accumulator planes never travel through memory.
template <int NTOK, bool DUAL>
struct StreamCfg {
    static constexpr int kMats = DUAL ? 2 : 1;
    static constexpr int kBytesB = NTOK * kSliceK;
    static constexpr int kBytesA = kSliceBytesA * kMats;
    static constexpr int kStageBytes = kBytesA + kBytesB;
    static constexpr int kStages = (200 * 1024) / kStageBytes > kMaxStages ? kMaxStages : (200 * 1024) / kStageBytes;
    static constexpr int kAccCols = NTOK * kMats;  // TMEM columns of one accumulator buffer
    static constexpr size_t kSmem = (size_t)kStages * kStageBytes + 1024;
    static_assert(2 * kAccCols <= 512, "two accumulator buffers must fit the 512 TMEM columns");
};

template <int NTOK, bool DUAL>
__global__ void __launch_bounds__(kGemmThreads, 1) lb_gemm_stream_kernel(const GemmParams p, int row_tiles, int ntiles) {
    using Cfg = StreamCfg<NTOK, DUAL>;
    constexpr int kStages = Cfg::kStages;
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ __align__(8) uint64_t load_bar[kMaxStages], empty_bar[kMaxStages], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base_s;
    __shared__ double s_os[NTOK], s_os_up[DUAL ? NTOK : 1];
    __shared__ int s_xsum[NTOK];
    __shared__ int s_failed;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    uint8_t* a_ring = smem;
    uint8_t* b_ring = smem + kStages * Cfg::kBytesA;
    const int ktot = p.kblocks;
    const int my_tiles = (int)blockIdx.x < ntiles ? (ntiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            lb_mbar_init(&load_bar[s], 1);
            lb_mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            lb_mbar_init(&acc_full[b], 1);
            lb_mbar_init(&acc_empty[b], kExpandThreads / 32);  // one arrival per epilogue warp
        }
        lb_fence_mbar_init();
        s_failed = 0;
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(lb_smem_u32(&tmem_base_s)), "r"(2 * Cfg::kAccCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;
    lb_pdl_launch_dependents();

    if (warp == kLoadWarp) {
        // ---------------- loads: per stage the activations of the tile's tokens and the code block(s) of its rows ----------------
        bool failed = false;
        uint32_t it = 0;
        // The weights do not depend on the quantizer that runs before this kernel: the code blocks of the first stages
        // are requested before the dependency wait, their activations after it (one barrier counts the bytes of both).
        int pre = 0;
        if (my_tiles > 0) {
            const int rt0 = (int)blockIdx.x % row_tiles;
            const size_t blk00 = (size_t)rt0 * ktot * kSliceBytesA;
            pre = ktot < kStages ? ktot : kStages;
            if (lane == 0) {
                for (int ks = 0; ks < pre; ++ks) {
                    lb_mbar_expect_tx(&load_bar[ks], (uint32_t)Cfg::kStageBytes);
                    lb_bulk_g2s(a_ring + (size_t)ks * Cfg::kBytesA, p.codes8 + blk00 + (size_t)ks * kSliceBytesA, (uint32_t)kSliceBytesA, &load_bar[ks]);
                    if (DUAL)
                        lb_bulk_g2s(a_ring + (size_t)ks * Cfg::kBytesA + kSliceBytesA, p.codes8_up + blk00 + (size_t)ks * kSliceBytesA,
                                    (uint32_t)kSliceBytesA, &load_bar[ks]);
                }
            }
        }
        lb_pdl_wait();
        for (int i = 0; i < my_tiles && !failed; ++i) {
            const int t = (int)blockIdx.x + i * (int)gridDim.x;
            const int rt = t % row_tiles, tok0 = (t / row_tiles) * NTOK;
            const int8_t* qbase = p.q + (size_t)(tok0 >> 8) * ktot * 32768 + (size_t)((tok0 & 255) >> 3) * 1024;
            const size_t blk0 = (size_t)rt * ktot * kSliceBytesA;
            for (int ks = 0; ks < ktot; ++ks, ++it) {
                const int s = (int)(it % kStages);
                if (it >= (uint32_t)kStages && !wait_bounded(&empty_bar[s], (it / kStages - 1) & 1)) {
                    failed = true;
                    break;
                }
                if (lane == 0) {
                    const bool a_done = i == 0 && ks < pre;  // requested before the dependency wait
                    if (!a_done) lb_mbar_expect_tx(&load_bar[s], (uint32_t)Cfg::kStageBytes);
                    lb_bulk_g2s(b_ring + (size_t)s * Cfg::kBytesB, qbase + (size_t)ks * 32768, (uint32_t)Cfg::kBytesB, &load_bar[s]);
                    if (!a_done) {
                        lb_bulk_g2s(a_ring + (size_t)s * Cfg::kBytesA, p.codes8 + blk0 + (size_t)ks * kSliceBytesA, (uint32_t)kSliceBytesA, &load_bar[s]);
                        if (DUAL)
                            lb_bulk_g2s(a_ring + (size_t)s * Cfg::kBytesA + kSliceBytesA, p.codes8_up + blk0 + (size_t)ks * kSliceBytesA,
                                        (uint32_t)kSliceBytesA, &load_bar[s]);
                    }
                }
                __syncwarp();
            }
        }
        if (failed && lane == 0) atomicExch(&s_failed, 1);
    } else if (warp == kMmaWarp) {
        // ---------------- MMA issuer ----------------
        const uint32_t idesc = (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(NTOK >> 3) << 17) | ((uint32_t)(kRowsPerCta >> 4) << 24);
        bool failed = false;
        uint32_t it = 0;
        for (int i = 0; i < my_tiles && !failed; ++i) {
            const int buf = i & 1;
            // the epilogue must have drained this buffer's previous tile
            if (i >= 2 && !wait_bounded(&acc_empty[buf], (uint32_t)(((i >> 1) - 1) & 1))) {
                failed = true;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t d = tmem_base + (uint32_t)(buf * Cfg::kAccCols);
            for (int ks = 0; ks < ktot; ++ks, ++it) {
                const int s = (int)(it % kStages);
                if (!wait_bounded(&load_bar[s], (it / kStages) & 1)) {
                    failed = true;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (lane == 0) {
                    const uint32_t a_addr = lb_smem_u32(a_ring + (size_t)s * Cfg::kBytesA);
                    const uint32_t b_addr = lb_smem_u32(b_ring + (size_t)s * Cfg::kBytesB);
#pragma unroll
                    for (int k = 0; k < kSliceK / 32; ++k)
                        mma_i8(d, smem_desc(a_addr + k * 256), smem_desc(b_addr + k * 256), idesc, (ks > 0 || k > 0) ? 1u : 0u);
                    if (DUAL) {
#pragma unroll
                        for (int k = 0; k < kSliceK / 32; ++k)
                            mma_i8(d + (uint32_t)NTOK, smem_desc(a_addr + kSliceBytesA + k * 256), smem_desc(b_addr + k * 256), idesc,
                                   (ks > 0 || k > 0) ? 1u : 0u);
                    }
                    mma_commit(&empty_bar[s]);
                }
                __syncwarp();
            }
            if (!failed && lane == 0) mma_commit(&acc_full[buf]);  // arrives when every MMA of the tile is done
            __syncwarp();
        }
        if (failed && lane == 0) atomicExch(&s_failed, 1);
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    } else {
        // ---------------- epilogue warps: tile i while the MMA warp is on tile i + 1 ----------------
        // a warp may only touch the 32 TMEM lanes of its quarter (warp % 4); the two warps of a quarter split the columns
        const int quarter = warp & 3, chalf = warp >> 2;
        bool failed = false;  // after a wait ran out the warp keeps walking the tiles (its named-barrier count must match) without touching TMEM or memory
        lb_pdl_wait();  // the per-token scales, the residual rows and the output buffer belong to earlier launches until here
        for (int i = 0; i < my_tiles; ++i) {
            const int t = (int)blockIdx.x + i * (int)gridDim.x;
            const int rt = t % row_tiles, tok0 = (t / row_tiles) * NTOK, buf = i & 1;
            asm volatile("bar.sync 1, 256;" ::: "memory");  // the previous tile's scales are no longer read
            for (int c = tid; c < NTOK; c += kExpandThreads) {
                const int tok = tok0 + c;
                s_os[c] = tok < p.tokens ? lb_output_scale(p.scale, p.amax[tok]) : 0.0;
                if (DUAL) s_os_up[c] = tok < p.tokens ? lb_output_scale(p.scale_up, p.amax[tok]) : 0.0;
                s_xsum[c] = tok < p.tokens ? p.xsum[tok] : 0;
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (!failed && !wait_bounded(&acc_full[buf], (uint32_t)((i >> 1) & 1))) {
                failed = true;
                atomicExch(&s_failed, 1);
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int r = rt * kRowsPerCta + quarter * 32 + lane;
            const bool row_ok = r < p.rows;
            const bool has_bias = row_ok && p.bias != nullptr;
            const double bias = has_bias ? (double)p.bias[r] : 0.0;
            const uint32_t tacc = tmem_base + (uint32_t)(buf * Cfg::kAccCols) + ((uint32_t)(quarter * 32) << 16);
            if (!failed) {
#pragma unroll 1
                for (int c0 = chalf * (NTOK / 2); c0 < (chalf + 1) * (NTOK / 2); c0 += 16) {
                    uint32_t v[16];
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                                   "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                                 : "r"(tacc + (uint32_t)c0)
                                 : "memory");
                    if (!DUAL) {
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        int raw[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) raw[j] = (int)v[j];
                        gemm_emit16(p, r, row_ok, false, tok0, c0, raw, s_os, s_xsum, bias, has_bias);
                    } else {
                        uint32_t u[16];
                        asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                                     : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]),
                                       "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15])
                                     : "r"(tacc + (uint32_t)(NTOK + c0))
                                     : "memory");
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        const bool has_bias_up = row_ok && p.bias_up != nullptr;
                        const double bias_up = has_bias_up ? (double)p.bias_up[r] : 0.0;
                        float f[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int xs = s_xsum[c0 + j];
                            double yg = __dmul_rn(gemm_i2d((int)v[j] - xs), s_os[c0 + j]);
                            double yu = __dmul_rn(gemm_i2d((int)u[j] - xs), s_os_up[c0 + j]);
                            if (has_bias) yg = __dadd_rn(yg, bias);
                            if (has_bias_up) yu = __dadd_rn(yu, bias_up);
                            f[j] = (float)lb_gate_product(yg, yu, p.act);
                        }
                        if (row_ok) {
                            const int ntok = p.tokens - (tok0 + c0);
                            const size_t o0 = (size_t)(tok0 + c0) * p.rows + r;
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                if (j < ntok) p.out[o0 + (size_t)j * p.rows] = f[j];
                        }
                    }
                }
            }
            // this warp's reads of the buffer are complete (wait::ld above): hand it back to the MMA warp
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
    }
    __syncthreads();
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * Cfg::kAccCols) : "memory");
    }
    if (tid == 0 && s_failed) atomicExch(p.status, 3);
}

// Measures what the tensor pipe can do on this shape of instruction: one CTA per SM, operands resident in shared memory
// (zeros), one thread issuing `iters` x 4 MMAs of M = 128, N = 256, K = 32 into one TMEM accumulator.  No loads, no
// expansion, no epilogue: the number the GEMM's tensor-pipe fraction is quoted against.
__global__ void __launch_bounds__(128, 1) lb_i8_peak_kernel(int iters, int* status) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ __align__(8) uint64_t done_bar;
    __shared__ uint32_t tmem_base_s;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int i = tid; i < (kSliceBytesA + 256 * kSliceK) / 16; i += blockDim.x) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0u, 0u, 0u, 0u);
    if (tid == 0) {
        lb_mbar_init(&done_bar, 1);
        lb_fence_mbar_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(lb_smem_u32(&tmem_base_s)), "r"(256) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;
    if (warp == 0) {
        const uint32_t idesc = (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(kRowsPerCta >> 4) << 24);
        if (lane == 0) {
            const uint32_t a_addr = lb_smem_u32(smem), b_addr = lb_smem_u32(smem + kSliceBytesA);
            for (int it = 0; it < iters; ++it) {
#pragma unroll
                for (int k = 0; k < 4; ++k) mma_i8(tmem_base, smem_desc(a_addr + k * 256), smem_desc(b_addr + k * 256), idesc, (it > 0 || k > 0) ? 1u : 0u);
            }
            mma_commit(&done_bar);
        }
        __syncwarp();
        if (!wait_bounded(&done_bar, 0) && lane == 0) atomicExch(status, 3);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256) : "memory");
    }
}

// Quantizer of the GEMM path: the GEMV prologues' arithmetic (plain absmax, or a block / inner RMSNorm first).  The
// output is laid out for the tensor core: [token/8][Kp/16][token%8][16 bytes], the bytes of every 16-column group in
// the order the A expansion produces (position 4j+b holds column 4b+j); columns up to Kp and tokens up to the padded
// count are zero; the per-token sum of the quantized values is written next to amax.  One CTA per (padded) token.
template <int PRO>
__global__ void __launch_bounds__(256) lb_quantize_gemm_kernel(const LbGemmQuant a, int Kp, int8_t* __restrict__ q,
                                                               float* __restrict__ amax_out, int* __restrict__ xsum_out) {
    extern __shared__ __align__(16) uint8_t qsm[];  // the token's row in its input precision: read from memory once
    __shared__ float red[8];
    __shared__ double redd[8];
    __shared__ int redi[8];
    constexpr bool f64 = PRO == LB_PRO_INNERNORM64;
    using VT = typename std::conditional<f64, double, float>::type;
    VT* vals = reinterpret_cast<VT*>(qsm);
    const int K = a.K, tid = threadIdx.x;
    // byte c of this token's row lives at: (256-token tile, k-slice c/128) block of 32 KB, + (token%256)/8 * 1 KB
    // + (16-byte chunk (c/16)%8) * 128 + (token%8) * 16 + c%16
    int8_t* qrow = q + (size_t)(blockIdx.x >> 8) * (Kp >> 7) * 32768 + (size_t)((blockIdx.x & 255) >> 3) * 1024 + (blockIdx.x & 7) * 16;
    auto chunk_ptr = [&](int ch) { return reinterpret_cast<uint4*>(qrow + (size_t)(ch >> 3) * 32768 + (ch & 7) * 128); };
    const int nchunks = Kp >> 4;
    if ((int)blockIdx.x >= a.tokens) {  // padding token: zeros
        for (int ch = tid; ch < nchunks; ch += blockDim.x) *chunk_ptr(ch) = make_uint4(0u, 0u, 0u, 0u);
        return;
    }
    const VT* row = reinterpret_cast<const VT*>(a.x) + (size_t)blockIdx.x * K;
    auto wt = [&](int i) { return (PRO != LB_PRO_F32 && a.norm_w && i < a.norm_w_len) ? (double)a.norm_w[i] : 1.0; };
    // pass 1: stage the row, sum of squares (norms) or absmax (plain rows)
    double ss = 0.0;
    float m = 0.0f;
    for (int i = tid; i < K; i += blockDim.x) {
        const VT v = row[i];
        vals[i] = v;
        if (PRO >= LB_PRO_BLOCKNORM) ss = __dadd_rn(ss, __dmul_rn((double)v, (double)v));
        else m = fmaxf(m, (float)fabs((double)v));
    }
    double root = 1.0, rr = 1.0;
    if (PRO >= LB_PRO_BLOCKNORM) {
        ss = lb_warp_sum(ss);
        if ((tid & 31) == 0) redd[tid >> 5] = ss;
        __syncthreads();
        ss = 0.0;
        for (int i = 0; i < 8; ++i) ss += redd[i];
        root = sqrt(__dadd_rn(__ddiv_rn(ss, (double)K), a.eps));
        rr = __ddiv_rn(1.0, root);
        // pass 2: normalise in place (each thread revisits the elements it staged), absmax of the result
        for (int i = tid; i < K; i += blockDim.x) {
            const double y = lb_pro_value<PRO>((double)vals[i], root, rr, wt(i));
            vals[i] = (VT)y;
            if (a.norm_out) a.norm_out[(size_t)blockIdx.x * K + i] = (float)y;
            m = fmaxf(m, (float)fabs(y));
        }
    }
    m = lb_warp_max(m);
    if ((tid & 31) == 0) red[tid >> 5] = m;
    __syncthreads();  // also: every staged / normalised value is visible to the whole CTA
    m = red[0];
    for (int i = 1; i < 8; ++i) m = fmaxf(m, red[i]);
    if (m < 1e-5f) m = 1e-5f;
    const double s = __ddiv_rn(127.0, (double)m);
    // pass 3: one 16-column chunk per thread and step -> one 16-byte store; byte 4j+b of the chunk holds column 4b+j
    int sum = 0;
    for (int ch = tid; ch < nchunks; ch += blockDim.x) {
        uint32_t wds[4] = {0u, 0u, 0u, 0u};
        const int base = ch << 4;
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            const int col = base + k;  // k = 4b + j -> destination byte 4j + b
            int v = 0;
            if (col < K) v = lb_quant_i8((double)vals[col], s);
            sum += v;
            const int j = k & 3, b = k >> 2;
            wds[j] |= (uint32_t)(v & 0xff) << (8 * b);
        }
        *chunk_ptr(ch) = make_uint4(wds[0], wds[1], wds[2], wds[3]);
    }
    sum = lb_warp_sum_i(sum);
    if ((tid & 31) == 0) redi[tid >> 5] = sum;
    __syncthreads();
    if (tid == 0) {
        int tot = 0;
        for (int i = 0; i < 8; ++i) tot += redi[i];
        amax_out[blockIdx.x] = m;
        xsum_out[blockIdx.x] = tot;
    }
}

// The same quantizer with the token's row held in registers: thread t owns the 16-column chunks t, t + T, ... (CPT of them),
// loads each with four 16-byte loads (all in flight together), and never stages the row in shared memory; one block
// reduction for the norm's sum of squares, one for the absmax.  The arithmetic per element is that of the kernel above;
// only the order of the float64 additions inside the sum of squares differs (per-thread partial sums).
template <int PRO, int CPT>
__global__ void __launch_bounds__(256) lb_quantize_gemm_regs_kernel(const LbGemmQuant a, int Kp, int8_t* __restrict__ q,
                                                                    float* __restrict__ amax_out, int* __restrict__ xsum_out) {
    __shared__ float red[8];
    __shared__ double redd[8];
    __shared__ int redi[8];
    constexpr bool f64 = PRO == LB_PRO_INNERNORM64;
    using VT = typename std::conditional<f64, double, float>::type;
    const int K = a.K, tid = threadIdx.x, T = blockDim.x, nwarps = T >> 5;
    int8_t* qrow = q + (size_t)(blockIdx.x >> 8) * (Kp >> 7) * 32768 + (size_t)((blockIdx.x & 255) >> 3) * 1024 + (blockIdx.x & 7) * 16;
    auto chunk_ptr = [&](int ch) { return reinterpret_cast<uint4*>(qrow + (size_t)(ch >> 3) * 32768 + (ch & 7) * 128); };
    const int nchunks = Kp >> 4;
    // programmatic dependent launch: the GEMM that follows may set itself up (barriers, tensor memory, first weight
    // blocks) while this kernel runs; this kernel reads its rows, and overwrites the activation image the previous GEMM
    // was reading, only after everything before it is complete
    lb_pdl_launch_dependents();
    lb_pdl_wait();
    if ((int)blockIdx.x >= a.tokens) {  // padding token: zeros
        for (int ch = tid; ch < nchunks; ch += T) *chunk_ptr(ch) = make_uint4(0u, 0u, 0u, 0u);
        return;
    }
    const VT* row = reinterpret_cast<const VT*>(a.x) + (size_t)blockIdx.x * K;
    const bool vec = (K % (f64 ? 2 : 4)) == 0 && (reinterpret_cast<uintptr_t>(a.x) & 15) == 0;
    VT v[CPT][16];
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
        const int base = (tid + c * T) << 4;
        if (vec && base + 16 <= K) {
            if (f64) {
                const double2* src = reinterpret_cast<const double2*>(row + base);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const double2 d = src[k];
                    v[c][2 * k] = (VT)d.x;
                    v[c][2 * k + 1] = (VT)d.y;
                }
            } else {
                const float4* src = reinterpret_cast<const float4*>(row + base);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float4 d = src[k];
                    v[c][4 * k] = (VT)d.x;
                    v[c][4 * k + 1] = (VT)d.y;
                    v[c][4 * k + 2] = (VT)d.z;
                    v[c][4 * k + 3] = (VT)d.w;
                }
            }
        } else {
#pragma unroll
            for (int k = 0; k < 16; ++k) v[c][k] = base + k < K ? row[base + k] : (VT)0;
        }
    }
    float m = 0.0f;
    if (PRO >= LB_PRO_BLOCKNORM) {
        double ss = 0.0;
#pragma unroll
        for (int c = 0; c < CPT; ++c)
#pragma unroll
            for (int k = 0; k < 16; ++k) ss = __dadd_rn(ss, __dmul_rn((double)v[c][k], (double)v[c][k]));  // columns past K hold zero
        ss = lb_warp_sum(ss);
        if ((tid & 31) == 0) redd[tid >> 5] = ss;
        __syncthreads();
        ss = 0.0;
        for (int i = 0; i < nwarps; ++i) ss += redd[i];
        if (a.given_ss) ss = a.given_ss[blockIdx.x];
        const double root = sqrt(__dadd_rn(__ddiv_rn(ss, (double)(a.norm_count > 0 ? a.norm_count : K)), a.eps));
        const double rr = __ddiv_rn(1.0, root);
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
            const int base = (tid + c * T) << 4;
#pragma unroll
            for (int k = 0; k < 16; ++k) {
                const int col = base + k;
                if (col < K) {
                    const double w = (a.norm_w && col < a.norm_w_len) ? (double)__ldg(a.norm_w + col) : 1.0;
                    const double y = lb_pro_value<PRO>((double)v[c][k], root, rr, w);
                    v[c][k] = (VT)y;
                    if (a.norm_out) a.norm_out[(size_t)blockIdx.x * K + col] = (float)y;
                    m = fmaxf(m, (float)fabs(y));
                }
            }
        }
    } else {
#pragma unroll
        for (int c = 0; c < CPT; ++c)
#pragma unroll
            for (int k = 0; k < 16; ++k) m = fmaxf(m, (float)fabs((double)v[c][k]));
    }
    m = lb_warp_max(m);
    if ((tid & 31) == 0) red[tid >> 5] = m;
    __syncthreads();
    m = red[0];
    for (int i = 1; i < nwarps; ++i) m = fmaxf(m, red[i]);
    if (a.given_amax) m = a.given_amax[blockIdx.x];
    if (m < 1e-5f) m = 1e-5f;
    const double s = __ddiv_rn(127.0, (double)m);
    int sum = 0;
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
        const int ch = tid + c * T;
        if (ch < nchunks) {
            uint32_t wds[4] = {0u, 0u, 0u, 0u};
#pragma unroll
            for (int k = 0; k < 16; ++k) {  // k = 4b + j -> destination byte 4j + b
                const int qv = lb_quant_i8((double)v[c][k], s);
                sum += qv;
                wds[k & 3] |= (uint32_t)(qv & 0xff) << (8 * (k >> 2));
            }
            *chunk_ptr(ch) = make_uint4(wds[0], wds[1], wds[2], wds[3]);
        }
    }
    sum = lb_warp_sum_i(sum);
    if ((tid & 31) == 0) redi[tid >> 5] = sum;
    __syncthreads();
    if (tid == 0) {
        int tot = 0;
        for (int i = 0; i < nwarps; ++i) tot += redi[i];
        amax_out[blockIdx.x] = m;
        xsum_out[blockIdx.x] = tot;
    }
}

// gate product of a token block from the raw accumulators of the gate and up GEMMs (swigluGateProduct in float64,
// poly/swiglu.go:37-46,299-306): prod = float32(f(acc_g * os_g + b_g) * (acc_u * os_u + b_u))
__global__ void lb_gate_product_acc_kernel(const int32_t* __restrict__ acc_g, const int32_t* __restrict__ acc_u,
                                           const float* __restrict__ amax, int tokens, int inter, float scale_g, float scale_u,
                                           const float* __restrict__ bias_g, const float* __restrict__ bias_u, int act,
                                           float* __restrict__ prod) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)tokens * inter) return;
    const int tok = (int)(i / inter), r = (int)(i % inter);
    double yg = __dmul_rn((double)acc_g[i], lb_output_scale(scale_g, amax[tok]));
    double yu = __dmul_rn((double)acc_u[i], lb_output_scale(scale_u, amax[tok]));
    if (bias_g) yg = __dadd_rn(yg, (double)bias_g[r]);
    if (bias_u) yu = __dadd_rn(yu, (double)bias_u[r]);
    prod[i] = (float)lb_gate_product(yg, yu, act);
}

// Pre-expands a packed matrix into the GEMM's A image: per (row block of 128, k-slice of 128 columns) 16 KB in K-major
// no-swizzle core-matrix order, [row / 8][16-byte K chunk][row % 8][16 B], byte 4j+b of a chunk = code of column 4b+j of
// its 16-column group (the order the in-kernel expansion produces and the quantizer matches).  One thread per 16 bytes.
__global__ void lb_expand_codes_kernel(const uint32_t* __restrict__ tiles, int strips, int kblocks, uint8_t* __restrict__ codes8) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // (row block, k-slice, row in block, chunk)
    const int row_blocks = (strips + 7) / 8;
    const size_t total = (size_t)row_blocks * kblocks * 128 * 8;
    if (idx >= total) return;
    const int kc = (int)(idx & 7), row = (int)((idx >> 3) & 127);
    const size_t blk = idx >> 10;
    const int ks = (int)(blk % kblocks), rb = (int)(blk / kblocks);
    const int strip = rb * 8 + (row >> 4), r16 = row & 15;
    uint32_t x = 0x55555555u;  // rows past the matrix: weight 0
    if (strip < strips) {
        // lane (g,t) of a tile holds [row g, word t] [row g+8, word t] [row g, word 4+t] [row g+8, word 4+t]
        const int g = r16 & 7, t = kc & 3, slot = (r16 >> 3) | ((kc >> 2) << 1);
        x = tiles[((size_t)strip * kblocks + ks) * kTileWords + (size_t)(g * 4 + t) * 4 + slot];
    }
    const uint4 e = make_uint4(x & 0x03030303u, (x >> 2) & 0x03030303u, (x >> 4) & 0x03030303u, (x >> 6) & 0x03030303u);
    *reinterpret_cast<uint4*>(codes8 + blk * kSliceBytesA + (size_t)(row >> 3) * 1024 + kc * 128 + (row & 7) * 16) = e;
}

// layout of the GEMM scratch for `tokens` rows of Kp bytes: int8 rows, amax, sums
struct GemmScratch {
    int8_t* q;
    float* amax;
    int* xsum;
};
constexpr int kTokPad = 256;  // the activations are padded with zero rows to whole CTA tiles of either size
int padded_tokens(int tokens) { return (tokens + kTokPad - 1) / kTokPad * kTokPad; }
GemmScratch gemm_scratch_at(void* base, int tokens, int Kp) {
    GemmScratch g;
    const int pt = padded_tokens(tokens);
    g.q = (int8_t*)base;
    g.amax = (float*)((char*)base + (((size_t)pt * Kp + 255) & ~(size_t)255));
    g.xsum = (int*)(g.amax + pt);
    return g;
}

}  // namespace

int lb_gemm_quantize(loom_b200_ctx* ctx, const LbGemmQuant& a) {
    LB_REQUIRE(ctx, a.x && a.tokens > 0 && a.K > 0, "gemm_quantize: bad arguments");
    const int Kp = (a.K + kTileCols - 1) / kTileCols * kTileCols;
    // scratch: permuted int8 activations, amax, sum per token
    const int pt = padded_tokens(a.tokens);
    size_t need = (size_t)pt * Kp + 256 + (size_t)pt * 8 + 256;
    if (need > ctx->gemm_scratch_bytes) {  // its own buffer: layer calls keep their tensors in ctx->scratch
        if (ctx->capturing) return lb_fail(ctx, LOOM_B200_ERR_INVALID, "ternary_gemm: scratch would grow while recording a graph");
        LB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        if (ctx->gemm_scratch) cudaFree(ctx->gemm_scratch);
        ctx->gemm_scratch = nullptr;
        ctx->gemm_scratch_bytes = 0;
        LB_CUDA(ctx, cudaMalloc(&ctx->gemm_scratch, need + need / 4));
        ctx->gemm_scratch_bytes = need + need / 4;
    }
    GemmScratch g = gemm_scratch_at(ctx->gemm_scratch, a.tokens, Kp);
    // rows of up to 256 * CPT chunks of 16 columns stay in registers (float rows: CPT up to 8, float64 rows: up to 4)
    const int nchunks = Kp >> 4;
    const int cpt_need = (nchunks + 255) / 256;
    const int cpt = cpt_need <= 1 ? 1 : cpt_need <= 2 ? 2 : cpt_need <= 4 ? 4 : 8;
    const bool regs_ok = cpt_need <= (a.pro == LB_PRO_INNERNORM64 ? 4 : 8);
    LB_REQUIRE(ctx, !(a.given_ss || a.given_amax) || regs_ok, "gemm_quantize: rows of %d columns with agreed statistics are not supported", a.K);
    if ((ctx->opt_quant_regs || a.given_ss || a.given_amax) && regs_ok) {
        const int T = ((nchunks + cpt - 1) / cpt + 31) / 32 * 32;
        cudaLaunchConfig_t qcfg = {};
        qcfg.gridDim = dim3(pt);
        qcfg.blockDim = dim3(T);
        qcfg.stream = ctx->stream;
        cudaLaunchAttribute qattr[1];
        qattr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        qattr[0].val.programmaticStreamSerializationAllowed = 1;
        qcfg.attrs = qattr;
        qcfg.numAttrs = ctx->opt_pdl ? 1 : 0;
        cudaError_t qerr = cudaSuccess;
#define LB_QREG(PRO, CPT) qerr = cudaLaunchKernelEx(&qcfg, lb_quantize_gemm_regs_kernel<PRO, CPT>, a, Kp, g.q, g.amax, g.xsum)
#define LB_QREG_PRO(PRO)            \
    switch (cpt) {                  \
        case 1: LB_QREG(PRO, 1); break; \
        case 2: LB_QREG(PRO, 2); break; \
        case 4: LB_QREG(PRO, 4); break; \
        default: LB_QREG(PRO, 8); break; \
    }
        switch (a.pro) {
            case LB_PRO_F32: LB_QREG_PRO(LB_PRO_F32) break;
            case LB_PRO_BLOCKNORM: LB_QREG_PRO(LB_PRO_BLOCKNORM) break;
            case LB_PRO_INNERNORM: LB_QREG_PRO(LB_PRO_INNERNORM) break;
            case LB_PRO_INNERNORM64:
                switch (cpt) {
                    case 1: LB_QREG(LB_PRO_INNERNORM64, 1); break;
                    case 2: LB_QREG(LB_PRO_INNERNORM64, 2); break;
                    default: LB_QREG(LB_PRO_INNERNORM64, 4); break;
                }
                break;
            default: return lb_fail(ctx, LOOM_B200_ERR_INVALID, "gemm_quantize: prologue %d", a.pro);
        }
#undef LB_QREG_PRO
#undef LB_QREG
        LB_CUDA(ctx, qerr);
        ctx->launches++;
        return 0;
    }
    const size_t qsmem = (size_t)a.K * (a.pro == LB_PRO_INNERNORM64 ? 8 : 4);
    LB_REQUIRE(ctx, qsmem <= 200 * 1024, "gemm_quantize: rows of %d columns do not fit in shared memory", a.K);
    if (!(ctx->func_attr_mask & (1u << 25))) {
        LB_CUDA(ctx, cudaFuncSetAttribute(lb_quantize_gemm_kernel<LB_PRO_F32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        LB_CUDA(ctx, cudaFuncSetAttribute(lb_quantize_gemm_kernel<LB_PRO_BLOCKNORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        LB_CUDA(ctx, cudaFuncSetAttribute(lb_quantize_gemm_kernel<LB_PRO_INNERNORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        LB_CUDA(ctx, cudaFuncSetAttribute(lb_quantize_gemm_kernel<LB_PRO_INNERNORM64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        ctx->func_attr_mask |= 1u << 25;
    }
    switch (a.pro) {
        case LB_PRO_F32: lb_quantize_gemm_kernel<LB_PRO_F32><<<pt, 256, qsmem, ctx->stream>>>(a, Kp, g.q, g.amax, g.xsum); break;
        case LB_PRO_BLOCKNORM: lb_quantize_gemm_kernel<LB_PRO_BLOCKNORM><<<pt, 256, qsmem, ctx->stream>>>(a, Kp, g.q, g.amax, g.xsum); break;
        case LB_PRO_INNERNORM: lb_quantize_gemm_kernel<LB_PRO_INNERNORM><<<pt, 256, qsmem, ctx->stream>>>(a, Kp, g.q, g.amax, g.xsum); break;
        case LB_PRO_INNERNORM64: lb_quantize_gemm_kernel<LB_PRO_INNERNORM64><<<pt, 256, qsmem, ctx->stream>>>(a, Kp, g.q, g.amax, g.xsum); break;
        default: return lb_fail(ctx, LOOM_B200_ERR_INVALID, "gemm_quantize: prologue %d", a.pro);
    }
    LB_CHECK_LAUNCH(ctx, "lb_quantize_gemm_kernel");
    ctx->launches++;
    return 0;
}

const float* lb_gemm_last_amax(loom_b200_ctx* ctx, int tokens, int K) {
    const int Kp = (K + kTileCols - 1) / kTileCols * kTileCols;
    return gemm_scratch_at(ctx->gemm_scratch, tokens, Kp).amax;
}

// Builds the pre-expanded codes of a matrix on first use (4x its packed bytes).  Returns false when the cache is switched
// off, cannot be built while a graph is being recorded, or does not fit: the caller then expands inside the kernel.
static bool gemm_ensure_codes(loom_b200_ctx* ctx, const loom_b200_weight* wc) {
    if (!ctx->opt_gemm_cache) return false;
    if (wc->codes8) return true;
    if (ctx->capturing) return false;
    loom_b200_weight* w = const_cast<loom_b200_weight*>(wc);  // a cache: the matrix itself does not change
    const int row_blocks = (w->strips + 7) / 8;
    const size_t bytes = (size_t)row_blocks * w->kblocks * kSliceBytesA;
    size_t free_b = 0, total_b = 0;
    if (cudaMemGetInfo(&free_b, &total_b) != cudaSuccess || free_b < bytes + (total_b >> 3)) {  // keep an eighth of the device free
        cudaGetLastError();
        return false;
    }
    uint8_t* c = nullptr;
    if (cudaMalloc(&c, bytes) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    const size_t threads = (size_t)row_blocks * w->kblocks * 128 * 8;
    lb_expand_codes_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, ctx->stream>>>(w->tiles, w->strips, w->kblocks, c);
    if (cudaGetLastError() != cudaSuccess) {
        cudaFree(c);
        return false;
    }
    ctx->launches++;
    w->codes8 = c;
    ctx->gemm_codes_fresh = true;  // the next GEMM launch reads these before its dependency wait: it must not start early
    return true;
}

template <int NTOK, int MODE>
static int gemm_launch(loom_b200_ctx* ctx, const GemmParams& p, dim3 grid, unsigned attr_bit) {
    using Cfg = GemmCfg<NTOK, MODE>;
    if (!(ctx->func_attr_mask2 & attr_bit)) {
        LB_CUDA(ctx, cudaFuncSetAttribute(lb_gemm_ternary_i8_kernel<NTOK, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::kSmem));
        ctx->func_attr_mask2 |= attr_bit;
    }
    lb_gemm_ternary_i8_kernel<NTOK, MODE><<<grid, kGemmThreads, Cfg::kSmem, ctx->stream>>>(p);
    LB_CHECK_LAUNCH(ctx, "lb_gemm_ternary_i8_kernel");
    ctx->launches++;
    return 0;
}

// the persistent kernel: one CTA per SM (or per tile, if there are fewer tiles)
template <int NTOK, bool DUAL>
static int gemm_launch_stream(loom_b200_ctx* ctx, const GemmParams& p, unsigned attr_bit) {
    using Cfg = StreamCfg<NTOK, DUAL>;
    if (!(ctx->func_attr_mask2 & attr_bit)) {
        LB_CUDA(ctx, cudaFuncSetAttribute(lb_gemm_stream_kernel<NTOK, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::kSmem));
        ctx->func_attr_mask2 |= attr_bit;
    }
    const int row_tiles = (p.rows + kRowsPerCta - 1) / kRowsPerCta;
    const int ntiles = row_tiles * ((p.tokens + NTOK - 1) / NTOK);
    const int grid = ntiles < ctx->sm_count ? ntiles : ctx->sm_count;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = Cfg::kSmem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    // (a launch that follows the build of its code cache starts only when that build is complete and visible)
    cfg.numAttrs = ctx->opt_pdl && !ctx->gemm_codes_fresh ? 1 : 0;
    ctx->gemm_codes_fresh = false;
    LB_CUDA(ctx, cudaLaunchKernelEx(&cfg, lb_gemm_stream_kernel<NTOK, DUAL>, p, row_tiles, ntiles));
    ctx->launches++;
    return 0;
}

int lb_gemm_run(loom_b200_ctx* ctx, const loom_b200_weight* w, int tokens, const LbGemmOut& o) {
    LB_REQUIRE(ctx, w && tokens > 0 && (o.out || o.out_f64 || o.acc_out), "gemm_run: bad arguments");
    LB_REQUIRE(ctx, w->device == ctx->device, "ternary_gemm: weight lives on device %d, context on %d", w->device, ctx->device);
    const int Kp = w->kblocks * kTileCols;
    LB_REQUIRE(ctx, (size_t)padded_tokens(tokens) * Kp <= ctx->gemm_scratch_bytes, "gemm_run: no quantized activations for %d tokens of %d columns", tokens, w->cols);
    GemmScratch g = gemm_scratch_at(ctx->gemm_scratch, tokens, Kp);
    GemmParams p = {};
    p.tiles = w->tiles;
    p.rows = w->rows;
    p.strips = w->strips;
    p.kblocks = w->kblocks;
    p.scale = w->scale;
    p.q = g.q;
    p.amax = g.amax;
    p.xsum = g.xsum;
    p.tokens = tokens;
    p.Kp = Kp;
    p.bias = o.bias;
    p.residual = o.residual;
    p.act = o.act;
    p.out = o.out;
    p.out_f64 = o.out_f64;
    p.pre_out = o.pre_out;
    p.acc_out = o.acc_out;
    p.kv_hd = o.kv_hd;
    p.kv_msl = o.kv_msl;
    p.kv_pos0 = o.kv_pos0;
    p.status = ctx->status_dev;
    // phase trace: one row for the kernel and one per k-slice, kept contiguous (skipped if the ring of rows would wrap)
    p.trace = nullptr;
    if (ctx->trace_dev && (ctx->trace_seq % kTraceSlots) + w->kblocks + 2 < kTraceSlots) {
        p.trace = lb_trace_row(ctx, "gemm");
        for (int i = 0; i < w->kblocks; ++i) lb_trace_row(ctx, "gemm-slice");
    }
    // Tokens per CTA: 256 halves the weight expansion per MMA but also the number of CTAs; take the variant with the
    // smaller (waves x relative tile time), a 256-token tile costing about 1.6 times a 128-token one.
    const int row_tiles = (w->rows + kRowsPerCta - 1) / kRowsPerCta;
    const int ct128 = row_tiles * ((tokens + 127) / 128), ct256 = row_tiles * ((tokens + 255) / 256);
    const int sms = ctx->sm_count;
    const double cost128 = (double)((ct128 + sms - 1) / sms), cost256 = 1.6 * (double)((ct256 + sms - 1) / sms);
    bool wide = tokens > 128 && cost256 < cost128;
    if (ctx->opt_gemm_tile == 128) wide = false;
    if (ctx->opt_gemm_tile == 256) wide = true;
    const bool cached = gemm_ensure_codes(ctx, w);
    p.codes8 = w->codes8;
    // Split-K when the output tiles alone would leave more than half of the SMs idle: up to eight CTAs share a tile,
    // each at least four k-slices deep; their int32 partial sums meet in a zero-initialised scratch (exact).
    const int tiles = wide ? ct256 : ct128;
    int splits = 1;
    if (ctx->opt_gemm_splitk && tiles * 2 <= sms) {
        splits = sms / tiles;
        if (splits > w->kblocks / 4) splits = w->kblocks / 4;
        if (splits > 8) splits = 8;
        if (splits < 1) splits = 1;
        // measured: a k-slice costs a CTA about 0.5 us, the atomic hand-over of a split about 0.15 us per token of the tile + 2 us
        const int tile_tokens = tokens < (wide ? 256 : 128) ? tokens : (wide ? 256 : 128);
        if (splits > 1 && 0.5 * w->kblocks * (1.0 - 1.0 / splits) <= 0.15 * tile_tokens + 2.0) splits = 1;
    }
    if (splits > 1) {
        if (int rc = lb_ensure_fixup(ctx, (size_t)tokens * w->rows, (size_t)tiles)) return rc;
        p.part_acc = ctx->fix_acc;
        p.part_cnt = ctx->fix_cnt;
    }
    if (cached && splits == 1 && !p.trace && ctx->opt_gemm_stream) {
        // persistent kernel: a tile's time follows the bytes its stages load (32 KB per slice for 128 tokens, 48 KB for
        // 256), the launch's time the tiles of the busiest CTA
        bool wide_s = tokens > 128 && 48 * ((ct256 + sms - 1) / sms) <= 32 * ((ct128 + sms - 1) / sms);
        if (ctx->opt_gemm_tile == 128) wide_s = false;
        if (ctx->opt_gemm_tile == 256) wide_s = true;
        return wide_s ? gemm_launch_stream<256, false>(ctx, p, 1u << 26) : gemm_launch_stream<128, false>(ctx, p, 1u << 27);
    }
    if (wide) {
        dim3 grid(row_tiles, (tokens + 255) / 256, splits);
        return cached ? gemm_launch<256, GEMM_CACHED>(ctx, p, grid, 1u << 20) : gemm_launch<256, GEMM_EXPAND>(ctx, p, grid, 1u << 21);
    }
    dim3 grid(row_tiles, (tokens + 127) / 128, splits);
    return cached ? gemm_launch<128, GEMM_CACHED>(ctx, p, grid, 1u << 22) : gemm_launch<128, GEMM_EXPAND>(ctx, p, grid, 1u << 23);
}

// gate and up projections of the block quantized last, fused with the gate product: prod [tokens, inter] float32.  Returns
// LOOM_B200_ERR_UNSUPPORTED (without touching last_error's meaning for the caller) when the pre-expanded codes are not
// available; the caller then runs the two projections and the gate-product kernel.
int lb_gemm_run_swiglu(loom_b200_ctx* ctx, const loom_b200_weight* gate, const loom_b200_weight* up, int tokens, const float* bias_g,
                       const float* bias_u, int act, float* prod) {
    LB_REQUIRE(ctx, gate && up && tokens > 0 && prod, "gemm_run_swiglu: bad arguments");
    LB_REQUIRE(ctx, gate->rows == up->rows && gate->cols == up->cols, "gemm_run_swiglu: gate %dx%d and up %dx%d differ", gate->rows, gate->cols, up->rows, up->cols);
    if (!ctx->opt_gemm_stream || !gemm_ensure_codes(ctx, gate) || !gemm_ensure_codes(ctx, up)) return LOOM_B200_ERR_UNSUPPORTED;
    const int Kp = gate->kblocks * kTileCols;
    LB_REQUIRE(ctx, (size_t)padded_tokens(tokens) * Kp <= ctx->gemm_scratch_bytes, "gemm_run_swiglu: no quantized activations for %d tokens of %d columns", tokens, gate->cols);
    GemmScratch g = gemm_scratch_at(ctx->gemm_scratch, tokens, Kp);
    GemmParams p = {};
    p.tiles = gate->tiles;
    p.codes8 = gate->codes8;
    p.codes8_up = up->codes8;
    p.rows = gate->rows;
    p.strips = gate->strips;
    p.kblocks = gate->kblocks;
    p.scale = gate->scale;
    p.scale_up = up->scale;
    p.q = g.q;
    p.amax = g.amax;
    p.xsum = g.xsum;
    p.tokens = tokens;
    p.Kp = Kp;
    p.bias = bias_g;
    p.bias_up = bias_u;
    p.act = act;
    p.out = prod;
    p.status = ctx->status_dev;
    // 128 tokens per tile: two accumulators of 128 columns in each of the two TMEM buffers
    return gemm_launch_stream<128, true>(ctx, p, 1u << 25);
}

int lb_gemm_gate_product(loom_b200_ctx* ctx, const int32_t* acc_g, const int32_t* acc_u, int tokens, int inter, int K, float scale_g,
                         float scale_u, const float* bias_g, const float* bias_u, int act, float* prod) {
    const size_t n = (size_t)tokens * inter;
    lb_gate_product_acc_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(acc_g, acc_u, lb_gemm_last_amax(ctx, tokens, K), tokens, inter,
                                                                                      scale_g, scale_u, bias_g, bias_u, act, prod);
    LB_CHECK_LAUNCH(ctx, "lb_gate_product_acc_kernel");
    ctx->launches++;
    return 0;
}

extern "C" int loom_b200_selftest_i8_peak(loom_b200_ctx* ctx, int iters, double* tops_out) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "selftest_i8_peak: ctx is NULL");
    LB_REQUIRE(ctx, iters >= 1 && iters <= 1000000 && tops_out, "selftest_i8_peak: bad arguments");
    if (ctx->capturing) return lb_fail(ctx, LOOM_B200_ERR_INVALID, "selftest_i8_peak cannot be recorded");
    if (int rc = lb_set_device(ctx)) return rc;
    const size_t smem = kSliceBytesA + 256 * kSliceK + 1024;
    LB_CUDA(ctx, cudaFuncSetAttribute(lb_i8_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    cudaEvent_t e0, e1;
    LB_CUDA(ctx, cudaEventCreate(&e0));
    LB_CUDA(ctx, cudaEventCreate(&e1));
    lb_i8_peak_kernel<<<ctx->sm_count, 128, smem, ctx->stream>>>(iters / 8 + 1, ctx->status_dev);  // warm-up
    LB_CUDA(ctx, cudaEventRecord(e0, ctx->stream));
    lb_i8_peak_kernel<<<ctx->sm_count, 128, smem, ctx->stream>>>(iters, ctx->status_dev);
    LB_CUDA(ctx, cudaEventRecord(e1, ctx->stream));
    LB_CHECK_LAUNCH(ctx, "lb_i8_peak_kernel");
    if (int rc = lb_sync_checked(ctx)) return rc;
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    *tops_out = 2.0 * 128.0 * 256.0 * 32.0 * 4.0 * (double)iters * ctx->sm_count / ((double)ms * 1e-3) / 1e12;
    return 0;
}

int lb_ternary_gemm(loom_b200_ctx* ctx, const loom_b200_weight* w, int tokens, const float* x, const float* bias,
                    const float* residual, int activation, float* out, float* pre_out, int32_t* acc_out, float* amax_out);

extern "C" int loom_b200_ternary_gemm(loom_b200_ctx* ctx, const loom_b200_weight* w, int tokens, const float* x, const float* bias,
                                      const float* residual, int activation, float* out, int32_t* acc_out, float* amax_out) {
    return lb_ternary_gemm(ctx, w, tokens, x, bias, residual, activation, out, nullptr, acc_out, amax_out);
}

int lb_ternary_gemm(loom_b200_ctx* ctx, const loom_b200_weight* w, int tokens, const float* x, const float* bias,
                    const float* residual, int activation, float* out, float* pre_out, int32_t* acc_out, float* amax_out) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "ternary_gemm: ctx is NULL");
    LB_REQUIRE(ctx, w != nullptr, "ternary_gemm: weight is NULL");
    LB_REQUIRE(ctx, tokens >= 0, "ternary_gemm: tokens=%d", tokens);
    if (tokens == 0) return 0;
    LB_REQUIRE(ctx, x && (out || acc_out), "ternary_gemm: NULL buffer");
    if (int rc = lb_set_device(ctx)) return rc;
    LbGemmQuant qa = {};
    qa.pro = LB_PRO_F32;
    qa.x = x;
    qa.K = w->cols;
    qa.tokens = tokens;
    if (int rc = lb_gemm_quantize(ctx, qa)) return rc;
    LbGemmOut o = {};
    o.bias = bias;
    o.residual = residual;
    o.act = activation;
    o.out = out;
    o.pre_out = pre_out;
    o.acc_out = acc_out;
    if (int rc = lb_gemm_run(ctx, w, tokens, o)) return rc;
    if (amax_out)
        LB_CUDA(ctx, cudaMemcpyAsync(amax_out, lb_gemm_last_amax(ctx, tokens, w->cols), (size_t)tokens * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
    return 0;
}
