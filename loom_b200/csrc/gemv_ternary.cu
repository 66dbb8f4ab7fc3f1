// gemv_ternary.cu -- packed-ternary x int8 decode GEMV for sm_100a.
//
// Replaces ShaderTiledDenseBitNetTernaryQuantizedReduce (poly/wgpu_shaders.go:512-642) and, through its
// fused prologues/epilogues, the quantize, gate-product, inner-norm and residual dispatches around it
// (poly/wgpu_forward.go:167-180,257-281,367-389,420-428).  Arithmetic contract: poly/bitnet_cpu.go:45-106,
// 536-546,752-776.
//
// Shape of the kernel
//   * The weight stream is the only real traffic (2 bits per weight); everything else is per-token vectors.
//     Tiles (16 rows x 128 columns, 512 B) are laid out so that a warp's slice of the matrix is contiguous.
//   * Stream-K: the virtual tile list (strips x k-blocks) is cut into equal contiguous ranges, one per CTA,
//     and again into eight per-warp ranges.  Each warp streams its range through a private ring of shared
//     memory stages filled by 1-D bulk async copies (TMA engine) that complete on mbarriers; the first ring
//     fill is issued before griddepcontrol.wait, so under programmatic dependent launch the weights of
//     launch i+1 are already in flight while launch i finishes.
//   * Integer dot products: a lane holds four reference words (2 rows x 2 column groups).  Masking a word
//     with 0x03030303 << 2j leaves, in each byte, 4^j * code of one column; the four masked registers of a
//     lane are exactly an m16n8k32 u8 x s8 MMA A-fragment, with up to eight tokens in the N dimension.
//     Accumulators are kept per j and shifted back (exactly) at the end; sum(code*x) - sum(x) = sum(w*x).
//     A dp4a variant of the same loop is kept for comparison (batch 1 only).
//   * Partial strips are combined through int32 atomics in a zero-initialised scratch; the CTA that
//     completes a strip group runs the float64 epilogue and clears what it used.  Integer addition is
//     associative, so the result is bit-identical to the sequential CPU loop whatever the arrival order.
#include "gemv_ternary.cuh"

#include <type_traits>


namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kStageTiles = 8;                          // tiles per ring stage (4 KB)
constexpr int kStages = 3;                              // most stages per warp (the launch picks 1..3)
constexpr int kStageBytes = kStageTiles * kTileBytes;   // 4096
constexpr int kMaxM = 8;

__device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ int dp4a_u8s8(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

#define LB_TRACE(k) lb_trace(p.trace, (k))

struct Smem {
    uint8_t* ring;
    uint32_t* acts;   // M rows of (Kp+16) bytes, then a 32-byte zero block
    int* sacc;        // [local strip][token][16]
    int* xsum;        // [8]
    float* amax;      // [8]
    double* os;       // [3][8] output scale per segment and token
    double* red;      // [32]
    int* flag;        // [4]
    uint64_t* bars;   // [kWarps*kStages]
    void* stage;      // K floats (doubles for fp64 input) of prologue staging, or null
};

__device__ __forceinline__ const uint32_t* tile_ptr(const LbGemvParams& p, int v, int kb) {
    int s, local;
    if (p.interleave2) {
        s = v & 1;
        local = v >> 1;
    } else {
        s = 0;
        if (p.nseg > 1 && v >= p.seg[1].vstrip0) s = 1;
        if (p.nseg > 2 && v >= p.seg[2].vstrip0) s = 2;
        local = v - p.seg[s].vstrip0;
    }
    return p.seg[s].tiles + ((size_t)local * p.kblocks + kb) * kTileWords;
}

__device__ __forceinline__ double block_sum(double v, double* red) {
    v = lb_warp_sum(v);
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    double r = 0.0;
#pragma unroll
    for (int i = 0; i < kWarps; ++i) r += red[i];
    return r;
}

__device__ __forceinline__ float block_max(float v, double* red) {
    v = lb_warp_max(v);
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* rf = reinterpret_cast<float*>(red + 16);
    __syncthreads();
    if (lane == 0) rf[warp] = v;
    __syncthreads();
    float r = rf[0];
#pragma unroll
    for (int i = 1; i < kWarps; ++i) r = fmaxf(r, rf[i]);
    return r;
}

// The value the reference quantizes for column c of token row `row` (already rounded to float32 where the
// reference stores a float32), as a double.
template <int mode>
__device__ __forceinline__ double pro_value(const void* row, int c, double stat, double rstat, const float* nw, int nwlen) {
    if (mode == LB_PRO_INNERNORM64) {
        double w = (nw && c < nwlen) ? (double)nw[c] : 1.0;
        return __dmul_rn(((const double*)row)[c], __dmul_rn(stat, w));
    }
    float x = ((const float*)row)[c];
    if (mode == LB_PRO_F32) return (double)x;
    if (mode == LB_PRO_BLOCKNORM) {
        double g = nw ? (double)nw[c] : 1.0;
        return (double)(float)__dmul_rn(lb_div_by((double)x, stat, rstat), g);
    }
    double w = (nw && c < nwlen) ? (double)nw[c] : 1.0;  // LB_PRO_INNERNORM
    return (double)(float)__dmul_rn(__dmul_rn((double)x, stat), w);
}

// Prologue for fp32/fp64 inputs with K % 4 == 0: the row is copied once from global into a shared staging
// buffer (loads of several units in flight), then normalisation, absmax and quantization run as short rolled
// loops over 4-column units.  Code executed once per CTA is fetched cold, so the loops are kept small and
// reused rather than unrolled; the four columns of a unit give the instruction-level parallelism.
template <int PRO>
__device__ __forceinline__ void stage_row_fast(const LbGemvParams& p, const Smem& sm, int n, const void* row) {
    const int tid = threadIdx.x, K = p.K, units = K >> 2;
    const int Kp = p.kblocks * kTileCols, stride32 = (Kp + 16) / 4;
    constexpr bool f64 = PRO == LB_PRO_INNERNORM64;
    using VT = typename std::conditional<f64, double, float>::type;
    VT* tmp = reinterpret_cast<VT*>(sm.stage);
    const bool have_w = PRO != LB_PRO_F32 && p.norm_w != nullptr;
    double ss = 0.0;
    float m = 0.0f;
#pragma unroll 4
    for (int idx = tid; idx < units; idx += kThreads) {
        VT a0, a1, a2, a3;
        if (f64) {
            const double2 a = reinterpret_cast<const double2*>(row)[2 * idx], b = reinterpret_cast<const double2*>(row)[2 * idx + 1];
            a0 = (VT)a.x; a1 = (VT)a.y; a2 = (VT)b.x; a3 = (VT)b.y;
        } else {
            const float4 a = reinterpret_cast<const float4*>(row)[idx];
            a0 = (VT)a.x; a1 = (VT)a.y; a2 = (VT)a.z; a3 = (VT)a.w;
        }
        if (have_w && 4 * idx < p.norm_w_len) asm volatile("prefetch.global.L1 [%0];" ::"l"(p.norm_w + 4 * idx));
        tmp[4 * idx] = a0; tmp[4 * idx + 1] = a1; tmp[4 * idx + 2] = a2; tmp[4 * idx + 3] = a3;
        if (PRO >= LB_PRO_BLOCKNORM) {
            ss = __dadd_rn(ss, __dmul_rn((double)a0, (double)a0));
            ss = __dadd_rn(ss, __dmul_rn((double)a1, (double)a1));
            ss = __dadd_rn(ss, __dmul_rn((double)a2, (double)a2));
            ss = __dadd_rn(ss, __dmul_rn((double)a3, (double)a3));
        } else {
            m = fmaxf(fmaxf(m, fabsf((float)a0)), fmaxf(fabsf((float)a1), fmaxf(fabsf((float)a2), fabsf((float)a3))));
        }
    }
    if (PRO >= LB_PRO_BLOCKNORM) {
        ss = block_sum(ss, sm.red);
        const double mean = __dadd_rn(__ddiv_rn(ss, (double)K), p.eps);
        const double root = sqrt(mean);
        const double rr = __ddiv_rn(1.0, root);  // RN(1/rms): the inner norms' scale, the block norm's reciprocal
#pragma unroll 1
        for (int idx = tid; idx < units; idx += kThreads) {
            double w[4] = {1.0, 1.0, 1.0, 1.0};
            if (have_w) {
                if (4 * idx + 4 <= p.norm_w_len) {
                    const float4 g = reinterpret_cast<const float4*>(p.norm_w)[idx];
                    w[0] = (double)g.x; w[1] = (double)g.y; w[2] = (double)g.z; w[3] = (double)g.w;
                } else {
                    for (int k = 0; k < 4; ++k)
                        if (4 * idx + k < p.norm_w_len) w[k] = (double)p.norm_w[4 * idx + k];
                }
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const double x = (double)tmp[4 * idx + k];
                VT y;
                if (PRO == LB_PRO_BLOCKNORM) y = (VT)(float)__dmul_rn(lb_div_by(x, root, rr), w[k]);
                else if (f64) y = (VT)__dmul_rn(x, __dmul_rn(rr, w[k]));
                else y = (VT)(float)__dmul_rn(__dmul_rn(x, rr), w[k]);
                tmp[4 * idx + k] = y;
                m = fmaxf(m, (float)fabs((double)y));
            }
        }
    }
    m = block_max(m, sm.red);
    const float amax = m < 1e-5f ? 1e-5f : m;
    const double s = __ddiv_rn(127.0, (double)amax);
    const bool side = blockIdx.x == 0;
    int local_sum = 0;
    uint8_t* abytes = reinterpret_cast<uint8_t*>(sm.acts + (size_t)n * stride32);
#pragma unroll 1
    for (int idx = tid; idx < (Kp >> 2); idx += kThreads) {
        int q0 = 0, q1 = 0, q2 = 0, q3 = 0;
        if (idx < units) {
            const VT y0 = tmp[4 * idx], y1 = tmp[4 * idx + 1], y2 = tmp[4 * idx + 2], y3 = tmp[4 * idx + 3];
            q0 = lb_quant_i8((double)y0, s);
            q1 = lb_quant_i8((double)y1, s);
            q2 = lb_quant_i8((double)y2, s);
            q3 = lb_quant_i8((double)y3, s);
            local_sum += q0 + q1 + q2 + q3;
            if (side) {
                if (p.q_out)
                    reinterpret_cast<uint32_t*>(p.q_out + (size_t)n * K)[idx] =
                        (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) | ((uint32_t)(q3 & 0xff) << 24);
                if (p.norm_out)
                    reinterpret_cast<float4*>(p.norm_out + (size_t)n * K)[idx] = make_float4((float)y0, (float)y1, (float)y2, (float)y3);
            }
        }
        // unit idx = word r_b of 16-column chunk i: byte j of r_b is byte b of B_j (columns >= K stay zero)
        const int i = idx >> 2, b = idx & 3;
        const int kb = i >> 3, w8 = i & 7, h = w8 >> 2, t = w8 & 3;
        uint8_t* dst = abytes + (size_t)(kb * 32 + t * 8 + h) * 4 + b;
        dst[0] = (uint8_t)q0;
        dst[8] = (uint8_t)q1;
        dst[16] = (uint8_t)q2;
        dst[24] = (uint8_t)q3;
    }
    local_sum = lb_warp_sum_i(local_sum);
    if ((tid & 31) == 0 && local_sum != 0) atomicAdd(&sm.xsum[n], local_sum);
    if (tid < 3) sm.os[tid * kMaxM + n] = tid < p.nseg ? lb_output_scale(p.seg[tid].scale, amax) : 1.0;
    if (tid == 0) {
        sm.amax[n] = amax;
        if (side && p.amax_out) p.amax_out[n] = amax;
    }
    __syncthreads();  // the staging buffer is reused by the next token
}

// Quantizes the M activation rows into shared memory in the k-slot order the MMA B-fragments use, and
// leaves sum(q) and amax per token in shared memory.
template <int PRO>
__device__ __forceinline__ void stage_activations(const LbGemvParams& p, const Smem& sm) {
    const int tid = threadIdx.x;
    const int K = p.K, Kp = p.kblocks * kTileCols;
    const int stride32 = (Kp + 16) / 4;
    const int chunks = Kp / 16;
    if (tid < kMaxM) sm.xsum[tid] = 0;
    if (tid < 8) sm.acts[p.M * stride32 + tid] = 0;  // zero block for the lanes of absent tokens
    for (int n = 0; n < p.M; ++n) {
        constexpr bool q8 = PRO == LB_PRO_Q8;
        const void* row = q8 ? (const void*)((const int8_t*)p.x + (size_t)n * K)
                             : (PRO == LB_PRO_INNERNORM64 ? (const void*)((const double*)p.x + (size_t)n * K)
                                                            : (const void*)((const float*)p.x + (size_t)n * K));
        if (!q8) {
            const bool aligned16 = (((uintptr_t)row) & 15) == 0 && (!p.norm_w || (((uintptr_t)p.norm_w) & 15) == 0) &&
                                   (!p.norm_out || (((uintptr_t)p.norm_out) & 15) == 0) && (!p.q_out || (((uintptr_t)p.q_out) & 3) == 0);
            if ((K & 3) == 0 && sm.stage && aligned16) {
                stage_row_fast<PRO == LB_PRO_Q8 ? LB_PRO_F32 : PRO>(p, sm, n, row);
                continue;
            }
        }
        double stat = 0.0, rstat = 0.0;  // rms (or 1/rms for the inner norms) and, for the block norm, RN(1/rms)
        float amax;
        if (q8) {
            amax = p.amax_in[n];
        } else {
            if (PRO >= LB_PRO_BLOCKNORM) {
                double ss = 0.0;
                if (PRO == LB_PRO_INNERNORM64) {
                    for (int c = tid; c < K; c += kThreads) {
                        double v = ((const double*)row)[c];
                        ss = __dadd_rn(ss, __dmul_rn(v, v));
                    }
                } else {
                    for (int c = tid; c < K; c += kThreads) {
                        double v = (double)((const float*)row)[c];
                        ss = __dadd_rn(ss, __dmul_rn(v, v));
                    }
                }
                ss = block_sum(ss, sm.red);
                double mean = __dadd_rn(__ddiv_rn(ss, (double)K), p.eps);
                stat = PRO == LB_PRO_BLOCKNORM ? sqrt(mean) : __ddiv_rn(1.0, sqrt(mean));
                if (PRO == LB_PRO_BLOCKNORM) rstat = __ddiv_rn(1.0, stat);
            }
            float m = 0.0f;
            for (int c = tid; c < K; c += kThreads)
                m = fmaxf(m, (float)fabs(pro_value<PRO>(row, c, stat, rstat, p.norm_w, p.norm_w_len)));
            m = block_max(m, sm.red);
            amax = m < 1e-5f ? 1e-5f : m;
        }
        const double s = __ddiv_rn(127.0, (double)amax);
        const bool side = blockIdx.x == 0;
        int local_sum = 0;
        const bool vec_ok = q8 && ((((uintptr_t)row) & 15) == 0);
        for (int i = tid; i < chunks; i += kThreads) {
            uint32_t r[4] = {0u, 0u, 0u, 0u};
            const int c0 = i * 16;
            if (q8) {
                if (vec_ok && c0 + 16 <= K) {
                    uint4 v = *reinterpret_cast<const uint4*>((const int8_t*)row + c0);
                    r[0] = v.x; r[1] = v.y; r[2] = v.z; r[3] = v.w;
                } else {
                    for (int k = 0; k < 16; ++k)
                        if (c0 + k < K) r[k >> 2] |= (uint32_t)(uint8_t)((const int8_t*)row)[c0 + k] << (8 * (k & 3));
                }
            } else {
                for (int k = 0; k < 16; ++k) {
                    int c = c0 + k;
                    if (c < K) {
                        double v = pro_value<PRO>(row, c, stat, rstat, p.norm_w, p.norm_w_len);
                        int q = lb_quant_i8(v, s);
                        r[k >> 2] |= (uint32_t)(q & 0xff) << (8 * (k & 3));
                        if (side) {
                            if (p.q_out) p.q_out[(size_t)n * K + c] = (int8_t)q;
                            if (p.norm_out) p.norm_out[(size_t)n * K + c] = (float)v;
                        }
                    }
                }
            }
#pragma unroll
            for (int b = 0; b < 4; ++b) local_sum = __dp4a((int)r[b], 0x01010101, local_sum);
            // 4x4 byte transpose: B_j = { byte j of r0, r1, r2, r3 }
            uint32_t t0 = __byte_perm(r[0], r[1], 0x5140), t1 = __byte_perm(r[2], r[3], 0x5140);
            uint32_t t2 = __byte_perm(r[0], r[1], 0x7362), t3 = __byte_perm(r[2], r[3], 0x7362);
            uint32_t B0 = __byte_perm(t0, t1, 0x5410), B1 = __byte_perm(t0, t1, 0x7632);
            uint32_t B2 = __byte_perm(t2, t3, 0x5410), B3 = __byte_perm(t2, t3, 0x7632);
            const int kb = i >> 3, w8 = i & 7, h = w8 >> 2, t = w8 & 3;
            uint32_t* dst = sm.acts + (size_t)n * stride32 + kb * 32 + t * 8 + h;
            dst[0] = B0; dst[2] = B1; dst[4] = B2; dst[6] = B3;
        }
        local_sum = lb_warp_sum_i(local_sum);
        if ((tid & 31) == 0 && local_sum != 0) atomicAdd(&sm.xsum[n], local_sum);
        if (tid < 3) sm.os[tid * kMaxM + n] = tid < p.nseg ? lb_output_scale(p.seg[tid].scale, amax) : 1.0;
        if (tid == 0) {
            sm.amax[n] = amax;
            if (side && p.amax_out) p.amax_out[n] = amax;
        }
    }
    __syncthreads();
}

// Activations other than linear/ReLU/ReLU2 pull in transcendental code: keep it out of the straight-line path.
__device__ __noinline__ float activate_slow(float v, int act) { return lb_activate(v, act); }

__device__ __forceinline__ size_t out_index(const LbGemvParams& p, const LbGemvSeg& sg, int n, int r) {
    if (sg.out_ring > 0) return (size_t)((*p.pos_ptr + n) % sg.out_ring) * sg.rows + r;
    return (size_t)n * sg.rows + r;
}

// Epilogue of one finished row (or gate/up row pair).  vals = [group][M][16] complete sums of sum(code*x).
template <int EPI>
__device__ __forceinline__ void finish_row(const LbGemvParams& p, const Smem& sm, int group_first_vstrip, int e, int n,
                                           int i, const int* vals) {
    const int M = p.M;
    if (EPI == LB_EPI_SWIGLU) {
        if (e != 0) return;  // pairs are finished from the gate side
        const int r = (group_first_vstrip >> 1) * kTileRows + i;
        const LbGemvSeg& sg = p.seg[0];
        const LbGemvSeg& su = p.seg[1];
        if (r >= sg.rows) return;
        const int ag = vals[(0 * M + n) * 16 + i] - sm.xsum[n];
        const int au = vals[(1 * M + n) * 16 + i] - sm.xsum[n];
        double yg = __dmul_rn((double)ag, sm.os[0 * kMaxM + n]);
        double yu = __dmul_rn((double)au, sm.os[1 * kMaxM + n]);
        if (sg.bias) yg = __dadd_rn(yg, (double)sg.bias[r]);
        if (su.bias) yu = __dadd_rn(yu, (double)su.bias[r]);
        ((float*)sg.out)[(size_t)n * sg.rows + r] = (float)lb_gate_product(yg, yu, p.act);
        return;
    }
    const int v = group_first_vstrip + e;
    int s = 0;
    if (EPI == LB_EPI_QKV || EPI == LB_EPI_GENERIC) {
        if (p.nseg > 1 && v >= p.seg[1].vstrip0) s = 1;
        if (p.nseg > 2 && v >= p.seg[2].vstrip0) s = 2;
    }
    const LbGemvSeg& sg = p.seg[s];
    const int r = (v - sg.vstrip0) * kTileRows + i;
    if (r >= sg.rows) return;
    const int acc = vals[(e * M + n) * 16 + i] - sm.xsum[n];
    if (EPI == LB_EPI_GENERIC) {
        const size_t o = (size_t)n * sg.rows + r;
        if (sg.acc_out) sg.acc_out[o] = acc;
        if (sg.kind == LB_OUT_ACC || !sg.out) return;
    }
    double y = __dmul_rn((double)acc, sm.os[s * kMaxM + n]);
    if (sg.bias) y = __dadd_rn(y, (double)sg.bias[r]);
    if (EPI == LB_EPI_QKV) {
        const size_t o = out_index(p, sg, n, r);
        if (s == 0) ((double*)sg.out)[o] = y;
        else ((float*)sg.out)[o] = (float)y;
        return;
    }
    if (EPI == LB_EPI_RESID) {
        const size_t o = (size_t)n * sg.rows + r;
        float f = (float)y;
        if (p.residual) f = __fadd_rn(f, p.residual[o]);
        ((float*)sg.out)[o] = f;
        return;
    }
    // generic: per-segment kind, any activation, optional pre-activation copy
    const size_t o = (size_t)n * sg.rows + r;
    if (sg.kind == LB_OUT_F64) {
        ((double*)sg.out)[o] = y;
        return;
    }
    float f = (float)y;
    if (sg.pre_out) sg.pre_out[o] = f;
    if (p.act == LOOM_B200_ACT_RELU) f = f < 0.f ? 0.f : f;
    else if (p.act == LOOM_B200_ACT_RELU2) f = f < 0.f ? 0.f : __fmul_rn(f, f);
    else if (p.act != LOOM_B200_ACT_LINEAR) f = activate_slow(f, p.act);
    if (p.residual && s == 0) f = __fadd_rn(f, p.residual[o]);
    ((float*)sg.out)[o] = f;
}

template <bool MMA, int PRO, int EPI>
__global__ void __launch_bounds__(kThreads, 2) lb_gemv_ternary_kernel(const __grid_constant__ LbGemvParams p) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int KB = p.kblocks, M = p.M;
    const int Kp = KB * kTileCols;
    const int stride32 = (Kp + 16) / 4;

    Smem sm;
    {
        uint8_t* ptr = smem_raw;
        sm.ring = ptr;
        ptr += (size_t)kWarps * p.stages * kStageBytes;
        sm.acts = reinterpret_cast<uint32_t*>(ptr);
        ptr += (size_t)(M * stride32 + 8) * 4;
        ptr = reinterpret_cast<uint8_t*>(((uintptr_t)ptr + 15) & ~(uintptr_t)15);
        sm.sacc = reinterpret_cast<int*>(ptr);
        ptr += (size_t)p.max_local_strips * M * 16 * 4;
        sm.xsum = reinterpret_cast<int*>(ptr);
        ptr += 32;
        sm.amax = reinterpret_cast<float*>(ptr);
        ptr += 32;
        sm.red = reinterpret_cast<double*>(ptr);
        ptr += 256;
        sm.os = reinterpret_cast<double*>(ptr);
        ptr += 3 * kMaxM * 8;
        sm.flag = reinterpret_cast<int*>(ptr);
        ptr += 16;
        sm.bars = reinterpret_cast<uint64_t*>(ptr);
        ptr += kWarps * kStages * 8;
        sm.stage = p.stage_bytes > 0 ? (void*)ptr : nullptr;
    }

    // ---- tile ranges --------------------------------------------------------------------------------
    // aligned: every CTA owns whole strip groups (no cross-CTA fix-up); otherwise stream-K over tiles.
    int t0, t1;
    if (p.aligned) {
        const long long NG = p.total_tiles / (p.group * KB);
        t0 = (int)(NG * blockIdx.x / gridDim.x) * p.group * KB;
        t1 = (int)(NG * (blockIdx.x + 1) / gridDim.x) * p.group * KB;
    } else {
        const long long T = p.total_tiles;
        t0 = (int)(T * blockIdx.x / gridDim.x);
        t1 = (int)(T * (blockIdx.x + 1) / gridDim.x);
    }
    const int cta_tiles = t1 - t0;
    const int w0 = t0 + (int)((long long)cta_tiles * warp / kWarps);
    const int w1 = t0 + (int)((long long)cta_tiles * (warp + 1) / kWarps);
    const int first_group = cta_tiles > 0 ? (t0 / KB) / p.group : 0;
    const int local_v0 = first_group * p.group;  // virtual strip held in sacc slot 0

    LB_TRACE(0);
    if (tid < kWarps * kStages) lb_mbar_init(&sm.bars[tid], 1);
    for (int i = tid; i < p.max_local_strips * M * 16; i += kThreads) sm.sacc[i] = 0;
    if (tid == 0) lb_fence_mbar_init();
    __syncthreads();

    const int nstages = p.stages;
    uint8_t* my_ring = sm.ring + (size_t)warp * nstages * kStageBytes;
    uint64_t* my_bars = sm.bars + warp * kStages;

    // Cursors walk the warp's tile range chunk by chunk; a chunk never crosses a strip, so (strip, kblock)
    // advance without any division.
    struct Cursor {
        int pos, v, kb;
    };
    auto chunk_len = [&](const Cursor& c) {
        int len = KB - c.kb;
        if (len > kStageTiles) len = kStageTiles;
        if (len > w1 - c.pos) len = w1 - c.pos;
        return len;
    };
    auto advance = [&](Cursor& c, int len) {
        c.pos += len;
        c.kb += len;
        if (c.kb >= KB) {
            c.kb = 0;
            c.v++;
        }
    };
    auto issue = [&](int stage, const Cursor& c, int len) {  // lane 0 only
        if (p.debug >= 2) return;
        lb_mbar_expect_tx(&my_bars[stage], (uint32_t)len * kTileBytes);
        lb_bulk_g2s(my_ring + (size_t)stage * kStageBytes, tile_ptr(p, c.v, c.kb), (uint32_t)len * kTileBytes,
                    &my_bars[stage]);
    };

    // first ring fill: weights do not depend on the producer of the activations
    Cursor ic;
    ic.pos = w0;
    ic.v = w0 / KB;
    ic.kb = w0 - ic.v * KB;
    Cursor cc = ic;
    for (int s = 0; s < nstages && ic.pos < w1; ++s) {
        int len = chunk_len(ic);
        if (lane == 0) issue(s, ic, len);
        advance(ic, len);
    }

    lb_pdl_launch_dependents();  // the next launch may start prefetching its weights
    LB_TRACE(1);
    lb_pdl_wait();               // everything below may read what earlier launches wrote
    LB_TRACE(2);
    if (p.debug == 3) return;
    stage_activations<PRO>(p, sm);
    LB_TRACE(3);
    if (p.debug == 4) return;

    // ---- main loop ------------------------------------------------------------------------------------
    const int g = lane >> 2, t = lane & 3;
    const uint32_t* act_base;
    int act_kb_mul;
    if (MMA) {
        if (g < M) {
            act_base = sm.acts + (size_t)g * stride32 + t * 8;
            act_kb_mul = 32;
        } else {
            act_base = sm.acts + (size_t)M * stride32;  // zero block
            act_kb_mul = 0;
        }
    } else {
        act_base = sm.acts + t * 8;
        act_kb_mul = 32;
    }

    int acc[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[j][k] = 0;
    int cur_v = -1;
    bool failed = false;

    auto flush = [&]() {
        if (cur_v < 0) return;
        int* dst = sm.sacc + (size_t)(cur_v - local_v0) * M * 16;
        if (MMA) {
            // c0:(row g, n=2t) c1:(row g, n=2t+1) c2:(row g+8, n=2t) c3:(row g+8, n=2t+1)
            int v0 = acc[0][0] + (acc[1][0] >> 2) + (acc[2][0] >> 4) + (acc[3][0] >> 6);
            int v1 = acc[0][1] + (acc[1][1] >> 2) + (acc[2][1] >> 4) + (acc[3][1] >> 6);
            int v2 = acc[0][2] + (acc[1][2] >> 2) + (acc[2][2] >> 4) + (acc[3][2] >> 6);
            int v3 = acc[0][3] + (acc[1][3] >> 2) + (acc[2][3] >> 4) + (acc[3][3] >> 6);
            int n0 = 2 * t, n1 = 2 * t + 1;
            if (n0 < M) {
                atomicAdd(&dst[n0 * 16 + g], v0);
                atomicAdd(&dst[n0 * 16 + g + 8], v2);
            }
            if (n1 < M) {
                atomicAdd(&dst[n1 * 16 + g], v1);
                atomicAdd(&dst[n1 * 16 + g + 8], v3);
            }
        } else {
            // acc[j][0]: row g, acc[j][1]: row g+8 (this lane's k subset); reduce over t
            int v0 = (acc[0][0] + acc[0][2]) + ((acc[1][0] + acc[1][2]) >> 2) + ((acc[2][0] + acc[2][2]) >> 4) +
                     ((acc[3][0] + acc[3][2]) >> 6);
            int v1 = (acc[0][1] + acc[0][3]) + ((acc[1][1] + acc[1][3]) >> 2) + ((acc[2][1] + acc[2][3]) >> 4) +
                     ((acc[3][1] + acc[3][3]) >> 6);
            v0 += __shfl_xor_sync(0xffffffffu, v0, 1);
            v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
            v0 += __shfl_xor_sync(0xffffffffu, v0, 2);
            v1 += __shfl_xor_sync(0xffffffffu, v1, 2);
            if (t == 0) {
                atomicAdd(&dst[g], v0);
                atomicAdd(&dst[g + 8], v1);
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int k = 0; k < 4; ++k) acc[j][k] = 0;
    };

    auto tile_step = [&](const uint8_t* tile, const uint32_t* ab) {
        const uint4 w = *reinterpret_cast<const uint4*>(tile);
        const uint4 b01 = *reinterpret_cast<const uint4*>(ab);
        const uint4 b23 = *reinterpret_cast<const uint4*>(ab + 4);
        if (MMA) {
            mma_u8s8(acc[0], w.x & 0x03030303u, w.y & 0x03030303u, w.z & 0x03030303u, w.w & 0x03030303u, b01.x, b01.y);
            mma_u8s8(acc[1], w.x & 0x0c0c0c0cu, w.y & 0x0c0c0c0cu, w.z & 0x0c0c0c0cu, w.w & 0x0c0c0c0cu, b01.z, b01.w);
            mma_u8s8(acc[2], w.x & 0x30303030u, w.y & 0x30303030u, w.z & 0x30303030u, w.w & 0x30303030u, b23.x, b23.y);
            mma_u8s8(acc[3], w.x & 0xc0c0c0c0u, w.y & 0xc0c0c0c0u, w.z & 0xc0c0c0c0u, w.w & 0xc0c0c0c0u, b23.z, b23.w);
        } else {
            const uint32_t bh0[4] = {b01.x, b01.z, b23.x, b23.z};
            const uint32_t bh1[4] = {b01.y, b01.w, b23.y, b23.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t mk = 0x03030303u << (2 * j);
                acc[j][0] = dp4a_u8s8(w.x & mk, bh0[j], acc[j][0]);
                acc[j][2] = dp4a_u8s8(w.z & mk, bh1[j], acc[j][2]);
                acc[j][1] = dp4a_u8s8(w.y & mk, bh0[j], acc[j][1]);
                acc[j][3] = dp4a_u8s8(w.w & mk, bh1[j], acc[j][3]);
            }
        }
    };

    int cstage = 0;
    uint32_t cphase = 0;
    while (cc.pos < w1) {
        const int len = chunk_len(cc);
        if (p.debug != 2 && !failed && !lb_mbar_wait_bounded(&my_bars[cstage], cphase)) {
            failed = true;
            if (lane == 0) atomicExch(p.status, 1);
        }
        if (cc.v != cur_v) {
            flush();
            cur_v = cc.v;
        }
        const uint8_t* tile = my_ring + (size_t)cstage * kStageBytes + lane * 16;
        const uint32_t* ab = act_base + cc.kb * act_kb_mul;
        if (!failed && p.debug != 1) {
            if (len == kStageTiles) {
#pragma unroll
                for (int i = 0; i < kStageTiles; ++i) tile_step(tile + i * kTileBytes, ab + i * act_kb_mul);
            } else {
                for (int i = 0; i < len; ++i) tile_step(tile + i * kTileBytes, ab + i * act_kb_mul);
            }
        }
        advance(cc, len);
        __syncwarp();
        if (ic.pos < w1) {
            const int len2 = chunk_len(ic);
            if (lane == 0) {
                fence_proxy_async();
                issue(cstage, ic, len2);
            }
            advance(ic, len2);
        }
        if (++cstage == nstages) {
            cstage = 0;
            cphase ^= 1u;
        }
    }
    flush();
    __syncthreads();
    LB_TRACE(4);

    // ---- strip groups: finish what this CTA owns entirely, hand the rest to the fix-up ------------------
    if (cta_tiles <= 0) return;
    const int group_tiles = p.group * KB;
    const int last_group = ((t1 - 1) / KB) / p.group;
    const int per_group = p.group * M * 16;
    const int ngl = last_group - first_group + 1;
    // Only the first and the last group of a stream-K range can be shared with another CTA.
    auto mine_of = [&](int G) {
        const int gs = G * group_tiles, ge = gs + group_tiles;
        return (t1 < ge ? t1 : ge) - (t0 > gs ? t0 : gs);
    };
    const int mine_first = mine_of(first_group), mine_last = mine_of(last_group);
    const bool part_first = mine_first != group_tiles;
    const bool part_last = ngl > 1 && mine_last != group_tiles;
    if (tid < 2) sm.flag[tid] = 1;  // 1 = this CTA finishes the group
    if (part_first || part_last) {
        for (int i = tid; i < 2 * per_group; i += kThreads) {
            const int which = i / per_group, k = i - which * per_group;
            if (which == 0 ? !part_first : !part_last) continue;
            const int G = which == 0 ? first_group : last_group;
            const int v = sm.sacc[(size_t)(G - first_group) * per_group + k];
            if (v != 0) atomicAdd(&p.fix_acc[(size_t)G * per_group + k], v);
        }
        __threadfence();
        __syncthreads();
        if (tid == 0 && part_first) {
            unsigned old = atomicAdd(&p.fix_cnt[first_group], (unsigned)mine_first);
            sm.flag[0] = (old + (unsigned)mine_first == (unsigned)group_tiles) ? 1 : 0;
        }
        if (tid == 32 && part_last) {
            unsigned old = atomicAdd(&p.fix_cnt[last_group], (unsigned)mine_last);
            sm.flag[1] = (old + (unsigned)mine_last == (unsigned)group_tiles) ? 1 : 0;
        }
        __syncthreads();
        const bool take_first = part_first && sm.flag[0], take_last = part_last && sm.flag[1];
        if (take_first || take_last) {
            __threadfence();
            for (int i = tid; i < 2 * per_group; i += kThreads) {
                const int which = i / per_group, k = i - which * per_group;
                if (which == 0 ? !take_first : !take_last) continue;
                const int G = which == 0 ? first_group : last_group;
                sm.sacc[(size_t)(G - first_group) * per_group + k] = atomicExch(&p.fix_acc[(size_t)G * per_group + k], 0);
            }
            if (tid == 0 && take_first) p.fix_cnt[first_group] = 0;
            if (tid == 32 && take_last) p.fix_cnt[last_group] = 0;
        }
    }
    __syncthreads();
    const bool do_first = sm.flag[0] != 0, do_last = sm.flag[1] != 0;
    for (int idx = tid; idx < ngl * per_group; idx += kThreads) {
        const int gl = idx / per_group, i = idx - gl * per_group;
        if (gl == 0 && !do_first) continue;
        if (gl == ngl - 1 && ngl > 1 && !do_last) continue;
        const int e = i / (M * 16), rem = i - e * (M * 16);
        finish_row<EPI>(p, sm, (first_group + gl) * p.group, e, rem >> 4, rem & 15, sm.sacc + (size_t)gl * per_group);
    }
    LB_TRACE(5);
}

size_t gemv_smem_bytes(const LbGemvParams& p, int max_local) {
    int Kp = p.kblocks * kTileCols;
    size_t b = (size_t)kWarps * p.stages * kStageBytes;
    b += (size_t)(p.M * ((Kp + 16) / 4) + 8) * 4;
    b = (b + 15) & ~(size_t)15;
    b += (size_t)max_local * p.M * 16 * 4;
    b += 32 + 32 + 256 + 3 * kMaxM * 8 + 16;
    b += (size_t)kWarps * kStages * 8;
    b = (b + 15) & ~(size_t)15;
    b += (size_t)p.stage_bytes;
    return b;
}

}  // namespace

int lb_gemv_finalize_params(loom_b200_ctx* ctx, LbGemvParams& p) {
    LB_REQUIRE(ctx, p.nseg >= 1 && p.nseg <= 3, "gemv: %d segments", p.nseg);
    LB_REQUIRE(ctx, p.M >= 1 && p.M <= kMaxM, "gemv: %d tokens per pass (max %d)", p.M, kMaxM);
    LB_REQUIRE(ctx, p.K > 0, "gemv: K=%d", p.K);
    p.kblocks = (p.K + kTileCols - 1) / kTileCols;
    int v = 0;
    for (int s = 0; s < p.nseg; ++s) {
        LB_REQUIRE(ctx, p.seg[s].tiles && p.seg[s].rows > 0, "gemv: segment %d is empty", s);
        p.seg[s].strips = (p.seg[s].rows + kTileRows - 1) / kTileRows;
        p.seg[s].vstrip0 = v;
        v += p.seg[s].strips;
    }
    p.interleave2 = p.epi == LB_EPI_SWIGLU ? 1 : 0;
    if (p.interleave2) {
        LB_REQUIRE(ctx, p.nseg == 2 && p.seg[0].rows == p.seg[1].rows, "gemv: gate/up pair needs two equal matrices");
        LB_REQUIRE(ctx, p.seg[0].out != nullptr, "gemv: gate/up pair needs an output buffer");
        p.seg[0].vstrip0 = p.seg[1].vstrip0 = 0;
        p.group = 2;
    } else {
        p.group = 1;
    }
    long long tiles = (long long)v * p.kblocks;
    LB_REQUIRE(ctx, tiles < (1ll << 30), "gemv: matrix too large (%lld tiles)", tiles);
    p.total_tiles = (int)tiles;
    return 0;
}

int lb_launch_gemv(loom_b200_ctx* ctx, const LbGemvParams& pin) {
    LbGemvParams p = pin;
    int vstrips = p.total_tiles / p.kblocks;
    int ngroups = (vstrips + p.group - 1) / p.group;
    int grid = ctx->sm_count * ctx->opt_gemv_ctas_per_sm;
    // Enough strip groups to occupy the SMs: give every CTA whole groups and skip the cross-CTA fix-up.
    p.aligned = ctx->opt_gemv_partition == 1 ? 0 : (ctx->opt_gemv_partition == 2 ? 1 : (ngroups * 2 >= ctx->sm_count ? 1 : 0));
    if (p.aligned) {
        if (grid > ngroups) grid = ngroups;
        int gpc = (ngroups + grid - 1) / grid;
        p.max_local_strips = gpc * p.group;
    } else {
        if (grid > p.total_tiles) grid = p.total_tiles;
        if (grid < 1) grid = 1;
        int tpc = (p.total_tiles + grid - 1) / grid;
        p.max_local_strips = (tpc + p.kblocks - 2) / p.kblocks + 1 + 2 * (p.group - 1);
    }
    if (int rc = lb_ensure_fixup(ctx, (size_t)ngroups * p.group * p.M * 16, (size_t)ngroups)) return rc;
    p.fix_acc = ctx->fix_acc;
    p.fix_cnt = ctx->fix_cnt;
    p.status = ctx->status_dev;
    p.debug = ctx->opt_debug;
    p.trace = lb_trace_row(ctx, "gemv");
    // ring depth: as many stages as the busiest warp has chunks (a chunk = up to 8 tiles inside one strip), up to 3
    {
        int most = 1;
        const int KB = p.kblocks, gt = p.group * KB;
        const long long NG = p.total_tiles / gt;
        for (int b = 0; b < grid && most < kStages; ++b) {
            long long t0, t1;
            if (p.aligned) {
                t0 = (NG * b / grid) * gt;
                t1 = (NG * (b + 1) / grid) * gt;
            } else {
                t0 = (long long)p.total_tiles * b / grid;
                t1 = (long long)p.total_tiles * (b + 1) / grid;
            }
            const long long n = t1 - t0;
            for (int w = 0; w < kWarps && most < kStages; ++w) {
                long long w0 = t0 + n * w / kWarps, w1 = t0 + n * (w + 1) / kWarps;
                int chunks = 0;
                while (w0 < w1) {
                    long long len = KB - w0 % KB;
                    if (len > kStageTiles) len = kStageTiles;
                    if (len > w1 - w0) len = w1 - w0;
                    w0 += len;
                    ++chunks;
                }
                if (chunks > most) most = chunks;
            }
        }
        p.stages = most > kStages ? kStages : most;
    }
    // prologue staging: the activation row in its input precision, when it fits beside the ring
    p.stage_bytes = 0;
    if (p.pro != LB_PRO_Q8 && (p.K & 3) == 0) {
        size_t want = (size_t)p.K * (p.pro == LB_PRO_INNERNORM64 ? 8 : 4);
        if (gemv_smem_bytes(p, p.max_local_strips) + want <= 227 * 1024) p.stage_bytes = (int)want;
    }
    size_t smem = gemv_smem_bytes(p, p.max_local_strips);
    if (smem > 227 * 1024)
        return lb_fail(ctx, LOOM_B200_ERR_UNSUPPORTED, "gemv: K=%d with %d tokens needs %zu B of shared memory", p.K, p.M, smem);
    // one instantiation per (inner loop, prologue, epilogue) combination that a caller can reach
    using Kern = void (*)(const LbGemvParams);
    Kern kern = nullptr;
    int kid = -1;
    const bool use_dp4a = ctx->opt_gemv_variant == 1 && p.M == 1 && p.pro == LB_PRO_Q8 && p.epi == LB_EPI_GENERIC;
#define LB_PICK(id, mma, pro_, epi_)                                \
    if (kid < 0 && p.pro == pro_ && p.epi == epi_ && (mma) == !use_dp4a) { \
        kern = lb_gemv_ternary_kernel<mma, pro_, epi_>;             \
        kid = id;                                                   \
    }
    LB_PICK(0, true, LB_PRO_Q8, LB_EPI_GENERIC)
    LB_PICK(1, false, LB_PRO_Q8, LB_EPI_GENERIC)
    LB_PICK(2, true, LB_PRO_F32, LB_EPI_GENERIC)
    LB_PICK(3, true, LB_PRO_BLOCKNORM, LB_EPI_QKV)
    LB_PICK(4, true, LB_PRO_F32, LB_EPI_QKV)
    LB_PICK(5, true, LB_PRO_INNERNORM64, LB_EPI_RESID)
    LB_PICK(6, true, LB_PRO_BLOCKNORM, LB_EPI_SWIGLU)
    LB_PICK(7, true, LB_PRO_F32, LB_EPI_SWIGLU)
    LB_PICK(8, true, LB_PRO_INNERNORM, LB_EPI_RESID)
    LB_PICK(9, true, LB_PRO_INNERNORM64, LB_EPI_GENERIC)
    LB_PICK(10, true, LB_PRO_INNERNORM, LB_EPI_GENERIC)
    LB_PICK(11, true, LB_PRO_Q8, LB_EPI_SWIGLU)
#undef LB_PICK
    if (!kern) return lb_fail(ctx, LOOM_B200_ERR_UNSUPPORTED, "gemv: no kernel for prologue %d with epilogue %d", p.pro, p.epi);
    const unsigned attr_bit = 1u << kid;
    if (!(ctx->func_attr_mask & attr_bit)) {  // per device: the context pins the device
        LB_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        ctx->func_attr_mask |= attr_bit;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
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

extern "C" int loom_b200_ternary_linear(loom_b200_ctx* ctx, const loom_b200_weight* w, int batch, const int8_t* q,
                                        const float* amax, const float* bias, const float* residual, int activation,
                                        float* out, int32_t* acc_out) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "ternary_linear: ctx is NULL");
    LB_REQUIRE(ctx, w != nullptr, "ternary_linear: weight is NULL");
    LB_REQUIRE(ctx, batch >= 0, "ternary_linear: batch=%d", batch);
    if (batch == 0) return 0;
    LB_REQUIRE(ctx, q && amax, "ternary_linear: NULL activation buffers");
    LB_REQUIRE(ctx, out || acc_out, "ternary_linear: no output buffer");
    LB_REQUIRE(ctx, w->device == ctx->device, "ternary_linear: weight lives on device %d, context on %d", w->device, ctx->device);
    if (int rc = lb_set_device(ctx)) return rc;
    for (int b0 = 0; b0 < batch; b0 += kMaxM) {
        LbGemvParams p = {};
        p.nseg = 1;
        p.seg[0].tiles = w->tiles;
        p.seg[0].rows = w->rows;
        p.seg[0].scale = w->scale;
        p.seg[0].bias = bias;
        p.seg[0].out = out ? (void*)(out + (size_t)b0 * w->rows) : nullptr;
        p.seg[0].acc_out = acc_out ? acc_out + (size_t)b0 * w->rows : nullptr;
        p.seg[0].kind = out ? LB_OUT_F32 : LB_OUT_ACC;
        p.epi = LB_EPI_GENERIC;
        p.K = w->cols;
        p.M = batch - b0 < kMaxM ? batch - b0 : kMaxM;
        p.pro = LB_PRO_Q8;
        p.x = q + (size_t)b0 * w->cols;
        p.amax_in = amax + b0;
        p.act = activation;
        p.residual = residual ? residual + (size_t)b0 * w->rows : nullptr;
        if (int rc = lb_gemv_finalize_params(ctx, p)) return rc;
        if (int rc = lb_launch_gemv(ctx, p)) return rc;
    }
    return 0;
}
