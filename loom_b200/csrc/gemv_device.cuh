// gemv_device.cuh -- device-side pieces of the packed-ternary GEMV kernel (gemv_ternary.cu): shared-memory layout,
// activation staging with the fused normalise/quantize prologues, the per-tile integer MMA step and the epilogues.
#pragma once
#include "gemv_ternary.cuh"
#include "tp_xchg.cuh"

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

#define LB_TRACE(k)                       \
    do {                                  \
        if (!LEAN) lb_trace(p.trace, (k)); \
    } while (0)

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
    float* gain;      // norm_w copied before the dependency wait, or null
    int pos0;         // *pos_ptr, read once after the dependency wait (KV ring rows)
    uint32_t xseq_c;  // tensor-parallel exchange: sequence number of this launch's exchange of partial sums
};

template <int EPI = LB_EPI_GENERIC, bool LEAN = false>
__device__ __forceinline__ const uint32_t* tile_ptr(const LbGemvParams& p, int v, int kb) {
    int s, local;
    if (LEAN && EPI == LB_EPI_RESID) {  // one matrix
        s = 0;
        local = v;
    } else if (LEAN ? EPI == LB_EPI_SWIGLU : p.interleave2 != 0) {
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

template <int NW = kWarps>
__device__ __forceinline__ double block_sum(double v, double* red) {
    v = lb_warp_sum(v);
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    double r = 0.0;
#pragma unroll
    for (int i = 0; i < NW; ++i) r += red[i];
    return r;
}

template <int NW = kWarps>
__device__ __forceinline__ float block_max(float v, double* red) {
    v = lb_warp_max(v);
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* rf = reinterpret_cast<float*>(red + 16);
    __syncthreads();
    if (lane == 0) rf[warp] = v;
    __syncthreads();
    float r = rf[0];
#pragma unroll
    for (int i = 1; i < NW; ++i) r = fmaxf(r, rf[i]);
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
__device__ __forceinline__ double lb_wide(float v) { return (double)v; }
__device__ __forceinline__ double lb_wide(double v) { return v; }

// LEAN (the launcher checked): gains cover the whole row or are absent, no statistics supplied by the caller, no side outputs.
template <int PRO, int NW = kWarps, bool LEAN = false>
__device__ __forceinline__ void stage_row_fast(const LbGemvParams& p, const Smem& sm, int n, const void* row) {
    constexpr int kThreads = NW * 32;
    const int tid = threadIdx.x, K = p.K, units = K >> 2;
    const int Kp = p.kblocks * kTileCols, stride32 = (Kp + 16) / 4;
    constexpr bool f64 = PRO == LB_PRO_INNERNORM64;
    using VT = typename std::conditional<f64, double, float>::type;
    VT* tmp = reinterpret_cast<VT*>(sm.stage);
    const bool have_w = PRO != LB_PRO_F32 && p.norm_w != nullptr;
    double ss = 0.0;
    unsigned long long mdb = 0;
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
        if (!LEAN && have_w && !sm.gain && 4 * idx < p.norm_w_len) asm volatile("prefetch.global.L1 [%0];" ::"l"(p.norm_w + 4 * idx));
        tmp[4 * idx] = a0; tmp[4 * idx + 1] = a1; tmp[4 * idx + 2] = a2; tmp[4 * idx + 3] = a3;
        if (PRO >= LB_PRO_BLOCKNORM) {
            const double d0 = lb_wide(a0), d1 = lb_wide(a1), d2 = lb_wide(a2), d3 = lb_wide(a3);
            ss = __dadd_rn(ss, __dmul_rn(d0, d0));
            ss = __dadd_rn(ss, __dmul_rn(d1, d1));
            ss = __dadd_rn(ss, __dmul_rn(d2, d2));
            ss = __dadd_rn(ss, __dmul_rn(d3, d3));
        } else {
            m = fmaxf(fmaxf(m, fabsf((float)a0)), fmaxf(fabsf((float)a1), fmaxf(fabsf((float)a2), fabsf((float)a3))));
        }
    }
    if (PRO >= LB_PRO_BLOCKNORM) {
        // tensor-parallel row shards: the sum of squares over the whole (sharded) vector is supplied by the caller
        if (!LEAN && p.given_ss) ss = p.given_ss[n];
        else ss = block_sum<NW>(ss, sm.red);
        const double mean = __dadd_rn(__ddiv_rn(ss, (double)(p.norm_count > 0 ? p.norm_count : K)), p.eps);
        const double root = sqrt(mean);
        const double rr = __ddiv_rn(1.0, root);  // RN(1/rms): the inner norms' scale, the block norm's reciprocal
        const float* gw = (LEAN || sm.gain) ? sm.gain : p.norm_w;  // the shared copy was made while waiting for the producer of the row (lean: always)
#pragma unroll 2
        for (int idx = tid; idx < units; idx += kThreads) {
            double w[4] = {1.0, 1.0, 1.0, 1.0};
            if (have_w) {
                if (LEAN || 4 * idx + 4 <= p.norm_w_len) {
                    const float4 g = reinterpret_cast<const float4*>(gw)[idx];
                    w[0] = (double)g.x; w[1] = (double)g.y; w[2] = (double)g.z; w[3] = (double)g.w;
                } else {
                    for (int k = 0; k < 4; ++k)
                        if (4 * idx + k < p.norm_w_len) w[k] = (double)gw[4 * idx + k];
                }
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const double x = lb_wide(tmp[4 * idx + k]);
                VT y;
                if (PRO == LB_PRO_BLOCKNORM) y = (VT)(float)__dmul_rn(lb_div_by(x, root, rr), w[k]);
                else if (f64) y = (VT)__dmul_rn(x, __dmul_rn(rr, w[k]));
                else y = (VT)(float)__dmul_rn(__dmul_rn(x, rr), w[k]);
                tmp[4 * idx + k] = y;
                if (f64) mdb = lb_absmax_bits(mdb, (double)y);  // one narrowing at the end: rounding is monotone
                else m = fmaxf(m, fabsf((float)y));
            }
        }
    }
    if (f64) m = fmaxf(m, (float)__longlong_as_double((long long)mdb));
    if (!LEAN && p.given_amax) m = p.given_amax[n];  // absmax over the whole sharded vector (already floored by the caller or below)
    else m = block_max<NW>(m, sm.red);
    const float amax = m < 1e-5f ? 1e-5f : m;
    const double s = __ddiv_rn(127.0, (double)amax);
    const bool side = !LEAN && blockIdx.x == 0;
    int local_sum = 0;
    uint8_t* abytes = reinterpret_cast<uint8_t*>(sm.acts + (size_t)n * stride32);
    // the output scales need a float64 division: the last threads (which own the fewest units) start it before their loop
    if (tid >= kThreads - 3) {
        const int sg = tid - (kThreads - 3);
        sm.os[sg * kMaxM + n] = sg < p.nseg ? lb_output_scale(p.seg[sg].scale, amax) : 1.0;
    }
#pragma unroll 2
    for (int idx = tid; idx < (Kp >> 2); idx += kThreads) {
        int q0 = 0, q1 = 0, q2 = 0, q3 = 0;
        if (idx < units) {
            const VT y0 = tmp[4 * idx], y1 = tmp[4 * idx + 1], y2 = tmp[4 * idx + 2], y3 = tmp[4 * idx + 3];
            q0 = lb_quant_i8(lb_wide(y0), s);
            q1 = lb_quant_i8(lb_wide(y1), s);
            q2 = lb_quant_i8(lb_wide(y2), s);
            q3 = lb_quant_i8(lb_wide(y3), s);
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
    if (tid == 0) {
        sm.amax[n] = amax;
        if (side && p.amax_out) p.amax_out[n] = amax;
    }
    __syncthreads();  // the staging buffer is reused by the next token
}

// One token through the general prologue path: the row is read from global memory in every pass (no staging buffer, any
// alignment, int8 rows).  For the float prologues this is the rare path (rows that are not 16-byte aligned or do not fit
// the staging buffer).  (Keeping it out of line was tried: the call needs the shared-memory layout in local memory and
// the decode step lost 2 %.)
template <int PRO, int NW>
__device__ __forceinline__ void stage_row_general(const LbGemvParams& p, const Smem& sm, int n, const void* row) {
    constexpr int kThreads = NW * 32;
    constexpr bool q8 = PRO == LB_PRO_Q8;
    const int tid = threadIdx.x;
    const int K = p.K, Kp = p.kblocks * kTileCols;
    const int stride32 = (Kp + 16) / 4;
    const int chunks = Kp / 16;
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
            ss = block_sum<NW>(ss, sm.red);
            if (p.given_ss) ss = p.given_ss[n];
            double mean = __dadd_rn(__ddiv_rn(ss, (double)(p.norm_count > 0 ? p.norm_count : K)), p.eps);
            stat = PRO == LB_PRO_BLOCKNORM ? sqrt(mean) : __ddiv_rn(1.0, sqrt(mean));
            if (PRO == LB_PRO_BLOCKNORM) rstat = __ddiv_rn(1.0, stat);
        }
        float m = 0.0f;
        for (int c = tid; c < K; c += kThreads)
            m = fmaxf(m, (float)fabs(pro_value<PRO>(row, c, stat, rstat, p.norm_w, p.norm_w_len)));
        m = block_max<NW>(m, sm.red);
        if (p.given_amax) m = p.given_amax[n];
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

// Quantizes the M activation rows into shared memory in the k-slot order the MMA B-fragments use, and
// leaves sum(q) and amax per token in shared memory.
template <int PRO, int NW = kWarps, bool LEAN = false>
__device__ __forceinline__ void stage_activations(const LbGemvParams& p, const Smem& sm) {
    const int tid = threadIdx.x;
    const int K = p.K, Kp = p.kblocks * kTileCols;
    const int stride32 = (Kp + 16) / 4;
    if (tid < kMaxM) sm.xsum[tid] = 0;
    const int M = p.M;
    if (tid < 8) sm.acts[M * stride32 + tid] = 0;  // zero block for the lanes of absent tokens
    for (int n = 0; n < M; ++n) {
        constexpr bool q8 = PRO == LB_PRO_Q8;
        const void* row = q8 ? (const void*)((const int8_t*)p.x + (size_t)n * K)
                             : (PRO == LB_PRO_INNERNORM64 ? (const void*)((const double*)p.x + (size_t)n * K)
                                                            : (const void*)((const float*)p.x + (size_t)n * K));
        if (LEAN && !q8) {  // the launcher checked the conditions of the staged path
            stage_row_fast<PRO == LB_PRO_Q8 ? LB_PRO_F32 : PRO, NW, true>(p, sm, n, row);
            continue;
        }
        if (!q8) {
            const bool aligned16 = (((uintptr_t)row) & 15) == 0 && (!p.norm_w || (((uintptr_t)p.norm_w) & 15) == 0) &&
                                   (!p.norm_out || (((uintptr_t)p.norm_out) & 15) == 0) && (!p.q_out || (((uintptr_t)p.q_out) & 3) == 0);
            if ((K & 3) == 0 && sm.stage && aligned16) {
                stage_row_fast<PRO == LB_PRO_Q8 ? LB_PRO_F32 : PRO, NW>(p, sm, n, row);
                continue;
            }
        }
        stage_row_general<PRO, NW>(p, sm, n, row);
    }
    __syncthreads();
}

// Activations other than linear/ReLU/ReLU2 pull in transcendental code: keep it out of the straight-line path.
__device__ __noinline__ float activate_slow(float v, int act) { return lb_activate(v, act); }

__device__ __forceinline__ size_t out_index(const LbGemvParams& p, const Smem& sm, const LbGemvSeg& sg, int n, int r) {
    if (sg.out_ring > 0) {
        size_t base = 0;
        int pos;
        if (sg.seq_stride > 0) {  // one ring and one position per token
            pos = p.pos_ptr[n] % sg.out_ring;
            base = (size_t)n * (size_t)sg.seq_stride;
        } else {
            pos = (sm.pos0 + n) % sg.out_ring;
        }
        if (sg.ring_hd > 0) return base + ((size_t)(r / sg.ring_hd) * sg.out_ring + pos) * sg.ring_hd + r % sg.ring_hd;  // head-major KV ring
        return base + (size_t)pos * sg.rows + r;
    }
    return (size_t)n * sg.rows + r;
}

// Epilogue of one finished row (or gate/up row pair).  vals = [group][M][16] complete sums of sum(code*x).
template <int EPI, bool LEAN = false>
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
        const size_t o = out_index(p, sm, sg, n, r);
        if (s == 0) ((double*)sg.out)[o] = y;
        else ((float*)sg.out)[o] = (float)y;
        return;
    }
    if (EPI == LB_EPI_RESID || EPI == LB_EPI_TPSUM) {
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

}  // namespace
