// glue.cu -- decoder steps around the ternary projections (see glue.cuh).  Arithmetic follows the reference's
// CPU decoder: poly/mha.go:285-354 (q/k norm, RoPE, attention in float64 over a float32 KV ring),
// poly/norm.go:102-138 (RMSNorm), poly/transformer.go:659-719 (fp32 LM head, float64 accumulation),
// poly/sampling.go:45-55 (greedy = first maximum).
#include "glue.cuh"

namespace {

__device__ __forceinline__ double warp_max_d(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmax(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// block-wide reductions for blockDim.x <= 1024; every thread gets the same bits
__device__ __forceinline__ double block_sum_d(double v, double* red) {
    v = lb_warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    double r = 0.0;
    for (int i = 0; i < nw; ++i) r += red[i];
    return r;
}
__device__ __forceinline__ double block_max_d(double v, double* red) {
    v = warp_max_d(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    double r = red[0];
    for (int i = 1; i < nw; ++i) r = fmax(r, red[i]);
    return r;
}

__global__ void lb_embed_kernel(const float* __restrict__ emb, int vocab, int hidden, const int* __restrict__ tok,
                                float* __restrict__ x) {
    lb_pdl_launch_dependents();
    lb_pdl_wait();
    const int n = blockIdx.x;
    const int t = tok[n];
    const bool ok = t >= 0 && t < vocab;
    const float* src = emb + (size_t)(ok ? t : 0) * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) x[(size_t)n * hidden + i] = ok ? src[i] : 0.0f;
}

// One CTA per (token, head) over Q heads then K heads; hd/2 threads, thread d owns the pair (d, d+hd/2).
__global__ void lb_rope_kernel(const LbRopeParams p) {
    __shared__ double red[32];
    lb_pdl_launch_dependents();
    lb_pdl_wait();
    lb_trace(p.trace, 2);
    const int n = blockIdx.y, h = blockIdx.x, half = p.hd / 2, d = threadIdx.x;
    const int pos = p.seq_stride > 0 ? p.pos_ptr[n] : *p.pos_ptr + n;
    const bool is_q = h < p.heads;
    double v0, v1;
    float* krow = nullptr;
    double* qrow = nullptr;
    if (is_q) {
        qrow = p.q + (size_t)n * p.heads * p.hd + (size_t)h * p.hd;
        v0 = qrow[d];
        v1 = qrow[d + half];
    } else {
        const int kh = h - p.heads;
        krow = p.cache_k + (size_t)n * (size_t)p.seq_stride + ((size_t)kh * p.msl + (size_t)(pos % p.msl)) * p.hd;  // ring is head-major: [kv head][position][hd]
        v0 = (double)krow[d];
        v1 = (double)krow[d + half];
    }
    const float* gamma = is_q ? p.q_norm : p.k_norm;
    const int glen = is_q ? p.q_norm_len : p.k_norm_len;
    if (gamma && glen > 0) {  // per-head RMSNorm, poly/mha.go:584-646
        double ss = block_sum_d(__dadd_rn(__dmul_rn(v0, v0), __dmul_rn(v1, v1)), red);
        double rms = sqrt(__dadd_rn(__ddiv_rn(ss, (double)p.hd), p.qk_eps));
        if (rms != 0.0) {
            const int hh = is_q ? h : h - p.heads;
            const int nh = is_q ? p.heads : p.kv_heads;
            double inv = __ddiv_rn(1.0, rms);
            double s0 = 1.0, s1 = 1.0;
            if (glen == p.hd) {
                s0 = (double)gamma[d];
                s1 = (double)gamma[d + half];
            } else if (glen == nh * p.hd) {
                s0 = (double)gamma[(size_t)hh * p.hd + d];
                s1 = (double)gamma[(size_t)hh * p.hd + d + half];
            }
            v0 = __dmul_rn(__dmul_rn(v0, inv), s0);
            v1 = __dmul_rn(__dmul_rn(v1, inv), s1);
            if (!is_q) {  // the K row is float32 storage: the norm result is rounded before RoPE reads it back
                v0 = (double)(float)v0;
                v1 = (double)(float)v1;
            }
        }
    }
    const double angle = __ddiv_rn((double)pos, p.rope_div[d]);
    double sn, c;
    sincos(angle, &sn, &c);
    const double r0 = __dsub_rn(__dmul_rn(v0, c), __dmul_rn(v1, sn));
    const double r1 = __dadd_rn(__dmul_rn(v0, sn), __dmul_rn(v1, c));
    if (is_q) {
        qrow[d] = r0;
        qrow[d + half] = r1;
    } else {
        krow[d] = (float)r0;
        krow[d + half] = (float)r1;
    }
    lb_trace(p.trace, 5);
}

// One CTA per (head, token, split).  K and V rows of the CTA's positions are brought into shared memory by
// one 512-byte bulk async copy (TMA engine) per row, so that every HBM access of the kernel is in flight at
// once; a pair of threads then scores one position (half of the head dimension each) and output dimension d is
// owned by thread d of each of G = 256/hd position groups.  With splits > 1 the partial (max, sum, weighted V)
// of every split goes to scratch and the CTA that arrives last combines them.  Sums run in float64 like the
// reference's; their order (and the fused multiply-adds) differ from its sequential loops only in the last
// bits of a double.
constexpr int kAttnThreads = 256;
constexpr int kAttnTile = 80;  // positions per shared-memory tile

// K or V rows of positions pos0 .. pos0+rows-1 of one KV head: the ring is head-major ([kv head][position][hd]), so
// they are one contiguous block and ONE bulk copy brings them (the copy engine costs ~30 ns per copy whatever its
// size: a copy per 512-byte row, as a position-major ring needs, made the loads the longest part of the kernel).
// `head_ring` points at position 0 of the head; a chunk never wraps (positions stay below MaxSeqLen).
__device__ __forceinline__ void attn_fetch_rows(float* tile, const float* head_ring, int hd, int pos0, int rows, uint64_t* bar, int lane) {
    if (lane == 0) {
        lb_mbar_expect_tx(bar, (uint32_t)rows * hd * 4);
        lb_bulk_g2s(tile, head_ring + (size_t)pos0 * hd, (uint32_t)rows * hd * 4, bar);
    }
    __syncwarp();
}

__global__ void __launch_bounds__(kAttnThreads) lb_attention_kernel(const LbAttnParams p) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ double red[32];
    __shared__ double s_w[64], s_ls[64];
    __shared__ __align__(8) uint64_t bars[2];
    __shared__ int s_last;
    const int h = blockIdx.x, n = blockIdx.y, sp = blockIdx.z, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hd = p.hd, kvd = p.kv_heads * hd, qd = p.heads * hd;
    const int rowf = hd;      // tile rows are dense (one bulk copy per tile); the score loop staggers its start per position instead
    const int tile = p.tile;  // positions per shared-memory tile (at most kAttnTile)
    const int G = hd >= kAttnThreads ? 1 : kAttnThreads / hd;
    float* kt = reinterpret_cast<float*>(smem_raw);           // [tile, rowf]
    float* vt = kt + (size_t)tile * rowf;                // [tile, rowf]
    double* sq = reinterpret_cast<double*>(vt + (size_t)tile * rowf);  // [hd]
    double* sacc = sq + hd;                                   // [G, hd]
    double* sc = sacc + (size_t)G * hd;                       // [max_chunk]
    if (tid == 0) {
        lb_mbar_init(&bars[0], 1);
        lb_mbar_init(&bars[1], 1);
        lb_fence_mbar_init();
    }
    __syncthreads();
    lb_pdl_launch_dependents();
    lb_pdl_wait();
    lb_trace(p.trace, 2);
    const int last = p.seq_stride > 0 ? p.pos_ptr[n] : *p.pos_ptr + n;  // attends to positions 0..last
    const int total = last + 1;
    const int per = (total + p.splits - 1) / p.splits;
    const int k0 = sp * per;
    int k1 = k0 + per;
    if (k1 > total) k1 = total;
    const int cnt = k1 > k0 ? k1 - k0 : 0;
    const int kvh = h / (p.heads / p.kv_heads);
    const float* kbase = p.cache_k + (size_t)n * (size_t)p.seq_stride + (size_t)kvh * p.msl * hd;
    const float* vbase = p.cache_v + (size_t)n * (size_t)p.seq_stride + (size_t)kvh * p.msl * hd;
    const int ntiles = (cnt + tile - 1) / tile;
    bool failed = false;
    // first K and V tiles: every row of both is requested before anything else happens
    if (cnt > 0) {
        const int rows0 = cnt < tile ? cnt : tile;
        if (warp == 0) attn_fetch_rows(kt, kbase, hd, k0, rows0, &bars[0], lane);
        if (warp == 1) attn_fetch_rows(vt, vbase, hd, k0, rows0, &bars[1], lane);
    }
    const double scale = __ddiv_rn(1.0, sqrt((double)hd));
    for (int d = tid; d < hd; d += kAttnThreads) sq[d] = p.q[(size_t)n * qd + (size_t)h * hd + d];
    __syncthreads();
    // RoPE folded in (one-token steps): thread d < hd/2 owns the pair (d, d + hd/2) of the query and of the newest K row
    const bool fold_rope = p.rope_div != nullptr;
    double rsn = 0.0, rc = 1.0;
    if (fold_rope) {
        if (tid < hd / 2) {
            sincos(__ddiv_rn((double)last, p.rope_div[tid]), &rsn, &rc);
            const double v0 = sq[tid], v1 = sq[tid + hd / 2];
            sq[tid] = __dsub_rn(__dmul_rn(v0, rc), __dmul_rn(v1, rsn));
            sq[tid + hd / 2] = __dadd_rn(__dmul_rn(v0, rsn), __dmul_rn(v1, rc));
        }
        __syncthreads();
    }

    // scores: thread pair (2j, 2j+1) handles position j of the tile, each over half of the dimensions
    double mx = -1e9;
    const int half = tid & 1, hlen = hd / 2;
    for (int t = 0; t < ntiles; ++t) {
        const int base = t * tile;
        const int rows = cnt - base < tile ? cnt - base : tile;
        if (t > 0) {
            __syncthreads();  // everyone is done with the previous K tile
            if (warp == 0) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                attn_fetch_rows(kt, kbase, hd, k0 + base, rows, &bars[0], lane);
            }
        }
        if (!failed && !lb_mbar_wait_bounded(&bars[0], (uint32_t)(t & 1))) failed = true;
        if (fold_rope && last >= k0 + base && last < k0 + base + rows) {
            // the newest position is in this tile: its ring row is not written yet; take the unrotated row from k_new,
            // rotate it into the tile, and (one CTA per KV head) into the ring
            if (tid < hd / 2) {
                const double v0 = (double)p.k_new[(size_t)kvh * hd + tid], v1 = (double)p.k_new[(size_t)kvh * hd + tid + hd / 2];
                const float r0 = (float)__dsub_rn(__dmul_rn(v0, rc), __dmul_rn(v1, rsn));
                const float r1 = (float)__dadd_rn(__dmul_rn(v0, rsn), __dmul_rn(v1, rc));
                float* trow = kt + (size_t)(last - k0 - base) * rowf;
                trow[tid] = r0;
                trow[tid + hd / 2] = r1;
                if (h % (p.heads / p.kv_heads) == 0) {
                    float* grow = p.cache_k_w + ((size_t)kvh * p.msl + (size_t)(last % p.msl)) * hd;
                    grow[tid] = r0;
                    grow[tid + hd / 2] = r1;
                }
            }
            __syncthreads();
        }
        for (int j0 = 0; j0 < rows; j0 += kAttnThreads / 2) {
            const int j = j0 + (tid >> 1);
            double dot = 0.0;
            if (j < rows) {
                const float* kr = kt + (size_t)j * rowf + half * hlen;
                const double* qh = sq + half * hlen;
                double d0 = 0.0, d1 = 0.0;
                // rows are 512 B apart: starting every position four columns further keeps the 16-byte reads off each other's banks
                const int rot = (4 * (tid >> 1)) % hlen;
#pragma unroll 4
                for (int dd = 0; dd < hlen; dd += 4) {
                    int d = dd + rot;
                    if (d >= hlen) d -= hlen;
                    const float4 kv = *reinterpret_cast<const float4*>(kr + d);
                    d0 = fma(qh[d], (double)kv.x, d0);
                    d1 = fma(qh[d + 1], (double)kv.y, d1);
                    d0 = fma(qh[d + 2], (double)kv.z, d0);
                    d1 = fma(qh[d + 3], (double)kv.w, d1);
                }
                dot = d0 + d1;
            }
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            if (j < rows) {
                const double s = __dmul_rn(dot, scale);
                if (half == 0) sc[base + j] = s;
                mx = fmax(mx, s);
            }
        }
    }
    mx = block_max_d(mx, red);
    lb_trace(p.trace, 3);
    double den = 0.0;
    for (int j = tid; j < cnt; j += kAttnThreads) {
        const double e = exp(__dsub_rn(sc[j], mx));
        sc[j] = e;
        den = __dadd_rn(den, e);
    }
    den = block_sum_d(den, red);  // also orders the sc[] writes before the reads below

    // weighted V: group g takes positions g, g+G, ... of each tile
    const int d = G > 1 ? tid % hd : tid, grp = G > 1 ? tid / hd : 0;
    const bool owner = d < hd && grp < G;
    double a0 = 0.0, a1 = 0.0;
    for (int t = 0; t < ntiles; ++t) {
        const int base = t * tile;
        const int rows = cnt - base < tile ? cnt - base : tile;
        if (t > 0) {
            __syncthreads();
            if (warp == 1) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                attn_fetch_rows(vt, vbase, hd, k0 + base, rows, &bars[1], lane);
            }
        }
        if (!failed && !lb_mbar_wait_bounded(&bars[1], (uint32_t)(t & 1))) failed = true;
        if (owner) {
            for (int dd = d; dd < hd; dd += kAttnThreads) {  // hd > 256: a thread owns several dimensions (one accumulator pair each would be needed)
                int j = grp;
                for (; j + G < rows; j += 2 * G) {
                    a0 = fma(sc[base + j], (double)vt[(size_t)j * rowf + dd], a0);
                    a1 = fma(sc[base + j + G], (double)vt[(size_t)(j + G) * rowf + dd], a1);
                }
                if (j < rows) a0 = fma(sc[base + j], (double)vt[(size_t)j * rowf + dd], a0);
            }
        }
    }
    if (failed && tid == 0) atomicExch(p.status, 1);
    if (owner) sacc[(size_t)grp * hd + d] = a0 + a1;
    __syncthreads();
    if (owner && grp == 0) {
        double acc = sacc[d];
        for (int g = 1; g < G; ++g) acc += sacc[(size_t)g * hd + d];
        if (p.splits == 1) {
            p.out[(size_t)n * qd + (size_t)h * hd + d] = __ddiv_rn(acc, den);
        } else {
            double* part = p.part + ((size_t)(n * p.heads + h) * p.splits + sp) * (hd + 2);
            part[2 + d] = acc;
            if (d == 0) {
                part[0] = mx;
                part[1] = den;
            }
        }
    }
    lb_trace(p.trace, 4);
    if (p.splits == 1) return;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        unsigned old = atomicAdd(&p.cnt[n * p.heads + h], 1u);
        s_last = old + 1 == (unsigned)p.splits;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const double* base = p.part + (size_t)(n * p.heads + h) * p.splits * (hd + 2);
    // weights of the splits: exp(m_s - max m), one thread per split
    double ms = -1e9, ls = 0.0;
    if (tid < p.splits) {
        ms = __ldcg(base + (size_t)tid * (hd + 2));
        ls = __ldcg(base + (size_t)tid * (hd + 2) + 1);
    }
    double gm = ms;
    if (warp == 0 || p.splits > 32) gm = warp_max_d(gm);
    if (tid == 0) red[0] = gm;
    __syncthreads();
    if (p.splits > 32) {  // more than one warp holds split maxima
        if (lane == 0 && warp < 2) red[1 + warp] = gm;
        __syncthreads();
        if (tid == 0) red[0] = fmax(red[1], red[2]);
        __syncthreads();
    }
    gm = red[0];
    if (tid < p.splits) {
        s_w[tid] = ls == 0.0 ? 0.0 : exp(__dsub_rn(ms, gm));
        s_ls[tid] = ls;
    }
    __syncthreads();
    for (int dd = tid; dd < hd; dd += kAttnThreads) {
        double num = 0.0, dn = 0.0;
        // eight partial sums are requested before any is used: one L2 round trip per eight splits instead of one per split
        for (int s0 = 0; s0 < p.splits; s0 += 8) {
            double v[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = s0 + k < p.splits ? __ldcg(base + (size_t)(s0 + k) * (hd + 2) + 2 + dd) : 0.0;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                if (s0 + k < p.splits) {
                    const double w = s_w[s0 + k];
                    if (w != 0.0) {  // not an empty split
                        num = fma(v[k], w, num);
                        dn = fma(s_ls[s0 + k], w, dn);
                    }
                }
            }
        }
        p.out[(size_t)n * qd + (size_t)h * hd + dd] = __ddiv_rn(num, dn);
    }
    if (tid == 0) p.cnt[n * p.heads + h] = 0;
}

// fp32 LM head: every warp walks vocabulary rows; the hidden row is normalised once per CTA into shared
// memory as doubles.  Products of two floats are exact in double; only the summation order differs from
// the reference's sequential loop.
constexpr int kHeadThreads = 256;

__global__ void __launch_bounds__(kHeadThreads) lb_lm_head_kernel(const LbLmHeadParams p) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __shared__ double red[32];
    double* sh = reinterpret_cast<double*>(smem_raw);  // [hidden]
    lb_pdl_launch_dependents();
    lb_pdl_wait();
    lb_trace(p.trace, 2);
    const int H = p.hidden, tid = threadIdx.x;
    double ss = 0.0;
    for (int i = tid; i < H; i += kHeadThreads) {
        double v = (double)p.x[i];
        ss = __dadd_rn(ss, __dmul_rn(v, v));
    }
    ss = block_sum_d(ss, red);
    const double rms = sqrt(__dadd_rn(__ddiv_rn(ss, (double)H), p.eps));
    const double rrms = __ddiv_rn(1.0, rms);
    for (int i = tid; i < H; i += kHeadThreads) {
        double g = p.gain ? (double)p.gain[i] : 1.0;
        float y = (float)__dmul_rn(lb_div_by((double)p.x[i], rms, rrms), g);
        sh[i] = (double)y;
        if (blockIdx.x == 0 && p.hidden_out) p.hidden_out[i] = y;
    }
    __syncthreads();
    const int lane = tid & 31;
    const int warps_total = gridDim.x * (kHeadThreads / 32);
    const int H4 = H / 4;
    for (int v = blockIdx.x * (kHeadThreads / 32) + (tid >> 5); v < p.vocab; v += warps_total) {
        const float* row = p.head + (size_t)v * H;
        double acc = 0.0;
        if ((H & 3) == 0) {
            const float4* r4 = reinterpret_cast<const float4*>(row);
            int i = lane;
            for (; i + 96 < H4; i += 128) {
                const float4 a = __ldcs(r4 + i), b = __ldcs(r4 + i + 32), c = __ldcs(r4 + i + 64), d = __ldcs(r4 + i + 96);
                const double* s0 = sh + 4 * i;
                acc = fma((double)a.x, s0[0], acc); acc = fma((double)a.y, s0[1], acc);
                acc = fma((double)a.z, s0[2], acc); acc = fma((double)a.w, s0[3], acc);
                acc = fma((double)b.x, s0[128], acc); acc = fma((double)b.y, s0[129], acc);
                acc = fma((double)b.z, s0[130], acc); acc = fma((double)b.w, s0[131], acc);
                acc = fma((double)c.x, s0[256], acc); acc = fma((double)c.y, s0[257], acc);
                acc = fma((double)c.z, s0[258], acc); acc = fma((double)c.w, s0[259], acc);
                acc = fma((double)d.x, s0[384], acc); acc = fma((double)d.y, s0[385], acc);
                acc = fma((double)d.z, s0[386], acc); acc = fma((double)d.w, s0[387], acc);
            }
            for (; i < H4; i += 32) {
                const float4 a = __ldcs(r4 + i);
                const double* s0 = sh + 4 * i;
                acc = fma((double)a.x, s0[0], acc); acc = fma((double)a.y, s0[1], acc);
                acc = fma((double)a.z, s0[2], acc); acc = fma((double)a.w, s0[3], acc);
            }
        } else {
            for (int i = lane; i < H; i += 32) acc = fma((double)row[i], sh[i], acc);
        }
        acc = lb_warp_sum(acc);
        if (lane == 0) p.logits[v] = (float)acc;
    }
    lb_trace(p.trace, 5);
}

// Greedy argmax in two levels: every CTA reduces a slice to (value, first index); the CTA that arrives last
// reduces the per-CTA results, publishes the token and advances the cursors.
constexpr int kArgmaxCtas = 64;

__device__ __forceinline__ void argmax_merge(float& best, int& idx, float ov, int oi) {
    if (ov > best || (ov == best && oi < idx)) {
        best = ov;
        idx = oi;
    }
}

__global__ void __launch_bounds__(256) lb_argmax_advance_kernel(const float* __restrict__ logits, int vocab, int* tok,
                                                                int* out_tokens, int out_cap, int* step, int* pos,
                                                                float* part_val, int* part_idx, unsigned int* cnt) {
    __shared__ float sv[8];
    __shared__ int si[8];
    __shared__ int s_last;
    lb_pdl_launch_dependents();
    lb_pdl_wait();
    const int per = (vocab + gridDim.x - 1) / gridDim.x;
    const int lo = blockIdx.x * per, hi = min(vocab, lo + per);
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) argmax_merge(best, idx, logits[i], i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, best, o);
        int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        argmax_merge(best, idx, ov, oi);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) {
        sv[warp] = best;
        si[warp] = idx;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w) argmax_merge(best, idx, sv[w], si[w]);
        part_val[blockIdx.x] = best;
        part_idx[blockIdx.x] = idx;
        __threadfence();
        unsigned old = atomicAdd(cnt, 1u);
        s_last = old + 1 == gridDim.x;
    }
    __syncthreads();
    if (!s_last || threadIdx.x >= 32) return;
    __threadfence();
    best = -INFINITY;
    idx = 0x7fffffff;
    for (int i = lane; i < (int)gridDim.x; i += 32) argmax_merge(best, idx, __ldcg(part_val + i), __ldcg(part_idx + i));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, best, o);
        int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        argmax_merge(best, idx, ov, oi);
    }
    if (lane == 0) {
        if (idx == 0x7fffffff) idx = 0;  // only NaNs: the reference keeps index 0
        tok[0] = idx;
        if (out_tokens && step) {
            int s = *step;
            if (s < out_cap) out_tokens[s] = idx;
            *step = s + 1;
        }
        if (pos) *pos += 1;
        *cnt = 0;
    }
}

// Attention for head dimensions the tiled kernels do not take (not a multiple of 8, e.g. the reference's own smallest
// fixture with head_dim 2, poly/tests/bitnet_cpu_test.go:364-386): one warp per (head, token), plain loads, the same
// float64 arithmetic (poly/mha.go:316-354).  Scores of all positions sit in shared memory.
__global__ void __launch_bounds__(32) lb_attention_small_kernel(const LbAttnParams p) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    double* sc = reinterpret_cast<double*>(smem_raw);  // [positions]
    lb_pdl_launch_dependents();
    lb_pdl_wait();
    const int h = blockIdx.x, n = blockIdx.y, lane = threadIdx.x;
    const int hd = p.hd, qd = p.heads * hd;
    const int last = p.seq_stride > 0 ? p.pos_ptr[n] : *p.pos_ptr + n;
    const int kvh = h / (p.heads / p.kv_heads);
    const size_t seq_off = (size_t)n * (size_t)p.seq_stride;
    const float* kbase = p.cache_k + seq_off + (size_t)kvh * p.msl * hd;
    const float* vbase = p.cache_v + seq_off + (size_t)kvh * p.msl * hd;
    const double* q = p.q + (size_t)n * qd + (size_t)h * hd;
    const double scale = __ddiv_rn(1.0, sqrt((double)hd));
    double mx = -1e300;
    for (int j = lane; j <= last; j += 32) {
        double dot = 0.0;
        for (int d = 0; d < hd; ++d) dot = __dadd_rn(dot, __dmul_rn(q[d], (double)kbase[(size_t)j * hd + d]));
        const double s = __dmul_rn(dot, scale);
        sc[j] = s;
        mx = fmax(mx, s);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmax(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    double den = 0.0;
    for (int j = lane; j <= last; j += 32) {
        const double e = exp(__dsub_rn(sc[j], mx));
        sc[j] = e;
        den = __dadd_rn(den, e);
    }
    den = lb_warp_sum(den);
    __syncwarp();
    for (int d = 0; d < hd; ++d) {
        double acc = 0.0;
        for (int j = lane; j <= last; j += 32) acc = __dadd_rn(acc, __dmul_rn(sc[j], (double)vbase[(size_t)j * hd + d]));
        acc = lb_warp_sum(acc);
        if (lane == 0) p.out[(size_t)n * qd + (size_t)h * hd + d] = __ddiv_rn(acc, den);
    }
}

__global__ void lb_add_scalar_kernel(int* p, int delta) {
    lb_pdl_launch_dependents();
    lb_pdl_wait();
    if (threadIdx.x == 0) *p += delta;
}

// Causal attention of a block of prompt tokens.  One CTA per (KV head, tile of query tokens): the 64 query rows of
// a CTA are the heads of one GQA group times 64/group consecutive tokens, so every K and V tile that is brought
// into shared memory (64 positions, one 512-byte bulk copy per row) serves all of them.  Scores, the running
// softmax (maximum, sum, rescaling of the partial output when the maximum moves) and the weighted V sum are float64
// like the reference's loops (poly/mha.go:296-356); only the order of the float64 additions differs.
// A tile arrives as float32 in a staging buffer and is widened to float64 once, into a buffer K and V take turns in.
// Both products run on the float64 tensor-core MMA (mma.sync m8n8k4: 256 FMAs per instruction at the same peak as
// scalar FMAs, measured 63.9 FMA/clk/SM, but a quarter of the shared-memory traffic and an eighth of the issue
// slots): warp w owns score rows 16*(w/2).. and key columns 32*(w%2).., then output rows 16*(w/2).. and the
// dimensions of half w%2.  Row strides are chosen so that a fragment load touches every bank once.
constexpr int kPfRows = 64, kPfKeys = 64, kPfThreads = 256;

__device__ __forceinline__ void dmma_884(double (&c)[2], double a, double b) {
    asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};" : "+d"(c[0]), "+d"(c[1]) : "d"(a), "d"(b));
}

__global__ void __launch_bounds__(kPfThreads, 1) lb_attention_prefill_kernel(const LbAttnParams p) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar;
    __shared__ double s_m[kPfRows], s_l[kPfRows], s_alpha[kPfRows];
    __shared__ int s_qpos[kPfRows];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hd = p.hd, kvd = p.kv_heads * hd, qd = p.heads * hd;
    const int group = p.heads / p.kv_heads, TQ = kPfRows / group;
    const int kvh = blockIdx.x, qt = (int)gridDim.y - 1 - (int)blockIdx.y;  // long rows first
    const int tok0 = qt * TQ;
    // row strides in elements: +4 doubles (32 B) puts the 8 rows x 4 k of an A or K fragment on 32 distinct banks,
    // +8 doubles (64 B) does the same for the 4 keys x 8 dimensions of a V fragment
    const int qstride = hd + 4, kstride = hd + 4, vstride = hd + 8, rowf = hd, sstride = kPfKeys + 4;
    double* Qs = reinterpret_cast<double*>(smem_raw);                      // [64, hd+4] queries
    double* KV = Qs + (size_t)kPfRows * qstride;                           // [64, hd+8] the K tile, then the V tile, as float64
    double* Ss = KV + (size_t)kPfKeys * vstride;                           // [64, 68] scores, then softmax weights
    float* stage = reinterpret_cast<float*>(Ss + (size_t)kPfRows * sstride);  // [64, hd] float32 tile as copied
    if (tid == 0) {
        lb_mbar_init(&bar, 1);
        lb_fence_mbar_init();
    }
    __syncthreads();
    lb_pdl_launch_dependents();
    lb_pdl_wait();
    const int pos0 = *p.pos_ptr;
    const int ntok = p.M - tok0 < TQ ? p.M - tok0 : TQ;  // tokens of this tile
    const int max_pos = pos0 + tok0 + ntok - 1;
    const int ntiles = max_pos / kPfKeys + 1;
    const float* kbase = p.cache_k + (size_t)kvh * p.msl * hd;
    const float* vbase = p.cache_v + (size_t)kvh * p.msl * hd;
    auto tile_rows = [&](int t) { return max_pos + 1 - t * kPfKeys < kPfKeys ? max_pos + 1 - t * kPfKeys : kPfKeys; };
    if (warp == 0) attn_fetch_rows(stage, kbase, hd, 0, tile_rows(0), &bar, lane);
    // query rows: row r = (head hi of the group, token ti); rows of absent tokens are zero and never written back
    for (int idx = tid; idx < kPfRows * hd; idx += kPfThreads) {
        const int r = idx / hd, d = idx - r * hd;
        const int hi = r / TQ, ti = r - hi * TQ;
        double v = 0.0;
        if (ti < ntok) v = p.q[(size_t)(tok0 + ti) * qd + (size_t)(kvh * group + hi) * hd + d];
        Qs[(size_t)r * qstride + d] = v;
    }
    if (tid < kPfRows) {
        const int ti = tid % TQ;
        s_qpos[tid] = ti < ntok ? pos0 + tok0 + ti : -1;  // -1: nothing is attended, the row stays empty
        s_m[tid] = -1e300;
        s_l[tid] = 0.0;
    }
    __syncthreads();
    const double scale = __ddiv_rn(1.0, sqrt((double)hd));
    // fragment coordinates: an m8n8k4 A fragment is A[lane/4][lane%4], B is B[lane%4][lane/4], C is C[lane/4][2*(lane%4) + {0,1}]
    const int g = lane >> 2, t4 = lane & 3;
    const int wr = (warp >> 1) * 16;          // first score / output row of this warp
    const int wc = (warp & 1) * 32;           // first key column of this warp's scores
    const int wd = (warp & 1) * (hd / 2);     // first output dimension of this warp
    const int nfr = hd / 16;                  // 8-dimension fragments per warp (8 for head_dim 128)
    double o[2][8][2];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) o[i][j][0] = o[i][j][1] = 0.0;
    bool failed = false;
    uint32_t phase = 0;
    // staging (float32, rows of hd+4) -> KV (float64, rows of `stride`); rows beyond `rows` become zero
    auto widen = [&](int rows, int stride) {
        const int quads = hd / 4;
        for (int idx = tid; idx < kPfKeys * quads; idx += kPfThreads) {
            const int r = idx / quads, c = (idx - r * quads) * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (r < rows) v = *reinterpret_cast<const float4*>(stage + (size_t)r * rowf + c);
            double2* dst = reinterpret_cast<double2*>(KV + (size_t)r * stride + c);
            dst[0] = make_double2((double)v.x, (double)v.y);
            dst[1] = make_double2((double)v.z, (double)v.w);
        }
    };
    for (int t = 0; t < ntiles; ++t) {
        const int kpos0 = t * kPfKeys;
        const int krows = tile_rows(t);
        // ---- K tile: wait, widen, then the staging buffer is free for the V tile of the same positions ----
        if (!failed && !lb_mbar_wait_bounded(&bar, phase)) failed = true;
        phase ^= 1;
        widen(krows, kstride);
        __syncthreads();
        if (warp == 0) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            attn_fetch_rows(stage, vbase, hd, kpos0, krows, &bar, lane);
        }
        // ---- scores of this tile: S[16 x 32 per warp] = Q[16 x hd] * K^T ----
        {
            double c[2][4][2];
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) c[i][j][0] = c[i][j][1] = 0.0;
            const double* qa = Qs + (size_t)(wr + g) * qstride + t4;
            const double* kb = KV + (size_t)(wc + g) * kstride + t4;
#pragma unroll 4
            for (int d = 0; d < hd; d += 4) {
                const double a0 = qa[d], a1 = qa[(size_t)8 * qstride + d];
                double b[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) b[j] = kb[(size_t)(8 * j) * kstride + d];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    dmma_884(c[0][j], a0, b[j]);
                    dmma_884(c[1][j], a1, b[j]);
                }
            }
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    *reinterpret_cast<double2*>(Ss + (size_t)(wr + 8 * i + g) * sstride + wc + 8 * j + 2 * t4) =
                        make_double2(__dmul_rn(c[i][j][0], scale), __dmul_rn(c[i][j][1], scale));
        }
        __syncthreads();  // scores complete, the float64 K tile is free
        // ---- running softmax: four threads per row, sixteen keys each ----
        {
            const int r = tid >> 2, part = tid & 3;
            const int qpos = s_qpos[r];
            double* srow = Ss + (size_t)r * sstride + part * 16;
            double tmax = -1e300;
#pragma unroll 4
            for (int k = 0; k < 16; ++k)
                if (kpos0 + part * 16 + k <= qpos) tmax = fmax(tmax, srow[k]);
            tmax = fmax(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
            tmax = fmax(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
            const double m_old = s_m[r];
            const double m_new = fmax(m_old, tmax);
            double sum = 0.0;
#pragma unroll 4
            for (int k = 0; k < 16; ++k) {
                double e = 0.0;
                if (kpos0 + part * 16 + k <= qpos) e = exp(__dsub_rn(srow[k], m_new));
                srow[k] = e;
                sum = __dadd_rn(sum, e);
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            if (part == 0) {
                const double alpha = m_old > -1e299 ? exp(__dsub_rn(m_old, m_new)) : 0.0;
                s_alpha[r] = alpha;
                s_l[r] = __dadd_rn(__dmul_rn(s_l[r], alpha), sum);
                s_m[r] = m_new;
            }
        }
        // ---- V tile: wait, widen into the buffer K just left, request the next K tile ----
        if (!failed && !lb_mbar_wait_bounded(&bar, phase)) failed = true;
        phase ^= 1;
        widen(krows, vstride);
        __syncthreads();  // weights, rescale factors and the float64 V tile visible; staging free
        if (t + 1 < ntiles && warp == 0) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            attn_fetch_rows(stage, kbase, hd, kpos0 + kPfKeys, tile_rows(t + 1), &bar, lane);
        }
        // ---- weighted V: O[16 x hd/2 per warp] = alpha * O + P[16 x 64] * V ----
        {
            const double al0 = s_alpha[wr + g], al1 = s_alpha[wr + 8 + g];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                o[0][j][0] = __dmul_rn(o[0][j][0], al0);
                o[0][j][1] = __dmul_rn(o[0][j][1], al0);
                o[1][j][0] = __dmul_rn(o[1][j][0], al1);
                o[1][j][1] = __dmul_rn(o[1][j][1], al1);
            }
            const double* pa = Ss + (size_t)(wr + g) * sstride + t4;
            const double* vb = KV + (size_t)t4 * vstride + wd + g;
            const int kend = (krows + 3) & ~3;  // keys past krows carry zero weights and zero rows
#pragma unroll 2
            for (int k = 0; k < kend; k += 4) {
                const double a0 = pa[k], a1 = pa[(size_t)8 * sstride + k];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if (j < nfr) {
                        const double b = vb[(size_t)k * vstride + 8 * j];
                        dmma_884(o[0][j], a0, b);
                        dmma_884(o[1][j], a1, b);
                    }
                }
            }
        }
        __syncthreads();  // the float64 V tile and the weights are free
    }
    if (failed && tid == 0) atomicExch(p.status, 1);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = wr + 8 * i + g;
        const int hi = r / TQ, ti = r - hi * TQ;
        if (ti >= ntok) continue;
        const double den = s_l[r];
        double* orow = p.out + (size_t)(tok0 + ti) * qd + (size_t)(kvh * group + hi) * hd + wd + 2 * t4;
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (j < nfr) *reinterpret_cast<double2*>(orow + 8 * j) = make_double2(__ddiv_rn(o[i][j][0], den), __ddiv_rn(o[i][j][1], den));
    }
}

template <typename... Args>
cudaError_t launch_pdl(loom_b200_ctx* ctx, void (*kern)(Args...), dim3 grid, dim3 block, size_t smem, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->opt_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, args...);
}

}  // namespace

int lb_launch_embed(loom_b200_ctx* ctx, const float* emb, int vocab, int hidden, const int* tok_dev, int n, float* x) {
    LB_CUDA(ctx, launch_pdl(ctx, lb_embed_kernel, dim3(n), dim3(256), 0, emb, vocab, hidden, tok_dev, x));
    ctx->launches++;
    return 0;
}

int lb_launch_rope(loom_b200_ctx* ctx, const LbRopeParams& pin) {
    LbRopeParams p = pin;
    p.trace = lb_trace_row(ctx, "rope");
    LB_REQUIRE(ctx, p.hd % 2 == 0 && p.hd / 2 <= 1024, "rope: head_dim %d", p.hd);
    LB_CUDA(ctx, launch_pdl(ctx, lb_rope_kernel, dim3(p.heads + p.kv_heads, p.M), dim3(p.hd / 2), 0, p));
    ctx->launches++;
    return 0;
}

size_t lb_attn_part_elems(int M, int heads, int hd, int splits) { return (size_t)M * heads * splits * (hd + 2); }

int lb_launch_attention(loom_b200_ctx* ctx, const LbAttnParams& pin) {
    LbAttnParams p = pin;
    p.trace = lb_trace_row(ctx, "attention");
    p.status = ctx->status_dev;
    if (p.hd % 8 != 0) {  // small or odd head dimensions: the plain kernel
        LB_REQUIRE(ctx, p.rope_div == nullptr, "attention: RoPE cannot be folded in for head_dim %d", p.hd);
        LB_REQUIRE(ctx, p.heads % p.kv_heads == 0, "attention: %d heads over %d kv heads", p.heads, p.kv_heads);
        const size_t smem = (size_t)p.msl * sizeof(double);
        if (smem > 200 * 1024) return lb_fail(ctx, LOOM_B200_ERR_UNSUPPORTED, "attention: %d positions with head_dim %d", p.msl, p.hd);
        if (smem > 48 * 1024 && !(ctx->func_attr_mask2 & (1u << 16))) {
            LB_CUDA(ctx, cudaFuncSetAttribute(lb_attention_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            ctx->func_attr_mask2 |= 1u << 16;
        }
        p.trace = nullptr;
        LB_CUDA(ctx, launch_pdl(ctx, lb_attention_small_kernel, dim3(p.heads, p.M), dim3(32), smem, p));
        ctx->launches++;
        return 0;
    }
    LB_REQUIRE(ctx, p.heads % p.kv_heads == 0, "attention: %d heads over %d kv heads", p.heads, p.kv_heads);
    LB_REQUIRE(ctx, p.hd <= kAttnThreads, "attention: head_dim %d above %d is not supported", p.hd, kAttnThreads);
    LB_REQUIRE(ctx, p.splits >= 1 && p.splits <= 64, "attention: %d splits", p.splits);
    const int G = p.hd >= kAttnThreads ? 1 : kAttnThreads / p.hd;
    // tile: short tiles let more CTAs share an SM
    p.tile = ((p.max_chunk + 1) / 2 + 7) / 8 * 8;  // half of the longest chunk: two tiles at most when the ring is full
    if (p.tile > kAttnTile) p.tile = kAttnTile;
    if (p.tile < 8) p.tile = 8;
    size_t smem = (size_t)(p.hd + (size_t)G * p.hd + p.max_chunk) * sizeof(double) + 2 * (size_t)p.tile * p.hd * sizeof(float);
    if (smem > 200 * 1024) return lb_fail(ctx, LOOM_B200_ERR_UNSUPPORTED, "attention: %d positions per CTA need %zu B of shared memory", p.max_chunk, smem);
    if (smem > 48 * 1024 && !(ctx->func_attr_mask & (1u << 30))) {
        LB_CUDA(ctx, cudaFuncSetAttribute(lb_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        ctx->func_attr_mask |= 1u << 30;
    }
    LB_CUDA(ctx, launch_pdl(ctx, lb_attention_kernel, dim3(p.heads, p.M, p.splits), dim3(kAttnThreads), smem, p));
    ctx->launches++;
    return 0;
}

bool lb_attention_prefill_supported(const LbAttnParams& p) {
    const int group = p.kv_heads > 0 ? p.heads / p.kv_heads : 0;
    return p.kv_heads > 0 && p.heads % p.kv_heads == 0 && group >= 1 && group <= kPfRows && (kPfRows % group) == 0 &&
           p.hd % 16 == 0 && p.hd >= 16 && p.hd <= 128;
}

int lb_launch_attention_prefill(loom_b200_ctx* ctx, const LbAttnParams& pin) {
    LbAttnParams p = pin;
    p.trace = nullptr;
    p.status = ctx->status_dev;
    LB_REQUIRE(ctx, lb_attention_prefill_supported(p), "attention (prompt block): %d heads over %d kv heads of %d dimensions", p.heads,
               p.kv_heads, p.hd);
    const int TQ = kPfRows / (p.heads / p.kv_heads);
    const size_t smem = (size_t)kPfRows * (p.hd + 4) * sizeof(double) + (size_t)kPfKeys * (p.hd + 8) * sizeof(double) +
                        (size_t)kPfRows * (kPfKeys + 4) * sizeof(double) + (size_t)kPfKeys * p.hd * sizeof(float);
    if (!(ctx->func_attr_mask & (1u << 26))) {
        LB_CUDA(ctx, cudaFuncSetAttribute(lb_attention_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 216 * 1024));
        ctx->func_attr_mask |= 1u << 26;
    }
    LB_CUDA(ctx, launch_pdl(ctx, lb_attention_prefill_kernel, dim3(p.kv_heads, (p.M + TQ - 1) / TQ), dim3(kPfThreads), smem, p));
    ctx->launches++;
    return 0;
}

// the warp-per-row kernel with plain loads: hidden sizes the streaming kernel (lm_head.cu) has no room for, or unaligned tables
int lb_launch_lm_head_legacy(loom_b200_ctx* ctx, const LbLmHeadParams& pin) {
    LbLmHeadParams p = pin;
    p.trace = lb_trace_row(ctx, "lm_head");
    size_t smem = (size_t)p.hidden * sizeof(double);
    if (smem > 200 * 1024) return lb_fail(ctx, LOOM_B200_ERR_UNSUPPORTED, "lm_head: hidden %d too large", p.hidden);
    if (smem > 48 * 1024 && !(ctx->func_attr_mask & (1u << 29))) {
        LB_CUDA(ctx, cudaFuncSetAttribute(lb_lm_head_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        ctx->func_attr_mask |= 1u << 29;
    }
    int grid = ctx->sm_count * 4;
    int rows_per = (p.vocab + 7) / 8;
    if (grid > rows_per) grid = rows_per > 0 ? rows_per : 1;
    LB_CUDA(ctx, launch_pdl(ctx, lb_lm_head_kernel, dim3(grid), dim3(kHeadThreads), smem, p));
    ctx->launches++;
    return 0;
}

int lb_launch_argmax_advance(loom_b200_ctx* ctx, const float* logits, int vocab, int* tok, int* out_tokens, int out_cap,
                             int* step, int* pos) {
    // partial results live in the context scratch of the argmax (allocated once)
    if (!ctx->argmax_scratch) {
        if (ctx->capturing) return lb_fail(ctx, LOOM_B200_ERR_INVALID, "argmax scratch would be allocated while recording a graph");
        LB_CUDA(ctx, cudaMalloc(&ctx->argmax_scratch, kArgmaxCtas * 8 + 16));
        LB_CUDA(ctx, cudaMemsetAsync(ctx->argmax_scratch, 0, kArgmaxCtas * 8 + 16, ctx->stream));
    }
    float* pv = (float*)ctx->argmax_scratch;
    int* pi = (int*)(pv + kArgmaxCtas);
    unsigned int* cnt = (unsigned int*)(pi + kArgmaxCtas);
    int grid = kArgmaxCtas;
    if (grid > (vocab + 255) / 256) grid = (vocab + 255) / 256;
    if (grid < 1) grid = 1;
    LB_CUDA(ctx, launch_pdl(ctx, lb_argmax_advance_kernel, dim3(grid), dim3(256), 0, logits, vocab, tok, out_tokens, out_cap,
                            step, pos, pv, pi, cnt));
    ctx->launches++;
    return 0;
}

int lb_launch_add_scalar(loom_b200_ctx* ctx, int* pos, int delta) {
    LB_CUDA(ctx, launch_pdl(ctx, lb_add_scalar_kernel, dim3(1), dim3(32), 0, pos, delta));
    ctx->launches++;
    return 0;
}
