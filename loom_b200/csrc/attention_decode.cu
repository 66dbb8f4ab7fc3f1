// attention_decode.cu -- causal GQA attention of ONE new token over the fp32 KV ring, as a thread-block cluster.
//
// Arithmetic: poly/mha.go:292-354 (RoPE of the query and of the newest K row in float64, scores dot(Q, K_f32) / sqrt(hd),
// max-subtracted exp, sum(p*V) / sum(p), all float64 over float32 K/V rows).  Replaces the decode use of the WGSL
// tiled attention (ShaderTiledMHAN, poly/wgpu_shaders.go:1112-1388).
//
// Shape of the kernel
//   * One cluster per KV head; the S CTAs of a cluster split the positions 0..pos into S contiguous slices.  A CTA
//     brings its K and V rows into shared memory with ONE bulk async copy each (the ring is head-major, so a slice is
//     one contiguous block) and serves all query heads of the GQA group from them: every K/V element is converted
//     to float64 once and used by every head of the group.
//   * Scores: a warp owns a position at a time, a lane four dimensions of it (the query slices live in registers);
//     sixteen (position, head) sums are reduced across the warp together so that the shuffle count per position stays small.
//   * The S partial results (max, sum, weighted V) never touch global memory: every CTA stores its partials straight
//     into the shared memory of the CTA that owns the output dimensions (distributed shared memory), one cluster
//     barrier orders the stores, and every CTA combines and writes hd/S dimensions of every head.  No atomics, no
//     last-arriver re-read, no global scratch.
//   * The K/V rows of the NEXT decoder block are prefetched into L2 while this block computes.
// The per-(head, split) kernel in glue.cu stays for chunks of several tokens, q/k norms and shapes this one refuses.
#include "glue.cuh"

namespace {

constexpr int kAcThreads = 512;
constexpr int kAcWarps = kAcThreads / 32;
constexpr int kAcMaxG = 8;   // query heads per KV head
constexpr int kAcMaxS = 16;  // CTAs per cluster

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_nctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
// address of the same shared-memory location in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_rank(const void* smem_ptr, uint32_t rank) {
    uint32_t a = lb_smem_u32(smem_ptr), r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_cluster_f64(uint32_t addr, double v) {
    asm volatile("st.shared::cluster.f64 [%0], %1;" ::"r"(addr), "d"(v) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void l2_prefetch(const void* gptr, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(gptr), "r"(bytes) : "memory");
}

// Sums NV = 4*G values per lane across the 32 lanes of a warp.  Each step halves the values a lane carries (it keeps
// one half and sends the other to its partner), so NV values cost about NV double shuffles instead of 5*NV.  Afterwards
// lane L holds, in v[0], the complete sum of value index(L); lanes that differ only in the low (5 - log2 NV) bits hold the same.
template <int NV>
__device__ __forceinline__ void warp_reduce_halving(double (&v)[NV], int lane) {
    int off = 16;
#pragma unroll
    for (int n = NV; n > 1; n >>= 1) {
        const int half = n >> 1;
        const bool upper = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < half; ++i) {
            const double send = upper ? v[i] : v[i + half];
            const double keep = upper ? v[i + half] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
        off >>= 1;
    }
    for (; off > 0; off >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], off);
}
// the value index lane L ends up with: one index bit per halving step, taken from the lane bits 16, 8, 4, ...
template <int NV>
__device__ __forceinline__ int halving_index(int lane) {
    int idx = 0, off = 16;
#pragma unroll
    for (int n = NV; n > 1; n >>= 1) {
        idx += (lane & off) ? (n >> 1) : 0;
        off >>= 1;
    }
    return idx;
}

// LEAN: one token of one sequence, no phase trace (what a decode step launches); the code of the other forms is left out.
// (Fixing the head dimension at compile time as well measured no better.)
template <int G, bool LEAN = false>
__global__ void __launch_bounds__(kAcThreads, 1) lb_attention_cluster_kernel(const LbAttnParams p) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[2];
    __shared__ double s_red[kAcWarps], s_red2[kAcWarps];  // per-warp maxima, per-warp sums (separate: no barrier between the two reductions)
    __shared__ double s_m[G], s_l[G];        // this CTA's maximum and sum per head
    __shared__ double s_gw[kAcMaxS * G];     // combine: weight of every (slice, head)
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hd = p.hd, half = hd >> 1, kvh = blockIdx.y;
    const int n = LEAN ? 0 : blockIdx.z;  // token of the pass; with seq_stride > 0 every token is a sequence of its own
    const size_t seq_off = LEAN ? 0 : (size_t)n * (size_t)p.seq_stride;
    const uint32_t rank = cluster_ctarank(), S = cluster_nctarank();
    const int cmax = p.max_chunk;  // positions one CTA holds at most
    const int dps = hd / (int)S;   // output dimensions every CTA combines
    float* kt = reinterpret_cast<float*>(smem_raw);            // [cmax, hd]
    float* vt = kt + (size_t)cmax * hd;                        // [cmax, hd]
    double* red = reinterpret_cast<double*>(smem_raw);         // after the weighted sums: [warps, G, hd] over the tiles
    double* sq = reinterpret_cast<double*>(smem_raw + p.tile); // p.tile = bytes of the tile / reduction region
    double* sc = sq + G * hd;                                  // [G, cmax] scores, then softmax weights
    double* part = sc + (size_t)G * cmax;                      // [S, G, dps + 2] partials received from every slice
    if (tid == 0) {
        lb_mbar_init(&bars[0], 1);
        lb_mbar_init(&bars[1], 1);
        lb_fence_mbar_init();
    }
    __syncthreads();
    // every CTA of the cluster is running before anyone stores into a neighbour's shared memory (waited for below)
    asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
    lb_pdl_launch_dependents();
    lb_pdl_wait();
    if (!LEAN) lb_trace(p.trace, 2);
    const int last = (!LEAN && p.seq_stride > 0) ? p.pos_ptr[n] : *p.pos_ptr;  // the new token's position; it attends to 0..last
    const int total = last + 1;
    const int per = (total + (int)S - 1) / (int)S;
    const int k0 = (int)rank * per;
    int k1 = k0 + per;
    if (k1 > total) k1 = total;
    const int cnt = k1 > k0 ? k1 - k0 : 0;
    const float* kbase = p.cache_k + seq_off + (size_t)kvh * p.msl * hd;
    const float* vbase = p.cache_v + seq_off + (size_t)kvh * p.msl * hd;
    if (cnt > 0 && lane == 0) {
        if (warp == 0) {
            lb_mbar_expect_tx(&bars[0], (uint32_t)cnt * hd * 4);
            lb_bulk_g2s_stream(kt, kbase + (size_t)k0 * hd, (uint32_t)cnt * hd * 4, &bars[0], lb_policy_evict_first());
        } else if (warp == 1) {
            lb_mbar_expect_tx(&bars[1], (uint32_t)cnt * hd * 4);
            lb_bulk_g2s_stream(vt, vbase + (size_t)k0 * hd, (uint32_t)cnt * hd * 4, &bars[1], lb_policy_evict_first());
        } else if (warp == 2 && p.next_k) {  // the next block's rows of the same positions, into L2
            l2_prefetch(p.next_k + ((size_t)kvh * p.msl + k0) * hd, (uint32_t)cnt * hd * 4);
            l2_prefetch(p.next_v + ((size_t)kvh * p.msl + k0) * hd, (uint32_t)cnt * hd * 4);
        }
    }
    // queries of the group, rotated (RoPE): thread idx owns the pair (d, d + hd/2) of head g
    double rsn = 0.0, rc = 1.0;
    for (int idx = tid; idx < G * half; idx += kAcThreads) {
        const int g = idx / half, d = idx - g * half;
        double sn, c;
        sincos(__ddiv_rn((double)last, p.rope_div[d]), &sn, &c);
        if (idx < half) {
            rsn = sn;
            rc = c;
        }
        const double* qrow = p.q + (size_t)n * p.heads * hd + (size_t)(kvh * G + g) * hd;
        const double v0 = qrow[d], v1 = qrow[d + half];
        sq[g * hd + d] = __dsub_rn(__dmul_rn(v0, c), __dmul_rn(v1, sn));
        sq[g * hd + d + half] = __dadd_rn(__dmul_rn(v0, sn), __dmul_rn(v1, c));
    }
    bool failed = false;
    if (cnt > 0 && !lb_mbar_wait_bounded(&bars[0], 0)) failed = true;
    if (cnt > 0 && last >= k0 && last < k1) {
        // the newest position belongs to this slice: its ring row is not written yet; rotate the row the QKV projection
        // left in k_new into the tile and into the ring (threads 0..hd/2-1 hold the sine and cosine of their pair)
        if (tid < half) {
            const float* knew = p.k_new + (size_t)n * p.kv_heads * hd + (size_t)kvh * hd;
            const double v0 = (double)knew[tid], v1 = (double)knew[tid + half];
            const float r0 = (float)__dsub_rn(__dmul_rn(v0, rc), __dmul_rn(v1, rsn));
            const float r1 = (float)__dadd_rn(__dmul_rn(v0, rsn), __dmul_rn(v1, rc));
            float* trow = kt + (size_t)(last - k0) * hd;
            trow[tid] = r0;
            trow[tid + half] = r1;
            float* grow = p.cache_k_w + seq_off + ((size_t)kvh * p.msl + (size_t)(last % p.msl)) * hd;
            grow[tid] = r0;
            grow[tid + half] = r1;
        }
    }
    __syncthreads();

    // ---- scores: warp = position, lane = four dimensions; PP positions x G heads = 16 sums are reduced together ----
    const double scale = __ddiv_rn(1.0, sqrt((double)hd));
    const bool lane_on = 4 * lane < hd;
    {
        constexpr int PP = 16 / G;
        double qv[G][4];
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int c = 0; c < 4; ++c) qv[g][c] = lane_on ? sq[g * hd + 4 * lane + c] : 0.0;
        const int vi = halving_index<16>(lane);  // this lane finishes value vi = pp * G + g
        for (int j0 = warp * PP; j0 < cnt; j0 += kAcWarps * PP) {
            double acc[16];
#pragma unroll
            for (int pp = 0; pp < PP; ++pp) {
                float4 kv = make_float4(0.f, 0.f, 0.f, 0.f);
                if (lane_on && j0 + pp < cnt) kv = *reinterpret_cast<const float4*>(kt + (size_t)(j0 + pp) * hd + 4 * lane);
                const double k0d = (double)kv.x, k1d = (double)kv.y, k2d = (double)kv.z, k3d = (double)kv.w;
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    double a = __dmul_rn(qv[g][0], k0d);
                    a = fma(qv[g][1], k1d, a);
                    a = fma(qv[g][2], k2d, a);
                    a = fma(qv[g][3], k3d, a);
                    acc[pp * G + g] = a;
                }
            }
            warp_reduce_halving<16>(acc, lane);
            const int pp = vi / G, g = vi - pp * G;
            if ((lane & 1) == 0 && j0 + pp < cnt) sc[g * cmax + j0 + pp] = __dmul_rn(acc[0], scale);
        }
    }
    __syncthreads();
    if (!LEAN) lb_trace(p.trace, 3);

    // ---- softmax over this slice, per head: the warps w with w % G == g share head g ----
    {
        constexpr int WPG = kAcWarps / G;  // warps per head
        const int g = warp % G, wq = warp / G;
        double mx = -1e300;
        for (int j = wq * 32 + lane; j < cnt; j += WPG * 32) mx = fmax(mx, sc[g * cmax + j]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmax(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if (lane == 0) s_red[warp] = mx;
        __syncthreads();
        mx = s_red[g];
#pragma unroll
        for (int w = 1; w < WPG; ++w) mx = fmax(mx, s_red[g + w * G]);
        double sum = 0.0;
        for (int j = wq * 32 + lane; j < cnt; j += WPG * 32) {
            const double e = exp(__dsub_rn(sc[g * cmax + j], mx));
            sc[g * cmax + j] = e;
            sum = __dadd_rn(sum, e);
        }
        sum = lb_warp_sum(sum);
        if (lane == 0) s_red2[warp] = sum;
        __syncthreads();
        if (tid < G) {
            double l = 0.0;
            for (int w = 0; w < WPG; ++w) l += s_red2[tid + w * G];
            s_l[tid] = l;
        }
        if (wq == 0 && lane == 0) s_m[g] = mx;  // every warp of head g holds the same maximum
    }
    if (cnt > 0 && !lb_mbar_wait_bounded(&bars[1], 0)) failed = true;
    __syncthreads();

    // ---- weighted V: warp = position, lane = four dimensions, all heads of the group from one converted row ----
    double acc[G][4];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[g][c] = 0.0;
    if (lane_on) {
        for (int j = warp; j < cnt; j += kAcWarps) {
            const float4 vv = *reinterpret_cast<const float4*>(vt + (size_t)j * hd + 4 * lane);
            const double v0 = (double)vv.x, v1 = (double)vv.y, v2 = (double)vv.z, v3 = (double)vv.w;
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const double w = sc[g * cmax + j];
                acc[g][0] = fma(w, v0, acc[g][0]);
                acc[g][1] = fma(w, v1, acc[g][1]);
                acc[g][2] = fma(w, v2, acc[g][2]);
                acc[g][3] = fma(w, v3, acc[g][3]);
            }
        }
    }
    if (failed && tid == 0) atomicExch(p.status, 1);
    __syncthreads();  // every warp is done with the K and V tiles: the reduction buffer takes their place
    if (lane_on) {
#pragma unroll
        for (int g = 0; g < G; ++g)
            *reinterpret_cast<double4*>(red + ((size_t)warp * G + g) * hd + 4 * lane) = make_double4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
    }
    __syncthreads();
    if (!LEAN) lb_trace(p.trace, 4);

    // ---- hand this slice's partials to the CTAs that own the output dimensions ----
    asm volatile("barrier.cluster.wait.aligned;" ::: "memory");  // completes the arrive at the top: every CTA has started
    // part[(slice * G + g) * (dps + 2)] = { max, sum, dps weighted-V values } in the receiving CTA's shared memory
    for (int idx = tid; idx < G * hd; idx += kAcThreads) {
        const int g = idx / hd, d = idx - g * hd;
        double v = 0.0;
#pragma unroll 4
        for (int w = 0; w < kAcWarps; ++w) v += red[((size_t)w * G + g) * hd + d];  // fixed order: the same bits on every replay
        const uint32_t owner = (uint32_t)(d / dps);
        st_cluster_f64(map_to_rank(part + ((size_t)rank * G + g) * (dps + 2) + 2 + (d - (int)owner * dps), owner), v);
    }
    for (int idx = tid; idx < (int)S * G; idx += kAcThreads) {
        const uint32_t owner = (uint32_t)(idx / G);
        const int g = idx - (int)owner * G;
        double* slot = part + ((size_t)rank * G + g) * (dps + 2);
        st_cluster_f64(map_to_rank(slot, owner), cnt > 0 ? s_m[g] : -1e300);
        st_cluster_f64(map_to_rank(slot + 1, owner), cnt > 0 ? s_l[g] : 0.0);
    }
    cluster_sync_all();

    // ---- combine the S slices for this CTA's dps dimensions of every head ----
    for (int idx = tid; idx < (int)S * G; idx += kAcThreads) {
        const int g = idx % G;
        double gm = -1e300;
        for (int r = 0; r < (int)S; ++r) gm = fmax(gm, part[((size_t)r * G + g) * (dps + 2)]);
        const int r = idx / G;
        const double ms = part[((size_t)r * G + g) * (dps + 2)], ls = part[((size_t)r * G + g) * (dps + 2) + 1];
        s_gw[r * G + g] = ls == 0.0 ? 0.0 : exp(__dsub_rn(ms, gm));
    }
    __syncthreads();
    for (int idx = tid; idx < G * dps; idx += kAcThreads) {
        const int g = idx / dps, dd = idx - g * dps;
        double num = 0.0, dn = 0.0;
        for (int r = 0; r < (int)S; ++r) {
            const double w = s_gw[r * G + g];
            if (w != 0.0) {  // not an empty slice
                const double* slot = part + ((size_t)r * G + g) * (dps + 2);
                num = fma(slot[2 + dd], w, num);
                dn = fma(slot[1], w, dn);
            }
        }
        p.out[(size_t)n * p.heads * hd + (size_t)(kvh * G + g) * hd + (int)rank * dps + dd] = __ddiv_rn(num, dn);
    }
    if (!LEAN) lb_trace(p.trace, 5);
}

// ------------------------------------------------------------------------------------------------------------------
// The throughput form for a pass of several sequences (one new token each): ONE CTA per (sequence, KV head) streams the
// sequence's whole context through double-buffered 64-position tiles (one bulk copy per K and per V tile) and keeps a
// running softmax, all query heads of the GQA group served from the same tiles.  A pass of eight sequences launches
// kv_heads x 8 such CTAs, which fit the device at once; the cluster kernel above would need sixteen CTAs for each of them
// and run in waves.  q arrives rotated and the newest K row is already in the ring (lb_rope_kernel ran before).
// Arithmetic as above; the running softmax rescales by exp(m_old - m_new) per tile (float64).
constexpr int kAsThreads = 256;
constexpr int kAsWarps = kAsThreads / 32;
constexpr int kAsTile = 64;  // positions per tile

template <int G>
__global__ void __launch_bounds__(kAsThreads, 1) lb_attention_stream_kernel(const LbAttnParams p) {
    static_assert(G == 4 || G == 8, "group sizes the score reduction is laid out for");
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[4];  // [stage][K, V]
    __shared__ double s_red[kAsWarps], s_red2[kAsWarps];
    __shared__ double s_m[G], s_l[G], s_alpha[2][G];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hd = p.hd, kvh = blockIdx.x, n = blockIdx.y;
    const size_t seq_off = (size_t)n * (size_t)(p.seq_stride > 0 ? p.seq_stride : 0);
    const size_t tile_elems = (size_t)kAsTile * hd;
    float* kt = reinterpret_cast<float*>(smem_raw);                 // [2][64, hd]
    float* vt = kt + 2 * tile_elems;                                // [2][64, hd]
    double* sq = reinterpret_cast<double*>(vt + 2 * tile_elems);    // [G, hd] queries
    double* sc = sq + G * hd;                                       // [2][G, 64] scores, then weights, per tile parity
    double* red = reinterpret_cast<double*>(smem_raw);              // after the last tile: [warps, G, hd] over the tiles
    if (tid == 0) {
        for (int i = 0; i < 4; ++i) lb_mbar_init(&bars[i], 1);
        lb_fence_mbar_init();
    }
    __syncthreads();
    lb_pdl_launch_dependents();
    lb_pdl_wait();
    const int last = p.seq_stride > 0 ? p.pos_ptr[n] : *p.pos_ptr + n;  // the token's position; it attends to 0..last
    const int total = last + 1;
    const int ntiles = (total + kAsTile - 1) / kAsTile;
    const float* kbase = p.cache_k + seq_off + (size_t)kvh * p.msl * hd;
    const float* vbase = p.cache_v + seq_off + (size_t)kvh * p.msl * hd;
    const uint64_t pol = lb_policy_evict_first();
    auto rows_of = [&](int t) { return total - t * kAsTile < kAsTile ? total - t * kAsTile : kAsTile; };
    auto issue = [&](int t) {  // one thread
        const int st = t & 1, rows = rows_of(t);
        lb_mbar_expect_tx(&bars[2 * st], (uint32_t)rows * hd * 4);
        lb_bulk_g2s_stream(kt + st * tile_elems, kbase + (size_t)t * kAsTile * hd, (uint32_t)rows * hd * 4, &bars[2 * st], pol);
        lb_mbar_expect_tx(&bars[2 * st + 1], (uint32_t)rows * hd * 4);
        lb_bulk_g2s_stream(vt + st * tile_elems, vbase + (size_t)t * kAsTile * hd, (uint32_t)rows * hd * 4, &bars[2 * st + 1], pol);
    };
    if (tid == 0) {
        issue(0);
        if (ntiles > 1) issue(1);
    }
    for (int idx = tid; idx < G * hd; idx += kAsThreads) sq[idx] = p.q[(size_t)n * p.heads * hd + (size_t)kvh * G * hd + idx];
    if (tid < G) {
        s_m[tid] = -1e300;
        s_l[tid] = 0.0;
    }
    __syncthreads();
    const double scale = __ddiv_rn(1.0, sqrt((double)hd));
    const bool lane_on = 4 * lane < hd;
    constexpr int PP = 16 / G;           // positions whose G sums are reduced together
    constexpr int WPG = kAsWarps / G < 1 ? 1 : kAsWarps / G;  // warps that share a head in the softmax (G = 8: one)
    double qv[G][4];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int c = 0; c < 4; ++c) qv[g][c] = lane_on ? sq[g * hd + 4 * lane + c] : 0.0;
    const int vi = halving_index<16>(lane);
    double o[G][4];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int c = 0; c < 4; ++c) o[g][c] = 0.0;
    bool failed = false;
    for (int t = 0; t < ntiles; ++t) {
        const int st = t & 1, rows = rows_of(t);
        const uint32_t ph = (uint32_t)((t >> 1) & 1);
        const float* ktile = kt + st * tile_elems;
        const float* vtile = vt + st * tile_elems;
        double* sct = sc + (size_t)st * G * kAsTile;
        if (!failed && !lb_mbar_wait_bounded(&bars[2 * st], ph)) failed = true;
        // ---- scores of the tile: warp = eight positions, lane = four dimensions ----
        for (int j0 = warp * (kAsTile / kAsWarps); j0 < (warp + 1) * (kAsTile / kAsWarps); j0 += PP) {
            double acc[16];
#pragma unroll
            for (int pp = 0; pp < PP; ++pp) {
                float4 kv = make_float4(0.f, 0.f, 0.f, 0.f);
                if (lane_on && j0 + pp < rows) kv = *reinterpret_cast<const float4*>(ktile + (size_t)(j0 + pp) * hd + 4 * lane);
                const double k0d = (double)kv.x, k1d = (double)kv.y, k2d = (double)kv.z, k3d = (double)kv.w;
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    double a = __dmul_rn(qv[g][0], k0d);
                    a = fma(qv[g][1], k1d, a);
                    a = fma(qv[g][2], k2d, a);
                    a = fma(qv[g][3], k3d, a);
                    acc[pp * G + g] = a;
                }
            }
            warp_reduce_halving<16>(acc, lane);
            const int pp = vi / G, g = vi - pp * G;
            if ((lane & 1) == 0) sct[g * kAsTile + j0 + pp] = j0 + pp < rows ? __dmul_rn(acc[0], scale) : -1e300;  // absent positions: weight 0
        }
        __syncthreads();  // scores complete; every warp is past the weighted sum of tile t - 1
        if (tid == 0 && t >= 1 && t + 1 < ntiles) issue(t + 1);  // into the buffers tile t - 1 has just left
        // ---- running softmax, per head ----
        {
            const int g = warp % G, wq = warp / G;
            double mx = -1e300;
            for (int j = wq * 32 + lane; j < kAsTile; j += WPG * 32) mx = fmax(mx, sct[g * kAsTile + j]);
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) mx = fmax(mx, __shfl_xor_sync(0xffffffffu, mx, off));
            if (lane == 0) s_red[warp] = mx;
            __syncthreads();
            mx = s_red[g];
#pragma unroll
            for (int w = 1; w < WPG; ++w) mx = fmax(mx, s_red[g + w * G]);
            const double m_old = s_m[g];
            const double m_new = fmax(m_old, mx);
            double sum = 0.0;
            for (int j = wq * 32 + lane; j < kAsTile; j += WPG * 32) {
                const double e = j < rows ? exp(__dsub_rn(sct[g * kAsTile + j], m_new)) : 0.0;
                sct[g * kAsTile + j] = e;
                sum = __dadd_rn(sum, e);
            }
            sum = lb_warp_sum(sum);
            if (lane == 0) s_red2[warp] = sum;
            __syncthreads();  // weights and per-warp sums visible; everyone has read the old maximum
            if (wq == 0 && lane == 0) {
                double l = 0.0;
                for (int w = 0; w < WPG; ++w) l += s_red2[g + w * G];
                const double alpha = exp(__dsub_rn(m_old, m_new));  // 0 for the first tile (m_old = -1e300)
                s_alpha[st][g] = alpha;
                s_l[g] = __dadd_rn(__dmul_rn(s_l[g], alpha), l);
                s_m[g] = m_new;
            }
        }
        if (!failed && !lb_mbar_wait_bounded(&bars[2 * st + 1], ph)) failed = true;
        __syncthreads();  // rescale factors visible
        // ---- weighted V: warp = every eighth position, lane = four dimensions ----
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const double al = s_alpha[st][g];
#pragma unroll
            for (int c = 0; c < 4; ++c) o[g][c] = __dmul_rn(o[g][c], al);
        }
        if (lane_on) {
            for (int j = warp; j < rows; j += kAsWarps) {
                const float4 vv = *reinterpret_cast<const float4*>(vtile + (size_t)j * hd + 4 * lane);
                const double v0 = (double)vv.x, v1 = (double)vv.y, v2 = (double)vv.z, v3 = (double)vv.w;
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const double w = sct[g * kAsTile + j];
                    o[g][0] = fma(w, v0, o[g][0]);
                    o[g][1] = fma(w, v1, o[g][1]);
                    o[g][2] = fma(w, v2, o[g][2]);
                    o[g][3] = fma(w, v3, o[g][3]);
                }
            }
        }
    }
    if (failed && tid == 0) atomicExch(p.status, 1);
    __syncthreads();  // every warp is done with the tiles: the reduction buffer takes their place
    if (lane_on) {
#pragma unroll
        for (int g = 0; g < G; ++g)
            *reinterpret_cast<double4*>(red + ((size_t)warp * G + g) * hd + 4 * lane) = make_double4(o[g][0], o[g][1], o[g][2], o[g][3]);
    }
    __syncthreads();
    for (int idx = tid; idx < G * hd; idx += kAsThreads) {
        const int g = idx / hd, d = idx - g * hd;
        double v = 0.0;
#pragma unroll
        for (int w = 0; w < kAsWarps; ++w) v += red[((size_t)w * G + g) * hd + d];  // fixed order: the same bits on every replay
        p.out[(size_t)n * p.heads * hd + (size_t)(kvh * G + g) * hd + d] = __ddiv_rn(v, s_l[g]);
    }
}

template <int G>
int launch_stream_attention(loom_b200_ctx* ctx, const LbAttnParams& p) {
    const size_t smem = (size_t)4 * kAsTile * p.hd * sizeof(float) + (size_t)G * p.hd * 8 + (size_t)2 * G * kAsTile * 8;
    auto kern = lb_attention_stream_kernel<G>;
    const unsigned bit = 1u << (G == 4 ? 13 : 14);  // (bits 0-7: the cluster kernel, 8-12: the streaming head, 16, 20-27: others)
    if (!(ctx->func_attr_mask2 & bit)) {
        LB_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        ctx->func_attr_mask2 |= bit;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.kv_heads, p.M);
    cfg.blockDim = dim3(kAsThreads);
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

template <int G>
size_t cluster_smem(const LbAttnParams& p, int S, int* tile_bytes) {
    const int cmax = (p.msl + S - 1) / S;
    size_t tiles = (size_t)2 * cmax * p.hd * sizeof(float);
    const size_t red = (size_t)kAcWarps * G * p.hd * sizeof(double);
    if (red > tiles) tiles = red;
    tiles = (tiles + 127) & ~(size_t)127;
    *tile_bytes = (int)tiles;
    const int dps = p.hd / S;
    return tiles + (size_t)G * p.hd * 8 + (size_t)G * cmax * 8 + (size_t)S * G * (dps + 2) * 8;
}

template <int G>
int launch_cluster(loom_b200_ctx* ctx, LbAttnParams p, int S, bool probe_only, int* active_clusters) {
    int tile_bytes = 0;
    const size_t smem = cluster_smem<G>(p, S, &tile_bytes);
    if (smem > 200 * 1024) return LOOM_B200_ERR_UNSUPPORTED;
    p.tile = tile_bytes;
    p.max_chunk = (p.msl + S - 1) / S;
    const bool lean = !probe_only && !p.trace && p.M == 1 && p.seq_stride <= 0;
    auto kern = lean ? lb_attention_cluster_kernel<G, true> : lb_attention_cluster_kernel<G, false>;
    const unsigned bit = 1u << ((G == 1 ? 0 : G == 2 ? 1 : G == 4 ? 2 : 3) + (lean ? 4 : 0));  // one bit per instantiation, per context (= per device)
    if (!(ctx->func_attr_mask2 & bit)) {
        LB_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        LB_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
        ctx->func_attr_mask2 |= bit;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(S, p.kv_heads, p.M);
    cfg.blockDim = dim3(kAcThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = S;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->opt_pdl ? 2 : 1;
    if (probe_only) {
        cfg.numAttrs = 1;
        int n = 0;
        cudaError_t e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
        if (e != cudaSuccess) {
            cudaGetLastError();
            n = 0;
        }
        *active_clusters = n;
        return 0;
    }
    LB_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, p));
    ctx->launches++;
    return 0;
}

int dispatch_cluster(loom_b200_ctx* ctx, const LbAttnParams& p, int S, bool probe_only, int* active) {
    switch (p.heads / p.kv_heads) {
        case 1: return launch_cluster<1>(ctx, p, S, probe_only, active);
        case 2: return launch_cluster<2>(ctx, p, S, probe_only, active);
        case 4: return launch_cluster<4>(ctx, p, S, probe_only, active);
        case 8: return launch_cluster<8>(ctx, p, S, probe_only, active);
        default: return LOOM_B200_ERR_UNSUPPORTED;
    }
}

}  // namespace

int lb_attention_cluster_size(loom_b200_ctx* ctx, const LbAttnParams& p, bool one_wave) {
    if ((p.M != 1 && p.seq_stride <= 0) || !p.rope_div || !p.k_new || !p.cache_k_w) return 0;
    if (p.kv_heads <= 0 || p.heads % p.kv_heads != 0) return 0;
    const int G = p.heads / p.kv_heads;
    if (G != 1 && G != 2 && G != 4 && G != 8) return 0;
    if (p.hd % 16 != 0 || p.hd > 128 || p.hd < 16) return 0;
    // the largest cluster size the device can launch for this shape
    const int smax = ctx->opt_attn_cluster >= 2 && ctx->opt_attn_cluster < kAcMaxS ? ctx->opt_attn_cluster : kAcMaxS;  // option: 1 = the largest that fits, 2..16 = at most that
    for (int S = kAcMaxS; S >= 2; S >>= 1) {
        if (S > smax) continue;
        if (p.hd % S != 0) continue;
        int active = 0;
        if (dispatch_cluster(ctx, p, S, true, &active) != 0) continue;
        // One sequence: only when every KV head's cluster is resident at once (one wave) -- in waves the split kernel is the
        // faster one (measured at 8 KV heads: 511 against 464 tok/s).  Several sequences launch many clusters anyway and
        // take whatever size the device can launch: the clusters do not depend on one another.
        if (one_wave ? (active >= p.kv_heads || (S == 2 && active >= 1)) : active >= 1) return S;
    }
    return 0;
}

int lb_launch_attention_cluster(loom_b200_ctx* ctx, const LbAttnParams& pin, int S) {
    LbAttnParams p = pin;
    p.trace = lb_trace_row(ctx, "attention");
    p.status = ctx->status_dev;
    int rc = dispatch_cluster(ctx, p, S, false, nullptr);
    if (rc == LOOM_B200_ERR_UNSUPPORTED) return lb_fail(ctx, rc, "attention (cluster): shape not supported");
    return rc;
}

// A pass of several sequences through the streaming kernel: head dimension 128 (tiles of 64 x 512 B), four or eight query
// heads per KV head, plain attention (q rotated, the newest K row already in the ring).
bool lb_attention_stream_supported(const loom_b200_ctx* ctx, const LbAttnParams& p) {
    if (!ctx->opt_attn_stream || p.hd != 128 || p.kv_heads <= 0 || p.heads % p.kv_heads != 0) return false;
    const int G = p.heads / p.kv_heads;
    return G == 4 || G == 8;
}

int lb_launch_attention_stream(loom_b200_ctx* ctx, const LbAttnParams& pin) {
    LbAttnParams p = pin;
    p.status = ctx->status_dev;
    p.trace = nullptr;
    return p.heads / p.kv_heads == 4 ? launch_stream_attention<4>(ctx, p) : launch_stream_attention<8>(ctx, p);
}
