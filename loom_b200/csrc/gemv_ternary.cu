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
#include "gemv_device.cuh"


namespace {


// LEAN: the instantiation for the launches of a decode step -- aligned partition, the staged prologue (or int8 rows), no
// phase trace.  The code of the other paths (stream-K ranges and their fix-up, the general float prologue) is left out: code a launch never runs still
// costs it time (adding 200 instructions to an unused branch of the prologue slowed the decode step by 3 %).
template <bool MMA, int PRO, int EPI, bool LEAN = false>
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
        ptr += p.stage_bytes;
        sm.gain = p.gain_bytes > 0 ? reinterpret_cast<float*>(ptr) : nullptr;
        sm.pos0 = 0;
    }

    // ---- tile ranges --------------------------------------------------------------------------------
    // aligned: every CTA owns whole strip groups (no cross-CTA fix-up); otherwise stream-K over tiles.
    int t0, t1, first_group;
    const bool aligned = LEAN || p.aligned;
    if (aligned) {
        const int b = (int)blockIdx.x;
        const int g0 = b * p.part_q + (b < p.part_r ? b : p.part_r);
        const int g1 = g0 + p.part_q + (b < p.part_r ? 1 : 0);
        t0 = g0 * p.group * KB;
        t1 = g1 * p.group * KB;
        first_group = g0;
    } else {
        const long long T = p.total_tiles;
        t0 = (int)(T * blockIdx.x / gridDim.x);
        t1 = (int)(T * (blockIdx.x + 1) / gridDim.x);
        first_group = t1 > t0 ? (t0 / KB) / p.group : 0;
    }
    const int cta_tiles = t1 - t0;
    const int w0 = t0 + (int)(((unsigned)cta_tiles * (unsigned)warp) / (unsigned)kWarps);  // kWarps is a power of two
    const int w1 = t0 + (int)(((unsigned)cta_tiles * (unsigned)(warp + 1)) / (unsigned)kWarps);
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
    const uint64_t stream_policy = lb_policy_evict_first();  // the weights are read once per step
    auto issue = [&](int stage, const Cursor& c, int len) {  // lane 0 only
        lb_mbar_expect_tx(&my_bars[stage], (uint32_t)len * kTileBytes);
        lb_bulk_g2s_stream(my_ring + (size_t)stage * kStageBytes, tile_ptr<EPI, LEAN>(p, c.v, c.kb), (uint32_t)len * kTileBytes,
                           &my_bars[stage], stream_policy);
    };

    // first ring fill: weights do not depend on the producer of the activations
    Cursor ic;
    ic.pos = w0;
    if (LEAN || (aligned && KB > 1 && KB <= 256 && (unsigned)(w0 - t0) < 65536u)) {  // t0 is a strip boundary: only the small offset needs dividing (the lean launcher checked the ranges)
        const int dv = (int)__umulhi((unsigned)(w0 - t0), p.kb_magic);
        ic.v = local_v0 + dv;
        ic.kb = (w0 - t0) - dv * KB;
    } else {
        ic.v = w0 / KB;
        ic.kb = w0 - ic.v * KB;
    }
    Cursor cc = ic;
    for (int s = 0; s < nstages && ic.pos < w1; ++s) {
        int len = chunk_len(ic);
        if (lane == 0) issue(s, ic, len);
        advance(ic, len);
    }

    // the norm gains are weights too: copy them while the producer of the activations is still running
    if (sm.gain) {
        const int n4 = p.norm_w_len >> 2;
        for (int i = tid; i < n4; i += kThreads) reinterpret_cast<float4*>(sm.gain)[i] = __ldg(reinterpret_cast<const float4*>(p.norm_w) + i);
        if (!LEAN)  // (lean: the gains cover a row of K % 4 == 0 columns)
            for (int i = (n4 << 2) + tid; i < p.norm_w_len; i += kThreads) sm.gain[i] = __ldg(p.norm_w + i);
    }
    lb_pdl_launch_dependents();  // the next launch may start prefetching its weights
    LB_TRACE(1);
    lb_pdl_wait();               // everything below may read what earlier launches wrote
    LB_TRACE(2);
    if (p.pos_ptr) sm.pos0 = *p.pos_ptr;
    if (EPI == LB_EPI_TPSUM) sm.xseq_c = p.xchg_ctr[2];  // sequence number of this launch's exchange (moved on by the last CTA of the previous one)
    if (EPI == LB_EPI_RESID && M == 1 && cta_tiles > 0) {
        // the epilogue's operands of this CTA's rows: requested now, so that they are in L1 when the sums are done
        const int row0 = (t0 / KB) * kTileRows, nrows = ((t1 - 1) / KB + 1) * kTileRows - row0;
        if (tid < nrows && row0 + tid < p.seg[0].rows) {
            if (p.residual) asm volatile("prefetch.global.L1 [%0];" ::"l"(p.residual + row0 + tid));
            if (p.seg[0].bias) asm volatile("prefetch.global.L1 [%0];" ::"l"(p.seg[0].bias + row0 + tid));
        }
    }
    stage_activations<PRO, kWarps, LEAN>(p, sm);
    LB_TRACE(3);

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
    for (;;) {  // (one copy of the flush in the code: the sums of a strip are handed over when the next strip, or the end, comes up)
        const bool done = cc.pos >= w1;
        if (done || cc.v != cur_v) {
            flush();
            cur_v = cc.v;
        }
        if (done) break;
        const int len = chunk_len(cc);
        if (!failed && !lb_mbar_wait_bounded(&my_bars[cstage], cphase)) {
            failed = true;
            if (lane == 0) atomicExch(p.status, 1);
        }
        const uint8_t* tile = my_ring + (size_t)cstage * kStageBytes + lane * 16;
        const uint32_t* ab = act_base + cc.kb * act_kb_mul;
        if (!failed) {
            if (LEAN) {  // one rolled loop, two tiles per trip: half the code of the unrolled chunk plus its remainder loop
                int i = 0;
#pragma unroll 1
                for (; i + 2 <= len; i += 2) {
                    tile_step(tile + i * kTileBytes, ab + i * act_kb_mul);
                    tile_step(tile + (i + 1) * kTileBytes, ab + (i + 1) * act_kb_mul);
                }
                if (i < len) tile_step(tile + i * kTileBytes, ab + i * act_kb_mul);
            } else if (len == kStageTiles) {
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
    __syncthreads();
    LB_TRACE(4);

    // ---- strip groups: finish what this CTA owns entirely, hand the rest to the fix-up ------------------
    if (cta_tiles <= 0) return;
    const int group_tiles = p.group * KB;
    const int per_group = p.group * M * 16;
    if (EPI == LB_EPI_TPSUM) {
        // Row-parallel shard (always the aligned partition): this rank's corrected partial sums go to every other rank's
        // mailbox, then every output adds up what the ranks sent, in rank order (integer: exact), and finishes like
        // float(y + bias) + residual.  All stores first, then the polls, so that the NVLink latencies overlap.
        const int ngl_a = p.part_q + ((int)blockIdx.x < p.part_r ? 1 : 0);
        const LbGemvSeg& sg = p.seg[0];
        const uint32_t seq = sm.xseq_c;
        const size_t half = (size_t)(seq & 1);
        const int W = p.xchg_world, me = p.xchg_rank;
        for (int idx = tid; idx < ngl_a * per_group; idx += kThreads) {
            const int gl = idx / per_group, i = idx - gl * per_group;
            const int n = i >> 4, r = (first_group + gl) * kTileRows + (i & 15);
            if (r >= sg.rows) continue;
            const int mine = sm.sacc[idx] - sm.xsum[n];
            const size_t o = (size_t)n * sg.rows + r;
            for (int q = 0; q < W; ++q)
                if (q != me) ll_store((char*)p.xchg_peers[q] + kXRegionC + ((half * kXMaxRanks + me) * kXMaxAcc + o) * 8, (uint32_t)mine, seq);
        }
        bool ok = true;
        for (int idx = tid; idx < ngl_a * per_group; idx += kThreads) {
            const int gl = idx / per_group, i = idx - gl * per_group;
            const int n = i >> 4, r = (first_group + gl) * kTileRows + (i & 15);
            if (r >= sg.rows) continue;
            const size_t o = (size_t)n * sg.rows + r;
            int sum = 0;
            for (int q = 0; q < W; ++q) {
                uint32_t d = (uint32_t)(sm.sacc[idx] - sm.xsum[n]);
                if (q != me) ok = ll_wait((const char*)p.xchg_peers[me] + kXRegionC + ((half * kXMaxRanks + q) * kXMaxAcc + o) * 8, seq, &d) && ok;
                sum += (int)d;
            }
            double y = __dmul_rn((double)sum, sm.os[n]);
            if (sg.bias) y = __dadd_rn(y, (double)sg.bias[r]);
            float f = (float)y;
            if (p.residual) f = __fadd_rn(f, p.residual[o]);
            ((float*)sg.out)[o] = f;
        }
        if (!ok) atomicExch(p.status, 5);
        // the last CTA to get here moves the sequence numbers on (a CTA that starts late has read the old ones by now:
        // it cannot start before the launch's dependency is resolved, and it reads them right after)
        __syncthreads();
        if (tid == 0) {
            __threadfence();
            const unsigned int t = atomicAdd(&p.xchg_ctr[4], 1u);
            if (t == gridDim.x - 1) {
                p.xchg_ctr[4] = 0;
                __threadfence();
                p.xchg_ctr[2] = seq + 1;
            }
        }
        LB_TRACE(5);
        return;
    }
    if (aligned) {  // every group is this CTA's own: no fix-up, no flags
        const int ngl_a = p.part_q + ((int)blockIdx.x < p.part_r ? 1 : 0);
        for (int idx = tid; idx < ngl_a * per_group; idx += kThreads) {
            int gl, i, e, rem;
            if (LEAN) {  // a power-of-two token count (the launcher checked): shifts instead of divisions
                const int msh = 31 - __clz(M * 16), gsh = msh + (p.group == 2 ? 1 : 0);
                gl = idx >> gsh;
                i = idx & ((1 << gsh) - 1);
                e = i >> msh;
                rem = i & ((1 << msh) - 1);
            } else {
                if (per_group == 16) {
                    gl = idx >> 4;
                    i = idx & 15;
                } else {
                    gl = idx / per_group;
                    i = idx - gl * per_group;
                }
                e = i / (M * 16);
                rem = i - e * (M * 16);
            }
            finish_row<EPI, LEAN>(p, sm, (first_group + gl) * p.group, e, rem >> 4, rem & 15, sm.sacc + (size_t)gl * per_group);
        }
        LB_TRACE(5);
        return;
    }
    const int last_group = ((t1 - 1) / KB) / p.group;
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
        finish_row<EPI, LEAN>(p, sm, (first_group + gl) * p.group, e, rem >> 4, rem & 15, sm.sacc + (size_t)gl * per_group);
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
    b += (size_t)p.gain_bytes;
    return b;
}

}  // namespace

int lb_gemv_max_tokens(int K) {
    const int Kp = (K + kTileCols - 1) / kTileCols * kTileCols;
    const long long budget = 227 * 1024 - 2 * kWarps * kStageBytes - 12 * 1024;  // two ring stages, epilogue values, bookkeeping
    long long m = budget / (Kp + 16);
    return m >= kMaxM ? kMaxM : (m < 1 ? 1 : (int)m);
}

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

// Partition, ring depth and shared-memory footprint for a grid of SMs x cps CTAs.
static void gemv_plan(const loom_b200_ctx* ctx, LbGemvParams& p, int cps, int* grid_out, size_t* smem_out) {
    int vstrips = p.total_tiles / p.kblocks;
    int ngroups = (vstrips + p.group - 1) / p.group;
    int grid = ctx->sm_count * cps;
    // Enough strip groups to occupy the SMs: give every CTA whole groups and skip the cross-CTA fix-up.
    p.aligned = ctx->opt_gemv_partition == 1 ? 0 : (ctx->opt_gemv_partition == 2 ? 1 : (ngroups * 2 >= ctx->sm_count ? 1 : 0));
    if (p.epi == LB_EPI_TPSUM) p.aligned = 1;  // the exchange epilogue finishes whole rows inside one CTA
    if (p.aligned) {
        if (grid > ngroups) grid = ngroups;
        int gpc = (ngroups + grid - 1) / grid;
        p.max_local_strips = gpc * p.group;
        p.part_q = ngroups / grid;
        p.part_r = ngroups % grid;
        p.kb_magic = (unsigned)((0x100000000ull + (unsigned long long)p.kblocks - 1) / (unsigned long long)p.kblocks);
    } else {
        if (grid > p.total_tiles) grid = p.total_tiles;
        if (grid < 1) grid = 1;
        int tpc = (p.total_tiles + grid - 1) / grid;
        p.max_local_strips = (tpc + p.kblocks - 2) / p.kblocks + 1 + 2 * (p.group - 1);
    }
    // ring depth: as many stages as the busiest warp has chunks (a chunk = up to 8 tiles inside one strip), up to 3
    {
        int most = 1;
        const int KB = p.kblocks, gt = p.group * KB;
        const long long NG = p.total_tiles / gt;
        for (int b = 0; b < grid && most < kStages; ++b) {
            long long t0, t1;
            if (p.aligned) {
                const long long g0 = (long long)b * p.part_q + (b < p.part_r ? b : p.part_r);
                t0 = g0 * gt;
                t1 = (g0 + p.part_q + (b < p.part_r ? 1 : 0)) * gt;
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
    p.gain_bytes = 0;
    if (p.pro != LB_PRO_Q8 && (p.K & 3) == 0) {
        size_t want = (size_t)p.K * (p.pro == LB_PRO_INNERNORM64 ? 8 : 4);
        if (gemv_smem_bytes(p, p.max_local_strips) + want <= 227 * 1024) p.stage_bytes = (int)want;
    }
    if (p.stage_bytes > 0 && p.pro >= LB_PRO_BLOCKNORM && p.norm_w && p.norm_w_len > 0 && (((uintptr_t)p.norm_w) & 15) == 0) {
        const size_t want = ((size_t)p.norm_w_len * 4 + 15) & ~(size_t)15;
        if (gemv_smem_bytes(p, p.max_local_strips) + want <= 227 * 1024) p.gain_bytes = (int)want;
    }
    size_t smem = gemv_smem_bytes(p, p.max_local_strips);
    while (smem > 227 * 1024 && p.stages > 1) {  // wide inputs: a shallower ring before giving up
        --p.stages;
        smem = gemv_smem_bytes(p, p.max_local_strips);
    }
    *grid_out = grid;
    *smem_out = smem;
}

int lb_launch_gemv(loom_b200_ctx* ctx, const LbGemvParams& pin) {
    LbGemvParams p = pin;
    // Wide inputs, or three and more tokens: normalise and quantize once in a launch of its own (one CTA per token), then
    // stream the weights against the int8 rows.  The fused prologue is repeated by every CTA and costs it 4-6 us per token:
    // right for one or two tokens on the critical path of a decode step, wrong for a pass of eight.
    if (p.pro != LB_PRO_Q8 && (p.K >= kSplitQuantK || p.M >= kSplitQuantTokens) && (p.K & 3) == 0 && (((uintptr_t)p.x) & 15) == 0 &&
        (!p.norm_w || (((uintptr_t)p.norm_w) & 15) == 0) && (!p.norm_out || (((uintptr_t)p.norm_out) & 15) == 0) &&
        (!p.q_out || (((uintptr_t)p.q_out) & 3) == 0)) {
        const size_t qbytes = ((size_t)p.M * p.K + 255) & ~(size_t)255;
        if (int rc = lb_ensure_quant_scratch(ctx, qbytes + kMaxM * sizeof(float))) return rc;
        int8_t* q = p.q_out ? p.q_out : reinterpret_cast<int8_t*>(ctx->quant_scratch);
        float* amax = p.amax_out ? p.amax_out : reinterpret_cast<float*>((char*)ctx->quant_scratch + qbytes);
        if (int rc = lb_launch_norm_quantize(ctx, p, q, amax)) return rc;
        p.pro = LB_PRO_Q8;
        p.x = q;
        p.amax_in = amax;
        p.norm_w = nullptr;
        p.norm_w_len = 0;
        p.given_ss = nullptr;
        p.given_amax = nullptr;
        p.q_out = nullptr;
        p.amax_out = nullptr;
        p.norm_out = nullptr;
    }
    int vstrips = p.total_tiles / p.kblocks;
    int ngroups = (vstrips + p.group - 1) / p.group;
    int grid = 0;
    size_t smem = 0;
    int cps = ctx->opt_gemv_ctas_per_sm;
    if (p.K >= 16384 && cps > 1) cps = 1;  // very wide rows: every CTA stages the whole int8 row, so fewer, longer CTAs win (measured)
    gemv_plan(ctx, p, cps, &grid, &smem);
    // A grid sized for more CTAs per SM than the shared memory lets be resident would run in waves, and every
    // wave repeats the prologue: fall back to what fits (228 KB per SM, 1 KB reserved per CTA).
    while (cps > 1 && (smem + 1024) * (size_t)cps > 228 * 1024) {
        --cps;
        gemv_plan(ctx, p, cps, &grid, &smem);
    }
    if (int rc = lb_ensure_fixup(ctx, (size_t)ngroups * p.group * p.M * 16, (size_t)ngroups)) return rc;
    p.fix_acc = ctx->fix_acc;
    p.fix_cnt = ctx->fix_cnt;
    p.status = ctx->status_dev;
    p.trace = lb_trace_row(ctx, "gemv");
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
    LB_PICK(12, true, LB_PRO_Q8, LB_EPI_QKV)
    LB_PICK(13, true, LB_PRO_Q8, LB_EPI_RESID)
    LB_PICK(14, true, LB_PRO_BLOCKNORM, LB_EPI_GENERIC)
    LB_PICK(15, true, LB_PRO_Q8, LB_EPI_TPSUM)
#undef LB_PICK
    // the lean instantiations: the launches of a decode step (fused prologues), and their int8-row forms (a pass of several
    // sequences, tensor-parallel row shards, the plain ternary linear)
    // (cursor start by multiplication: 1 < k-blocks <= 256 and fewer than 65536 tiles per CTA; epilogue indices by shifts:
    //  a power-of-two token count)
    const bool lean_base = ctx->opt_gemv_lean && !p.trace && p.aligned && !use_dp4a && p.kblocks > 1 && p.kblocks <= 256 &&
                           (long long)(p.part_q + 1) * p.group * p.kblocks < 65536 && (p.M & (p.M - 1)) == 0;
    const bool lean = lean_base && (p.pro == LB_PRO_Q8 ||
                                    (p.stage_bytes > 0 && (p.K & 3) == 0 && (((uintptr_t)p.x) & 15) == 0 &&
                                     (!p.norm_w || ((((uintptr_t)p.norm_w) & 15) == 0 && p.norm_w_len == p.K && p.gain_bytes > 0)) && !p.norm_out && !p.q_out &&
                                     !p.amax_out && !p.given_ss && !p.given_amax));
#define LB_PICK_LEAN(id, pro_, epi_)                              \
    if (lean && p.pro == pro_ && p.epi == epi_) {                 \
        kern = lb_gemv_ternary_kernel<true, pro_, epi_, true>;    \
        kid = id;                                                 \
    }
    LB_PICK_LEAN(16, LB_PRO_BLOCKNORM, LB_EPI_QKV)
    LB_PICK_LEAN(17, LB_PRO_INNERNORM64, LB_EPI_RESID)
    LB_PICK_LEAN(18, LB_PRO_BLOCKNORM, LB_EPI_SWIGLU)
    LB_PICK_LEAN(19, LB_PRO_INNERNORM, LB_EPI_RESID)
    LB_PICK_LEAN(20, LB_PRO_Q8, LB_EPI_GENERIC)
    LB_PICK_LEAN(21, LB_PRO_Q8, LB_EPI_QKV)
    LB_PICK_LEAN(22, LB_PRO_Q8, LB_EPI_SWIGLU)
    LB_PICK_LEAN(23, LB_PRO_Q8, LB_EPI_RESID)
    LB_PICK_LEAN(24, LB_PRO_Q8, LB_EPI_TPSUM)
#undef LB_PICK_LEAN
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
    const int pass = lb_gemv_max_tokens(w->cols);  // tokens one pass carries: 8, fewer for very wide inputs
    for (int b0 = 0; b0 < batch; b0 += pass) {
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
        p.M = batch - b0 < pass ? batch - b0 : pass;
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
