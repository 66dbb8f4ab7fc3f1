// stream_program.cu -- a recorded list of ternary linears executed by ONE persistent launch.
//
// A decode step is a long chain of small matrix-vector products (1.6 - 8.8 MB of packed weights each).  Launched
// one by one, each of them pays its own start-up: cold instruction fetch, activation staging and an empty weight
// pipeline.  Here one CTA per SM stays resident for the whole list.  Every warp walks its slice of job after job
// and keeps its private shared-memory ring full with 1-D bulk async copies (TMA engine) that run several jobs
// ahead, so HBM keeps streaming weights while the CTA stages the next activation vector or writes an epilogue,
// and the instruction stream stays resident.  Jobs may depend on the job before them (grid_wait): all CTAs then
// meet at a bounded-wait grid barrier before staging activations; weight prefetch is never held back by it.
//
// Replaces a frame of DispatchDenseBitNetTernaryQuantized calls between BeginFrame and FlushFrame
// (poly/wgpu_kernels.go:416-475, poly/wgpu_context_native.go:263-276).
#include "gemv_device.cuh"

#include <vector>

struct LbJob {
    LbGemvParams p;
    int grid_wait;  // 1: every CTA must have finished the previous job before this one reads its inputs
    int pad[3];
};

struct LbStreamParams {
    const LbJob* jobs;
    int njobs;
    int stages;            // ring stages per warp
    int acts_bytes;        // largest staged activation block over all jobs
    int sacc_ints;         // largest per-CTA accumulator block
    int stage_bytes;       // largest prologue staging buffer
    unsigned int* barrier; // grid barrier counter (zero at launch)
    int* status;
};

struct loom_b200_program {
    LbJob* jobs_dev = nullptr;
    unsigned int* barrier_dev = nullptr;
    LbStreamParams sp{};
    size_t smem = 0;
    int grid = 0;
    uint64_t bytes = 0;  // algorithmic bytes of one run
};

namespace {

constexpr int kPStagesMax = 6;

// my slice of a job: whole strip groups per CTA, then eight contiguous warp ranges
__device__ __forceinline__ void warp_range(const LbGemvParams& p, int warp, int& w0, int& w1) {
    const int gt = p.group * p.kblocks;
    const long long NG = p.total_tiles / gt;
    const int t0 = (int)(NG * blockIdx.x / gridDim.x) * gt, t1 = (int)(NG * (blockIdx.x + 1) / gridDim.x) * gt;
    const int n = t1 - t0;
    w0 = t0 + (int)((long long)n * warp / kWarps);
    w1 = t0 + (int)((long long)n * (warp + 1) / kWarps);
}

struct JCursor {
    int job, pos, v, kb, w1, KB;
};

__device__ __forceinline__ void cursor_enter(JCursor& c, const LbJob* jobs, int njobs, int job, int warp) {
    // moves to the first job at or after `job` in which this warp has tiles
    for (; job < njobs; ++job) {
        int w0, w1;
        warp_range(jobs[job].p, warp, w0, w1);
        if (w0 < w1) {
            c.job = job;
            c.KB = jobs[job].p.kblocks;
            c.pos = w0;
            c.w1 = w1;
            c.v = w0 / c.KB;
            c.kb = w0 - c.v * c.KB;
            return;
        }
    }
    c.job = njobs;
    c.pos = c.w1 = 0;
}

__device__ __forceinline__ int cursor_len(const JCursor& c) {
    int len = c.KB - c.kb;
    if (len > kStageTiles) len = kStageTiles;
    if (len > c.w1 - c.pos) len = c.w1 - c.pos;
    return len;
}

__device__ __forceinline__ void cursor_advance(JCursor& c, int len) {
    c.pos += len;
    c.kb += len;
    if (c.kb >= c.KB) {
        c.kb = 0;
        c.v++;
    }
}

// Bounded grid barrier: returns false when the wait ran out (the caller raises the status word and goes on).
__device__ __forceinline__ bool grid_barrier(unsigned int* counter, unsigned int target) {
    __shared__ int ok;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(counter, 1u);
        int good = 0;
        for (unsigned it = 0; it < 20000000u; ++it) {
            unsigned v;
            asm volatile("ld.acquire.gpu.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
            if (v >= target) {
                good = 1;
                break;
            }
        }
        __threadfence();
        ok = good;
    }
    __syncthreads();
    return ok != 0;
}

template <int PRO>
__device__ __noinline__ void stage_job(const LbGemvParams& p, const Smem& sm) {
    stage_activations<PRO>(p, sm);
}

template <int EPI>
__device__ __noinline__ void finish_job(const LbGemvParams& p, const Smem& sm, int first_group, int ngl) {
    const int per_group = p.group * p.M * 16;
    for (int idx = threadIdx.x; idx < ngl * per_group; idx += kThreads) {
        const int gl = idx / per_group, i = idx - gl * per_group;
        const int e = i / (p.M * 16), rem = i - e * (p.M * 16);
        finish_row<EPI>(p, sm, (first_group + gl) * p.group, e, rem >> 4, rem & 15, sm.sacc + (size_t)gl * per_group);
    }
}

__global__ void __launch_bounds__(kThreads, 1) lb_stream_kernel(const __grid_constant__ LbStreamParams sp) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ LbGemvParams job;  // the current job's parameter block
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nstages = sp.stages;

    Smem sm;
    {
        uint8_t* ptr = smem_raw;
        sm.ring = ptr;
        ptr += (size_t)kWarps * nstages * kStageBytes;
        sm.acts = reinterpret_cast<uint32_t*>(ptr);
        ptr += sp.acts_bytes;
        sm.sacc = reinterpret_cast<int*>(ptr);
        ptr += (size_t)sp.sacc_ints * 4;
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
        ptr += kWarps * kPStagesMax * 8;
        sm.stage = sp.stage_bytes > 0 ? (void*)ptr : nullptr;
        sm.gain = nullptr;  // the program reads norm gains from global memory
        sm.pos0 = 0;
    }
    if (tid < kWarps * nstages) lb_mbar_init(&sm.bars[tid], 1);
    if (tid == 0) lb_fence_mbar_init();
    __syncthreads();

    uint8_t* my_ring = sm.ring + (size_t)warp * nstages * kStageBytes;
    uint64_t* my_bars = sm.bars + warp * nstages;
    JCursor ic, cc;
    cursor_enter(ic, sp.jobs, sp.njobs, 0, warp);
    cc = ic;
    unsigned issued = 0, consumed = 0;  // chunks of this warp, over the whole program
    bool failed = false;

    // keeps this warp's ring full, running ahead into later jobs
    auto pump = [&]() {
        while (issued - consumed < (unsigned)nstages && ic.job < sp.njobs) {
            const int len = cursor_len(ic);
            if (lane == 0) {
                const int stage = (int)(issued % (unsigned)nstages);
                lb_mbar_expect_tx(&my_bars[stage], (uint32_t)len * kTileBytes);
                lb_bulk_g2s(my_ring + (size_t)stage * kStageBytes, tile_ptr(sp.jobs[ic.job].p, ic.v, ic.kb), (uint32_t)len * kTileBytes,
                            &my_bars[stage]);
            }
            ++issued;
            cursor_advance(ic, len);
            if (ic.pos >= ic.w1) cursor_enter(ic, sp.jobs, sp.njobs, ic.job + 1, warp);
        }
    };
    pump();

    const int g = lane >> 2, t = lane & 3;
    unsigned barriers_done = 0;
    for (int j = 0; j < sp.njobs; ++j) {
        __syncthreads();  // the previous job's epilogue is done with the shared buffers
        {
            const uint32_t* src = reinterpret_cast<const uint32_t*>(&sp.jobs[j].p);
            uint32_t* dst = reinterpret_cast<uint32_t*>(&job);
            for (int i = tid; i < (int)(sizeof(LbGemvParams) / 4); i += kThreads) dst[i] = src[i];
        }
        const int grid_wait = sp.jobs[j].grid_wait;
        if (grid_wait) {
            ++barriers_done;
            if (!grid_barrier(sp.barrier, barriers_done * gridDim.x) && tid == 0) atomicExch(sp.status, 2);
        }
        __syncthreads();
        const LbGemvParams& p = job;
        if (p.pos_ptr) sm.pos0 = *p.pos_ptr;
        const int KB = p.kblocks, M = p.M;
        const int gt = p.group * KB;
        const long long NG = p.total_tiles / gt;
        const int g0 = (int)(NG * blockIdx.x / gridDim.x), g1 = (int)(NG * (blockIdx.x + 1) / gridDim.x);
        const int ngl = g1 - g0;
        lb_trace(p.trace, 0);
        if (ngl > 0) {
            for (int i = tid; i < ngl * p.group * M * 16; i += kThreads) sm.sacc[i] = 0;
        }
        lb_trace(p.trace, 2);
        if (ngl > 0) {  // a CTA without rows in this job has nothing to stage
            switch (p.pro) {
                case LB_PRO_Q8: stage_job<LB_PRO_Q8>(p, sm); break;
                case LB_PRO_F32: stage_job<LB_PRO_F32>(p, sm); break;
                case LB_PRO_BLOCKNORM: stage_job<LB_PRO_BLOCKNORM>(p, sm); break;
                case LB_PRO_INNERNORM: stage_job<LB_PRO_INNERNORM>(p, sm); break;
                default: stage_job<LB_PRO_INNERNORM64>(p, sm); break;
            }
        }
        lb_trace(p.trace, 3);

        // ---- dot products of this warp's tiles of job j ----
        if (cc.job == j) {
            const int Kp = KB * kTileCols, stride32 = (Kp + 16) / 4;
            const uint32_t* act_base;
            int act_kb_mul;
            if (g < M) {
                act_base = sm.acts + (size_t)g * stride32 + t * 8;
                act_kb_mul = 32;
            } else {
                act_base = sm.acts + (size_t)M * stride32;  // zero block
                act_kb_mul = 0;
            }
            const int local_v0 = g0 * p.group;
            int acc[4][4];
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) acc[a][b] = 0;
            int cur_v = -1;
            auto flush = [&]() {
                if (cur_v < 0) return;
                int* dst = sm.sacc + (size_t)(cur_v - local_v0) * M * 16;
                const int v0 = acc[0][0] + (acc[1][0] >> 2) + (acc[2][0] >> 4) + (acc[3][0] >> 6);
                const int v1 = acc[0][1] + (acc[1][1] >> 2) + (acc[2][1] >> 4) + (acc[3][1] >> 6);
                const int v2 = acc[0][2] + (acc[1][2] >> 2) + (acc[2][2] >> 4) + (acc[3][2] >> 6);
                const int v3 = acc[0][3] + (acc[1][3] >> 2) + (acc[2][3] >> 4) + (acc[3][3] >> 6);
                const int n0 = 2 * t, n1 = 2 * t + 1;
                if (n0 < M) {
                    atomicAdd(&dst[n0 * 16 + g], v0);
                    atomicAdd(&dst[n0 * 16 + g + 8], v2);
                }
                if (n1 < M) {
                    atomicAdd(&dst[n1 * 16 + g], v1);
                    atomicAdd(&dst[n1 * 16 + g + 8], v3);
                }
#pragma unroll
                for (int a = 0; a < 4; ++a)
#pragma unroll
                    for (int b = 0; b < 4; ++b) acc[a][b] = 0;
            };
            auto tile_step = [&](const uint8_t* tile, const uint32_t* ab) {
                const uint4 w = *reinterpret_cast<const uint4*>(tile);
                const uint4 b01 = *reinterpret_cast<const uint4*>(ab);
                const uint4 b23 = *reinterpret_cast<const uint4*>(ab + 4);
                mma_u8s8(acc[0], w.x & 0x03030303u, w.y & 0x03030303u, w.z & 0x03030303u, w.w & 0x03030303u, b01.x, b01.y);
                mma_u8s8(acc[1], w.x & 0x0c0c0c0cu, w.y & 0x0c0c0c0cu, w.z & 0x0c0c0c0cu, w.w & 0x0c0c0c0cu, b01.z, b01.w);
                mma_u8s8(acc[2], w.x & 0x30303030u, w.y & 0x30303030u, w.z & 0x30303030u, w.w & 0x30303030u, b23.x, b23.y);
                mma_u8s8(acc[3], w.x & 0xc0c0c0c0u, w.y & 0xc0c0c0c0u, w.z & 0xc0c0c0c0u, w.w & 0xc0c0c0c0u, b23.z, b23.w);
            };
            while (cc.job == j) {
                const int len = cursor_len(cc);
                const int stage = (int)(consumed % (unsigned)nstages);
                const uint32_t parity = (consumed / (unsigned)nstages) & 1u;
                if (!failed && !lb_mbar_wait_bounded(&my_bars[stage], parity)) {
                    failed = true;
                    if (lane == 0) atomicExch(sp.status, 1);
                }
                if (cc.v != cur_v) {
                    flush();
                    cur_v = cc.v;
                }
                const uint8_t* tile = my_ring + (size_t)stage * kStageBytes + lane * 16;
                const uint32_t* ab = act_base + cc.kb * act_kb_mul;
                if (!failed) {
                    if (len == kStageTiles) {
#pragma unroll
                        for (int i = 0; i < kStageTiles; ++i) tile_step(tile + i * kTileBytes, ab + i * act_kb_mul);
                    } else {
                        for (int i = 0; i < len; ++i) tile_step(tile + i * kTileBytes, ab + i * act_kb_mul);
                    }
                }
                cursor_advance(cc, len);
                if (cc.pos >= cc.w1) cursor_enter(cc, sp.jobs, sp.njobs, cc.job + 1, warp);
                ++consumed;
                __syncwarp();
                if (lane == 0) fence_proxy_async();
                pump();
            }
            flush();
        }
        __syncthreads();
        lb_trace(p.trace, 4);
        if (ngl > 0) {
            switch (p.epi) {
                case LB_EPI_GENERIC: finish_job<LB_EPI_GENERIC>(p, sm, g0, ngl); break;
                case LB_EPI_QKV: finish_job<LB_EPI_QKV>(p, sm, g0, ngl); break;
                case LB_EPI_RESID: finish_job<LB_EPI_RESID>(p, sm, g0, ngl); break;
                default: finish_job<LB_EPI_SWIGLU>(p, sm, g0, ngl); break;
            }
        }
        lb_trace(p.trace, 5);
    }
}

}  // namespace

// ---- host side -------------------------------------------------------------------------------------------

int lb_program_build(loom_b200_ctx* ctx, const std::vector<LbJob>& jobs_in, loom_b200_program** out) {
    *out = nullptr;
    LB_REQUIRE(ctx, !jobs_in.empty(), "program: no jobs");
    if (ctx->capturing) return lb_fail(ctx, LOOM_B200_ERR_INVALID, "a program cannot be built while recording a graph");
    std::vector<LbJob> jobs = jobs_in;
    const int grid = ctx->sm_count;
    int acts_bytes = 0, sacc_ints = 0, stage_bytes = 0;
    uint64_t bytes = 0;
    for (auto& jb : jobs) {
        LbGemvParams& p = jb.p;
        p.aligned = 1;
        const int vstrips = p.total_tiles / p.kblocks;
        const int ngroups = vstrips / p.group;
        const int gpc = (ngroups + grid - 1) / grid;
        p.max_local_strips = gpc * p.group;
        const int Kp = p.kblocks * kTileCols;
        const int a = p.M * (Kp + 16) + 32;
        if (a > acts_bytes) acts_bytes = a;
        const int s = p.max_local_strips * p.M * 16;
        if (s > sacc_ints) sacc_ints = s;
        p.stage_bytes = 0;
        if (p.pro != LB_PRO_Q8 && (p.K & 3) == 0) p.stage_bytes = p.K * (p.pro == LB_PRO_INNERNORM64 ? 8 : 4);
        if (p.stage_bytes > stage_bytes) stage_bytes = p.stage_bytes;
        p.stages = 0;
        p.fix_acc = nullptr;
        p.fix_cnt = nullptr;
        p.status = ctx->status_dev;
        p.trace = lb_trace_row(ctx, "stream-job");
        for (int s2 = 0; s2 < p.nseg; ++s2) bytes += (uint64_t)p.seg[s2].strips * p.kblocks * kTileBytes + (uint64_t)p.M * p.seg[s2].rows * 4;
        bytes += (uint64_t)p.M * p.K;
    }
    acts_bytes = (acts_bytes + 15) & ~15;
    size_t fixed = (size_t)acts_bytes + (size_t)sacc_ints * 4 + 32 + 32 + 256 + 3 * kMaxM * 8 + 16 + (size_t)kWarps * kPStagesMax * 8 + 16;
    size_t stage_room = (size_t)((stage_bytes + 15) & ~15);
    // dynamic shared memory left beside the kernel's static part (the job block and the job table)
    cudaFuncAttributes fattr;
    LB_CUDA(ctx, cudaFuncGetAttributes(&fattr, lb_stream_kernel));
    const size_t dyn_max = ((size_t)227 * 1024 - fattr.sharedSizeBytes) & ~(size_t)1023;
    const size_t budget = dyn_max - 1024;
    // the staging buffer is optional (the slow generic prologue works without it); the ring needs at least 2 stages
    if (fixed + stage_room + (size_t)kWarps * 2 * kStageBytes > budget) {
        stage_room = 0;
        for (auto& jb : jobs) jb.p.stage_bytes = 0;
        stage_bytes = 0;
    }
    LB_REQUIRE(ctx, fixed + stage_room + (size_t)kWarps * 2 * kStageBytes <= budget, "program: activations of %d bytes do not fit in shared memory", acts_bytes);
    int stages = (int)((budget - fixed - stage_room) / ((size_t)kWarps * kStageBytes));
    if (stages > kPStagesMax) stages = kPStagesMax;
    auto* prog = new loom_b200_program();
    prog->grid = grid;
    prog->bytes = bytes;
    prog->smem = (size_t)kWarps * stages * kStageBytes + fixed + stage_room;
    cudaError_t e = cudaMalloc(&prog->jobs_dev, jobs.size() * sizeof(LbJob));
    if (e == cudaSuccess) e = cudaMalloc(&prog->barrier_dev, 64);
    if (e == cudaSuccess) e = cudaMemcpyAsync(prog->jobs_dev, jobs.data(), jobs.size() * sizeof(LbJob), cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(prog->barrier_dev, 0, 64, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e == cudaSuccess && !(ctx->func_attr_mask & (1u << 28))) {
        e = cudaFuncSetAttribute(lb_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn_max);
        ctx->func_attr_mask |= 1u << 28;
    }
    if (e != cudaSuccess) {
        if (prog->jobs_dev) cudaFree(prog->jobs_dev);
        if (prog->barrier_dev) cudaFree(prog->barrier_dev);
        delete prog;
        return lb_fail(ctx, LOOM_B200_ERR_CUDA, "program: %s", cudaGetErrorString(e));
    }
    prog->sp.jobs = prog->jobs_dev;
    prog->sp.njobs = (int)jobs.size();
    prog->sp.stages = stages;
    prog->sp.acts_bytes = acts_bytes;
    prog->sp.sacc_ints = sacc_ints;
    prog->sp.stage_bytes = stage_bytes;
    prog->sp.barrier = prog->barrier_dev;
    prog->sp.status = ctx->status_dev;
    *out = prog;
    return 0;
}

int lb_program_launch(loom_b200_ctx* ctx, loom_b200_program* prog) {
    bool needs_barrier = true;  // cooperative launch also guarantees that every CTA is resident at once
    LB_CUDA(ctx, cudaMemsetAsync(prog->barrier_dev, 0, 4, ctx->stream));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(prog->grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = prog->smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = needs_barrier ? 1 : 0;
    LB_CUDA(ctx, cudaLaunchKernelEx(&cfg, lb_stream_kernel, prog->sp));
    ctx->launches++;
    return 0;
}

extern "C" {

int loom_b200_linear_program_create(loom_b200_ctx* ctx, int n, const loom_b200_linear_job* jobs, loom_b200_program** out) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "linear_program_create: ctx is NULL");
    LB_REQUIRE(ctx, out != nullptr, "linear_program_create: out is NULL");
    *out = nullptr;
    LB_REQUIRE(ctx, n > 0 && jobs, "linear_program_create: no jobs");
    if (int rc = lb_set_device(ctx)) return rc;
    std::vector<LbJob> list((size_t)n);
    for (int i = 0; i < n; ++i) {
        const loom_b200_linear_job& jb = jobs[i];
        LB_REQUIRE(ctx, jb.w && jb.q && jb.amax && jb.out, "linear_program_create: job %d has a NULL pointer", i);
        LB_REQUIRE(ctx, jb.batch >= 1 && jb.batch <= kMaxM, "linear_program_create: job %d has batch %d (1..%d)", i, jb.batch, kMaxM);
        LB_REQUIRE(ctx, jb.w->device == ctx->device, "linear_program_create: job %d weight lives on device %d", i, jb.w->device);
        LbJob& o = list[i];
        memset(&o, 0, sizeof(o));
        LbGemvParams& p = o.p;
        p.nseg = 1;
        p.seg[0].tiles = jb.w->tiles;
        p.seg[0].rows = jb.w->rows;
        p.seg[0].scale = jb.w->scale;
        p.seg[0].bias = jb.bias;
        p.seg[0].out = jb.out;
        p.seg[0].kind = LB_OUT_F32;
        p.K = jb.w->cols;
        p.M = jb.batch;
        p.pro = LB_PRO_Q8;
        p.x = jb.q;
        p.amax_in = jb.amax;
        p.epi = LB_EPI_GENERIC;
        p.act = jb.activation;
        p.residual = jb.residual;
        o.grid_wait = jb.depends_on_previous ? 1 : 0;
        if (int rc = lb_gemv_finalize_params(ctx, p)) return rc;
    }
    return lb_program_build(ctx, list, out);
}

int loom_b200_program_run(loom_b200_ctx* ctx, loom_b200_program* prog) {
    if (!ctx) return lb_fail(nullptr, LOOM_B200_ERR_INVALID, "program_run: ctx is NULL");
    LB_REQUIRE(ctx, prog != nullptr, "program_run: program is NULL");
    if (int rc = lb_set_device(ctx)) return rc;
    return lb_program_launch(ctx, prog);
}

uint64_t loom_b200_program_bytes(const loom_b200_program* prog) { return prog ? prog->bytes : 0; }

void loom_b200_program_free(loom_b200_ctx* ctx, loom_b200_program* prog) {
    if (!prog) return;
    if (ctx) {
        cudaSetDevice(ctx->device);
        cudaStreamSynchronize(ctx->stream);
    }
    if (prog->jobs_dev) cudaFree(prog->jobs_dev);
    if (prog->barrier_dev) cudaFree(prog->barrier_dev);
    delete prog;
}

}  // extern "C"
