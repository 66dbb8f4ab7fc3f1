// tp_xchg.cuh -- the peer-memory exchange of the tensor-parallel path: mailbox layout and the 8-byte {value, sequence}
// store / poll pair, shared by the stand-alone exchange kernels (tp.cu) and the GEMV that carries the exchange in its
// own prologue and epilogue (gemv_ternary.cu).
//
// Every rank owns a mailbox in its own HBM and maps every other rank's mailbox (CUDA IPC).  A value travels as an
// 8-byte {data, sequence} pair written with one store straight into the receiver's mailbox over NVLink; the receiver
// polls its own memory until the sequence number of the current exchange shows up (the scheme NCCL calls LL).  No
// kernel ever loads from a peer: only plain stores cross NVLink.  Two alternating halves per region let a rank run
// one exchange ahead of a slow peer without overwriting what that peer has not read yet; it cannot run two ahead
// because finishing an exchange needs every peer's contribution to it.  Every poll is bounded: on expiry the kernel
// raises the context status word (5) and carries on with whatever it has, so a missing peer never hangs the GPU.
#pragma once
#include "common.cuh"

constexpr int kXMaxRanks = 8;
constexpr int kXMaxAcc = 8 * 8192;  // int32 accumulators one exchange can carry (tokens x rows)
constexpr size_t kXRegionA = 0;                                                     // [2][ranks][8 tokens][lo, hi] sum of squares
constexpr size_t kXRegionB = kXRegionA + 2 * kXMaxRanks * 8 * 2 * 8;                // [2][ranks][8 tokens] absmax
constexpr size_t kXRegionC = kXRegionB + 2 * kXMaxRanks * 8 * 8;                    // [2][ranks][kXMaxAcc] accumulators
constexpr size_t kXRegionD = kXRegionC + 2 * (size_t)kXMaxRanks * kXMaxAcc * 8;      // [2][ranks][8 rows][value, index] greedy choice of a vocabulary slice
constexpr size_t kXBytes = kXRegionD + 2 * kXMaxRanks * 8 * 2 * 8;
constexpr unsigned int kXSpin = 40000000u;  // polls before giving up (of the order of a second)

__device__ __forceinline__ void ll_store(void* p, uint32_t data, uint32_t seq) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(data), "r"(seq) : "memory");
}
__device__ __forceinline__ bool ll_wait(const void* p, uint32_t seq, uint32_t* data) {
    for (unsigned int i = 0; i < kXSpin; ++i) {
        uint32_t d, f;
        asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(d), "=r"(f) : "l"(p) : "memory");
        if (f == seq) {
            *data = d;
            return true;
        }
    }
    *data = 0;
    return false;
}
