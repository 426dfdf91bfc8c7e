// Peer-memory exchange: state of a symmetric buffer and the device-side hand-shake
// that ends a push (shared by the push kernel and the GEMM's pushing epilogue).
#pragma once

#include "tm_cuda_internal.cuh"

constexpr int kSymmMaxWorld = 16;
constexpr uint32_t kSymmTail = 512;        // u32 flags[16] | u32 seq @64 | u32 block counter @68 | u32 status @72 | pair-exchange number @80, its block counter @84
constexpr uint32_t kSymmSpinLimit = 1u << 24;

struct tm_symm_state {
    int world = 1, rank = 0;
    size_t payload = 0;                    // bytes before the flag tail
    void *peer[kSymmMaxWorld] = {};        // this buffer on every rank (own entry = local pointer)
    void **d_peer = nullptr;               // the same table in device memory
};

// Called by every block once all of its threads' peer stores are fenced to system scope and the
// block has synchronised: the block that counts in last raises this rank's sequence flag on every
// rank and waits, with an iteration limit, until every sender's flag on this rank has reached the
// same number.  Returns for all other blocks at once.  `s_flag` is two words of shared memory.
__device__ __forceinline__ void tm_symm_finish(float *const *peer, uint32_t tail_off, uint32_t world, uint32_t rank,
                                               uint32_t *s_flag) {
    uint32_t *tail = (uint32_t *)(peer[rank] + tail_off);
    if (threadIdx.x == 0) {
        const uint32_t prev = atomicAdd(tail + 68, 1u);
        s_flag[0] = prev == gridDim.x * gridDim.y - 1u ? 1u : 0u;
        if (s_flag[0]) {
            tail[68] = 0u;                 // ready for the next launch
            s_flag[1] = tail[64] + 1u;
            tail[64] = s_flag[1];
        }
    }
    __syncthreads();
    if (!s_flag[0]) return;
    const uint32_t seq = s_flag[1];
    if (threadIdx.x < world) {
        __threadfence_system();
        uint32_t *remote = (uint32_t *)(peer[threadIdx.x] + tail_off) + rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(seq) : "memory");
        const uint32_t *mine = tail + threadIdx.x;  // sender threadIdx.x on this rank; numbers only grow
        uint32_t spin = 0, v = 0;
        for (;;) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
            if ((int32_t)(v - seq) >= 0) break;
            if (++spin > kSymmSpinLimit) {
                atomicOr(tail + 72, 1u);   // gave up: the consumer will read stale rows; the host sees the status
                break;
            }
        }
    }
}
