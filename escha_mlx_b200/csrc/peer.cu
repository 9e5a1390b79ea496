// Cross-GPU barrier for the fused GEMV + all-gather: after a rank's GEMV epilogue has
// stored its output block into every peer's gathered buffer (peer-mapped memory over
// NVLink), the ranks meet here before anyone reads its buffer.  The reference is
// single-device; this has no counterpart there.
//
// Each rank owns an array of 32-bit words in peer-accessible memory:
//   [0, n)   arrival words: word r holds the latest epoch rank r has announced to us
//   [n]      this rank's epoch counter (only this kernel touches it)
//   [n + 1]  status: set to 1 if a wait below gave up
// One launch per rank, one warp, lane g talks to rank g: it stores the new epoch into
// rank g's arrival word for us (release, system scope, after a system-wide fence so the
// epilogue's peer stores are ordered before it), then polls our arrival word for rank g
// (acquire, system scope) until it reaches the epoch.  The epoch lives on the device, so
// the launch is identical every time and can be replayed from a CUDA graph.
//
// The launch is chained with programmatic dependent launch (unless ESCHA_B200_PDL=off), so
// only its polling, not its launch latency, sits between producer and consumer.
//
// The kernels of different ranks run on different GPUs at the same time; ranks must
// never share a GPU.  The poll is bounded (about two seconds): a rank that never shows
// up raises the status word instead of hanging the others.
#include "common.cuh"
#include "kernels.h"

namespace escha {

namespace {

constexpr uint32_t kPollLimit = 1u << 24;
uint32_t g_poll_limit = kPollLimit;   // host side; a test shortens it

__device__ __forceinline__ void store_release_sys(int32_t* p, int32_t v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int32_t load_acquire_sys(const int32_t* p) {
    int32_t v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(32)
peer_barrier_kernel(const PeerBarrierParams p, const uint32_t poll_limit) {
    const int lane = threadIdx.x, n = p.nranks;
    // chained to its neighbours in the stream (programmatic dependent launch): the warp is
    // resident while the producing kernel drains and the consumer's CTAs are scheduled while
    // it polls; it waits here until the producer has completed and its stores are visible
    grid_launch_dependents();
    grid_dependency_wait();
    int32_t epoch = 0;
    if (lane == 0) {
        epoch = p.local[n] + 1;
        p.local[n] = epoch;
    }
    epoch = __shfl_sync(0xFFFFFFFFu, epoch, 0);
    __threadfence_system();
    const bool talks = lane < n && lane != p.rank;
    if (talks) store_release_sys(p.peer[lane] + p.rank, epoch);
    if (talks) {
        bool seen = false;
        for (uint32_t it = 0; it < poll_limit; ++it) {
            if (load_acquire_sys(p.local + lane) - epoch >= 0) {
                seen = true;
                break;
            }
            __nanosleep(100);
        }
        if (!seen) atomicExch(p.local + n + 1, 1);
    }
    __syncwarp();
}

}  // namespace

void peer_barrier_poll_limit(unsigned polls) { g_poll_limit = polls ? polls : kPollLimit; }

cudaError_t launch_peer_barrier(const PeerBarrierParams& p, cudaStream_t st) {
    return launch_chained(peer_barrier_kernel, dim3(1), dim3(32), 0, st, p, g_poll_limit);
}

}  // namespace escha
