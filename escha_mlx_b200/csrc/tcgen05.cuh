// tcgen05 / tensor-memory / TMA primitives shared by the prefill GEMM kernels.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace escha {

// Bounded wait that does not poll: a waiting warp must not take issue slots from the
// decode warps, which are what limits this kernel.
__device__ __forceinline__ bool mbar_wait_relaxed(uint32_t bar, uint32_t parity,
                                                  uint32_t limit = 1u << 21) {
    // try_wait with a suspend-time hint parks the thread in hardware until the phase
    // completes or the hint (in nanoseconds) runs out: one instruction per microsecond of
    // waiting instead of a polling loop
    // (`limit` tries: about two seconds by default; a test shortens it)
    for (uint32_t it = 0; it < limit; ++it) {
        uint32_t ok;
        asm volatile(
            "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3; selp.u32 %0, 1, 0, p; }"
            : "=r"(ok) : "r"(bar), "r"(parity), "r"(1000u) : "memory");
        if (ok) return true;
    }
    return false;
}

// Bounded wait for the single-thread service roles (loaders, the issuing thread): test, then
// sleep.  Their polls share issue slots with the decode warps, so they poll rarely.
__device__ __forceinline__ bool mbar_wait_sleepy(uint32_t bar, uint32_t parity, uint32_t ns) {
    for (uint32_t it = 0; it < (1u << 22); ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        __nanosleep(ns);
    }
    return false;
}

// true in exactly one lane of a converged warp
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{ .reg .pred p; elect.sync _|p, 0xFFFFFFFF; selp.u32 %0, 1, 0, p; }" : "=r"(pred)::"memory");
    return pred != 0;
}

// ---- tcgen05 / tensor-memory primitives (one CTA per group)
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
                 "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// writes made through the generic proxy (st.shared, cp.async) become visible to the
// tensor core's reads of shared memory
__device__ __forceinline__ void fence_async_proxy() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T, f16 inputs, f32 accumulate
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                         uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// arrive on an mbarrier of this CTA once all tcgen05.mma issued so far have completed
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(bar) : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns of tensor memory -> 16 registers per thread
__device__ __forceinline__ void tmem_ld16(uint32_t addr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
          "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
          "=r"(v[14]), "=r"(v[15])
        : "r"(addr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64
// halves) with the 128-byte swizzle: 8-row groups 1024 bytes apart, descriptor
// version 1, layout type 2.  `addr` is the shared address of the first row (1024-byte
// aligned tile) plus 32 bytes per 16 channels already consumed.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    return static_cast<uint64_t>((addr >> 4) & 0x3FFFu) | (uint64_t(1) << 16) |
           (uint64_t(1024 >> 4) << 32) | (uint64_t(1) << 46) | (uint64_t(2) << 61);
}
// Instruction descriptor: f16 x f16 -> f32, both operands K-major, M = 128 (output
// channels: the decoded weights are the A operand), N = rows of activations (128 or 256).
__host__ __device__ constexpr uint32_t idesc_for(uint32_t n) {
    return (1u << 4) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}

// byte offset of (row, 16-byte chunk) inside a swizzled [rows][128 B] tile
__device__ __forceinline__ uint32_t sw128(uint32_t row, uint32_t chunk) {
    return row * 128u + ((chunk ^ (row & 7u)) << 4);
}

// 2-D tiled TMA load (no multicast): box at element coordinates (x, y) of the tensor the
// map describes -> shared memory, completion counted in bytes on an mbarrier of this CTA.
// x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, int32_t x, int32_t y,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(bar) : "memory");
}

// 32 lanes x 16 consecutive 32-bit columns: 16 registers per thread -> tensor memory
__device__ __forceinline__ void tmem_st16(uint32_t addr, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(addr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]),
          "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]),
          "r"(v[14]), "r"(v[15]) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]^T: the A operand (128 lanes x 8 columns per instruction,
// two consecutive K elements per 32-bit cell) comes from tensor memory
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b,
                                            uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}

// ---- thread-block clusters: barrier over all CTAs of the cluster, and reads of another CTA's
// shared memory (distributed shared memory)
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// 16 bytes at shared address `addr` (an address of this CTA's window) of the cluster's CTA `rank`
__device__ __forceinline__ float4 ld_cluster_f4(uint32_t addr, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
    return v;
}

// Tensor map of the [M, IC] binary16 activations for boxes of 64 channels x rows_per_box rows,
// 128-byte swizzle (defined with the shared-memory-operand kernel).
cudaError_t encode_x_map(CUtensorMap* map, const __half* xh, int M, int IC, int rows_per_box);

}  // namespace escha
