// Shared device helpers for the escha coded-projection kernels (sm_100a).
//
// Numeric contract (escha_mlx/ref.py:37-48, escha_mlx/msl.py:34-41 of the
// reference): a 16-bit trellis state x decodes to
//     r = ((x * 0xCBAC1FED) & 0x8FFF8FFF) ^ 0x3B603B60          (32-bit)
//     w = fp16(lo16(r)) + fp16(hi16(r))                         (one RNE fp16 add)
// Everything here is compiled without fast-math; the fp16 add is the hardware
// binary16 adder (__hadd / __hadd2), never a float add.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdlib>
#include <cstring>
#include <utility>

namespace escha {

constexpr float kRS = 0.088388347648f;  // 1/sqrt(128) as the format pins it (ref.py:30)

__device__ __forceinline__ uint32_t cba_hash(uint32_t state16) {
    return ((state16 * 0xCBAC1FEDu) & 0x8FFF8FFFu) ^ 0x3B603B60u;
}

__device__ __forceinline__ __half2 as_half2(uint32_t r) {
    return *reinterpret_cast<__half2*>(&r);
}

__device__ __forceinline__ uint32_t as_u32(__half2 h) {
    return *reinterpret_cast<uint32_t*>(&h);
}

// Scalar decode: one state -> one half.
__device__ __forceinline__ __half cba_decode(uint32_t state16) {
    __half2 h = as_half2(cba_hash(state16));
    return __hadd(__low2half(h), __high2half(h));
}

// Decode into both halves of a register: (w, w).  The tensor-core GEMV feeds
// this straight into an mma A-fragment register against a (x, 0) B register.
__device__ __forceinline__ uint32_t cba_decode_dup(uint32_t state16) {
    __half2 h = as_half2(cba_hash(state16));
    return as_u32(__hadd2(__low2half2(h), __high2half2(h)));
}

// Hot-loop form of the decode.  With both 32-bit constants written as literals
// the compiler emits two logic instructions per weight (an AND-immediate and an
// XOR-immediate; a three-input logic op takes only one immediate), and the
// integer pipe is what limits the GEMV.  Taking the mask and the xor value as
// run-time registers makes it one three-input op: (p & mask) ^ x = LUT 0x6A.
__device__ __forceinline__ uint32_t cba_decode_dup(uint32_t state16, uint32_t mask, uint32_t x) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(r) : "r"(state16 * 0xCBAC1FEDu), "r"(mask), "r"(x));
    __half2 h = as_half2(r);
    return as_u32(__hadd2(__low2half2(h), __high2half2(h)));
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

// ---------------------------------------------------------------------------
// Window extraction (escha_mlx/ref.py:64-93; msl.py:45-81).  `w` points at the
// tile's 8K words (any address space); lane is the lane index within the warp.
// Produces the lane's eight 16-bit states, zero-extended.
// ---------------------------------------------------------------------------

// Multipliers 2^k handed to the hot loop as run-time values: `x * m` with an
// opaque m is always an IMAD (multiply pipe), whereas `x << k` may be placed on
// the integer pipe, which the decode saturates first.
struct ShiftMuls {
    uint32_t m2, m4, m16, m32, m64, m128;
};

struct LaneK2 {
    uint32_t i0, i1, sel;  // word indices and the byte selector that forms the window
    __device__ __forceinline__ explicit LaneK2(uint32_t lane) {
        i1 = lane >> 1;          // (lane*8) >> 4
        i0 = (i1 + 15u) & 15u;   // previous word, tail-biting wrap
        // even lane: window = (w[i0] << 16) | (w[i1] >> 16); odd lane: w[i1]
        sel = (lane & 1u) ? 0x3210u : 0x5432u;
    }
};

// State j is the 16-bit window of wv at bit 2*(7-j).  Left shifts bring every
// window to a byte boundary; the byte permute then extracts it zero-extended, so
// no separate mask is needed.
__device__ __forceinline__ void states_k2(uint32_t w0, uint32_t w1, uint32_t sel, uint32_t s[8]) {
    const uint32_t wv = prmt(w1, w0, sel);
    const uint32_t z1 = wv << 2, z2 = wv << 4, z3 = wv << 6;
    s[7] = prmt(wv, 0u, 0x4410u);   // bit 0
    s[3] = prmt(wv, 0u, 0x4421u);   // bit 8
    s[6] = prmt(z3, 0u, 0x4421u);   // bit 2  -> 8
    s[2] = prmt(z3, 0u, 0x4432u);   // bit 10 -> 16
    s[5] = prmt(z2, 0u, 0x4421u);   // bit 4  -> 8
    s[1] = prmt(z2, 0u, 0x4432u);   // bit 12 -> 16
    s[4] = prmt(z1, 0u, 0x4421u);   // bit 6  -> 8
    s[0] = prmt(z1, 0u, 0x4432u);   // bit 14 -> 16
}
__device__ __forceinline__ void states_k2(uint32_t w0, uint32_t w1, uint32_t sel,
                                          const ShiftMuls& m, uint32_t s[8]) {
    const uint32_t wv = prmt(w1, w0, sel);
    const uint32_t z1 = wv * m.m4, z2 = wv * m.m16, z3 = wv * m.m64;
    s[7] = prmt(wv, 0u, 0x4410u);
    s[3] = prmt(wv, 0u, 0x4421u);
    s[6] = prmt(z3, 0u, 0x4421u);
    s[2] = prmt(z3, 0u, 0x4432u);
    s[5] = prmt(z2, 0u, 0x4421u);
    s[1] = prmt(z2, 0u, 0x4432u);
    s[4] = prmt(z1, 0u, 0x4421u);
    s[0] = prmt(z1, 0u, 0x4432u);
}

// K = 3: the reference forms merged = (w[i0] << 32) | w[i2] and takes 32-bit
// windows at bit sh and sh + 12 (ref.py:78-93).  i0 is always the word before i2
// and sh is always a multiple of 8 (it cycles 8, 16, 24, 0 with the lane), so
// u = merged >> sh is a byte selection; the eight states are the 16-bit windows
// of u at bits 21, 18, 15, 12, 9, 6, 3, 0.
struct LaneK3 {
    uint32_t i0, i2, sh;    // word indices (mod 24) and the window shift
    uint32_t selA, selB;    // byte selectors: A = u[0:32), B = u[16:48)
    __device__ __forceinline__ explicit LaneK3(uint32_t lane) {
        uint32_t b1 = (lane * 8u + 257u) * 3u;
        uint32_t b0 = b1 - 16u;
        uint32_t b2 = b1 + 21u;
        uint32_t j0 = b0 >> 5;
        uint32_t j2 = (b2 - 1u) >> 5;
        sh = ((j2 + 1u) << 5) - b2;
        i0 = j0 % 24u;
        i2 = j2 % 24u;
        const uint32_t b = sh >> 3;
        selA = b | ((b + 1u) << 4) | ((b + 2u) << 8) | ((b + 3u) << 12);
        selB = (b + 2u) | ((b + 3u) << 4) | ((b + 4u) << 8) | (min(b + 5u, 7u) << 12);
    }
};

__device__ __forceinline__ void states_k3(uint32_t whi, uint32_t wlo, uint32_t sh, uint32_t s[8]) {
    uint64_t merged = (static_cast<uint64_t>(whi) << 32) | static_cast<uint64_t>(wlo);
    const uint32_t w7 = static_cast<uint32_t>(merged >> sh);
    const uint32_t w3 = static_cast<uint32_t>(merged >> (sh + 12u));
    // windows at bits 9, 6, 3, 0 of each word: left-shift to a byte boundary
    // (9 -> 16, 6 -> 8, 3 -> 8), then a zero-extending byte permute
    s[0] = prmt(w3 << 7, 0u, 0x4432u);
    s[1] = prmt(w3 << 2, 0u, 0x4421u);
    s[2] = prmt(w3 << 5, 0u, 0x4421u);
    s[3] = prmt(w3, 0u, 0x4410u);
    s[4] = prmt(w7 << 7, 0u, 0x4432u);
    s[5] = prmt(w7 << 2, 0u, 0x4421u);
    s[6] = prmt(w7 << 5, 0u, 0x4421u);
    s[7] = prmt(w7, 0u, 0x4410u);
}
// Hot-loop form: two byte selections instead of 64-bit shifts, and every shift as a
// multiply by 2^k (multiply pipe): the byte permutes and the decode's mask/xor already
// saturate the integer pipe (measured: +1.1% on the batch-1 layer against a version that
// kept three of the seven shifts on the integer pipe).
__device__ __forceinline__ void states_k3(uint32_t whi, uint32_t wlo, uint32_t selA,
                                          uint32_t selB, const ShiftMuls& m, uint32_t s[8]) {
    const uint32_t A = prmt(wlo, whi, selA), B = prmt(wlo, whi, selB);
    s[7] = prmt(A, 0u, 0x4410u);                 // bit 0
    s[6] = prmt(A * m.m32, 0u, 0x4421u);         // bit 3  -> 8
    s[5] = prmt(A * m.m4, 0u, 0x4421u);          // bit 6  -> 8
    s[4] = prmt(A * m.m128, 0u, 0x4432u);        // bit 9  -> 16
    s[3] = prmt(A * m.m16, 0u, 0x4432u);         // bit 12 -> 16
    const uint32_t m8 = m.m4 * m.m2;             // loop-invariant
    s[2] = prmt(A * m.m2, 0u, 0x4432u);          // bit 15 -> 16
    s[1] = prmt(B * m.m64, 0u, 0x4421u);         // bit 18 = bit 2 of B -> 8
    s[0] = prmt(B * m8, 0u, 0x4421u);            // bit 21 = bit 5 of B -> 8
}

template <int K>
struct LaneConsts;
template <>
struct LaneConsts<2> : LaneK2 {
    __device__ __forceinline__ explicit LaneConsts(uint32_t lane) : LaneK2(lane) {}
    __device__ __forceinline__ uint32_t ia() const { return i0; }
    __device__ __forceinline__ uint32_t ib() const { return i1; }
    __device__ __forceinline__ void states(uint32_t wa, uint32_t wb, uint32_t s[8]) const {
        states_k2(wa, wb, sel, s);
    }
    __device__ __forceinline__ void states(uint32_t wa, uint32_t wb, const ShiftMuls& m,
                                           uint32_t s[8]) const {
        states_k2(wa, wb, sel, m, s);
    }
};
template <>
struct LaneConsts<3> : LaneK3 {
    __device__ __forceinline__ explicit LaneConsts(uint32_t lane) : LaneK3(lane) {}
    __device__ __forceinline__ uint32_t ia() const { return i0; }
    __device__ __forceinline__ uint32_t ib() const { return i2; }
    __device__ __forceinline__ void states(uint32_t wa, uint32_t wb, uint32_t s[8]) const {
        states_k3(wa, wb, sh, s);
    }
    __device__ __forceinline__ void states(uint32_t wa, uint32_t wb, const ShiftMuls& m,
                                           uint32_t s[8]) const {
        states_k3(wa, wb, selA, selB, m, s);
    }
};

// ---------------------------------------------------------------------------
// 128-point unnormalised Sylvester WHT across one warp (escha_mlx/ref.py:204-218).
// Element i of the block lives in lane i>>2, register i&3.  Stage h pairs i with
// i^h; the low index receives a+b, the high index a-b, exactly the operands the
// in-place reference butterfly uses at every stage, so results are bit-identical.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void wht128_warp(float v[4], uint32_t lane) {
    {   // h = 1
        float a = v[0], b = v[1], c = v[2], d = v[3];
        v[0] = __fadd_rn(a, b); v[1] = __fsub_rn(a, b);
        v[2] = __fadd_rn(c, d); v[3] = __fsub_rn(c, d);
    }
    {   // h = 2
        float a = v[0], b = v[1], c = v[2], d = v[3];
        v[0] = __fadd_rn(a, c); v[2] = __fsub_rn(a, c);
        v[1] = __fadd_rn(b, d); v[3] = __fsub_rn(b, d);
    }
#pragma unroll
    for (uint32_t m = 1; m < 32; m <<= 1) {  // h = 4*m
        const bool high = (lane & m) != 0;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            float mine = v[r];
            float other = __shfl_xor_sync(0xFFFFFFFFu, mine, m);
            v[r] = high ? __fsub_rn(other, mine) : __fadd_rn(mine, other);
        }
    }
}

// cp.async helpers (16-byte, L2-only caching: the code stream is read once).
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async16_shared(uint32_t smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
    asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}


// ---------------------------------------------------------------------------
// mbarrier + bulk-copy (TMA, untiled) helpers.  Every wait is bounded: a wait
// that gives up returns false and the caller records an error and leaves, so a
// logic error can never spin a GPU forever.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
// Programmatic dependent launch.  launch_dependents: the next kernel in the stream
// may be scheduled once every CTA of this grid has executed it (or exited).  wait:
// blocks until the kernels this grid depends on have completed and their writes are
// visible; a no-op for a grid launched without a programmatic dependency.
__device__ __forceinline__ void grid_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void grid_dependency_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// Host side of the same: launch `kernel` so that it may be scheduled while the previous
// kernel of the stream drains.  The kernel must call grid_dependency_wait() before it
// touches anything an earlier kernel may have written.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                    cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// The same, unless ESCHA_B200_PDL=off (read once per process): then a plain launch, and the
// kernel's grid_dependency_wait() is a no-op.  For the small kernels between the products
// (transforms, SwiGLU, plane sums): they call launch_dependents and wait first thing, so only
// launch latency and set-up overlap the previous kernel's tail.
inline bool pdl_allowed() {
    static const bool on = [] {
        const char* v = std::getenv("ESCHA_B200_PDL");
        return v == nullptr || std::strcmp(v, "off") != 0;
    }();
    return on;
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                  cudaStream_t st, Args&&... args) {
    if (pdl_allowed()) return launch_dependent(kernel, grid, block, smem, st, std::forward<Args>(args)...);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// launch_chained for a grid of thread-block clusters of (1, cluster_y, 1) CTAs
template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                          cudaStream_t st, unsigned cluster_y, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = cluster_y;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_allowed() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
constexpr uint32_t kMbarWaitLimit = 1u << 22;  // try_wait attempts before giving up
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t it = 0; it < kMbarWaitLimit; ++it)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// The same with the bound as a parameter: `limit` rounds of 32 tries (a try blocks in
// hardware for some tens of cycles by itself).
__device__ __forceinline__ bool mbar_wait_n(uint32_t bar, uint32_t parity, uint32_t limit) {
    for (uint32_t it = 0; it < limit; ++it)
#pragma unroll 1
        for (int k = 0; k < 32; ++k)
            if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// global -> shared bulk copy (16-byte aligned addresses, size a multiple of 16),
// completion signalled on an mbarrier of this CTA.  No multicast.
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes,
                                              uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void named_barrier_sync(uint32_t id, uint32_t threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Arrive at a named barrier without waiting (the waiting side uses named_barrier_sync with
// the same thread count).
__device__ __forceinline__ void named_barrier_arrive(uint32_t id, uint32_t threads) {
    asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// mma.sync m16n8k16, f16 x f16 -> f32 accumulate.
__device__ __forceinline__ void mma16816(float d[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

}  // namespace escha
