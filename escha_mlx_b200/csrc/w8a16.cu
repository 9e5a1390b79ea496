// int8-weight linear of the MoE block's shared expert and the dense int8
// projections: y = f16( f32(x) @ f32( f16( f32(w8) * f32(scale) ) )^T )
// (escha_mlx/ref.py:308-311 w8a16; the reference runs it through
// mx.quantized_matmul after an exact repack, escha_mlx/quant.py:82-143).
// w8 is [N, Kd] int8 row-major with one f16 scale per output row.
//
// The per-weight rounding f16(w8 * scale) is a single HMUL2: int8 and scale are
// both exact in binary16 and the hardware rounds the exact product once.
// One warp owns one output row n and up to 8 activation rows; lanes stride over
// Kd in 16-byte pieces (16 weights), accumulate in f32 and reduce by shuffles.
#include "common.cuh"
#include "kernels.h"

namespace escha {

namespace {

// two int8 (bytes b0, b1 of a 16-bit lane) -> half2, exact: place each byte in the
// mantissa of 1024.0 with the sign bit flipped (u = b ^ 0x80), then subtract 1152.
__device__ __forceinline__ __half2 i8x2_to_half2(uint32_t word, uint32_t sel) {
    const uint32_t v = prmt(word ^ 0x80808080u, 0x64646464u, sel);
    return __hsub2(as_half2(v), as_half2(0x64806480u));  // 1024 + 128
}

template <int R>
__global__ void __launch_bounds__(256)
w8a16_kernel(const __half* __restrict__ x, const int8_t* __restrict__ w8,
             const __half* __restrict__ scale, __half* __restrict__ y, int M, int N, int Kd) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const uint32_t r0 = blockIdx.y * R;
    if (n >= static_cast<uint32_t>(N)) return;
    const __half2 sc2 = __half2half2(scale[n]);
    const int8_t* wrow = w8 + static_cast<size_t>(n) * Kd;
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.0f;
    for (uint32_t k = lane * 16u; k < static_cast<uint32_t>(Kd); k += 512u) {
        const uint4 wv = *reinterpret_cast<const uint4*>(wrow + k);
        const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
        float wf[16];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float2 lo = __half22float2(__hmul2(i8x2_to_half2(ww[q], 0x4140u), sc2));
            const float2 hi = __half22float2(__hmul2(i8x2_to_half2(ww[q], 0x4342u), sc2));
            wf[4 * q + 0] = lo.x; wf[4 * q + 1] = lo.y;
            wf[4 * q + 2] = hi.x; wf[4 * q + 3] = hi.y;
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const uint32_t row = min(r0 + r, static_cast<uint32_t>(M) - 1u);
            const uint4* xp = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * Kd + k);
            const uint4 xa = xp[0], xb = xp[1];
            const uint32_t xw[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float2 xf = __half22float2(as_half2(xw[i]));
                acc[r] = __fmaf_rn(xf.x, wf[2 * i], acc[r]);
                acc[r] = __fmaf_rn(xf.y, wf[2 * i + 1], acc[r]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        float a = acc[r];
#pragma unroll
        for (uint32_t m = 16; m > 0; m >>= 1) a = __fadd_rn(a, __shfl_xor_sync(0xFFFFFFFFu, a, m));
        if (lane == 0 && r0 + r < static_cast<uint32_t>(M))
            y[static_cast<size_t>(r0 + r) * N + n] = __float2half_rn(a);
    }
}

// Embedding rows of an int8 table: out[r, :] = f16( f32(w8[ids[r], :]) * f32(scale[ids[r]]) ),
// the per-weight rounding of the int8 linear (EschaQ8Embedding, escha_mlx/quant.py:249-262).
// One warp per row, 16 weights per lane and step.
__global__ void __launch_bounds__(256)
q8_embed_kernel(const int64_t* __restrict__ ids, const int8_t* __restrict__ w8,
                const __half* __restrict__ scale, __half* __restrict__ out, int rows, int N, int Kd) {
    const uint32_t lane = threadIdx.x & 31u;
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= rows) return;
    long id = ids[r];
    if (id < 0 || id >= N) id = 0;   // callers validate; never read out of bounds
    const __half2 sc2 = __half2half2(scale[id]);
    const int8_t* wrow = w8 + static_cast<size_t>(id) * Kd;
    __half* orow = out + static_cast<size_t>(r) * Kd;
    for (uint32_t k = lane * 16u; k < static_cast<uint32_t>(Kd); k += 512u) {
        const uint4 wv = *reinterpret_cast<const uint4*>(wrow + k);
        const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
        uint32_t o[8];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            o[2 * q] = as_u32(__hmul2(i8x2_to_half2(ww[q], 0x4140u), sc2));
            o[2 * q + 1] = as_u32(__hmul2(i8x2_to_half2(ww[q], 0x4342u), sc2));
        }
        uint4* dst = reinterpret_cast<uint4*>(orow + k);
        dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
        dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
    }
}

}  // namespace

cudaError_t launch_q8_embed(const int64_t* ids, const int8_t* w8, const __half* scale, __half* out,
                            int rows, int N, int Kd, cudaStream_t st) {
    q8_embed_kernel<<<(rows + 7) / 8, 256, 0, st>>>(ids, w8, scale, out, rows, N, Kd);
    return cudaGetLastError();
}

cudaError_t launch_w8a16(const __half* x, const int8_t* w8, const __half* scale, __half* y, int M,
                         int N, int Kd, cudaStream_t st) {
    const int warps = 8;
    if (M == 1) {
        dim3 grid((N + warps - 1) / warps, 1);
        w8a16_kernel<1><<<grid, warps * 32, 0, st>>>(x, w8, scale, y, M, N, Kd);
    } else if (M <= 4) {
        dim3 grid((N + warps - 1) / warps, 1);
        w8a16_kernel<4><<<grid, warps * 32, 0, st>>>(x, w8, scale, y, M, N, Kd);
    } else {
        dim3 grid((N + warps - 1) / warps, (M + 7) / 8);
        w8a16_kernel<8><<<grid, warps * 32, 0, st>>>(x, w8, scale, y, M, N, Kd);
    }
    return cudaGetLastError();
}

}  // namespace escha
