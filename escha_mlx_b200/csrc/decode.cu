// decode_tiles: packed trellis code stream -> fp16 bare weight [IC, OC].
// Replaces the reference's escha_decode_tiles_k{2,3}[_lut] Metal kernels
// (escha_mlx/msl.py:183-202, wrapper :1404-1421).  Correctness anchor of the
// whole path: the output must equal ref.reconstruct bit for bit.
//
// One warp decodes one 16x16 tile (lane L owns 8 values, placed as
// ref.lane_positions says); a 256-thread CTA covers one kt row of eight tiles,
// transposes through shared memory and writes 16 rows of 256 contiguous bytes.
#include "common.cuh"
#include "kernels.h"

namespace escha {

__global__ void lut_init_kernel(__half* lut) {
    uint32_t s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s < 65536u) lut[s] = cba_decode(s);
}

template <int K, bool LUT>
__global__ void __launch_bounds__(256)
decode_tiles_kernel(const uint32_t* __restrict__ code, const __half* __restrict__ lut,
                    __half* __restrict__ w, int TN, int OC) {
    constexpr int WPT = 8 * K;
    __shared__ __align__(16) __half tile[16][128 + 8];
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t ntb = blockIdx.x, kt = blockIdx.y;
    const uint32_t nt = ntb * 8u + warp;
    if (nt < static_cast<uint32_t>(TN)) {
        const uint32_t* wp = code + (static_cast<size_t>(kt) * TN + nt) * WPT;
        LaneConsts<K> lc(lane);
        uint32_t s[8];
        lc.states(__ldg(wp + lc.ia()), __ldg(wp + lc.ib()), s);
        const uint32_t g = lane >> 2, t = lane & 3u;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            // value j: input row 2t + (j&1) + 8*((j>>1)&1), output column g + 8*(j>=4)
            const uint32_t row = 2u * t + (j & 1) + ((j >> 1) & 1) * 8u;
            const uint32_t col = g + (j >= 4 ? 8u : 0u);
            tile[row][warp * 16u + col] = LUT ? lut[s[j]] : cba_decode(s[j]);
        }
    }
    __syncthreads();
    // 16 rows x 128 halves = 256 x 16-byte pieces, one per thread
    const uint32_t row = threadIdx.x >> 4, piece = threadIdx.x & 15u;
    const uint32_t col0 = ntb * 128u + piece * 8u;
    if (col0 < static_cast<uint32_t>(OC)) {
        const uint4 v = *reinterpret_cast<const uint4*>(&tile[row][piece * 8u]);
        *reinterpret_cast<uint4*>(w + (static_cast<size_t>(kt) * 16u + row) * OC + col0) = v;
    }
}

cudaError_t launch_lut_init(__half* lut, cudaStream_t st) {
    lut_init_kernel<<<256, 256, 0, st>>>(lut);
    return cudaGetLastError();
}

cudaError_t launch_decode_tiles(const uint32_t* code, int K, int IC, int OC, const __half* lut,
                                __half* w, cudaStream_t st) {
    const int TK = IC / 16, TN = OC / 16;
    dim3 grid((TN + 7) / 8, TK), block(256);
    if (K == 2) {
        if (lut) decode_tiles_kernel<2, true><<<grid, block, 0, st>>>(code, lut, w, TN, OC);
        else decode_tiles_kernel<2, false><<<grid, block, 0, st>>>(code, lut, w, TN, OC);
    } else {
        if (lut) decode_tiles_kernel<3, true><<<grid, block, 0, st>>>(code, lut, w, TN, OC);
        else decode_tiles_kernel<3, false><<<grid, block, 0, st>>>(code, lut, w, TN, OC);
    }
    return cudaGetLastError();
}

}  // namespace escha
