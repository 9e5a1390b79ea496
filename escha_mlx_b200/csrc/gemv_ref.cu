// Per-row coded GEMV in the reference kernels' exact accumulation order.
// Replaces escha_moe_gemv_k{K}[_direct][_lut] / escha_gemv_dense_k{K}... and,
// through the optional split argument, escha_..._sk{S}
// (escha_mlx/msl.py:205-435, wrapper :1424-1478).
//
//   mid[r, :] = f32(xh[r, :]) @ f32(decode(code[row_expert[r]]))
//
// A 256-thread CTA covers 128 output channels of one row; warp sg owns output
// tile ocb*8+sg and walks kt ascending.  Per tile a lane adds its values
// j=0..3 into acc0 and j=4..7 into acc1 in ascending j, and the four lanes that
// share a column are combined with xor-1 then xor-2 shuffles -- the order every
// scalar kernel of the reference uses, so this kernel is bit-identical to them
// and to the CPU oracle's restatement.  It is the bit-comparable baseline the
// tensor-core kernel in gemv_mma.cu is checked against, not the fast path.
#include "common.cuh"
#include "kernels.h"

namespace escha {

template <int K, bool LUT>
__global__ void __launch_bounds__(256)
gemv_ref_kernel(const __half* __restrict__ xh, const uint32_t* __restrict__ code,
                const int32_t* __restrict__ row_expert, const int32_t* __restrict__ row_map,
                const __half* __restrict__ lut, float* __restrict__ out, int M, int TK, int TN,
                int splits) {
    constexpr int WPT = 8 * K;
    const uint32_t lane = threadIdx.x & 31u, sg = threadIdx.x >> 5;
    const uint32_t ocb = blockIdx.x, split = blockIdx.z;
    const uint32_t slot = blockIdx.y;
    // row_map lets the row-blocked entry points reuse this kernel: slot -> row
    // index, entries >= M are padding and produce nothing.
    const uint32_t row = row_map ? static_cast<uint32_t>(row_map[slot]) : slot;
    if (row >= static_cast<uint32_t>(M)) return;
    const int IC = TK * 16, OC = TN * 16;
    const uint32_t* base = code;
    if (row_expert) base += static_cast<size_t>(row_expert[row]) * TK * TN * WPT;
    const __half* xbase = xh + static_cast<size_t>(row) * IC;

    const uint32_t kps = TK / splits, kt0 = split * kps, kt1 = kt0 + kps;
    LaneConsts<K> lc(lane);
    const uint32_t xrow = (lane & 3u) * 2u;
    float acc0 = 0.0f, acc1 = 0.0f;
    for (uint32_t kt = kt0; kt < kt1; ++kt) {
        const uint32_t* wp = base + (static_cast<size_t>(kt) * TN + ocb * 8u + sg) * WPT;
        uint32_t s[8];
        lc.states(__ldg(wp + lc.ia()), __ldg(wp + lc.ib()), s);
        const __half2 xv0 = *reinterpret_cast<const __half2*>(xbase + kt * 16u + xrow);
        const __half2 xv1 = *reinterpret_cast<const __half2*>(xbase + kt * 16u + xrow + 8u);
        const float x0 = __low2float(xv0), x1 = __high2float(xv0);
        const float x8 = __low2float(xv1), x9 = __high2float(xv1);
        float d[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) d[j] = __half2float(LUT ? lut[s[j]] : cba_decode(s[j]));
        // half x half products are exact in f32, so fused and unfused forms agree
        acc0 = __fmaf_rn(x0, d[0], acc0);
        acc0 = __fmaf_rn(x1, d[1], acc0);
        acc0 = __fmaf_rn(x8, d[2], acc0);
        acc0 = __fmaf_rn(x9, d[3], acc0);
        acc1 = __fmaf_rn(x0, d[4], acc1);
        acc1 = __fmaf_rn(x1, d[5], acc1);
        acc1 = __fmaf_rn(x8, d[6], acc1);
        acc1 = __fmaf_rn(x9, d[7], acc1);
    }
    acc0 = __fadd_rn(acc0, __shfl_xor_sync(0xFFFFFFFFu, acc0, 1));
    acc0 = __fadd_rn(acc0, __shfl_xor_sync(0xFFFFFFFFu, acc0, 2));
    acc1 = __fadd_rn(acc1, __shfl_xor_sync(0xFFFFFFFFu, acc1, 1));
    acc1 = __fadd_rn(acc1, __shfl_xor_sync(0xFFFFFFFFu, acc1, 2));
    if ((lane & 3u) == 0u) {
        const uint32_t col = lane >> 2;  // 2*((lane&~4)>>3) + ((lane>>2)&1)
        const size_t ob = (static_cast<size_t>(split) * M + row) * OC + ocb * 128u + sg * 16u;
        out[ob + col] = acc0;
        out[ob + col + 8u] = acc1;
    }
}

// Fixed-order reduction of split-K partials: out = ((p0 + p1) + p2) + ...
__global__ void splitk_sum_kernel(const float* __restrict__ part, float* __restrict__ out,
                                  long n, int splits) {
    long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float a = part[i];
    for (int s = 1; s < splits; ++s) a = __fadd_rn(a, part[static_cast<long>(s) * n + i]);
    out[i] = a;
}

cudaError_t launch_gemv_ref(const __half* xh, const uint32_t* code, const int32_t* row_expert,
                            const int32_t* row_map, int slots, const __half* lut, float* out,
                            float* part, int M, int IC, int OC, int K, int splits,
                            cudaStream_t st) {
    const int TK = IC / 16, TN = OC / 16;
    dim3 grid(OC / 128, slots, splits), block(256);
    float* dst = splits > 1 ? part : out;
#define ESCHA_LAUNCH(KK, LL)                                                                   \
    gemv_ref_kernel<KK, LL><<<grid, block, 0, st>>>(xh, code, row_expert, row_map, lut, dst, M, \
                                                    TK, TN, splits)
    if (K == 2) { if (lut) ESCHA_LAUNCH(2, true); else ESCHA_LAUNCH(2, false); }
    else        { if (lut) ESCHA_LAUNCH(3, true); else ESCHA_LAUNCH(3, false); }
#undef ESCHA_LAUNCH
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess || splits <= 1) return e;
    const long n = static_cast<long>(M) * OC;
    splitk_sum_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, st>>>(part, out, n, splits);
    return cudaGetLastError();
}

}  // namespace escha
