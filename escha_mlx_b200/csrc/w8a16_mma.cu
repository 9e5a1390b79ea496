// Tensor-core int8-weight linear for up to 32 rows per pass:
//   y[r, n] = f16( sum_k f32(x[r, k]) * f32( f16( f32(w8[n, k]) * f32(scale[n]) ) ) )
// (escha_mlx/ref.py:308-311 w8a16; mx.quantized_matmul in EschaQ8Linear,
// escha_mlx/quant.py:129-143), with two optional fusions used by the MoE block's
// shared expert (escha_mlx/models/qwen3_5_moe.py:255-273):
//   input    x[r, k] = f16( (g * sigmoid(g)) * u ),  g, u = gate/up halves of gu[r]
//   epilogue out[r, n] = f16( f32(routed[r, n]) + f32(y[r, n]) * sigmoid(gate_logit[r]) )
//            where routed[r, n] is the fixed slot-order combine of the expert rows.
//
// Shape of the work: int8 weights are one byte each and convert to binary16 in
// 1.75 instructions per weight (xor + byte permute into the mantissa of 1024,
// subtract 1152, multiply by the row scale: every step exact but the last, which
// rounds once as the contract demands), so unlike the trellis-coded GEMV this
// kernel is bound by HBM, and the design goal is bytes in flight:
//   * a CTA owns 16 output rows (one mma M tile); its 8 warps split the input
//     dimension in 64-channel chunks, so a [4096, 2048] matrix is 256 CTAs x 8
//     warps, each lane streaming 16-byte pieces of two weight rows;
//   * weights go global -> registers (read once, no reuse to stage for);
//     activations are the mma B operand read through L1/L2 (a few KB per warp);
//   * mma.m16n8k16 contracts over 16 input channels in any order as long as A and
//     B agree, so lane t takes the four consecutive bytes 16t+4s .. 16t+4s+3 of a
//     chunk in step s -- whole 16-byte loads, no shuffles;
//   * the 8 warps' partial sums meet in shared memory and are added in warp
//     order, so the result is bit-reproducible.
#include "common.cuh"
#include "kernels.h"

namespace escha {

namespace {

__device__ __forceinline__ float sigmoid_f32(float v) {
    return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-v)));
}

// bytes (lo, hi) of a biased word (int8 ^ 0x80) -> half2 of the int8 values times scale
__device__ __forceinline__ uint32_t i8pair(uint32_t biased, uint32_t sel, __half2 sc2) {
    const uint32_t v = prmt(biased, 0x64646464u, sel);                   // 1024 + (b ^ 0x80)
    const __half2 w = __hsub2(as_half2(v), as_half2(0x64806480u));        // - 1152: exact int8
    return as_u32(__hmul2(w, sc2));                                      // one rounding
}

// 16 consecutive input channels of one row as 8 words of two halves
template <int IN>
__device__ __forceinline__ void load_x16(const Q8Params& p, int row, int k, uint32_t (&xw)[8]) {
    if (IN == kQ8InputPlain) {
        const uint4* src = reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(row) * p.Kd + k);
        const uint4 a = src[0], b = src[1];
        xw[0] = a.x; xw[1] = a.y; xw[2] = a.z; xw[3] = a.w;
        xw[4] = b.x; xw[5] = b.y; xw[6] = b.z; xw[7] = b.w;
    } else {
        // x = f16((g * sigmoid(g)) * u) from the merged gate/up row [2 * Kd]
        const uint4* gs = reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(row) * 2 * p.Kd + k);
        const uint4* us = reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(row) * 2 * p.Kd + p.Kd + k);
        const uint4 g0 = gs[0], g1 = gs[1], u0 = us[0], u1 = us[1];
        const uint32_t gw[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
        const uint32_t uw[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float2 g = __half22float2(as_half2(gw[i])), u = __half22float2(as_half2(uw[i]));
            const float a = __fmul_rn(__fmul_rn(g.x, sigmoid_f32(g.x)), u.x);
            const float b = __fmul_rn(__fmul_rn(g.y, sigmoid_f32(g.y)), u.y);
            xw[i] = as_u32(__floats2half2_rn(a, b));
        }
    }
}

template <int NT, int IN, int EP>
__global__ void __launch_bounds__(256)
w8a16_mma_kernel(const Q8Params p) {
    __shared__ float s_red[8][16][8 * NT + 1];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    // the linear this CTA belongs to (one unless several share the launch) and its 16 rows
    const int8_t* w8 = p.w8;
    const __half* scale = p.scale;
    __half* yout = p.y;
    int N = p.N, n0 = blockIdx.x * 16;
    if (p.nseg > 0) {
        int sg = 0;
        while (sg + 1 < p.nseg && static_cast<int>(blockIdx.x) >= p.blk0[sg + 1]) ++sg;
        w8 = p.seg_w8[sg]; scale = p.seg_scale[sg]; yout = p.seg_y[sg]; N = p.seg_N[sg];
        n0 = (static_cast<int>(blockIdx.x) - p.blk0[sg]) * 16;
    }
    const int r0 = blockIdx.y * (8 * NT);
    const int chunks = p.Kd >> 6;
    const int cbase = chunks / 8, crem = chunks % 8;
    // scheduled early (programmatic dependent launch): wait for the producers of the inputs
    grid_launch_dependents();
    grid_dependency_wait();
    const int c0 = warp * cbase + min(warp, crem), cn = cbase + (warp < crem ? 1 : 0);

    const int8_t* wa_row = w8 + static_cast<size_t>(n0 + g) * p.Kd + 16 * t;
    const int8_t* wb_row = wa_row + static_cast<size_t>(8) * p.Kd;
    const __half2 sa = __half2half2(scale[n0 + g]), sb = __half2half2(scale[n0 + g + 8]);
    int xrow[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) xrow[nt] = min(r0 + 8 * nt + g, p.M - 1);

    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][i] = 0.0f;

    // enough independent 16-byte loads in flight per lane to cover the DRAM latency
    constexpr int kUnroll = NT == 1 ? 4 : 2;
#pragma unroll kUnroll
    for (int c = c0; c < c0 + cn; ++c) {
        const int k = c * 64;
        const uint4 wa = __ldg(reinterpret_cast<const uint4*>(wa_row + k));
        const uint4 wb = __ldg(reinterpret_cast<const uint4*>(wb_row + k));
        const uint32_t ua[4] = {wa.x ^ 0x80808080u, wa.y ^ 0x80808080u, wa.z ^ 0x80808080u,
                                wa.w ^ 0x80808080u};
        const uint32_t ub[4] = {wb.x ^ 0x80808080u, wb.y ^ 0x80808080u, wb.z ^ 0x80808080u,
                                wb.w ^ 0x80808080u};
        uint32_t a0[4], a1[4], a2[4], a3[4];
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            a0[s] = i8pair(ua[s], 0x4140u, sa);   // row g,     channels 16t+4s, +1
            a2[s] = i8pair(ua[s], 0x4342u, sa);   // row g,     channels 16t+4s+2, +3
            a1[s] = i8pair(ub[s], 0x4140u, sb);   // row g + 8
            a3[s] = i8pair(ub[s], 0x4342u, sb);
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            uint32_t xw[8];
            load_x16<IN>(p, xrow[nt], k + 16 * t, xw);
#pragma unroll
            for (int s = 0; s < 4; ++s)
                mma16816(acc[nt], a0[s], a1[s], a2[s], a3[s], xw[2 * s], xw[2 * s + 1]);
        }
    }

    // accumulator (row g / g+8, token 2t / 2t+1 of tile nt) -> shared, then warp-order sum
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        s_red[warp][g][8 * nt + 2 * t] = acc[nt][0];
        s_red[warp][g][8 * nt + 2 * t + 1] = acc[nt][1];
        s_red[warp][g + 8][8 * nt + 2 * t] = acc[nt][2];
        s_red[warp][g + 8][8 * nt + 2 * t + 1] = acc[nt][3];
    }
    __syncthreads();
    for (int idx = tid; idx < 16 * 8 * NT; idx += 256) {
        const int j = idx >> 4, rr = idx & 15;   // token j of this pass, output row rr
        const int row = r0 + j;
        if (row >= p.M) continue;
        float v = s_red[0][rr][j];
#pragma unroll
        for (int w = 1; w < 8; ++w) v = __fadd_rn(v, s_red[w][rr][j]);
        const __half y = __float2half_rn(v);
        const size_t o = static_cast<size_t>(row) * N + n0 + rr;
        if (EP == kQ8StorePlain) {
            yout[o] = y;
        } else {
            // routed-expert combine for this (token, channel), then the gated add
            float comb = 0.0f;
            for (int s = 0; s < p.top_k; ++s) {
                const size_t er = static_cast<size_t>(row) * p.top_k + s;
                const float w16 = __half2float(__float2half_rn(p.scores[er]));
                // expert parallel: every rank's rows were gathered side by side; a row
                // is valid in the copy of the rank that owns its expert
                const size_t src = p.ids ? static_cast<size_t>(p.ids[er] / p.experts_per_rank) *
                                               p.M * p.top_k + er
                                         : er;
                comb = __fadd_rn(comb, __fmul_rn(__half2float(p.d16[src * p.N + n0 + rr]), w16));
            }
            const float routed = __half2float(__float2half_rn(comb));
            const float gate = sigmoid_f32(p.gate_logit[row]);
            p.y[o] = __float2half_rn(__fadd_rn(routed, __fmul_rn(__half2float(y), gate)));
        }
    }
}

template <int IN, int EP>
cudaError_t launch_nt(const Q8Params& p, cudaStream_t st) {
    const int rows = p.M < 32 ? p.M : 32;
    const int nt = (rows + 7) / 8;
    const dim3 grid(p.nseg > 0 ? p.blk0[p.nseg] : p.N / 16, (p.M + 8 * nt - 1) / (8 * nt));
    switch (nt) {
        case 1: return launch_dependent(w8a16_mma_kernel<1, IN, EP>, grid, dim3(256), 0, st, p);
        case 2: return launch_dependent(w8a16_mma_kernel<2, IN, EP>, grid, dim3(256), 0, st, p);
        case 3: return launch_dependent(w8a16_mma_kernel<3, IN, EP>, grid, dim3(256), 0, st, p);
        default: return launch_dependent(w8a16_mma_kernel<4, IN, EP>, grid, dim3(256), 0, st, p);
    }
}

}  // namespace

bool w8a16_mma_supports(int N, int Kd) { return N % 16 == 0 && Kd % 64 == 0 && N > 0 && Kd > 0; }

cudaError_t launch_w8a16_mma(const Q8Params& p, cudaStream_t st) {
    if (p.input == kQ8InputPlain)
        return p.epilogue == kQ8StorePlain ? launch_nt<kQ8InputPlain, kQ8StorePlain>(p, st)
                                           : launch_nt<kQ8InputPlain, kQ8StoreGatedAdd>(p, st);
    return p.epilogue == kQ8StorePlain ? launch_nt<kQ8InputSwiglu, kQ8StorePlain>(p, st)
                                       : launch_nt<kQ8InputSwiglu, kQ8StoreGatedAdd>(p, st);
}

}  // namespace escha
