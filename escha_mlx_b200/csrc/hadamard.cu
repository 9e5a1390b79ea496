// Scaled 128-block Hadamard transforms around the coded product.
// Replaces escha_scaled_had[_dense], escha_scaled_had_out[_dense] and the
// two-projection *_pair dispatches of the reference
// (escha_mlx/msl.py:875-977, wrappers :1029-1067 and :1481-1527):
//     input :  xh = f16( H128( f32(x) * rin[e] ) * RS )
//     output:  y  = f16( (H128(mid) * RS) * rout[e] )     (two f32 multiplies, in that order)
// One warp owns one (row, 128-block): each lane holds four consecutive
// channels, two butterfly stages run in registers and five through warp
// shuffles -- no shared memory and no barriers.  Every multiply/add is an
// explicit round-to-nearest intrinsic so no FMA contraction can move a
// rounding point; the result is bit-identical to ref.input_transform /
// ref.output_transform.
#include "common.cuh"
#include "kernels.h"

namespace escha {

struct HadShard {
    const void* src;    // f16 rows (input transform) or f32 mid (output transform)
    const float* vec;   // rin / rout: [dim] or [E, dim]
    __half* out;
    int dim;            // IC or OC of this shard
};

template <bool OUTPUT>
__global__ void __launch_bounds__(256)
scaled_had_kernel(HadShard s0, HadShard s1, const int32_t* __restrict__ row_expert, int M,
                  float rs) {
    grid_launch_dependents();
    grid_dependency_wait();
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const uint32_t nb0 = s0.dim >> 7, nb1 = s1.dim >> 7;
    const uint32_t per_row = nb0 + nb1;
    const uint32_t row = unit / per_row;
    if (row >= static_cast<uint32_t>(M)) return;
    uint32_t blk = unit - row * per_row;
    const bool second = blk >= nb0;
    const HadShard& s = second ? s1 : s0;
    if (second) blk -= nb0;

    const size_t off = static_cast<size_t>(row) * s.dim + blk * 128u + lane * 4u;
    const size_t voff = (row_expert ? static_cast<size_t>(row_expert[row]) * s.dim : 0) +
                        blk * 128u + lane * 4u;
    const float4 sc = *reinterpret_cast<const float4*>(s.vec + voff);
    float v[4];
    if (OUTPUT) {
        const float4 m = *reinterpret_cast<const float4*>(static_cast<const float*>(s.src) + off);
        v[0] = m.x; v[1] = m.y; v[2] = m.z; v[3] = m.w;
    } else {
        const uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const __half*>(s.src) + off);
        const float2 a = __half22float2(as_half2(raw.x)), b = __half22float2(as_half2(raw.y));
        v[0] = __fmul_rn(a.x, sc.x); v[1] = __fmul_rn(a.y, sc.y);
        v[2] = __fmul_rn(b.x, sc.z); v[3] = __fmul_rn(b.y, sc.w);
    }
    wht128_warp(v, lane);
    float o[4];
    if (OUTPUT) {
        o[0] = __fmul_rn(__fmul_rn(v[0], rs), sc.x); o[1] = __fmul_rn(__fmul_rn(v[1], rs), sc.y);
        o[2] = __fmul_rn(__fmul_rn(v[2], rs), sc.z); o[3] = __fmul_rn(__fmul_rn(v[3], rs), sc.w);
    } else {
        o[0] = __fmul_rn(v[0], rs); o[1] = __fmul_rn(v[1], rs);
        o[2] = __fmul_rn(v[2], rs); o[3] = __fmul_rn(v[3], rs);
    }
    uint2 packed;
    packed.x = as_u32(__floats2half2_rn(o[0], o[1]));
    packed.y = as_u32(__floats2half2_rn(o[2], o[3]));
    *reinterpret_cast<uint2*>(s.out + off) = packed;
}

// Up to four input transforms of the SAME rows, each with its own scale vector (Q/K/V, gate/up),
// in one launch: the rows are read once.  With `up` given the rows are the gate half of a
// SwiGLU MLP and the input is h = f16( f16(silu(gate)) * up ) (ref.py:296-301), formed here
// instead of by a kernel of its own and a round trip through memory -- the fusion of
// _FusedMLP (escha_mlx/models/qwen3_5.py:63-198).  Bit-identical to the separate launches.
struct HadMany {
    const __half* rows;
    const __half* up;        // nullptr: plain rows
    const float* rin[4];
    __half* out[4];
    int n, dim;
};

// kHadManyUnits 128-blocks per warp, all loads issued before any butterfly.  Measured at 256 rows:
// four blocks per warp take the SwiGLU form of a 17408-wide input from 16.4 to 12.3 us, but a
// three-output transform of a 5120-wide input from 8.6 to 12.2 us (fewer warps, longer serial
// chains), and everything at 32 rows gets slower -- so only the large SwiGLU case uses four.
template <int kHadManyUnits>
__global__ void __launch_bounds__(256)
scaled_had_many_kernel(HadMany s, int M, float rs) {
    grid_launch_dependents();
    grid_dependency_wait();
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t per_row = s.dim >> 7;
    const uint32_t total = static_cast<uint32_t>(M) * per_row;      // [M, dim] is total x 128 halves
    const uint32_t unit0 = (blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * kHadManyUnits;
    if (unit0 >= total) return;
    uint2 raw[kHadManyUnits], ur[kHadManyUnits];
#pragma unroll
    for (int u = 0; u < kHadManyUnits; ++u) {
        const uint32_t unit = min(unit0 + u, total - 1u);   // clamped: the tail re-reads the last block
        const size_t off = static_cast<size_t>(unit) * 128u + lane * 4u;
        raw[u] = *reinterpret_cast<const uint2*>(s.rows + off);
        if (s.up) ur[u] = *reinterpret_cast<const uint2*>(s.up + off);
    }
#pragma unroll
    for (int u = 0; u < kHadManyUnits; ++u) {
        const uint32_t unit = unit0 + u;
        if (unit >= total) break;
        const uint32_t blk = unit % per_row;
        const size_t off = static_cast<size_t>(unit) * 128u + lane * 4u;
        __half2 lo = as_half2(raw[u].x), hi = as_half2(raw[u].y);
        if (s.up) {
            const float2 g0 = __half22float2(lo), g1 = __half22float2(hi);
            const __half2 u0 = as_half2(ur[u].x), u1 = as_half2(ur[u].y);
            auto act = [](float g, __half up) {
                const __half sg = __float2half_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))));
                return __hmul(sg, up);
            };
            lo = __halves2half2(act(g0.x, __low2half(u0)), act(g0.y, __high2half(u0)));
            hi = __halves2half2(act(g1.x, __low2half(u1)), act(g1.y, __high2half(u1)));
        }
        const float2 a = __half22float2(lo), b = __half22float2(hi);
#pragma unroll 1
        for (int i = 0; i < s.n; ++i) {
            const float4 sc = *reinterpret_cast<const float4*>(s.rin[i] + blk * 128u + lane * 4u);
            float v[4] = {__fmul_rn(a.x, sc.x), __fmul_rn(a.y, sc.y), __fmul_rn(b.x, sc.z),
                          __fmul_rn(b.y, sc.w)};
            wht128_warp(v, lane);
            uint2 packed;
            packed.x = as_u32(__floats2half2_rn(__fmul_rn(v[0], rs), __fmul_rn(v[1], rs)));
            packed.y = as_u32(__floats2half2_rn(__fmul_rn(v[2], rs), __fmul_rn(v[3], rs)));
            *reinterpret_cast<uint2*>(s.out[i] + off) = packed;
        }
    }
}

cudaError_t launch_scaled_had_many(const __half* rows, const __half* up, int n,
                                   const float* const* rins, __half* const* outs, int M, int dim,
                                   float rs, cudaStream_t st) {
    HadMany s{};
    s.rows = rows;
    s.up = up;
    s.n = n;
    s.dim = dim;
    for (int i = 0; i < n; ++i) {
        s.rin[i] = rins[i];
        s.out[i] = outs[i];
    }
    const long units = static_cast<long>(M) * (dim / 128);
    if (up != nullptr && units >= 16384)
        return launch_chained(scaled_had_many_kernel<4>, dim3(static_cast<unsigned>((units + 31) / 32)),
                              dim3(256), 0, st, s, M, rs);
    return launch_chained(scaled_had_many_kernel<1>, dim3(static_cast<unsigned>((units + 7) / 8)),
                          dim3(256), 0, st, s, M, rs);
}

// Plain unnormalised H128 on f32 blocks (the reference's moe.had_blocks, which
// calls mx.hadamard_transform(scale=1.0): escha_mlx/moe.py:19-27).
__global__ void __launch_bounds__(256)
had128_kernel(const float* __restrict__ x, float* __restrict__ out, long nblocks) {
    const uint32_t lane = threadIdx.x & 31u;
    const long blk = static_cast<long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (blk >= nblocks) return;
    const float4 m = *reinterpret_cast<const float4*>(x + blk * 128 + lane * 4u);
    float v[4] = {m.x, m.y, m.z, m.w};
    wht128_warp(v, lane);
    *reinterpret_cast<float4*>(out + blk * 128 + lane * 4u) = make_float4(v[0], v[1], v[2], v[3]);
}

cudaError_t launch_had128(const float* x, float* out, long nblocks, cudaStream_t st) {
    const int warps = 8;
    had128_kernel<<<static_cast<unsigned>((nblocks + warps - 1) / warps), warps * 32, 0, st>>>(
        x, out, nblocks);
    return cudaGetLastError();
}

cudaError_t launch_scaled_had(bool output, const void* src0, const float* vec0, __half* out0,
                              int dim0, const void* src1, const float* vec1, __half* out1,
                              int dim1, const int32_t* row_expert, int M, float rs,
                              cudaStream_t st) {
    HadShard s0{src0, vec0, out0, dim0}, s1{src1, vec1, out1, dim1};
    const long units = static_cast<long>(M) * ((dim0 + dim1) / 128);
    const int warps = 8;
    dim3 grid(static_cast<unsigned>((units + warps - 1) / warps)), block(warps * 32);
    if (output) return launch_chained(scaled_had_kernel<true>, grid, block, 0, st, s0, s1, row_expert, M, rs);
    return launch_chained(scaled_had_kernel<false>, grid, block, 0, st, s0, s1, row_expert, M, rs);
}

}  // namespace escha
