// Prefill row-blocked coded GEMM on the 5th-generation tensor cores:
//     mid[r, :] = f32(xh[r, :]) @ f32(decode(code))        for M = tens to hundreds of rows
// -- the product behind dense_gemm_mat / dense_gemm_rows at prefill sizes
// (escha_mlx/msl.py:1608-1782, :1785-1841 of the reference, which runs it on 8x8
// simdgroup-matrix fragments with R = 16 rows per decode).
//
// At these row counts the decoded tile is a real dense contraction, so the trellis
// decode and the matrix product are split between the two machines an SM has:
//
//   16 decode warps  read the code stream (each warp half of a 16-channel column of tiles),
//                    walk the trellis windows in registers, and write binary16
//                    weights into a shared-memory ring in the K-major, 128-byte
//                    swizzled layout tcgen05 consumes: each weight is decoded ONCE
//                    for up to 256 rows.
//   1 code warp      streams the CTA's slice of the code into a shared-memory ring with
//                    bulk copies (cp.async.bulk, no multicast), so the decode warps
//                    never wait on a global load.
//   1 loader thread  brings the matching slice of the activations with one tiled TMA load
//                    per chunk (cp.async.bulk.tensor, 128-byte swizzle, no multicast;
//                    rows past M are zero-filled) into a ring of its own.
//   1 issuing thread feeds tcgen05.mma (M = 128 channels x N = 128 or 256 rows x K = 16
//                    per instruction, both operands from shared memory) with fp32
//                    accumulators in tensor memory; tcgen05.commit hands each ring
//                    slot back to the producers when the tensor core is done with it.
//   4 warps          read the accumulators back with tcgen05.ld and store fp32.
//
// One CTA owns a 128-channel output block (one Hadamard block) for up to 256 rows
// and a range of the input dimension; with splits > 1 each split writes its own
// partial [M, OC] plane, summed afterwards in split order (deterministic).  The
// output transform runs as its own kernel on the summed mid.
//
// Every wait on an mbarrier is bounded; a wait that gives up raises the status word,
// the CTA drains, frees its tensor memory and leaves.
#include <cstdlib>
#include <cstring>

#include "kernels.h"
#include "tcgen05.cuh"

namespace escha {

namespace {

constexpr int kBStages = 6;                       // decoded-weight ring (16 KiB slots)
constexpr int kAStages = 3;                       // activation ring (16 KiB per 128 rows per slot)
constexpr int kChunkK = 64;                       // input channels per ring slot
constexpr int kTileN = 128;                       // output channels per CTA
constexpr int kBBytes = kTileN * kChunkK * 2;     // 16 KiB of decoded weights per slot
constexpr int kABytesPerMt = 128 * kChunkK * 2;   // 16 KiB of activations per 128 rows
constexpr int kDecodeWarps = 16;
constexpr int kCodeStages = 6;                    // code-stream ring depth (chunks)
constexpr int kThreadsTc = (kDecodeWarps + 3) * 32;   // + activation loader, issuing and code warps

__device__ int g_gemm_status = 0;

template <int K, int MT>
__global__ void __launch_bounds__(kThreadsTc, 1)
gemm_tc_kernel(const __grid_constant__ GemmTcParams p, const __grid_constant__ CUtensorMap xmap) {
    constexpr int WPT = 8 * K;
    constexpr uint32_t kABytes = MT * kABytesPerMt;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t s_bfull[kBStages], s_bempty[kBStages];
    __shared__ __align__(8) uint64_t s_afull[kAStages], s_aempty[kAStages];
    __shared__ __align__(8) uint64_t s_cfull[kCodeStages], s_cempty[kCodeStages], s_done;
    __shared__ uint32_t s_tmem;

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t ocb = blockIdx.x, split = blockIdx.y, r0 = blockIdx.z * (128u * MT);
    // dynamic shared memory is only guaranteed 16-byte alignment: round up to the
    // 1024 bytes the swizzle pattern is anchored to
    const uint32_t aring = (smem_u32(smem_raw) + 1023u) & ~1023u;   // [kAStages][rows][128 B]
    const uint32_t bring = aring + kAStages * kABytes;              // [kBStages][128][128 B]
    const uint32_t bfull0 = smem_u32(s_bfull), bempty0 = smem_u32(s_bempty);
    const uint32_t afull0 = smem_u32(s_afull), aempty0 = smem_u32(s_aempty);
    const uint32_t cfull0 = smem_u32(s_cfull), cempty0 = smem_u32(s_cempty), done = smem_u32(&s_done);
    constexpr uint32_t kRowBytes = 8u * WPT * 4u;          // one tile row of the CTA's 8 tile columns
    constexpr uint32_t kCodeChunkBytes = 4u * kRowBytes;   // four tile rows = 64 input channels
    const uint32_t code0 = bring + kBStages * kBBytes;     // code ring follows the operand rings

    const uint32_t nchunk_all = static_cast<uint32_t>(p.IC) / kChunkK;
    const uint32_t S = p.splits, cbase = nchunk_all / S, crem = nchunk_all % S;
    const uint32_t c_first = split * cbase + min(split, crem);
    const uint32_t nchunk = cbase + (split < crem ? 1u : 0u);

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < kBStages; ++s) {
            mbar_init(bfull0 + 8u * s, kDecodeWarps);
            mbar_init(bempty0 + 8u * s, 1u);
        }
#pragma unroll
        for (int s = 0; s < kAStages; ++s) {
            mbar_init(afull0 + 8u * s, 1u);    // the loader's arrive.expect_tx
            mbar_init(aempty0 + 8u * s, 1u);
        }
#pragma unroll
        for (int s = 0; s < kCodeStages; ++s) {
            mbar_init(cfull0 + 8u * s, 1u);             // the code warp's arrive.expect_tx
            mbar_init(cempty0 + 8u * s, kDecodeWarps);  // one arrival per decode warp
        }
        mbar_init(done, 1u);
        mbar_fence_init();
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(&s_tmem), 128u * MT);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = s_tmem;

    bool ok = true;
    if (warp < kDecodeWarps) {
        // ---- decode warps: warp w owns output channels 16(w&7) .. +15 of the block and
        // tile rows 2(w>>3), 2(w>>3)+1 of every 64-channel chunk
        const LaneConsts<K> lc(lane);
        const uint32_t g = lane >> 2, t = lane & 3u;
        const uint32_t wn = warp & 7u, q0 = 2u * (warp >> 3);
        const uint32_t hmask = p.hash_mask, hxor = p.hash_xor;
        const ShiftMuls muls{p.mul2, p.mul4, p.mul16, p.mul32, p.mul64, p.mul128};
        const uint32_t my_words = code0 + q0 * kRowBytes + wn * (WPT * 4u);
        const uint32_t row_lo = 16u * wn + g, row_hi = row_lo + 8u;
        for (uint32_t c = 0; c < nchunk; ++c) {
            // this warp's two tiles of the chunk: two words per lane and tile from the code ring
            const uint32_t cslot = c % kCodeStages;
            if (!mbar_wait_relaxed(cfull0 + 8u * cslot, (c / kCodeStages) & 1u)) {
                ok = false;
                break;
            }
            uint32_t wa[2], wb[2];
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const uint32_t tp = my_words + cslot * kCodeChunkBytes + q * kRowBytes;
                asm volatile("ld.shared.b32 %0, [%1];" : "=r"(wa[q]) : "r"(tp + 4u * lc.ia()));
                asm volatile("ld.shared.b32 %0, [%1];" : "=r"(wb[q]) : "r"(tp + 4u * lc.ib()));
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(cempty0 + 8u * cslot);
            uint32_t a[2][8];
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                uint32_t s[8];
                lc.states(wa[q], wb[q], muls, s);
#pragma unroll
                for (int j = 0; j < 8; ++j) a[q][j] = cba_decode_dup(s[j], hmask, hxor);
            }
            const uint32_t slot = c % kBStages;
            if (c >= kBStages && !mbar_wait_relaxed(bempty0 + 8u * slot, ((c / kBStages) - 1u) & 1u)) {
                ok = false;
                break;
            }
            const uint32_t bslot = bring + slot * kBBytes;
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                // value j sits at (channel g + 8*(j>=4), input 2t + (j&1) + 8*((j>>1)&1)) of
                // its tile row: pairs (0,1), (2,3), (4,5), (6,7) are two consecutive inputs
                const uint32_t c_lo = 2u * (q0 + q), c_hi = c_lo + 1u;   // 16-byte chunks of the row
                const uint32_t p01 = prmt(a[q][0], a[q][1], 0x5410u), p23 = prmt(a[q][2], a[q][3], 0x5410u);
                const uint32_t p45 = prmt(a[q][4], a[q][5], 0x5410u), p67 = prmt(a[q][6], a[q][7], 0x5410u);
                asm volatile("st.shared.b32 [%0], %1;" ::"r"(bslot + sw128(row_lo, c_lo) + 4u * t), "r"(p01) : "memory");
                asm volatile("st.shared.b32 [%0], %1;" ::"r"(bslot + sw128(row_lo, c_hi) + 4u * t), "r"(p23) : "memory");
                asm volatile("st.shared.b32 [%0], %1;" ::"r"(bslot + sw128(row_hi, c_lo) + 4u * t), "r"(p45) : "memory");
                asm volatile("st.shared.b32 [%0], %1;" ::"r"(bslot + sw128(row_hi, c_hi) + 4u * t), "r"(p67) : "memory");
            }
            fence_async_proxy();
            __syncwarp();
            if (lane == 0) mbar_arrive(bfull0 + 8u * slot);
        }
    } else if (warp == kDecodeWarps) {
        // ---- activation loader: one tiled TMA load per chunk (rows r0.., 64 channels, written
        // in the 128-byte swizzle; rows past M are filled with zeros by the copy engine)
        if (lane == 0) {
            for (uint32_t c = 0; c < nchunk; ++c) {
                const uint32_t slot = c % kAStages;
                if (c >= kAStages && !mbar_wait_relaxed(aempty0 + 8u * slot, ((c / kAStages) - 1u) & 1u)) {
                    ok = false;
                    break;
                }
                mbar_arrive_expect_tx(afull0 + 8u * slot, kABytes);
                tma_load_2d(aring + slot * kABytes, &xmap, static_cast<int32_t>((c_first + c) * kChunkK),
                            static_cast<int32_t>(r0), afull0 + 8u * slot);
            }
        }
    } else if (warp == kDecodeWarps + 2) {
        // ---- code warp: bulk copies (TMA, untiled, no multicast) of the CTA's slice of the
        // code stream, one copy per tile row (8 tiles side by side), four rows per chunk
        const uint32_t TN = static_cast<uint32_t>(p.OC) >> 4;
        const size_t kt_words = static_cast<size_t>(TN) * WPT;   // words from tile row kt to kt+1
        const uint32_t* grow = p.code + (static_cast<size_t>(c_first) * 4u + lane) * kt_words +
                               static_cast<size_t>(ocb) * 8u * WPT;
        for (uint32_t c = 0; c < nchunk; ++c) {
            const uint32_t cslot = c % kCodeStages;
            if (c >= kCodeStages &&
                !mbar_wait_relaxed(cempty0 + 8u * cslot, ((c / kCodeStages) - 1u) & 1u)) {
                ok = false;
                break;
            }
            if (lane == 0) mbar_arrive_expect_tx(cfull0 + 8u * cslot, kCodeChunkBytes);
            __syncwarp();
            if (lane < 4)
                bulk_copy_g2s(code0 + cslot * kCodeChunkBytes + lane * kRowBytes, grow, kRowBytes,
                              cfull0 + 8u * cslot);
            grow += 4u * kt_words;
        }
    } else if (lane == 0) {
        // ---- the issuing thread (warp kDecodeWarps + 1)
        for (uint32_t c = 0; c < nchunk; ++c) {
            const uint32_t bs = c % kBStages, as = c % kAStages;
            if (!mbar_wait_relaxed(bfull0 + 8u * bs, (c / kBStages) & 1u) ||
                !mbar_wait_relaxed(afull0 + 8u * as, (c / kAStages) & 1u)) {
                ok = false;
                break;
            }
            tc_fence_after_sync();
            const uint32_t bslot = bring + bs * kBBytes, aslot = aring + as * kABytes;
            // D[channel][row] += W[channel][k] * X[row][k]: one instruction per 16 channels of
            // K covers all 128 x (128 MT) outputs, so each weight tile is fetched once
#pragma unroll
            for (uint32_t k16 = 0; k16 < kChunkK / 16; ++k16)
                umma_f16(tmem, smem_desc_sw128(bslot + 32u * k16), smem_desc_sw128(aslot + 32u * k16),
                         idesc_for(128u * MT), (c | k16) != 0u);
            // both slots are free once these MMAs have read them
            umma_commit(bempty0 + 8u * bs);
            umma_commit(aempty0 + 8u * as);
        }
        if (ok) umma_commit(done);
    }
    if (!ok && lane == 0) atomicExch(&g_gemm_status, 1);

    // ---- epilogue: warps 0..3 own accumulator lanes 32w .. 32w+31 (= output channels of the
    // block); columns are activation rows.
    const bool fused_out = p.rout != nullptr;   // only with splits == 1 (checked by the host)
    float* const stage = reinterpret_cast<float*>(smem_raw + (aring - smem_u32(smem_raw)));
    if (warp < 4) {
        bool ready = __shfl_sync(0xFFFFFFFFu, ok ? 1 : 0, 0) != 0 && nchunk > 0;
        if (ready && !mbar_wait_relaxed(done, 0u)) {
            ready = false;
            if (lane == 0) atomicExch(&g_gemm_status, 2);
        }
        tc_fence_after_sync();
        if (ready) {
            float* plane = p.out + static_cast<size_t>(split) * p.M * p.OC + ocb * 128u + 32u * warp + lane;
#pragma unroll 1
            for (uint32_t col = 0; col < 128u * MT; col += 16u) {
                if (r0 + col >= static_cast<uint32_t>(p.M)) break;   // uniform: no rows left
                uint32_t v[16];
                tmem_ld16(tmem + ((32u * warp) << 16) + col, v);
                tmem_ld_wait();
                if (fused_out) {
                    // transpose through shared memory (the rings are idle now): [row][channel]
#pragma unroll
                    for (uint32_t i = 0; i < 16u; ++i)
                        stage[(col + i) * 128u + 32u * warp + lane] = __uint_as_float(v[i]);
                } else {
                    // for one row a warp stores 32 consecutive floats
#pragma unroll
                    for (uint32_t i = 0; i < 16u; ++i) {
                        const uint32_t row = r0 + col + i;
                        if (row < static_cast<uint32_t>(p.M))
                            plane[static_cast<size_t>(row) * p.OC] = __uint_as_float(v[i]);
                    }
                }
            }
        }
    }
    if (fused_out) {
        // every warp of the CTA: one row per step, four consecutive channels per lane ->
        // 128-point butterflies across the warp, scales, binary16 store
        __syncthreads();
        const uint32_t nwarps = kThreadsTc / 32u;
        const uint32_t rows_here = min(128u * MT, static_cast<uint32_t>(p.M) - r0);
        const float4 sc = *reinterpret_cast<const float4*>(p.rout + ocb * 128u + lane * 4u);
        for (uint32_t r = warp; r < rows_here; r += nwarps) {
            const float4 a = *reinterpret_cast<const float4*>(stage + r * 128u + lane * 4u);
            float v[4] = {a.x, a.y, a.z, a.w};
            wht128_warp(v, lane);
            uint2 packed;
            packed.x = as_u32(__floats2half2_rn(__fmul_rn(__fmul_rn(v[0], p.rs), sc.x),
                                                __fmul_rn(__fmul_rn(v[1], p.rs), sc.y)));
            packed.y = as_u32(__floats2half2_rn(__fmul_rn(__fmul_rn(v[2], p.rs), sc.z),
                                                __fmul_rn(__fmul_rn(v[3], p.rs), sc.w)));
            *reinterpret_cast<uint2*>(p.y16 + static_cast<size_t>(r0 + r) * p.OC + ocb * 128u + lane * 4u) = packed;
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 128u * MT);
}

}  // namespace

// cuTensorMapEncodeTiled, resolved through the runtime (the library does not link libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

cudaError_t encode_x_map(CUtensorMap* map, const __half* xh, int M, int IC, int rows_per_box) {
    // resolved once per process (the initialisation of a function-local static is safe from
    // several host threads); nullptr if the driver does not offer the entry point
    static const EncodeTiledFn fn = [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        const cudaError_t e =
            cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q);
        return (e == cudaSuccess && q == cudaDriverEntryPointSuccess) ? reinterpret_cast<EncodeTiledFn>(sym)
                                                                      : static_cast<EncodeTiledFn>(nullptr);
    }();
    if (!fn) return cudaErrorNotSupported;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(IC), static_cast<cuuint64_t>(M)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(IC) * 2u};   // bytes between rows
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(kChunkK), static_cast<cuuint32_t>(rows_per_box)};
    const cuuint32_t estr[2] = {1u, 1u};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2u, const_cast<__half*>(xh), dims,
                          strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

namespace {

template <int K, int MT>
cudaError_t launch_tc(const GemmTcParams& p, cudaStream_t st) {
    const size_t smem = static_cast<size_t>(kAStages) * MT * kABytesPerMt +
                        static_cast<size_t>(kBStages) * kBBytes +
                        static_cast<size_t>(kCodeStages) * 4u * (8u * 8u * K * 4u) + 1024;
    static SmemLimit limit;
    cudaError_t e = limit.ensure(gemm_tc_kernel<K, MT>, smem);
    if (e != cudaSuccess) return e;
    CUtensorMap xmap;
    e = encode_x_map(&xmap, p.xh, p.M, p.IC, 128 * MT);
    if (e != cudaSuccess) return e;
    const dim3 grid(p.OC / 128, p.splits, (p.M + 128 * MT - 1) / (128 * MT));
    gemm_tc_kernel<K, MT><<<grid, kThreadsTc, smem, st>>>(p, xmap);
    return cudaGetLastError();
}

}  // namespace

// ESCHA_B200_TC_WEIGHTS=tmem (default) | smem: which operand path the decoded weights take
bool gemm_tc_uses_tmem() {
    static const bool through_tmem = [] {
        const char* e = std::getenv("ESCHA_B200_TC_WEIGHTS");
        return e == nullptr || std::strcmp(e, "smem") != 0;
    }();
    return through_tmem;
}

cudaError_t launch_gemm_tc(const GemmTcParams& p, cudaStream_t st) {
    if (gemm_tc_uses_tmem() && gemm_tcm_supports(p)) return launch_gemm_tcm(p, st);
    const bool two = p.M > 128;
    if (p.K == 2) return two ? launch_tc<2, 2>(p, st) : launch_tc<2, 1>(p, st);
    return two ? launch_tc<3, 2>(p, st) : launch_tc<3, 1>(p, st);
}

namespace {
// mid = ((plane0 + plane1) + plane2) + ... in split order
__global__ void sum_planes_kernel(const float4* __restrict__ planes, float4* __restrict__ mid,
                                  size_t n4, int splits) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n4) return;
    float4 a = planes[i];
    for (int s = 1; s < splits; ++s) {
        const float4 b = planes[static_cast<size_t>(s) * n4 + i];
        a.x = __fadd_rn(a.x, b.x); a.y = __fadd_rn(a.y, b.y);
        a.z = __fadd_rn(a.z, b.z); a.w = __fadd_rn(a.w, b.w);
    }
    mid[i] = a;
}
}  // namespace

namespace {
// y = f16( (H128(plane0 + plane1 + ...) * rs) * rout ): the split-order sum and the output
// transform (escha_mlx/ref.py:226-228) in one pass; one warp per (row, 128-channel block).
__global__ void __launch_bounds__(256)
planes_out_kernel(const float* __restrict__ planes, const float* __restrict__ rout,
                  __half* __restrict__ y, int M, int OC, int splits, float rs) {
    grid_launch_dependents();
    grid_dependency_wait();
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const uint32_t per_row = static_cast<uint32_t>(OC) >> 7;
    const uint32_t row = unit / per_row;
    if (row >= static_cast<uint32_t>(M)) return;
    const uint32_t blk = unit - row * per_row;
    const size_t off = static_cast<size_t>(row) * OC + blk * 128u + lane * 4u;
    const size_t plane = static_cast<size_t>(M) * OC;
    const float4 a = *reinterpret_cast<const float4*>(planes + off);
    float v[4] = {a.x, a.y, a.z, a.w};
    for (int s = 1; s < splits; ++s) {
        const float4 b = *reinterpret_cast<const float4*>(planes + s * plane + off);
        v[0] = __fadd_rn(v[0], b.x); v[1] = __fadd_rn(v[1], b.y);
        v[2] = __fadd_rn(v[2], b.z); v[3] = __fadd_rn(v[3], b.w);
    }
    wht128_warp(v, lane);
    const float4 sc = *reinterpret_cast<const float4*>(rout + blk * 128u + lane * 4u);
    uint2 packed;
    packed.x = as_u32(__floats2half2_rn(__fmul_rn(__fmul_rn(v[0], rs), sc.x),
                                        __fmul_rn(__fmul_rn(v[1], rs), sc.y)));
    packed.y = as_u32(__floats2half2_rn(__fmul_rn(__fmul_rn(v[2], rs), sc.z),
                                        __fmul_rn(__fmul_rn(v[3], rs), sc.w)));
    *reinterpret_cast<uint2*>(y + off) = packed;
}
// the same for up to three projections of one launch
struct PlanesOutMany {
    const float* planes[3];
    const float* rout[3];
    __half* y[3];
    int OC[3];
    int n;
};
__global__ void __launch_bounds__(256)
planes_out_many_kernel(PlanesOutMany s, int M, int splits, float rs) {
    grid_launch_dependents();
    grid_dependency_wait();
    const uint32_t lane = threadIdx.x & 31u;
    uint32_t unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    // units are laid out projection after projection, M * (OC / 128) each
    uint32_t pj = 0;
    while (pj + 1u < static_cast<uint32_t>(s.n) &&
           unit >= static_cast<uint32_t>(M) * (static_cast<uint32_t>(s.OC[pj]) >> 7)) {
        unit -= static_cast<uint32_t>(M) * (static_cast<uint32_t>(s.OC[pj]) >> 7);
        ++pj;
    }
    const uint32_t OC = static_cast<uint32_t>(s.OC[pj]);
    const uint32_t per_row = OC >> 7;
    const uint32_t row = unit / per_row;
    if (row >= static_cast<uint32_t>(M)) return;
    const uint32_t blk = unit - row * per_row;
    const size_t off = static_cast<size_t>(row) * OC + blk * 128u + lane * 4u;
    const size_t plane = static_cast<size_t>(M) * OC;
    const float* planes = s.planes[pj];
    const float4 a = *reinterpret_cast<const float4*>(planes + off);
    float v[4] = {a.x, a.y, a.z, a.w};
    for (int i = 1; i < splits; ++i) {
        const float4 b = *reinterpret_cast<const float4*>(planes + i * plane + off);
        v[0] = __fadd_rn(v[0], b.x); v[1] = __fadd_rn(v[1], b.y);
        v[2] = __fadd_rn(v[2], b.z); v[3] = __fadd_rn(v[3], b.w);
    }
    wht128_warp(v, lane);
    const float4 sc = *reinterpret_cast<const float4*>(s.rout[pj] + blk * 128u + lane * 4u);
    uint2 packed;
    packed.x = as_u32(__floats2half2_rn(__fmul_rn(__fmul_rn(v[0], rs), sc.x),
                                        __fmul_rn(__fmul_rn(v[1], rs), sc.y)));
    packed.y = as_u32(__floats2half2_rn(__fmul_rn(__fmul_rn(v[2], rs), sc.z),
                                        __fmul_rn(__fmul_rn(v[3], rs), sc.w)));
    *reinterpret_cast<uint2*>(s.y[pj] + off) = packed;
}
}  // namespace

cudaError_t launch_planes_out_many(int n, const float* const* planes, const float* const* routs,
                                   __half* const* ys, const int* OCs, int M, int splits, float rs,
                                   cudaStream_t st) {
    PlanesOutMany s{};
    s.n = n;
    long units = 0;
    for (int i = 0; i < n; ++i) {
        s.planes[i] = planes[i];
        s.rout[i] = routs[i];
        s.y[i] = ys[i];
        s.OC[i] = OCs[i];
        units += static_cast<long>(M) * (OCs[i] / 128);
    }
    return launch_chained(planes_out_many_kernel, dim3(static_cast<unsigned>((units + 7) / 8)),
                          dim3(256), 0, st, s, M, splits, rs);
}

cudaError_t launch_planes_out(const float* planes, const float* rout, __half* y, int M, int OC,
                              int splits, float rs, cudaStream_t st) {
    const long units = static_cast<long>(M) * (OC / 128);
    return launch_chained(planes_out_kernel, dim3(static_cast<unsigned>((units + 7) / 8)), dim3(256), 0,
                          st, planes, rout, y, M, OC, splits, rs);
}

cudaError_t launch_sum_planes(const float* planes, float* mid, size_t n, int splits, cudaStream_t st) {
    const size_t n4 = n / 4;
    sum_planes_kernel<<<static_cast<unsigned>((n4 + 255) / 256), 256, 0, st>>>(
        reinterpret_cast<const float4*>(planes), reinterpret_cast<float4*>(mid), n4, splits);
    return cudaGetLastError();
}

cudaError_t gemm_tc_status(int* host_status) {
    int a = 0, b = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&a, g_gemm_status, sizeof(int));
    if (e == cudaSuccess) e = gemm_tcm_status(&b);
    *host_status = a != 0 ? a : b;
    return e;
}

}  // namespace escha
