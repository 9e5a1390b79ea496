// Prefill coded GEMM on tcgen05 with the decoded weights handed to the tensor core through
// TENSOR MEMORY instead of shared memory:
//     mid[r, :] = f32(xh[r, :]) @ f32(decode(code))
// (the product of escha_mlx/msl.py:1608-1782, :1785-1841 of the reference at prefill sizes).
//
// The shared-memory-operand kernel (gemm_tc.cu) is limited by its decode warps, and 40 of the
// 96 instructions they spend per 16x16 tile go into getting the weights into the swizzled
// shared-memory layout: pairing, four scattered 4-byte stores with their addresses, a proxy
// fence and a barrier round per 64 channels.  Here the weights are the A operand of
// tcgen05.mma read from tensor memory, whose layout is "lane = output channel, column = two
// consecutive input channels": a decode thread that owns ONE output channel writes 32 weights
// of that channel with a single tcgen05.st and no address arithmetic at all.
//
// That needs the trellis walked channel-major rather than in the mma-fragment order of the
// GEMV kernels.  State i of a tile is the 16-bit window that ends K(i+1) bits into the tile's
// MSB-first bit stream (escha_mlx/ref.py:64-93), and the value at (channel c, input k) of the
// tile is state 32(c&7) + 8((k&7)>>1) + 4(c>>3) + 2(k>>3) + (k&1) (ref.py:96-134).  So the 16
// inputs of one channel are four runs of four consecutive states; each run lies within one
// 32-bit window that a byte permute cuts out of two adjacent words of the stream.
//
//   warp 0           issues tcgen05.mma (A from tensor memory, B = activations from shared
//                    memory, fp32 accumulators in tensor memory: 128 channels x 128 or 256 rows
//                    x 16 per instruction).  Its loop is warp-uniform with one elected lane
//                    issuing; one tcgen05.commit per stage hands its ring slots back.  Measured: a commit returns
//                    only when the instructions before it have run, so this warp is paced by
//                    the tensor core (about 128 cycles per instruction) and must not also wait
//                    for issue slots behind the decode warps -- hence the CTA's first warp.
//   warp 1           one thread: tiled TMA loads of the activations, two boxes of 64 channels x
//                    up to 256 rows per stage (128-byte swizzle, no multicast, rows past M
//                    zero-filled).
//   warp 2           bulk copies of the CTA's slice of the code stream into a ring.
//   warps 4..19      decode: warp w owns channels 32(w&3)..+31 of the CTA's 128 (the tensor-
//                    memory lanes a warp may address) and input channels 32((w-4)>>2)..+31 of
//                    every 128-channel stage: lane = channel, 32 weights per lane and stage.
//   epilogue         the decode warps read the accumulators back (tcgen05.ld), each a quarter
//                    of the columns of its lanes; with a fused output transform the tile is
//                    transposed through the idle activation ring and every warp runs
//                    128-point butterflies on its rows.
//
// Tensor memory: columns 0..255 accumulators, 256..511 four weight stages of 64 columns.
// Every wait on an mbarrier is bounded; a wait that gives up raises the status word, the CTA
// drains, frees its tensor memory and leaves.
#include "kernels.h"
#include "tcgen05.cuh"

namespace escha {

namespace {

constexpr int kStageK = 128;                      // input channels per weight stage
constexpr int kWStages = 4;                       // weight stages in tensor memory
constexpr uint32_t kWStageCols = kStageK / 2;     // two binary16 per 32-bit column
constexpr uint32_t kWCol0 = 256;                  // weight stages follow the accumulators
constexpr uint32_t kTmemCols = 512;
constexpr int kXStages = 3;                       // activation ring slots (128 channels each)
constexpr int kFreeBars = 12;                     // a common multiple of the two ring depths
constexpr int kXChunkK = 64;
constexpr int kXBytesPerMt = 128 * kXChunkK * 2;  // 16 KiB of activations per 128 rows
constexpr int kDecodeWarps = 16;
constexpr int kCodeStages = 4;                    // code ring depth (stages of 128 channels)
constexpr int kServiceWarps = 4;                   // issuing warp, two loader warps, one spare
constexpr int kThreadsTcm = (kServiceWarps + kDecodeWarps) * 32;

__device__ int g_gemm_tcm_status = 0;

// Per-lane constants of the channel-major walk.  g = channel & 7, hi = channel >> 3 within the
// tile.  Run t (inputs 2t, 2t+1, 2t+8, 2t+9) ends at stream byte Eb(t) (rounded up to a byte;
// the 3-bit stream of a low channel ends 4 bits earlier, which moves into the state shifts):
//   K = 2: Eb = 8g + 2t + hi + 1         K = 3: Eb = 12g + 3t + 2 + hi
// The window is stream bytes Eb-4 .. Eb-1, r bytes into the pair of words (p, p+1):
//   K = 2: p = 2g-1, 2g-1, 2g, 2g  r = 1+hi, 3+hi, 1+hi, 3+hi
//   K = 3: p = 3g-1, 3g, 3g+1, 3g+1  r = 2+hi, 1+hi, hi, 3+hi
// and prmt(later word, earlier word, 0x7654 - 0x1111 r) cuts it out.
template <int K>
struct ChannelLane;

template <>
struct ChannelLane<2> {
    static constexpr int kWords = 3;
    uint32_t off[3];       // byte offsets of words 2g-1 (wrapping), 2g, 2g+1 within the tile
    uint32_t sel_even, sel_odd;
    __device__ __forceinline__ ChannelLane(uint32_t l16, const GemmTcParams&) {
        const uint32_t g = l16 & 7u, hi = l16 >> 3;
        off[0] = 4u * ((2u * g + 15u) & 15u);
        off[1] = 8u * g;
        off[2] = 8u * g + 4u;
        sel_even = 0x7654u - 0x1111u * (1u + hi);
        sel_odd = 0x7654u - 0x1111u * (3u + hi);
    }
    // states of inputs (2t, 2t+1, 2t+8, 2t+9), t = 0..3, in s[4t .. 4t+3]
    __device__ __forceinline__ void states(const uint32_t (&w)[3], const ShiftMuls& m,
                                           uint32_t (&s)[16]) const {
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const uint32_t win = prmt(w[(t >> 1) + 1], w[t >> 1], (t & 1) ? sel_odd : sel_even);
            s[4 * t + 0] = prmt(win * m.m4, 0u, 0x4421u);    // bit 6 -> 8
            s[4 * t + 1] = prmt(win * m.m16, 0u, 0x4421u);   // bit 4 -> 8
            s[4 * t + 2] = prmt(win * m.m64, 0u, 0x4421u);   // bit 2 -> 8
            s[4 * t + 3] = prmt(win, 0u, 0x4410u);           // bit 0
        }
    }
};

template <>
struct ChannelLane<3> {
    static constexpr int kWords = 4;
    uint32_t off[4];       // words 3g-1 (wrapping), 3g, 3g+1, 3g+2
    uint32_t sel[4];
    uint32_t mul[4], bsel[4];   // per state of a run: multiplier (a left shift) and byte selector
    __device__ __forceinline__ ChannelLane(uint32_t l16, const GemmTcParams& p) {
        const uint32_t g = l16 & 7u, hi = l16 >> 3;
        off[0] = 4u * ((3u * g + 23u) % 24u);
        off[1] = 12u * g;
        off[2] = 12u * g + 4u;
        off[3] = 12u * g + 8u;
        sel[0] = 0x7654u - 0x1111u * (2u + hi);
        sel[1] = 0x7654u - 0x1111u * (1u + hi);
        sel[2] = 0x7654u - 0x1111u * hi;
        sel[3] = 0x7654u - 0x1111u * (3u + hi);
        // state shifts: high channel 9, 6, 3, 0; low channel 13, 10, 7, 4.  Each is done as a
        // multiply that moves the window to a byte boundary and a byte selection.  The
        // multipliers come from kernel parameters so that they stay multiplies.
        const uint32_t one = p.mul2 >> 1, eight = p.mul4 * p.mul2;
        mul[0] = hi ? p.mul128 : eight;    bsel[0] = 0x4432u;
        mul[1] = hi ? p.mul4 : p.mul64;    bsel[1] = hi ? 0x4421u : 0x4432u;
        mul[2] = hi ? p.mul32 : p.mul2;    bsel[2] = 0x4421u;
        mul[3] = hi ? one : p.mul16;       bsel[3] = hi ? 0x4410u : 0x4421u;
    }
    __device__ __forceinline__ void states(const uint32_t (&w)[4], const ShiftMuls&,
                                           uint32_t (&s)[16]) const {
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const int pw = t < 3 ? t : 2;
            const uint32_t win = prmt(w[pw + 1], w[pw], sel[t]);
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) s[4 * t + jj] = prmt(win * mul[jj], 0u, bsel[jj]);
        }
    }
};

template <int K, int MT>
__global__ void __launch_bounds__(kThreadsTcm, 1)
gemm_tcm_kernel(const __grid_constant__ GemmTcParams p, const __grid_constant__ CUtensorMap xmap0,
                const __grid_constant__ CUtensorMap xmap1, const __grid_constant__ CUtensorMap xmap2) {
    constexpr int WPT = 8 * K;
    constexpr uint32_t kXHalfBytes = MT * kXBytesPerMt;    // one 64-channel box of activations
    constexpr uint32_t kXBytes = 2u * kXHalfBytes;         // a stage: 128 channels
    constexpr uint32_t kRowBytes = 8u * WPT * 4u;          // one tile row of the CTA's 8 tile columns
    constexpr uint32_t kCodeStageBytes = 8u * kRowBytes;   // eight tile rows = 128 input channels
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // s_free[c % kFreeBars] completes when the tensor core is done with stage c: ONE commit per
    // stage releases both the stage's weight columns and its activation slot (a tcgen05.commit
    // holds the issuing thread until the instructions before it have run, so every commit saved
    // is time on the critical path).  The ring depths differ, hence a barrier per stage modulo
    // their common multiple.
    __shared__ __align__(8) uint64_t s_wfull[kWStages], s_xfull[kXStages], s_free[kFreeBars];
    __shared__ __align__(8) uint64_t s_cfull[kCodeStages], s_cempty[kCodeStages], s_done;
    __shared__ uint32_t s_tmem;

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t split = blockIdx.y, r0 = blockIdx.z * (128u * MT);
    // which projection of the launch this column block belongs to
    uint32_t ocb = blockIdx.x;
    const uint32_t* code_p = p.code;
    float* out_p = p.out;
    const float* rout_p = p.rout;
    __half* y16_p = p.y16;
    uint32_t OCp = static_cast<uint32_t>(p.OC);
    const CUtensorMap* xm = &xmap0;
    if (p.nproj > 1 && ocb >= static_cast<uint32_t>(p.more[0].cb0)) {
        const int j = (p.nproj > 2 && ocb >= static_cast<uint32_t>(p.more[1].cb0)) ? 1 : 0;
        ocb -= static_cast<uint32_t>(p.more[j].cb0);
        code_p = p.more[j].code;
        out_p = p.more[j].out;
        rout_p = p.more[j].rout;
        y16_p = p.more[j].y16;
        OCp = static_cast<uint32_t>(p.more[j].OC);
        xm = j ? &xmap2 : &xmap1;
    }
    const uint32_t xring = (smem_u32(smem_raw) + 1023u) & ~1023u;   // [kXStages][2][rows][128 B]
    const uint32_t code0 = xring + kXStages * kXBytes;              // [kCodeStages][8][kRowBytes]
    const uint32_t wfull0 = smem_u32(s_wfull), xfull0 = smem_u32(s_xfull), free0 = smem_u32(s_free);
    const uint32_t cfull0 = smem_u32(s_cfull), cempty0 = smem_u32(s_cempty), done = smem_u32(&s_done);

    const uint32_t nstage_all = static_cast<uint32_t>(p.IC) / kStageK;
    const uint32_t S = p.splits, sbase = nstage_all / S, srem = nstage_all % S;
    const uint32_t s_first = split * sbase + min(split, srem);
    const uint32_t nstage = sbase + (split < srem ? 1u : 0u);

    grid_launch_dependents();
    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < kWStages; ++s) mbar_init(wfull0 + 8u * s, kDecodeWarps);
#pragma unroll
        for (int s = 0; s < kXStages; ++s) mbar_init(xfull0 + 8u * s, 1u);
#pragma unroll
        for (int s = 0; s < kFreeBars; ++s) mbar_init(free0 + 8u * s, 1u);
#pragma unroll
        for (int s = 0; s < kCodeStages; ++s) {
            mbar_init(cfull0 + 8u * s, 1u);
            mbar_init(cempty0 + 8u * s, kDecodeWarps);
        }
        mbar_init(done, 1u);
        mbar_fence_init();
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(&s_tmem), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = s_tmem;
    // the set-up above overlapped the previous kernel's tail; its results are needed from here
    grid_dependency_wait();

    bool ok = true;
    if (warp >= kServiceWarps) {
        // ---- decode warps
        const uint32_t qd = warp & 3u, kq = (warp - kServiceWarps) >> 2;
        const ChannelLane<K> cl(lane & 15u, p);
        const uint32_t hmask = p.hash_mask, hxor = p.hash_xor;
        const ShiftMuls muls{p.mul2, p.mul4, p.mul16, p.mul32, p.mul64, p.mul128};
        // the lane's tile: tile rows 2kq, 2kq+1 of the stage, tile column 2qd + (lane >> 4)
        const uint32_t my_code = code0 + 2u * kq * kRowBytes + (2u * qd + (lane >> 4)) * (WPT * 4u);
        const uint32_t my_cols = tmem + ((32u * qd) << 16) + kWCol0 + 16u * kq;
        for (uint32_t c = 0; c < nstage; ++c) {
            const uint32_t cslot = c % kCodeStages;
            if (!mbar_wait_relaxed(cfull0 + 8u * cslot, (c / kCodeStages) & 1u, p.wait_limit)) {
                ok = false;
                break;
            }
            uint32_t wd[2][ChannelLane<K>::kWords];
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const uint32_t tp = my_code + cslot * kCodeStageBytes + q * kRowBytes;
#pragma unroll
                for (int i = 0; i < ChannelLane<K>::kWords; ++i)
                    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(wd[q][i]) : "r"(tp + cl.off[i]));
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(cempty0 + 8u * cslot);
            uint32_t v[16];
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                uint32_t s[16];
                cl.states(wd[q], muls, s);
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    // inputs (2t, 2t+1) -> column t, (2t+8, 2t+9) -> column t+4 of this step
                    const uint32_t a0 = cba_decode_dup(s[4 * t + 0], hmask, hxor);
                    const uint32_t a1 = cba_decode_dup(s[4 * t + 1], hmask, hxor);
                    const uint32_t a2 = cba_decode_dup(s[4 * t + 2], hmask, hxor);
                    const uint32_t a3 = cba_decode_dup(s[4 * t + 3], hmask, hxor);
                    v[8 * q + t] = prmt(a0, a1, 0x5410u);
                    v[8 * q + t + 4] = prmt(a2, a3, 0x5410u);
                }
            }
            const uint32_t wslot = c % kWStages;
            if (c >= kWStages && !mbar_wait_relaxed(free0 + 8u * ((c - kWStages) % kFreeBars),
                                                    ((c - kWStages) / kFreeBars) & 1u, p.wait_limit)) {
                ok = false;
                break;
            }
            tc_fence_after_sync();
            tmem_st16(my_cols + wslot * kWStageCols, v);
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(wfull0 + 8u * wslot);
        }
    } else if (warp == 0) {
        // ---- the issuing warp.  It is the CTA's first warp and runs its loop warp-uniformly
        // (addresses and descriptors stay in uniform registers); one elected lane issues.
        const uint32_t idesc = idesc_for(128u * MT);
        for (uint32_t c = 0; c < nstage; ++c) {
            const uint32_t ws = c % kWStages, xs = c % kXStages;
            if (!mbar_wait_relaxed(wfull0 + 8u * ws, (c / kWStages) & 1u, p.wait_limit) ||
                !mbar_wait_relaxed(xfull0 + 8u * xs, (c / kXStages) & 1u, p.wait_limit)) {
                ok = false;
                break;
            }
            tc_fence_after_sync();
            const uint32_t wcols = tmem + kWCol0 + ws * kWStageCols;
            const uint32_t xslot = xring + xs * kXBytes;
            if (elect_one()) {
                // D[channel][row] += W[channel][k] * X[row][k], 16 input channels per instruction
#pragma unroll
                for (uint32_t k16 = 0; k16 < 8u; ++k16) {
                    umma_f16_ts(tmem, wcols + 8u * k16,
                                smem_desc_sw128(xslot + (k16 >> 2) * kXHalfBytes + 32u * (k16 & 3u)),
                                idesc, (c | k16) != 0u);
                }
                // the stage's weight columns and activation slot are free once these have run
                umma_commit(free0 + 8u * (c % kFreeBars));
                if (c + 1u == nstage) umma_commit(done);
            }
            __syncwarp();
        }
    } else if (warp == 1) {
        // ---- activation loader: two tiled TMA loads (64 channels each) per stage
        if (lane == 0) {
            for (uint32_t c = 0; c < nstage; ++c) {
                const uint32_t slot = c % kXStages;
                if (c >= kXStages && !mbar_wait_relaxed(free0 + 8u * ((c - kXStages) % kFreeBars),
                                                        ((c - kXStages) / kFreeBars) & 1u, p.wait_limit)) {
                    ok = false;
                    break;
                }
                mbar_arrive_expect_tx(xfull0 + 8u * slot, kXBytes);
                const int32_t x0 = static_cast<int32_t>((s_first + c) * kStageK);
                tma_load_2d(xring + slot * kXBytes, xm, x0, static_cast<int32_t>(r0),
                            xfull0 + 8u * slot);
                tma_load_2d(xring + slot * kXBytes + kXHalfBytes, xm, x0 + kXChunkK,
                            static_cast<int32_t>(r0), xfull0 + 8u * slot);
            }
        }
    } else if (warp == 2) {
        // ---- code warp: bulk copies (untiled, no multicast), one per tile row, eight per stage
        const uint32_t TN = OCp >> 4;
        const size_t kt_words = static_cast<size_t>(TN) * WPT;   // words from tile row kt to kt+1
        const uint32_t* grow = code_p + (static_cast<size_t>(s_first) * 8u + lane) * kt_words +
                               static_cast<size_t>(ocb) * 8u * WPT;
        for (uint32_t c = 0; c < nstage; ++c) {
            const uint32_t cslot = c % kCodeStages;
            if (c >= kCodeStages &&
                !mbar_wait_relaxed(cempty0 + 8u * cslot, ((c / kCodeStages) - 1u) & 1u, p.wait_limit)) {
                ok = false;
                break;
            }
            if (lane == 0) mbar_arrive_expect_tx(cfull0 + 8u * cslot, kCodeStageBytes);
            __syncwarp();
            if (lane < 8 && !p.test_stall)   // the test hook announces the bytes and never sends them
                bulk_copy_g2s(code0 + cslot * kCodeStageBytes + lane * kRowBytes, grow, kRowBytes,
                              cfull0 + 8u * cslot);
            grow += 8u * kt_words;
        }
    }
    if (!ok && lane == 0) atomicExch(&g_gemm_tcm_status, 1);

    // ---- epilogue: accumulator lanes are output channels of the block, columns activation rows
    const bool fused_out = rout_p != nullptr;   // splits == 1, or a cluster launch of S <= 8 CTAs
    float* const stage = reinterpret_cast<float*>(smem_raw + (xring - smem_u32(smem_raw)));
    if (warp >= kServiceWarps) {
        // warp w reads lanes 32(w&3).. (the only ones it may address) and a quarter of the columns
        const uint32_t qd = warp & 3u, cq = (warp - kServiceWarps) >> 2;
        bool ready = __shfl_sync(0xFFFFFFFFu, ok ? 1 : 0, 0) != 0 && nstage > 0;
        if (ready && !mbar_wait_relaxed(done, 0u, p.wait_limit)) {
            ready = false;
            if (lane == 0) atomicExch(&g_gemm_tcm_status, 2);
        }
        tc_fence_after_sync();
        if (ready) {
            float* plane = out_p + static_cast<size_t>(split) * p.M * OCp + ocb * 128u + 32u * qd + lane;
#pragma unroll 1
            for (uint32_t col = cq * (32u * MT); col < (cq + 1u) * (32u * MT); col += 16u) {
                if (r0 + col >= static_cast<uint32_t>(p.M)) break;   // uniform: no rows left
                uint32_t v[16];
                tmem_ld16(tmem + ((32u * qd) << 16) + col, v);
                tmem_ld_wait();
                if (fused_out) {
                    // transpose through shared memory (the rings are idle now): [row][channel]
#pragma unroll
                    for (uint32_t i = 0; i < 16u; ++i)
                        stage[(col + i) * 128u + 32u * qd + lane] = __uint_as_float(v[i]);
                } else {
#pragma unroll
                    for (uint32_t i = 0; i < 16u; ++i) {
                        const uint32_t row = r0 + col + i;
                        if (row < static_cast<uint32_t>(p.M))
                            plane[static_cast<size_t>(row) * OCp] = __uint_as_float(v[i]);
                    }
                }
            }
        }
    }
    if (fused_out) {
        // every warp of the CTA: one row per step, four consecutive channels per lane ->
        // 128-point butterflies across the warp, scales, binary16 store.
        // A launch split along K runs as clusters of S CTAs (one per split, same output block):
        // every CTA leaves its partial tile in its own shared memory, and after a cluster barrier
        // CTA s sums rows s, s+S, ... over all S tiles in split order through distributed shared
        // memory -- the split-order plane sum without planes, a second launch or memory traffic.
        __syncthreads();
        const bool cluster_sum = S > 1u;
        if (cluster_sum) cluster_sync_all();
        const uint32_t nwarps = kThreadsTcm / 32u;
        const uint32_t rows_here = min(128u * MT, static_cast<uint32_t>(p.M) - r0);
        const float4 sc = *reinterpret_cast<const float4*>(rout_p + ocb * 128u + lane * 4u);
        const uint32_t r_first = cluster_sum ? split + S * warp : warp;
        const uint32_t r_step = cluster_sum ? S * nwarps : nwarps;
        for (uint32_t r = r_first; r < rows_here; r += r_step) {
            float v[4];
            if (cluster_sum) {
                const uint32_t at = xring + (r * 128u + lane * 4u) * 4u;
                const float4 a = ld_cluster_f4(at, 0u);
                v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
                for (uint32_t i = 1; i < S; ++i) {
                    const float4 b = ld_cluster_f4(at, i);
                    v[0] = __fadd_rn(v[0], b.x); v[1] = __fadd_rn(v[1], b.y);
                    v[2] = __fadd_rn(v[2], b.z); v[3] = __fadd_rn(v[3], b.w);
                }
            } else {
                const float4 a = *reinterpret_cast<const float4*>(stage + r * 128u + lane * 4u);
                v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
            }
            wht128_warp(v, lane);
            uint2 packed;
            packed.x = as_u32(__floats2half2_rn(__fmul_rn(__fmul_rn(v[0], p.rs), sc.x),
                                                __fmul_rn(__fmul_rn(v[1], p.rs), sc.y)));
            packed.y = as_u32(__floats2half2_rn(__fmul_rn(__fmul_rn(v[2], p.rs), sc.z),
                                                __fmul_rn(__fmul_rn(v[3], p.rs), sc.w)));
            *reinterpret_cast<uint2*>(y16_p + static_cast<size_t>(r0 + r) * OCp + ocb * 128u + lane * 4u) = packed;
        }
        // no CTA may leave while another still reads its tile
        if (cluster_sum) cluster_sync_all();
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

template <int K, int MT>
cudaError_t launch_tcm(const GemmTcParams& p, const __half* const* xh_more, cudaStream_t st) {
    const size_t smem = static_cast<size_t>(kXStages) * 2u * MT * kXBytesPerMt +
                        static_cast<size_t>(kCodeStages) * 8u * (8u * 8u * K * 4u) + 1024;
    static SmemLimit limit;
    cudaError_t e = limit.ensure(gemm_tcm_kernel<K, MT>, smem);
    if (e != cudaSuccess) return e;
    CUtensorMap xmap[3];
    e = encode_x_map(&xmap[0], p.xh, p.M, p.IC, 128 * MT);
    if (e != cudaSuccess) return e;
    xmap[1] = xmap[0];
    xmap[2] = xmap[0];
    int blocks = p.OC / 128;
    for (int j = 0; j + 1 < p.nproj; ++j) {
        e = encode_x_map(&xmap[1 + j], xh_more[j], p.M, p.IC, 128 * MT);
        if (e != cudaSuccess) return e;
        blocks += p.more[j].OC / 128;
    }
    const dim3 grid(blocks, p.splits, (p.M + 128 * MT - 1) / (128 * MT));
    if (p.rout != nullptr && p.splits > 1)   // the splits of an output block form a cluster
        return launch_chained_cluster(gemm_tcm_kernel<K, MT>, grid, dim3(kThreadsTcm), smem, st,
                                      static_cast<unsigned>(p.splits), p, xmap[0], xmap[1], xmap[2]);
    return launch_chained(gemm_tcm_kernel<K, MT>, grid, dim3(kThreadsTcm), smem, st, p, xmap[0], xmap[1],
                          xmap[2]);
}

}  // namespace

// whether a launch with a transform vector and `splits` > 1 sums its splits inside the kernel.
// Clusters of up to 4 CTAs: each CTA holds a whole SM, and with clusters of 7 (a 2-GPU shard of
// the 27B-class o/down projections) a layer step measured 267 us against 245 us with planes.
bool gemm_tcm_cluster_sum(int IC, int splits) {
    return splits > 1 && splits <= 4 && IC % kStageK == 0 && splits <= IC / kStageK;
}

bool gemm_tcm_supports(const GemmTcParams& p) {
    return p.IC % kStageK == 0 && p.splits >= 1 && p.splits <= p.IC / kStageK;
}

namespace {
int g_tcm_stall = 0;                    // host side; tests only
unsigned g_tcm_wait_limit = 1u << 21;   // about two seconds per wait
}  // namespace

void gemm_tcm_test_stall(int on, unsigned limit) {
    g_tcm_stall = on ? 1 : 0;
    g_tcm_wait_limit = (on && limit) ? limit : (1u << 21);
}

cudaError_t launch_gemm_tcm_many(const GemmTcParams& p_in, const __half* const* xh_more, cudaStream_t st) {
    GemmTcParams p = p_in;
    p.wait_limit = g_tcm_wait_limit;
    p.test_stall = g_tcm_stall;
    const bool two = p.M > 128;
    if (p.K == 2) return two ? launch_tcm<2, 2>(p, xh_more, st) : launch_tcm<2, 1>(p, xh_more, st);
    return two ? launch_tcm<3, 2>(p, xh_more, st) : launch_tcm<3, 1>(p, xh_more, st);
}

cudaError_t launch_gemm_tcm(const GemmTcParams& p, cudaStream_t st) {
    GemmTcParams one = p;
    one.nproj = 1;
    return launch_gemm_tcm_many(one, nullptr, st);
}


cudaError_t gemm_tcm_status(int* host_status) {
    return cudaMemcpyFromSymbol(host_status, g_gemm_tcm_status, sizeof(int));
}

}  // namespace escha
