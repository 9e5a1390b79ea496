// Tensor-core coded GEMV / small-batch GEMM with split-K, optional fused input
// transform (incl. SwiGLU) and fused output transform, for one or several
// projections of the same input per launch.  This is the fast path behind
// moe_gemv / dense_gemv / dense_gemm_rows[_direct[_out]] / dense_gemm_pair[_out] /
// moe_gemm_rows of the reference's kernel layer (escha_mlx/msl.py:1366-1478,
// :1785-1950): the same product
//
//     mid[r, :] = f32(xh[r, :]) @ f32(decode(code[expert(r)]))
//
// optionally preceded in the same kernel by  xh = f16(H128(x * rin) * RS)  and
// followed by  y = f16((H128(mid) * RS) * rout).
//
// Why it looks the way it does on B200:
//  * The reference's lane -> tile-position map (ref.lane_positions) is exactly
//    the A-fragment ownership of mma.m16n8k16 for the transposed tile, so the
//    eight halves a lane decodes go from registers straight into the tensor
//    core; the activations are the B operand (up to 8 rows per mma column
//    block), accumulation is fp32.  No cvt, no FMA chain, no shuffle reduction,
//    and up to 16 rows share one decode for free.
//  * The kernel is bound by instruction issue, not by HBM: integer-pipe ops
//    (byte permute, logic) and multiply-pipe ops (IMAD, HADD2) both issue at half
//    rate on this part, and a decoded weight needs two of each.  So each weight
//    is kept as (w, w) in one register -- one HADD2 with half-select operands --
//    and multiplied against (x, 0): that spends an idle half of the tensor core
//    instead of two more byte permutes per weight pair.
//  * The code stream is read exactly once: a producer warp issues bulk copies
//    (cp.async.bulk, the untiled TMA form, no multicast) of whole eight-tile rows
//    into a shared-memory ring guarded by full/empty mbarriers, so the eight
//    decode warps spend no instruction on address generation; their main loop
//    has no block-wide barrier except when the activation chunk is re-staged (every 256 to 2048 input
//    channels, depending on how many rows share the decode).
//  * 128 output channels per CTA = one Hadamard block, so the CTA that
//    completes a block runs the output transform with warp butterflies.
//  * Split-K over 128-channel input blocks fills the 148 SMs for any shape.
//    Partials go to caller-provided scratch; the CTA that arrives last for an
//    output block sums them in ascending split order (no float atomics), so the
//    result is bit-reproducible run to run for a given (shape, splits).
#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "kernels.h"

namespace escha {

namespace {

constexpr int NS = 6;              // bulk-copy ring depth (128-channel blocks) per CTA
constexpr int kXBudgetBytes = 32 * 1024;  // shared memory spent on staged activations

// 128-channel blocks of activations staged per chunk: as many as the budget
// allows for the job's rows (plus the zero row), between 2 and 16.  A staged row
// is blocks*128 + 16 words; the +16 keeps the LDS.128 fragment loads conflict-free.
inline int x_chunk_blocks(int xrows) {
    int b = kXBudgetBytes / ((xrows + 1) * 520);
    return b > 16 ? 16 : (b < 2 ? 2 : b);
}

template <bool FUSED_OUT>
__device__ __forceinline__ void finalize_row(float v[4], uint32_t lane, const float* rout_blk,
                                             const GemvProblem& pr, size_t off, float rs) {
    void* const out = pr.out;
    if (FUSED_OUT) {
        const float4 sc = *reinterpret_cast<const float4*>(rout_blk + lane * 4u);
        wht128_warp(v, lane);
        uint2 packed;
        packed.x = as_u32(__floats2half2_rn(__fmul_rn(__fmul_rn(v[0], rs), sc.x),
                                            __fmul_rn(__fmul_rn(v[1], rs), sc.y)));
        packed.y = as_u32(__floats2half2_rn(__fmul_rn(__fmul_rn(v[2], rs), sc.z),
                                            __fmul_rn(__fmul_rn(v[3], rs), sc.w)));
        *reinterpret_cast<uint2*>(static_cast<__half*>(out) + off) = packed;
        // the same block into the gathered row of every other GPU (plain stores over NVLink)
        for (int g = 0; g < pr.npeer; ++g)
            *reinterpret_cast<uint2*>(static_cast<__half*>(pr.peer[g]) + off) = packed;
    } else {
        const float4 q = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(static_cast<float*>(out) + off) = q;
        for (int g = 0; g < pr.npeer; ++g)
            *reinterpret_cast<float4*>(static_cast<float*>(pr.peer[g]) + off) = q;
    }
}

__device__ __forceinline__ __half swiglu_half(__half g16, __half u16) {
    const float g = __half2float(g16);
    const __half s = __float2half_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))));
    return __hmul(s, u16);
}

// Stage `cnt` 128-channel blocks (starting at block blk0) of the job's rows into
// shared memory as (x, 0) words, applying the input transform when fused.  Within
// each 16-channel group the words are ordered c0 c8 c1 c9 ... c7 c15, so that one
// 16-byte load at word 4t hands lane t the B fragments of both mma of a tile:
// (x[2t], x[2t+8]) and (x[2t+1], x[2t+9]).
__device__ __forceinline__ void stage_activations(const GemvMmaParams& p, const __half* xsrc, const float* rin,
                                                  const int* s_rows, int nrows, uint32_t blk0,
                                                  uint32_t cnt, uint32_t* s_x, uint32_t XS,
                                                  uint32_t tid) {
    const uint32_t lane = tid & 31u, warp = tid >> 5;
    if (p.input == kInputTransformed) {
        const uint32_t grp_per_row = cnt * 8u;  // 16-channel groups per row
        const uint32_t total = static_cast<uint32_t>(nrows) * grp_per_row;
        for (uint32_t idx = tid; idx < total; idx += 256u) {
            const uint32_t r = idx / grp_per_row, v = idx - r * grp_per_row;
            const uint4* src = reinterpret_cast<const uint4*>(
                xsrc + static_cast<size_t>(s_rows[r] / p.x_row_div) * p.x_stride + blk0 * 128u +
                v * 16u);
            const uint4 lo = src[0], hi = src[1];  // channels 0..7 and 8..15 of the group
            uint4* dst = reinterpret_cast<uint4*>(s_x + r * XS + v * 16u);
            // staged order c0 c8 c1 c9 ... c7 c15, each as a (x, 0) word
            dst[0] = make_uint4(lo.x & 0xFFFFu, hi.x & 0xFFFFu, lo.x >> 16, hi.x >> 16);
            dst[1] = make_uint4(lo.y & 0xFFFFu, hi.y & 0xFFFFu, lo.y >> 16, hi.y >> 16);
            dst[2] = make_uint4(lo.z & 0xFFFFu, hi.z & 0xFFFFu, lo.z >> 16, hi.z >> 16);
            dst[3] = make_uint4(lo.w & 0xFFFFu, hi.w & 0xFFFFu, lo.w >> 16, hi.w >> 16);
        }
        return;
    }
    // fused input transform: one warp per (row, block), butterflies in registers
    const uint32_t units = static_cast<uint32_t>(nrows) * cnt;
    for (uint32_t u = warp; u < units; u += 8u) {
        const uint32_t r = u / cnt, b = u - r * cnt;
        const size_t xoff = static_cast<size_t>(s_rows[r] / p.x_row_div) * p.x_stride +
                            (blk0 + b) * 128u + lane * 4u;
        uint2 raw = *reinterpret_cast<const uint2*>(xsrc + xoff);
        if (p.input == kInputSwiglu) {
            const uint2 up = *reinterpret_cast<const uint2*>(p.x_up + xoff);
            const __half2 g0 = as_half2(raw.x), g1 = as_half2(raw.y);
            const __half2 u0 = as_half2(up.x), u1 = as_half2(up.y);
            raw.x = as_u32(__halves2half2(swiglu_half(__low2half(g0), __low2half(u0)),
                                          swiglu_half(__high2half(g0), __high2half(u0))));
            raw.y = as_u32(__halves2half2(swiglu_half(__low2half(g1), __low2half(u1)),
                                          swiglu_half(__high2half(g1), __high2half(u1))));
        }
        const float4 sc = *reinterpret_cast<const float4*>(rin + (blk0 + b) * 128u + lane * 4u);
        const float2 a = __half22float2(as_half2(raw.x)), c = __half22float2(as_half2(raw.y));
        float v[4] = {__fmul_rn(a.x, sc.x), __fmul_rn(a.y, sc.y), __fmul_rn(c.x, sc.z),
                      __fmul_rn(c.y, sc.w)};
        wht128_warp(v, lane);
        // lane holds channels 4*lane..4*lane+3 of the block: group lane/4, channel
        // c = 4*(lane%4)+i within it, staged at word 2*(c%8) + c/8
        uint32_t* dst = s_x + r * XS + b * 128u + (lane >> 2) * 16u + ((lane & 1u) * 8u) +
                        ((lane >> 1) & 1u);
        dst[0] = __half_as_ushort(__float2half_rn(__fmul_rn(v[0], p.rs)));
        dst[2] = __half_as_ushort(__float2half_rn(__fmul_rn(v[1], p.rs)));
        dst[4] = __half_as_ushort(__float2half_rn(__fmul_rn(v[2], p.rs)));
        dst[6] = __half_as_ushort(__float2half_rn(__fmul_rn(v[3], p.rs)));
    }
}

// Error word set by a kernel whose bounded wait gave up (never expected).
__device__ int g_gemv_status = 0;

constexpr int kConsumerThreads = 256;   // 8 decode warps
constexpr int kThreads = kConsumerThreads + 32;  // + 1 producer warp
constexpr uint32_t kBarSlot0 = 2;       // named barriers 2..7: the ring's slots (1: the decode warps' own)

// Each weight is rounded to binary16 exactly as the format defines it, w = f16(lo) + f16(hi),
// and kept as (w, w) against activations staged as (x, 0).  GRP = true is the form for expert
// row jobs, where a CTA may take several consecutive output blocks (p.ocb_group); the dense
// form is compiled without that loop (measured: 1.8% on the batch-1 layer).
template <int K, int MT, bool GRP>
__global__ void __launch_bounds__(kThreads, 3)
gemv_mma_kernel(const __grid_constant__ GemvMmaParams p) {
    constexpr int WPT = 8 * K;
    constexpr int ROW_WORDS = 8 * WPT;          // one kt row of the CTA's eight tiles
    constexpr int STAGE_WORDS = 8 * ROW_WORDS;  // eight kt rows = one 128-channel block
    constexpr int ROWS = 8 * MT;
    extern __shared__ __align__(128) uint32_t smem[];
    uint32_t* const s_code = smem;                    // [NS][8 kt][8 tiles][WPT]
    uint32_t* const s_x = smem + NS * STAGE_WORDS;    // [rows + 1][XS] as (x, 0) words; then,
                                                      // with G > 1, [ROWS][128] accumulators
    __shared__ __align__(8) uint64_t s_full[NS];
    __shared__ int s_rows[16];
    __shared__ int s_last;

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3u;
    // a CTA covers G consecutive output blocks of one projection (G > 1 only for unsplit
    // launches whose input range fits one staged chunk: the rows are staged once for all G)
    const uint32_t G = GRP ? static_cast<uint32_t>(p.ocb_group) : 1u;
    const uint32_t gocb = blockIdx.x * G, split = blockIdx.y, job = blockIdx.z;
    const uint32_t nblk = p.IC >> 7;

    // which projection of the launch this output block belongs to (uniform per CTA)
    int pi = 0;
#pragma unroll
    for (int q = 1; q < kMaxProblems; ++q)
        if (q < p.nprob && gocb >= static_cast<uint32_t>(p.prob[q].ocb0)) pi = q;
    const GemvProblem& pr = p.prob[pi];
    const uint32_t ocb = gocb - pr.ocb0;
    const uint32_t OC = pr.OC, TN = OC >> 4;

    // Programmatic dependent launch: let the next kernel of the stream be scheduled
    // as soon as every CTA of this one has started, so that its start-up overlaps
    // this kernel's tail.  Everything a launch reads that an earlier kernel may have
    // written sits behind grid_dependency_wait(): the row jobs right here, the
    // activations below.  With kPdlPrefetch the producer warp of a dense launch does
    // not wait: it streams weights (which nothing in flight writes) while the
    // previous kernel drains.
    if (p.pdl != kPdlOff) grid_launch_dependents();
    if (p.pdl == kPdlWaitFirst || (p.pdl == kPdlPrefetch && p.jobs)) grid_dependency_wait();

    int expert = 0, nrows, xrows;
    if (p.jobs) {
        const RowJob* jb = p.jobs + job;
        expert = jb->expert;
        nrows = jb->nrows;
        xrows = ROWS;
        if (tid < 16) s_rows[tid] = jb->rows[tid];
    } else {
        const int r0 = static_cast<int>(job) * ROWS;
        nrows = min(ROWS, p.M - r0);
        xrows = min(ROWS, p.M);
        if (tid < 16) s_rows[tid] = r0 + static_cast<int>(tid);
    }
    // this CTA's range of 128-channel input blocks; projections of one launch may
    // use different split factors (each keeps the factor it has when launched alone)
    const uint32_t S = pr.splits, SMAX = p.splits;
    if (nrows <= 0 || split >= S) return;  // uniform for the CTA

    const uint32_t bbase = nblk / S, brem = nblk % S;
    const uint32_t b0 = split * bbase + min(split, brem);
    const uint32_t nb = bbase + (split < brem ? 1u : 0u);

    const uint32_t tile_row_words = TN * WPT;  // words between kt and kt+1 in the stream
    const uint32_t full0 = smem_u32(s_full);
    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < NS; ++s) {
            mbar_init(full0 + 8u * s, 1u);    // the producer's arrive.expect_tx
        }
        mbar_fence_init();
    }
    __syncthreads();

    if (warp == 8) {
        // ---- producer warp: bulk copies (TMA, untiled, no multicast) of the CTA's
        // eight-tile rows, one copy per kt row, eight rows per stage
        const uint32_t* const gbase = pr.code + static_cast<size_t>(expert) * (p.IC >> 4) * tile_row_words +
                                      ocb * ROW_WORDS +
                                      (static_cast<size_t>(b0) * 8u + lane) * tile_row_words;
        const uint32_t dst0 = smem_u32(s_code) + lane * (ROW_WORDS * 4u);
        uint32_t st = 0;   // stages issued so far
        for (uint32_t o = 0; o < G; ++o) {
            const uint32_t* grow = gbase + o * ROW_WORDS;
            for (uint32_t i = 0; i < nb; ++i, ++st) {
                const uint32_t slot = st % NS;
                // The slot is free once all eight decode warps have arrived at its barrier.  The
                // producer is parked there by the hardware: a polling wait would take issue
                // slots on its sub-partition, and the slowest sub-partition paces the CTA.
                if (st >= NS) named_barrier_sync(kBarSlot0 + slot, kThreads);
                if (lane == 0) mbar_arrive_expect_tx(full0 + 8u * slot, STAGE_WORDS * 4u);
                __syncwarp();
                if (lane < 8 && !p.test_stall)
                    bulk_copy_g2s(dst0 + slot * (STAGE_WORDS * 4u), grow, ROW_WORDS * 4u,
                                  full0 + 8u * slot);
                grow += static_cast<size_t>(8u) * tile_row_words;
            }
        }
        return;
    }

    // ---- decode warps
    const LaneConsts<K> lc(lane);
    const uint32_t XCB = p.xcb, XS = XCB * 128u + 16u;  // blocks per chunk, words per staged row
    // zero row: B columns past the job's last row read it instead of branching
    uint32_t* const zero_row = s_x + static_cast<uint32_t>(xrows) * XS;
    for (uint32_t i = tid; i < XS; i += kConsumerThreads) zero_row[i] = 0u;

    const uint32_t* xrow[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        const int slot = static_cast<int>(g) + 8 * mt;
        xrow[mt] = (slot < nrows ? s_x + slot * XS : zero_row) + 4u * t;
    }
    const float* rin = pr.rin ? pr.rin + static_cast<size_t>(expert) * p.IC : nullptr;
    const __half* xsrc = pr.x ? pr.x : p.x;
    const uint32_t hmask = p.hash_mask, hxor = p.hash_xor;
    const ShiftMuls muls{p.mul2, p.mul4, p.mul16, p.mul32, p.mul64, p.mul128};
    const uint32_t* const wa0 = s_code + warp * WPT + lc.ia();
    const uint32_t* const wb0 = s_code + warp * WPT + lc.ib();

    if (p.pdl == kPdlPrefetch && !p.jobs) grid_dependency_wait();

    bool ok = true;
    uint32_t slot = 0, phase = 0;
    // with G > 1 the accumulators cannot borrow the code ring (it is never drained between
    // output blocks): they get their own rows behind the activations
    float* const s_acc = G > 1 ? reinterpret_cast<float*>(s_x + (static_cast<uint32_t>(xrows) + 1u) * XS)
                               : reinterpret_cast<float*>(s_code);
    const size_t out_ld = pr.out_ld ? static_cast<size_t>(pr.out_ld) : OC;
  for (uint32_t o = 0; o < G; ++o) {
    // two independent accumulator sets per column block: the two mma of a tile
    // do not wait on each other, and each chain advances once per tile
    float dA[MT][4], dB[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) dA[mt][i] = dB[mt][i] = 0.0f;
    for (uint32_t c0 = 0; c0 < nb; c0 += XCB) {
        const uint32_t cnt = min(XCB, nb - c0);
        if (o == 0) {   // G > 1 means one chunk: staged once, reused by every output block
            named_barrier_sync(1, kConsumerThreads);
            stage_activations(p, xsrc, rin, s_rows, nrows, b0 + c0, cnt, s_x, XS, tid);
            named_barrier_sync(1, kConsumerThreads);
        }
        for (uint32_t cb = 0; cb < cnt; ++cb) {
            // a wait that gives up is recorded; the warp stops waiting but keeps walking the
            // stages and arriving everywhere, so that nobody in the CTA is left alone at a barrier
            if (ok && !mbar_wait_n(full0 + 8u * slot, phase, p.wait_limit)) ok = false;
            const uint32_t* wa = wa0 + slot * STAGE_WORDS;
            const uint32_t* wb = wb0 + slot * STAGE_WORDS;
            const uint32_t* xr[MT];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) xr[mt] = xrow[mt] + cb * 128u;
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                uint32_t s[8], a[8];
                lc.states(wa[kk * ROW_WORDS], wb[kk * ROW_WORDS], muls, s);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    a[j] = cba_decode_dup(s[j], hmask, hxor);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    // (x[2t], x[2t+8], x[2t+1], x[2t+9]) as (x, 0) words
                    const uint4 b = *reinterpret_cast<const uint4*>(xr[mt] + kk * 16);
                    // value j sits at (channel g + 8*(j>=4), input 2t + (j&1) + 8*((j>>1)&1))
                    mma16816(dA[mt], a[0], a[4], a[2], a[6], b.x, b.y);
                    mma16816(dB[mt], a[1], a[5], a[3], a[7], b.z, b.w);
                }
            }
            named_barrier_arrive(kBarSlot0 + slot, kThreads);  // this warp is done with the slot
            if (++slot == NS) { slot = 0; phase ^= 1u; }
        }
    }
    // what this CTA computed after a give-up is void; the status word says so
    if (!ok && lane == 0) atomicExch(&g_gemv_status, 2);
    named_barrier_sync(1, kConsumerThreads);

    // accumulators -> shared [ROWS][128] (with G == 1 in the drained code ring)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        const uint32_t ch = warp * 16u + g, n0 = 2u * t + 8u * mt;
        s_acc[n0 * 128u + ch] = __fadd_rn(dA[mt][0], dB[mt][0]);
        s_acc[(n0 + 1u) * 128u + ch] = __fadd_rn(dA[mt][1], dB[mt][1]);
        s_acc[n0 * 128u + ch + 8u] = __fadd_rn(dA[mt][2], dB[mt][2]);
        s_acc[(n0 + 1u) * 128u + ch + 8u] = __fadd_rn(dA[mt][3], dB[mt][3]);
    }
    named_barrier_sync(1, kConsumerThreads);

    const float* rout_blk =
        pr.rout ? pr.rout + static_cast<size_t>(expert) * OC + (ocb + o) * 128u : nullptr;

    if (S == 1) {
        for (uint32_t r = warp; r < static_cast<uint32_t>(nrows); r += 8u) {
            const float4 a4 = *reinterpret_cast<const float4*>(s_acc + r * 128u + lane * 4u);
            float v[4] = {a4.x, a4.y, a4.z, a4.w};
            const size_t off = static_cast<size_t>(s_rows[r]) * out_ld + pr.out_col0 + (ocb + o) * 128u + lane * 4u;
            if (pr.rout) finalize_row<true>(v, lane, rout_blk, pr, off, p.rs);
            else finalize_row<false>(v, lane, rout_blk, pr, off, p.rs);
        }
        // stores into other GPUs' buffers: one system-wide fence per CTA, after its last output
        // block (a fence per block makes every warp wait out an NVLink round trip each time)
        if (pr.npeer && o + 1u == G) __threadfence_system();
        continue;   // the next output block of this CTA (the barrier before its rows are
                    // written keeps them from overtaking the reads above)
    }

    // split-K: publish this CTA's partial, last arriver reduces in split order
    const size_t unit_floats = static_cast<size_t>(ROWS) * 128u;
    const size_t nocb = static_cast<size_t>(p.total_ocb);
    float* const my_part =
        p.part + ((static_cast<size_t>(job) * SMAX + split) * nocb + gocb) * unit_floats;
    for (uint32_t r = warp; r < static_cast<uint32_t>(nrows); r += 8u)
        __stcg(reinterpret_cast<float4*>(my_part + r * 128u + lane * 4u),
               *reinterpret_cast<const float4*>(s_acc + r * 128u + lane * 4u));
    __threadfence();
    named_barrier_sync(1, kConsumerThreads);
    if (tid == 0) {
        int32_t* ctr = p.counters + static_cast<size_t>(job) * nocb + gocb;
        const int prev = atomicAdd(ctr, 1);
        const int last = prev == static_cast<int>(S) - 1;
        if (last) *ctr = 0;  // every split has arrived: leave the counter clean for the next launch
        s_last = last;
    }
    named_barrier_sync(1, kConsumerThreads);
    if (!s_last) return;
    __threadfence();
    const float* const part0 =
        p.part + (static_cast<size_t>(job) * SMAX * nocb + gocb) * unit_floats;
    for (uint32_t r = warp; r < static_cast<uint32_t>(nrows); r += 8u) {
        float v[4];
        for (uint32_t s = 0; s < S; ++s) {
            const float4 q = __ldcg(reinterpret_cast<const float4*>(
                part0 + static_cast<size_t>(s) * nocb * unit_floats + r * 128u + lane * 4u));
            if (s == 0) { v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w; }
            else {
                v[0] = __fadd_rn(v[0], q.x); v[1] = __fadd_rn(v[1], q.y);
                v[2] = __fadd_rn(v[2], q.z); v[3] = __fadd_rn(v[3], q.w);
            }
        }
        const size_t off = static_cast<size_t>(s_rows[r]) * out_ld + pr.out_col0 + ocb * 128u + lane * 4u;
        if (pr.rout) finalize_row<true>(v, lane, rout_blk, pr, off, p.rs);
        else finalize_row<false>(v, lane, rout_blk, pr, off, p.rs);
    }
    if (pr.npeer) __threadfence_system();
  }   // output blocks of this CTA (split launches have one)
}

template <int K, int MT, bool GRP>
cudaError_t launch_t(const GemvMmaParams& p, int xrows, cudaStream_t st) {
    constexpr int STAGE_WORDS = 8 * 8 * 8 * K;
    const size_t XS = static_cast<size_t>(p.xcb) * 128u + 16u;
    const size_t smem =
        (static_cast<size_t>(NS * STAGE_WORDS) + static_cast<size_t>(xrows + 1) * XS +
         (p.ocb_group > 1 ? static_cast<size_t>(p.rows_per_job) * 128u : 0u)) * 4u;
    static SmemLimit limit;   // per device: largest size already enabled
    cudaError_t e = limit.ensure(gemv_mma_kernel<K, MT, GRP>, smem);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.total_ocb / p.ocb_group, p.splits, p.njobs);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = p.pdl != kPdlOff ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, gemv_mma_kernel<K, MT, GRP>, p);
}

}  // namespace

// ESCHA_B200_PDL = off | wait | prefetch (default): how launches use programmatic
// dependent launch; read once per process.  "prefetch" lets a dense launch request the
// first stages of its weight stream before the previous kernel of the stream has
// finished.  Only kernels that signal their dependents early can be overlapped that
// way, which in a stream of this library's launches means this library's own kernels,
// and none of them writes a code stream; "wait" is for a caller whose own kernels do
// both.
static int pdl_mode() {
    static const int mode = [] {
        const char* v = std::getenv("ESCHA_B200_PDL");
        if (!v) return static_cast<int>(kPdlPrefetch);
        if (!std::strcmp(v, "off")) return static_cast<int>(kPdlOff);
        if (!std::strcmp(v, "wait")) return static_cast<int>(kPdlWaitFirst);
        return static_cast<int>(kPdlPrefetch);
    }();
    return mode;
}

cudaError_t gemv_mma_status(int* host_status) {
    int zero = 0;
    cudaError_t e = cudaMemcpyFromSymbol(host_status, g_gemv_status, sizeof(int));
    if (e != cudaSuccess) return e;
    if (*host_status != 0) e = cudaMemcpyToSymbol(g_gemv_status, &zero, sizeof(int));
    return e;
}

size_t gemv_mma_part_floats(int njobs, int splits, int total_ocb, int rows_per_job) {
    if (splits <= 1) return 0;
    return static_cast<size_t>(njobs) * splits * total_ocb * rows_per_job * 128u;
}

// ESCHA_B200_GEMV_KERNEL=stream selects the persistent kernel (gemv_stream.cu) for every
// launch; otherwise this file's one-CTA-per-(block, split) kernel runs everything it can:
// launches whose projections all have one rate and that do not ask for the shared-memory
// table.  Read once per process.
static bool prefer_stream_kernel() {
    static const bool on = [] {
        const char* v = std::getenv("ESCHA_B200_GEMV_KERNEL");
        return v != nullptr && !std::strcmp(v, "stream");
    }();
    return on;
}
static bool table_mode() {
    static const bool on = [] {
        const char* s = std::getenv("ESCHA_B200_LUT_STATES");
        if (s && *s) return std::atoi(s) >= 2;
        const char* l = std::getenv("ESCHA_MLX_LUT");
        return l != nullptr && *l && std::strcmp(l, "0") != 0;
    }();
    return on;
}

cudaError_t launch_gemv_mma(const GemvMmaParams& params, cudaStream_t st) {
    bool mixed = false;
    for (int i = 1; i < params.nprob; ++i)
        if (params.prob[i].K && params.prob[i].K != params.prob[0].K) mixed = true;
    if (prefer_stream_kernel() || table_mode() || mixed) {
        GemvMmaParams q = params;
        q.pdl = pdl_mode();
        return launch_gemv_stream(q, st);
    }
    GemvMmaParams p = params;
    gemv_test_hooks(&p.test_stall, &p.wait_limit);
    const int rows = p.rows_per_job;
    const int xrows = p.jobs ? rows : (p.M < rows ? p.M : rows);
    p.xcb = x_chunk_blocks(xrows);
    p.pdl = pdl_mode();
    // Output blocks per CTA.  Expert streams at many rows come as thousands of short CTAs
    // (the second expert leg: four input blocks each) that all stage the same rows; when the
    // launch is unsplit, its input range fits one staged chunk and every projection's block
    // count allows it, a CTA takes 4 (or 2) consecutive output blocks and stages once, as
    // long as that still leaves two waves of CTAs.  Measured on the 35B-A3B-class layer at 64
    // tokens: second expert leg 89 -> 70 us.
    p.ocb_group = 1;
    if (p.jobs && p.splits == 1 && (p.IC >> 7) <= p.xcb) {
        for (int gsize = 4; gsize >= 2; gsize >>= 1) {
            bool fits = static_cast<long>(p.njobs) * (p.total_ocb / gsize) >= 2L * 3 * 148;
            for (int i = 0; i < p.nprob && fits; ++i) fits = (p.prob[i].OC / 128) % gsize == 0;
            if (fits) { p.ocb_group = gsize; break; }
        }
    }
    if (p.jobs) {
        if (p.K == 2) return rows == 8 ? launch_t<2, 1, true>(p, xrows, st) : launch_t<2, 2, true>(p, xrows, st);
        return rows == 8 ? launch_t<3, 1, true>(p, xrows, st) : launch_t<3, 2, true>(p, xrows, st);
    }
    if (p.K == 2) return rows == 8 ? launch_t<2, 1, false>(p, xrows, st) : launch_t<2, 2, false>(p, xrows, st);
    return rows == 8 ? launch_t<3, 1, false>(p, xrows, st) : launch_t<3, 2, false>(p, xrows, st);
}

}  // namespace escha
