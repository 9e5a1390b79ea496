// Persistent form of the tensor-core coded GEMV / small-batch GEMM: the fast path behind
// moe_gemv / dense_gemv / dense_gemm_rows[_direct[_out]] / dense_gemm_pair[_out] /
// moe_gemm_rows of the reference's kernel layer (escha_mlx/msl.py:1366-1478, :1785-1950),
//
//     mid[r, :] = f32(xh[r, :]) @ f32(decode(code[expert(r)]))
//
// optionally preceded in the same kernel by  xh = f16(H128(x * rin) * RS)  (also with the
// SwiGLU of two inputs in front) and followed by  y = f16((H128(mid) * RS) * rout),
// for up to eight projections per launch, each with its own rate (2 or 3 bits), width
// and code stream.
//
// Shape of the kernel on B200:
//  * One CTA per resident slot (three per SM), alive for the whole launch.  The work of
//    a launch is a list of ITEMS fixed by the shapes alone: (projection, row job, a few
//    consecutive 128-channel output blocks, one range of 128-channel input blocks).
//    CTAs take items in list order -- the first by block index, the rest from a counter
//    in the caller's workspace -- so however many projections a launch holds there is
//    one ramp-up and one tail, every SM stays busy until the list is empty, and nothing
//    about the result depends on which CTA ran which item.
//  * Ten warps, three roles, no block-wide barrier between them:
//      warp 8, feeder: resolves items and streams their code (cp.async.bulk, the untiled
//        TMA form, no multicast) into a ring of 128-channel stages, running as far ahead
//        of the decode as the ring allows, across item boundaries;
//      warp 9, finisher: takes each finished block's accumulators from shared memory and
//        does the epilogue (split-K partials and their ordered sum, output transform,
//        stores), so that no decode warp ever waits on global memory;
//      warps 0-7, decode: together they bring an item's activation rows into one of two
//        shared buffers as (x, 0) words (applying the input transform when it is fused);
//        then each owns 16 of the block's 128 output channels; ref.lane_positions
//        is exactly the A-fragment ownership of mma.m16n8k16 for the transposed tile, so
//        the eight halves a lane decodes go from registers into mma.sync against the
//        activations as B operand (up to 16 rows share one decode), fp32 accumulate.
//    Stages, activation buffers and item descriptors are handed over through mbarriers
//    with bounded, hardware-suspended waits.
//  * Each weight is kept as (w, w) in one register -- one HADD2 with half-select operands,
//    the format's binary16 rounding point -- against (x, 0): that spends an idle half of
//    the tensor core instead of two byte permutes per weight pair.  The loop is bound by
//    instruction issue (about 41 instructions per 16x16 tile), not by HBM.
//  * Optionally (NLUT > 0) some or all of a lane's eight states are looked up in a
//    65536-entry binary16 table held in shared memory instead of being hashed
//    (escha_mlx/msl.py:17-22, :114-115 of the reference: every kernel has such a twin).
//    The zero-extended table entry (w, 0) multiplies (x, 0) to the same bits as (w, w).
//  * Split-K partials go to the caller's scratch; the CTA that arrives last for an output
//    block sums them in ascending split order (no float atomics) and runs the output
//    transform with warp butterflies: bit-reproducible for a given (shape, split factor).
#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "kernels.h"

namespace escha {

namespace {

constexpr int kDecodeWarps = 8;
constexpr int kFeederWarp = 8;
constexpr int kFinisherWarp = 9;
constexpr int kStreamThreads = (kDecodeWarps + 2) * 32;
constexpr int kStreamMinBlocks = 3;   // resident CTAs per SM the kernel is built for
constexpr int kItemQ = 3;        // item descriptors in flight per CTA: the one being decoded and the next
                                 // (a CTA that claimed further ahead would sit on work others could do)
constexpr int kXBufs = 3;        // activation buffers: one in use, one staged ahead, one draining
constexpr int kLutBytes = 65536 * 2;

struct ItemDesc {
    int32_t kind;                // 1: work, 0: the list is exhausted
    int32_t pi, job, ocb, nocb, split, b0, nb, expert, nrows, K;
    int32_t rows[16];
};

// Bounded wait of the two service warps: test, then sleep about a microsecond.  They wait most
// of the time (for a free ring slot, for a finished block) and nothing needs them within
// less than that, so their polls should not take issue slots from the decode warps.
__device__ __forceinline__ bool mbar_wait_service(uint32_t bar, uint32_t parity, uint32_t limit) {
    for (uint32_t it = 0; it < limit; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        __nanosleep(200);
    }
    return false;
}

__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
    uint32_t v;
    asm volatile("{ .reg .u16 t; ld.shared.u16 t, [%1]; cvt.u32.u16 %0, t; }" : "=r"(v) : "r"(addr));
    return v;
}

__device__ __forceinline__ __half swiglu_half(__half g16, __half u16) {
    const float g = __half2float(g16);
    const __half s = __float2half_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))));
    return __hmul(s, u16);
}

// Error word set by a kernel whose bounded wait gave up (never expected).
__device__ int g_stream_status = 0;

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

// Stage warp `part`'s share (of `nparts`) of `cnt` 128-channel blocks (from block blk0) of an
// item's rows into a shared buffer as (x, 0) words.  Within each 16-channel group the words are
// ordered c0 c8 c1 c9 ... c7 c15, so that one 16-byte load at word 4t hands lane t the B
// fragments of both mma of a tile: (x[2t], x[2t+8]) and (x[2t+1], x[2t+9]).
__device__ __forceinline__ void stage_rows(const GemvMmaParams& p, const GemvProblem& pr,
                                           const ItemDesc& it, uint32_t blk0, uint32_t cnt,
                                           uint32_t* s_x, uint32_t XS, uint32_t lane,
                                           uint32_t part, uint32_t nparts) {
    const __half* xsrc = pr.x ? pr.x : p.x;
    const uint32_t IC = static_cast<uint32_t>(pr.IC);
    const int nrows = it.nrows;
    if (p.input == kInputTransformed) {
        const uint32_t grp_per_row = cnt * 8u;  // 16-channel groups per row
        const uint32_t total = static_cast<uint32_t>(nrows) * grp_per_row;
        for (uint32_t idx = part * 32u + lane; idx < total; idx += nparts * 32u) {
            const uint32_t r = idx / grp_per_row, v = idx - r * grp_per_row;
            const uint4* src = reinterpret_cast<const uint4*>(
                xsrc + static_cast<size_t>(it.rows[r] / p.x_row_div) * p.x_stride + blk0 * 128u +
                v * 16u);
            const uint4 lo = src[0], hi = src[1];  // channels 0..7 and 8..15 of the group
            uint4* dst = reinterpret_cast<uint4*>(s_x + r * XS + v * 16u);
            dst[0] = make_uint4(lo.x & 0xFFFFu, hi.x & 0xFFFFu, lo.x >> 16, hi.x >> 16);
            dst[1] = make_uint4(lo.y & 0xFFFFu, hi.y & 0xFFFFu, lo.y >> 16, hi.y >> 16);
            dst[2] = make_uint4(lo.z & 0xFFFFu, hi.z & 0xFFFFu, lo.z >> 16, hi.z >> 16);
            dst[3] = make_uint4(lo.w & 0xFFFFu, hi.w & 0xFFFFu, lo.w >> 16, hi.w >> 16);
        }
        return;
    }
    // fused input transform: one (row, block) unit per butterfly
    const float* rin = pr.rin + static_cast<size_t>(it.expert) * IC;
    const uint32_t units = static_cast<uint32_t>(nrows) * cnt;
    for (uint32_t u = part; u < units; u += nparts) {
        const uint32_t r = u / cnt, b = u - r * cnt;
        const size_t xoff = static_cast<size_t>(it.rows[r] / p.x_row_div) * p.x_stride +
                            (blk0 + b) * 128u + lane * 4u;
        uint2 raw = *reinterpret_cast<const uint2*>(xsrc + xoff);
        const float4 sc = *reinterpret_cast<const float4*>(rin + (blk0 + b) * 128u + lane * 4u);
        if (p.input == kInputSwiglu) {
            const uint2 up = *reinterpret_cast<const uint2*>(p.x_up + xoff);
            const __half2 g0 = as_half2(raw.x), g1 = as_half2(raw.y);
            const __half2 u0 = as_half2(up.x), u1 = as_half2(up.y);
            raw.x = as_u32(__halves2half2(swiglu_half(__low2half(g0), __low2half(u0)),
                                          swiglu_half(__high2half(g0), __high2half(u0))));
            raw.y = as_u32(__halves2half2(swiglu_half(__low2half(g1), __low2half(u1)),
                                          swiglu_half(__high2half(g1), __high2half(u1))));
        }
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

// Everything the roles of a CTA share.
struct Shared {
    uint64_t full[8];                        // code ring (up to 8 stages)
    uint64_t item_full[kItemQ], item_empty[kItemQ];
    uint64_t x_full[kXBufs], x_empty[kXBufs];
    uint64_t acc_full[2], acc_empty[2];      // a finished block's accumulators in s_acc
    ItemDesc item[kItemQ];
};

// Item index -> descriptor fields that depend on shapes only.
__device__ __forceinline__ uint32_t div_magic(uint32_t n, unsigned long long magic) {
    return static_cast<uint32_t>((static_cast<unsigned long long>(n) * magic) >> 40);
}
__device__ __forceinline__ void resolve_item(const GemvMmaParams& p, int id, ItemDesc& d) {
    int pi = 0;
#pragma unroll
    for (int q = 1; q < kMaxProblems; ++q)
        if (q < p.nprob && id >= p.prob[q].item0) pi = q;
    const GemvProblem& pr = p.prob[pi];
    const uint32_t rel = static_cast<uint32_t>(id - pr.item0);
    const uint32_t S = static_cast<uint32_t>(pr.splits), ngroups = static_cast<uint32_t>(pr.ngroups);
    const uint32_t rest = div_magic(rel, pr.magic_s), split = rel - rest * S;
    const uint32_t job = div_magic(rest, pr.magic_g), grp = rest - job * ngroups;
    const int nocb = pr.OC >> 7, opi = pr.opi;
    const int bbase = pr.bbase, brem = pr.brem;
    d.pi = pi;
    d.job = static_cast<int>(job);
    d.ocb = static_cast<int>(grp) * opi;
    d.nocb = min(opi, nocb - d.ocb);
    d.split = static_cast<int>(split);
    d.b0 = d.split * bbase + min(d.split, brem);
    d.nb = bbase + (d.split < brem ? 1 : 0);
}

// Hardware barriers between the decode warps and a service warp.  The service warps (feeder,
// finisher) wait most of the time; a polled wait, however sparse, costs them instructions on
// the two sub-partitions they live on, and since a stage is only free once all eight decode
// warps are through with it, the slowest sub-partition paces the whole CTA (measured: 98
// cycles per tile with polled service waits against 75 without service warps at all).  A
// named barrier parks the service warp in hardware: the eight decode warps arrive (without
// waiting), the service warp syncs.  These waits cannot time out; they do not need to,
// because the decode warps' own waits are all bounded and a decode warp that gave up still
// walks every stage of every item and arrives everywhere.
constexpr uint32_t kBarThreads = (kDecodeWarps + 1) * 32;
constexpr uint32_t kBarSlot0 = 1;    // ids 1..8: code ring slots
constexpr uint32_t kBarAcc0 = 9;     // ids 9, 10: accumulator buffers
// mbarrier arrive by lane 0 without a divergent branch
__device__ __forceinline__ void mbar_arrive_lane0(uint32_t bar, uint32_t lane) {
    asm volatile("{ .reg .pred p; setp.eq.u32 p, %1, 0; @p mbarrier.arrive.shared::cta.b64 _, [%0]; }"
                 ::"r"(bar), "r"(lane) : "memory");
}

// The slow half of a wait, kept out of line so the decode loop stays small.  try_wait blocks
// for a hardware-defined short time by itself; no sleep in between, the data is usually
// about to land.
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, uint32_t limit) {
    for (uint32_t it = 0; it < limit; ++it)
#pragma unroll 1
        for (int k = 0; k < 8; ++k)
            if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ bool mbar_wait_fast(uint32_t bar, uint32_t parity, uint32_t limit) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, limit);
}

template <int K, int MT, int NLUT>
__device__ __forceinline__ void decode_block(const uint32_t* wa, const uint32_t* wb,
                                             const uint32_t* const (&xr)[MT], float (&dA)[MT][4],
                                             float (&dB)[MT][4], const LaneConsts<K>& lc,
                                             const ShiftMuls& muls, uint32_t hmask, uint32_t hxor,
                                             uint32_t lut) {
    constexpr int ROW_WORDS = 64 * K;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
        uint32_t s[8], a[8];
        lc.states(wa[kk * ROW_WORDS], wb[kk * ROW_WORDS], muls, s);
#pragma unroll
        for (int j = 0; j < 8; ++j)
            a[j] = (j < NLUT) ? lds_u16(lut + s[j] + s[j]) : cba_decode_dup(s[j], hmask, hxor);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            // (x[2t], x[2t+8], x[2t+1], x[2t+9]) as (x, 0) words
            const uint4 b = *reinterpret_cast<const uint4*>(xr[mt] + kk * 16);
            // value j sits at (channel g + 8*(j>=4), input 2t + (j&1) + 8*((j>>1)&1))
            mma16816(dA[mt], a[0], a[4], a[2], a[6], b.x, b.y);
            mma16816(dB[mt], a[1], a[5], a[3], a[7], b.z, b.w);
        }
    }
}

// What a decode warp keeps about the rings between items.
struct RingPos {
    uint32_t slot_off;   // word offset of the current code stage
    uint32_t slot8;      // 8 * slot: byte offset of the stage's full barrier
    uint32_t slot, phase;
    uint32_t xc;         // activation chunks consumed
    // staging runs one chunk ahead of the decode: next chunk to stage = chunk sc0 of item sq
    uint32_t sq, sn;     // item index of the staging cursor, chunks staged so far
    int sc0;
    bool sdone;          // the cursor has reached the end of the list (or a wait gave up)
};

// Stage this warp's share of the next chunk in list order (possibly the next item's first).
// `block` = false is the look-ahead: if the chunk belongs to an item whose descriptor is not
// out yet, nothing happens (the feeder may itself be waiting for this warp to free ring slots).
// Returns false if nothing was staged.
template <int MT>
__device__ __forceinline__ bool stage_next(const GemvMmaParams& p, Shared& sh, uint32_t* s_x, uint32_t XS,
                                           uint32_t xrows, RingPos& rp, uint32_t lane, uint32_t warp,
                                           bool block, bool& ok) {
    const uint32_t limit = p.wait_limit;
    const uint32_t qs = rp.sq % kItemQ;
    const uint32_t ibar = smem_u32(sh.item_full) + 8u * qs, ipar = (rp.sq / kItemQ) & 1u;
    if (!block) {
        if (!mbar_try_wait(ibar, ipar)) return false;
    } else if (!mbar_wait_fast(ibar, ipar, limit)) {
        rp.sdone = true;
        ok = false;
        return false;
    }
    const ItemDesc& it = sh.item[qs];
    if (it.kind == 0) { rp.sdone = true; return false; }
    const uint32_t xb = rp.sn % kXBufs;
    if (ok && rp.sn >= kXBufs &&
        !mbar_wait_fast(smem_u32(sh.x_empty) + 8u * xb, ((rp.sn / kXBufs) - 1u) & 1u, limit)) ok = false;
    const int cnt = min(p.xcb, it.nb - rp.sc0);
    stage_rows(p, p.prob[it.pi], it, static_cast<uint32_t>(it.b0 + rp.sc0), static_cast<uint32_t>(cnt),
               s_x + xb * xrows * XS, XS, lane, warp, kDecodeWarps);
    __syncwarp();
    mbar_arrive_lane0(smem_u32(sh.x_full) + 8u * xb, lane);
    ++rp.sn;
    rp.sc0 += p.xcb;
    if (rp.sc0 >= it.nb) { rp.sc0 = 0; ++rp.sq; }
    return true;
}

// One item's products for one output block: walk the item's input blocks, decoding each
// stage's 8 x 8 tiles into the accumulators.  K is a template parameter, so everything about
// the stage layout is an immediate; what the per-block path needs is kept in registers.
template <int K, int MT, int NLUT>
__device__ __forceinline__ bool item_block(const GemvMmaParams& p, Shared& sh, const uint32_t* s_code,
                                           const uint32_t* s_x, uint32_t XS, uint32_t xrows,
                                           int nb, int nrows, bool first_ocb, bool last_ocb,
                                           RingPos& rp, uint32_t lane, uint32_t warp, uint32_t lut,
                                           float (&dA)[MT][4], float (&dB)[MT][4], bool ok) {
    constexpr int WPT = 8 * K;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t NS = p.nstages, SLOT = p.slot_words, limit = p.wait_limit;
    const uint32_t full0 = smem_u32(sh.full);
    const uint32_t xfull0 = smem_u32(sh.x_full), xempty0 = smem_u32(sh.x_empty);
    const LaneConsts<K> lc(lane);
    const uint32_t hmask = p.hash_mask, hxor = p.hash_xor;
    const ShiftMuls muls{p.mul2, p.mul4, p.mul16, p.mul32, p.mul64, p.mul128};
    const uint32_t* const wa0 = s_code + warp * WPT + lc.ia();
    const uint32_t* const wb0 = s_code + warp * WPT + lc.ib();
    const uint32_t xcb = p.xcb;
    const bool live = p.test_stall != 2;   // false only in the decode-only measurement mode
    for (int c0 = 0; c0 < nb; c0 += xcb, ++rp.xc) {
        const uint32_t xb = rp.xc % kXBufs;
        const int cnt = min(static_cast<int>(xcb), nb - c0);
        bool look = false;   // the next chunk still has to be staged by this warp
        if (first_ocb) {
            // this chunk's rows were staged while the previous chunk was being decoded; stage
            // the chunk after it now (every decode warp its share), then make sure all eight
            // shares of this one have landed
            if (rp.sn == rp.xc)
                stage_next<MT>(p, sh, const_cast<uint32_t*>(s_x), XS, xrows, rp, lane, warp, true, ok);
            if (!rp.sdone && rp.sn == rp.xc + 1u)
                look = !stage_next<MT>(p, sh, const_cast<uint32_t*>(s_x), XS, xrows, rp, lane, warp, false, ok) &&
                       !rp.sdone;
            if (ok && !mbar_wait_fast(xfull0 + 8u * xb, (rp.xc / kXBufs) & 1u, limit)) ok = false;
        }
        const uint32_t* xbuf = s_x + xb * xrows * XS + 4u * t;
        const uint32_t* xr[MT];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            // columns past the job's last row repeat row 0: their results are never stored
            const int rslot = static_cast<int>(g) + 8 * mt;
            xr[mt] = xbuf + (rslot < nrows ? rslot : 0) * XS;
        }
        for (int cb = 0; cb < cnt; ++cb) {
            // the look-ahead again if the next item's descriptor was not out yet
            if (look)
                look = !stage_next<MT>(p, sh, const_cast<uint32_t*>(s_x), XS, xrows, rp, lane, warp, false, ok) &&
                       !rp.sdone;
            if (live && ok && !mbar_try_wait(full0 + rp.slot8, rp.phase) &&
                !mbar_wait_slow(full0 + rp.slot8, rp.phase, limit)) ok = false;
            decode_block<K, MT, NLUT>(wa0 + rp.slot_off, wb0 + rp.slot_off, xr, dA, dB, lc, muls, hmask, hxor, lut);
            if (live) named_barrier_arrive(kBarSlot0 + rp.slot, kBarThreads);   // done with the stage
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) xr[mt] += 128;
            rp.slot_off += SLOT;
            rp.slot8 += 8u;
            if (++rp.slot == NS) { rp.slot = 0; rp.slot8 = 0; rp.slot_off = 0; rp.phase ^= 1u; }
        }
        if (last_ocb) {
            __syncwarp();
            mbar_arrive_lane0(xempty0 + 8u * xb, lane);
        }
    }
    return ok;
}

template <int MT, int NLUT>
__global__ void __launch_bounds__(kStreamThreads, NLUT ? 1 : kStreamMinBlocks)
gemv_stream_kernel(const __grid_constant__ GemvMmaParams p) {
    constexpr int ROWS = 8 * MT;
    extern __shared__ __align__(128) uint32_t smem[];
    __shared__ __align__(16) Shared sh;
    const uint32_t NS = p.nstages, SLOT = p.slot_words;
    const uint32_t XS = p.xcb * 128u + 16u;           // words per staged row
    const uint32_t xrows = p.xrows;
    uint32_t* const s_code = smem;                              // [NS][SLOT]
    uint32_t* const s_x = s_code + NS * SLOT;                   // [kXBufs][xrows][XS]
    float* const s_acc = reinterpret_cast<float*>(s_x + kXBufs * xrows * XS);   // [2][ROWS][128]
    uint32_t* const s_lut = reinterpret_cast<uint32_t*>(s_acc + 2 * ROWS * 128);   // 128 KiB when NLUT

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t full0 = smem_u32(sh.full);
    const uint32_t ifull0 = smem_u32(sh.item_full), iempty0 = smem_u32(sh.item_empty);
    const uint32_t xfull0 = smem_u32(sh.x_full), xempty0 = smem_u32(sh.x_empty);
    const uint32_t accfull0 = smem_u32(sh.acc_full), accempty0 = smem_u32(sh.acc_empty);
    const uint32_t limit = p.wait_limit;

    if (tid == 0) {
        for (uint32_t s = 0; s < NS; ++s) {
            mbar_init(full0 + 8u * s, 1u);               // the producer's arrive.expect_tx
        }
        for (int q = 0; q < kItemQ; ++q) {
            mbar_init(ifull0 + 8u * q, 1u);
            mbar_init(iempty0 + 8u * q, kDecodeWarps + 1u);   // decode warps + the finisher
        }
        for (int b = 0; b < kXBufs; ++b) {
            mbar_init(xfull0 + 8u * b, kDecodeWarps);    // every decode warp stages a share
            mbar_init(xempty0 + 8u * b, kDecodeWarps);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(accfull0 + 8u * b, kDecodeWarps);
            mbar_init(accempty0 + 8u * b, 1u);
        }
        mbar_fence_init();
    }
    // Programmatic dependent launch: the next kernel of the stream may be scheduled as
    // soon as every CTA of this one has started.  Everything a launch reads that an
    // earlier kernel may have written (row jobs, activations, the work counter) sits
    // behind grid_dependency_wait().
    if (p.pdl != kPdlOff) grid_launch_dependents();
    if (NLUT) {
        // the table: 65536 binary16 weights, filled once per CTA
        __half* lut16 = reinterpret_cast<__half*>(s_lut);
        for (uint32_t i = tid; i < 65536u; i += kStreamThreads) lut16[i] = cba_decode(i);
    }
    __syncthreads();
    const int total = p.total_items;

    if (warp == kFeederWarp) {
        // ---- feeder: resolves items, stages their activation rows, streams their code
        uint32_t rslot = 0, lap = 0;  // ring position and how many times the ring has wrapped
        uint32_t q = 0;               // items published
        int id = blockIdx.x;
        bool ok = true;

        // One stage = the eight kt rows of a 128-channel input block for one output block,
        // one bulk copy per row (lanes 0..7).  `wait` = false issues only into a slot that is
        // free right now and reports whether it did.
        auto issue_stage = [&](const uint32_t* grow, uint32_t row_bytes) {
            // the slot is free once all eight decode warps have arrived at its barrier
            if (lap > 0) named_barrier_sync(kBarSlot0 + rslot, kBarThreads);
            if (lane == 0) mbar_arrive_expect_tx(full0 + 8u * rslot, 8u * row_bytes);
            __syncwarp();
            if (lane < 8 && p.test_stall != 1)
                bulk_copy_g2s(smem_u32(s_code + rslot * SLOT) + lane * row_bytes, grow, row_bytes,
                              full0 + 8u * rslot);
            if (++rslot == NS) { rslot = 0; ++lap; }
        };

        // Weights are never written by a kernel of this library, so with kPdlPrefetch a dense
        // launch requests the first stages of its first item before waiting for the previous
        // kernel of the stream: its start-up overlaps that kernel's tail.
        int pre = 0;
        if (p.pdl == kPdlPrefetch && !p.jobs && id < total && p.test_stall != 2) {
            ItemDesc d;
            resolve_item(p, id, d);
            const GemvProblem& pr = p.prob[d.pi];
            const uint32_t WPT = 8u * static_cast<uint32_t>(pr.K), ROW_WORDS = 8u * WPT;
            const size_t tile_row_words = static_cast<size_t>(static_cast<uint32_t>(pr.OC) >> 4) * WPT;
            const uint32_t* grow = pr.code + (static_cast<size_t>(d.b0) * 8u + lane) * tile_row_words +
                                   static_cast<size_t>(d.ocb) * ROW_WORDS;
            const int cnt = min(min(p.xcb, d.nb), static_cast<int>(NS));
            for (; pre < cnt; ++pre, grow += 8u * tile_row_words) issue_stage(grow, ROW_WORDS * 4u);
        }
        if (p.pdl != kPdlOff) grid_dependency_wait();

        for (;;) {
            ItemDesc d;
            const bool work = ok && id < total;
            if (work) {
                resolve_item(p, id, d);
                if (p.jobs) {
                    const RowJob* jb = p.jobs + d.job;
                    d.expert = jb->expert;
                    d.nrows = jb->nrows;
                } else {
                    d.expert = 0;
                    d.nrows = min(ROWS, p.M - d.job * ROWS);
                }
            }
            // the id after this one: by block stride, or from the shared counter (the
            // atomic's answer is not needed until this item's code has been issued)
            int next = id + static_cast<int>(gridDim.x);
            if (p.sched && work && lane == 0) next = static_cast<int>(gridDim.x) + atomicAdd(p.sched, 1);
            if (work && d.nrows <= 0) {   // an empty row job
                id = p.sched ? __shfl_sync(0xFFFFFFFFu, next, 0) : next;
                continue;
            }
            // publish the descriptor
            const uint32_t qs = q % kItemQ;
            if (ok && q >= kItemQ && !mbar_wait_service(iempty0 + 8u * qs, ((q / kItemQ) - 1u) & 1u, limit))
                ok = false;
            ItemDesc& pub = sh.item[qs];
            if (lane == 0) {
                pub.kind = work ? 1 : 0;
                if (work) {
                    pub.pi = d.pi; pub.job = d.job; pub.ocb = d.ocb; pub.nocb = d.nocb; pub.split = d.split;
                    pub.b0 = d.b0; pub.nb = d.nb; pub.expert = d.expert; pub.nrows = d.nrows;
                    pub.K = p.prob[d.pi].K;
                }
            }
            if (work && lane < 16)
                pub.rows[lane] = p.jobs ? p.jobs[d.job].rows[lane] : d.job * ROWS + static_cast<int>(lane);
            __syncwarp();
            if (lane == 0) mbar_arrive(ifull0 + 8u * qs);
            ++q;
            if (!work) break;
            // the item's code: for each output block, its range of input blocks, stage by stage
            // as the decode warps free slots
            const GemvProblem& pr = p.prob[d.pi];
            const uint32_t WPT = 8u * static_cast<uint32_t>(pr.K), ROW_WORDS = 8u * WPT;
            const size_t tile_row_words = static_cast<size_t>(static_cast<uint32_t>(pr.OC) >> 4) * WPT;
            const uint32_t* base = pr.code +
                static_cast<size_t>(d.expert) * (static_cast<uint32_t>(pr.IC) >> 4) * tile_row_words +
                (static_cast<size_t>(d.b0) * 8u + lane) * tile_row_words;
            for (int o = 0; o < d.nocb; ++o) {
                const uint32_t* grow = base + static_cast<size_t>(d.ocb + o) * ROW_WORDS;
                for (int c0 = 0; c0 < d.nb; c0 += p.xcb) {
                    const int cnt = min(p.xcb, d.nb - c0);
                    int b = 0;
                    if (pre > 0) {   // the first chunk's first stages went out before the dependency wait
                        b = pre;
                        grow += static_cast<size_t>(pre) * 8u * tile_row_words;
                        pre = 0;
                    }
                    if (p.test_stall == 2) b = cnt;   // measurement aid: decode from whatever the ring holds
                    for (; b < cnt; ++b) {
                        issue_stage(grow, ROW_WORDS * 4u);
                        grow += 8u * tile_row_words;
                    }
                }
            }
            id = p.sched ? __shfl_sync(0xFFFFFFFFu, next, 0) : next;
        }
        if (!ok && lane == 0) atomicExch(&g_stream_status, 1);
        // Leave the work counter clean for the next launch: the last CTA whose feeder
        // has run out of items resets it (no feeder fetches after its own exhaustion).
        if (p.sched && lane == 0) {
            __threadfence();
            if (atomicAdd(p.sched + 1, 1) == static_cast<int>(gridDim.x) - 1) {
                p.sched[0] = 0;
                p.sched[1] = 0;
            }
        }
        return;
    }
    if (p.pdl != kPdlOff) grid_dependency_wait();

    if (warp == kFinisherWarp) {
        // ---- finisher: everything that happens to a finished block's accumulators.  The
        // decode warps leave them in one of two shared buffers and go on decoding; this warp
        // transforms and stores the rows (unsplit item) or publishes the partial, counts the
        // block's splits and, if this was the last one, sums the partials in ascending split
        // order and transforms the rows.  All global-memory latency of the epilogue stays here.
        uint32_t q = 0, na = 0;   // items consumed, blocks finished
        bool ok = true;
        for (;;) {
            const uint32_t qs = q % kItemQ;
            if (!mbar_wait_service(ifull0 + 8u * qs, (q / kItemQ) & 1u, limit)) { ok = false; break; }
            const ItemDesc& it = sh.item[qs];
            if (it.kind == 0) break;
            const GemvProblem& pr = p.prob[it.pi];
            const int nrows = it.nrows;
            const uint32_t S = static_cast<uint32_t>(pr.splits);
            const uint32_t OC = static_cast<uint32_t>(pr.OC);
            const size_t out_ld = pr.out_ld ? static_cast<size_t>(pr.out_ld) : OC;
            for (int o = 0; o < it.nocb; ++o, ++na) {
                const uint32_t ab = na & 1u;
                named_barrier_sync(kBarAcc0 + ab, kBarThreads);   // all eight decode warps have left their rows
                const float* const acc = s_acc + ab * (ROWS * 128);
                const uint32_t ocb = static_cast<uint32_t>(it.ocb + o);
                const uint32_t gocb = static_cast<uint32_t>(pr.ocb0) + ocb;
                const float* rout_blk =
                    pr.rout ? pr.rout + static_cast<size_t>(it.expert) * OC + ocb * 128u : nullptr;
                if (S == 1) {
                    for (int r = 0; r < nrows; ++r) {
                        const float4 a4 = *reinterpret_cast<const float4*>(acc + r * 128 + lane * 4u);
                        float v[4] = {a4.x, a4.y, a4.z, a4.w};
                        const size_t off = static_cast<size_t>(it.rows[r]) * out_ld + pr.out_col0 + ocb * 128u + lane * 4u;
                        if (pr.rout) finalize_row<true>(v, lane, rout_blk, pr, off, p.rs);
                        else finalize_row<false>(v, lane, rout_blk, pr, off, p.rs);
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(accempty0 + 8u * ab);
                    if (pr.npeer) __threadfence_system();
                    continue;
                }
                const size_t unit_floats = static_cast<size_t>(ROWS) * 128u;
                const size_t nocb_all = static_cast<size_t>(p.total_ocb);
                const size_t SMAX = static_cast<size_t>(p.splits);
                const size_t job = static_cast<size_t>(it.job);
                float* const my_part =
                    p.part + ((job * SMAX + static_cast<size_t>(it.split)) * nocb_all + gocb) * unit_floats;
                for (int r = 0; r < nrows; ++r)
                    __stcg(reinterpret_cast<float4*>(my_part + r * 128 + lane * 4u),
                           *reinterpret_cast<const float4*>(acc + r * 128 + lane * 4u));
                __syncwarp();
                if (lane == 0) mbar_arrive(accempty0 + 8u * ab);   // the buffer is free again
                __threadfence();
                __syncwarp();
                int prev = 0;
                int32_t* ctr = p.counters + job * nocb_all + gocb;
                if (lane == 0) prev = atomicAdd(ctr, 1);
                prev = __shfl_sync(0xFFFFFFFFu, prev, 0);
                if (prev != static_cast<int>(S) - 1) continue;
                if (lane == 0) *ctr = 0;   // every split has arrived: leave the counter clean for the next launch
                __threadfence();
                const float* const part0 = p.part + (job * SMAX * nocb_all + gocb) * unit_floats;
                for (int r = 0; r < nrows; ++r) {
                    float v[4] = {0.f, 0.f, 0.f, 0.f};
                    for (uint32_t s0 = 0; s0 < S; s0 += 4u) {
                        float4 qv[4];
#pragma unroll
                        for (uint32_t i = 0; i < 4u; ++i)
                            if (s0 + i < S)
                                qv[i] = __ldcg(reinterpret_cast<const float4*>(
                                    part0 + static_cast<size_t>(s0 + i) * nocb_all * unit_floats + r * 128 + lane * 4u));
#pragma unroll
                        for (uint32_t i = 0; i < 4u; ++i) {
                            if (s0 + i >= S) break;
                            if (s0 + i == 0) { v[0] = qv[i].x; v[1] = qv[i].y; v[2] = qv[i].z; v[3] = qv[i].w; }
                            else {
                                v[0] = __fadd_rn(v[0], qv[i].x); v[1] = __fadd_rn(v[1], qv[i].y);
                                v[2] = __fadd_rn(v[2], qv[i].z); v[3] = __fadd_rn(v[3], qv[i].w);
                            }
                        }
                    }
                    const size_t off = static_cast<size_t>(it.rows[r]) * out_ld + pr.out_col0 + ocb * 128u + lane * 4u;
                    if (pr.rout) finalize_row<true>(v, lane, rout_blk, pr, off, p.rs);
                    else finalize_row<false>(v, lane, rout_blk, pr, off, p.rs);
                }
                if (pr.npeer) __threadfence_system();
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(iempty0 + 8u * qs);
            ++q;
        }
        if (!ok && lane == 0) atomicExch(&g_stream_status, 2);
        return;
    }

    // ---- decode warps.  Each runs on its own: it waits for descriptors, activation chunks,
    // code stages and a free accumulator buffer itself, never touches global memory, and has
    // no barrier with the other seven.  A warp whose wait gave up stops waiting (ok = false)
    // but keeps the control flow the descriptors dictate; what it computes from then on is
    // void and the status word says so.
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t lut = smem_u32(s_lut);
    RingPos rp{0u, 0u, 0u, 0u, 0u, 0u, 0u, 0, false};
    uint32_t q = 0, na = 0;   // items consumed, blocks finished
    bool ok = true;
    for (;;) {
        const uint32_t qs = q % kItemQ;
        if (!mbar_wait_fast(ifull0 + 8u * qs, (q / kItemQ) & 1u, limit)) { ok = false; break; }
        const ItemDesc& it = sh.item[qs];
        if (it.kind == 0) break;
        const int nrows = it.nrows, nb = it.nb, nocb_item = it.nocb, Kp = it.K;
        const uint32_t xc_item = rp.xc;
        for (int o = 0; o < nocb_item; ++o, ++na) {
            float dA[MT][4], dB[MT][4];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int i = 0; i < 4; ++i) dA[mt][i] = dB[mt][i] = 0.0f;
            rp.xc = xc_item;
            if (Kp == 2)
                ok = item_block<2, MT, NLUT>(p, sh, s_code, s_x, XS, xrows, nb, nrows, o == 0,
                                             o == nocb_item - 1, rp, lane, warp, lut, dA, dB, ok);
            else
                ok = item_block<3, MT, NLUT>(p, sh, s_code, s_x, XS, xrows, nb, nrows, o == 0,
                                             o == nocb_item - 1, rp, lane, warp, lut, dA, dB, ok);
            // hand the block's accumulators to the finisher
            const uint32_t ab = na & 1u;
            if (ok && na >= 2u && !mbar_wait_fast(accempty0 + 8u * ab, ((na >> 1) - 1u) & 1u, limit)) ok = false;
            float* const acc = s_acc + ab * (ROWS * 128);
            const uint32_t ch = warp * 16u + g;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const uint32_t n0 = 2u * t + 8u * mt;
                acc[n0 * 128u + ch] = __fadd_rn(dA[mt][0], dB[mt][0]);
                acc[(n0 + 1u) * 128u + ch] = __fadd_rn(dA[mt][1], dB[mt][1]);
                acc[n0 * 128u + ch + 8u] = __fadd_rn(dA[mt][2], dB[mt][2]);
                acc[(n0 + 1u) * 128u + ch + 8u] = __fadd_rn(dA[mt][3], dB[mt][3]);
            }
            named_barrier_arrive(kBarAcc0 + ab, kBarThreads);
        }
        __syncwarp();
        mbar_arrive_lane0(iempty0 + 8u * qs, lane);
        ++q;
    }
    if (!ok && lane == 0) atomicExch(&g_stream_status, 3);
}

// ---- host side

// Shared memory per CTA that keeps three CTAs on an SM (228 KiB per SM, 1 KiB reserved per CTA).
constexpr size_t kSmemBudget3 = (228 / kStreamMinBlocks - 2) * 1024;
constexpr size_t kSmemBudget1 = 226 * 1024;

template <int MT, int NLUT>
cudaError_t launch_stream_t(const GemvMmaParams& p, size_t smem, int grid, cudaStream_t st) {
    static SmemLimit limit;   // per device: largest size already enabled
    cudaError_t e = limit.ensure(gemv_stream_kernel<MT, NLUT>, smem);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kStreamThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = p.pdl != kPdlOff ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, gemv_stream_kernel<MT, NLUT>, p);
}

int g_test_stall = 0;
unsigned g_test_limit = 0;

int env_int(const char* name, int dflt) {
    const char* v = std::getenv(name);
    return v && *v ? std::atoi(v) : dflt;
}

}  // namespace

void gemv_stream_test_stall(int on, unsigned limit) {
    g_test_stall = on;
    g_test_limit = limit;
}

void gemv_test_hooks(int* stall, unsigned* limit) {
    *stall = g_test_stall;
    *limit = g_test_limit ? g_test_limit : (1u << 21);
}

cudaError_t gemv_stream_status(int* host_status) {
    int zero = 0;
    cudaError_t e = cudaMemcpyFromSymbol(host_status, g_stream_status, sizeof(int));
    if (e != cudaSuccess) return e;
    if (*host_status != 0) e = cudaMemcpyToSymbol(g_stream_status, &zero, sizeof(int));
    return e;
}

// Table mode of the decode (read once per process): ESCHA_MLX_LUT=1 looks all eight of a
// lane's states up in the shared-memory table (the reference's `_lut` kernel twins);
// ESCHA_B200_LUT_STATES=2 is the hybrid that looks two up and hashes six.
static int lut_states() {
    static const int n = [] {
        int v = env_int("ESCHA_B200_LUT_STATES", -1);
        if (v < 0) {
            const char* l = std::getenv("ESCHA_MLX_LUT");
            v = (l && *l && std::strcmp(l, "0") != 0) ? 8 : 0;
        }
        return v >= 8 ? 8 : (v >= 2 ? 2 : 0);
    }();
    return n;
}

cudaError_t launch_gemv_stream(const GemvMmaParams& params, cudaStream_t st) {
    GemvMmaParams p = params;
    const int ROWS = p.rows_per_job;
    const int nlut = lut_states();
    int dev = 0, sms = 148;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    static int sm_count[64] = {0};
    if (dev >= 0 && dev < 64 && sm_count[dev]) sms = sm_count[dev];
    else {
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) sm_count[dev] = sms;
    }
    const int ctas = (nlut ? 1 : kStreamMinBlocks) * sms;

    // rows an activation buffer holds, and blocks per staged chunk: about 10 KiB per buffer
    p.xrows = p.jobs ? ROWS : (p.M < ROWS ? p.M : ROWS);
    int xcb = 10240 / (p.xrows * 512);
    p.xcb = xcb > 16 ? 16 : (xcb < 1 ? 1 : xcb);

    // the item list
    int maxK = 2, total = 0;
    static const int opi_pin = env_int("ESCHA_B200_OPI", 0);
    for (int i = 0; i < p.nprob; ++i) {
        GemvProblem& pr = p.prob[i];
        if (pr.K == 0) pr.K = p.K;
        if (pr.IC == 0) pr.IC = p.IC;
        if (pr.K > maxK) maxK = pr.K;
        const int nocb = pr.OC / 128, nblk = pr.IC / 128;
        const int nb_max = (nblk + pr.splits - 1) / pr.splits;
        // Output blocks per item.  Blocks of one item share one staging of the rows, which
        // matters when that staging is a large part of the item (row jobs with a fused
        // input transform over a short K range); it needs the whole range in one chunk.
        int opi = 1;
        if (nb_max <= p.xcb && p.jobs && p.input != kInputTransformed) {
            while (opi < 8 && nocb % (opi * 2) == 0 &&
                   static_cast<long>(p.njobs) * (nocb / (opi * 2)) * pr.splits >= 4L * ctas)
                opi *= 2;
        }
        if (opi_pin > 0 && nb_max <= p.xcb) opi = opi_pin < nocb ? opi_pin : nocb;
        pr.opi = opi;
        pr.item0 = total;
        pr.ngroups = (nocb + opi - 1) / opi;
        pr.bbase = nblk / pr.splits;
        pr.brem = nblk % pr.splits;
        pr.magic_s = ((1ull << 40) + pr.splits - 1) / pr.splits;
        pr.magic_g = ((1ull << 40) + pr.ngroups - 1) / pr.ngroups;
        total += p.njobs * pr.ngroups * pr.splits;
    }
    if (total >= (1 << 24)) return cudaErrorInvalidValue;   // div_magic's range
    p.total_items = total;
    p.slot_words = 8 * 8 * 8 * maxK;
    const size_t x_bytes = static_cast<size_t>(kXBufs) * p.xrows * (p.xcb * 128u + 16u) * 4u;
    const size_t acc_bytes = 2u * static_cast<size_t>(ROWS) * 128u * 4u;
    const size_t budget = nlut ? kSmemBudget1 - kLutBytes : kSmemBudget3;
    long ns = (static_cast<long>(budget) - static_cast<long>(x_bytes + acc_bytes)) / (p.slot_words * 4);
    if (ns > 8) ns = 8;
    if (ns < 2) ns = 2;
    p.nstages = static_cast<int>(ns);
    const size_t smem = static_cast<size_t>(p.nstages) * p.slot_words * 4u + x_bytes + acc_bytes +
                        (nlut ? kLutBytes : 0);
    static const int dry = env_int("ESCHA_B200_DRY", 0);
    p.test_stall = dry ? 2 : g_test_stall;
    p.wait_limit = g_test_limit ? g_test_limit : (1u << 21);
    const int grid = total < ctas ? total : ctas;
    if (grid <= 0) return cudaSuccess;
    if (ROWS == 8) {
        if (nlut == 0) return launch_stream_t<1, 0>(p, smem, grid, st);
        if (nlut == 2) return launch_stream_t<1, 2>(p, smem, grid, st);
        return launch_stream_t<1, 8>(p, smem, grid, st);
    }
    if (nlut == 0) return launch_stream_t<2, 0>(p, smem, grid, st);
    if (nlut == 2) return launch_stream_t<2, 2>(p, smem, grid, st);
    return launch_stream_t<2, 8>(p, smem, grid, st);
}

}  // namespace escha
