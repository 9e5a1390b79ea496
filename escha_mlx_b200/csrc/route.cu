// Router of the MoE block in one launch: gate logits, top-k, softmax over the k
// values, the shared expert's gate logit, and the grouping of (token, slot) rows
// into per-expert jobs for the expert GEMV.
//
// Reference: EschaSparseMoeBlock.__call__ / route (escha_mlx/models/
// qwen3_5_moe.py:255-273; ref.py:326-331): fp32 logits from the fp16 gate linear
// rounded once through binary16, top-k, softmax over the selected values; and
// moe.build_groups (escha_mlx/moe.py:30-83) for the grouping.  The reference
// issues these as half a dozen framework ops; at decode batch sizes each of them
// costs more to launch than to run, so here they are one kernel:
//
//   phase 1 (grid: gate rows x tiles of 8 tokens)  one CTA per (row, tile): its 8
//                        warps split the hidden dimension, so every lane issues all of
//                        its loads at once; partial sums meet in shared memory and
//                        are added in warp order, rounded through binary16.
//   phase 2 (the last CTA to finish a tile)  one warp per token: k rounds of warp
//                        arg-max (ties to the lower expert index, i.e. a stable
//                        descending sort), softmax over the k values.
//   phase 3 (the last tile to finish)  rows -> RowJobs (ascending expert, ascending
//                        row inside an expert), restricted to this rank's experts
//                        [e_lo, e_hi) under expert parallelism.
//
// "Last" is decided with one counter per tile plus one for the launch, all zero on
// entry and left zero.
#include "common.cuh"
#include "kernels.h"

namespace escha {

namespace {

constexpr int kMaxExpertsPerLane = 32;  // E <= 1024

__device__ __forceinline__ float round_through_half(float v) {
    return __half2float(__float2half_rn(v));
}

__device__ __forceinline__ float dot8(const uint4& w, const uint4& x, float acc) {
    const uint32_t ww[4] = {w.x, w.y, w.z, w.w}, xx[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 a = __half22float2(as_half2(ww[i])), b = __half22float2(as_half2(xx[i]));
        acc = __fmaf_rn(a.x, b.x, acc);
        acc = __fmaf_rn(a.y, b.y, acc);
    }
    return acc;
}

// k rounds of warp arg-max over one token's logits (NV per lane), ties to the lower expert
// index; softmax over the k selected values; lane s writes the s-th selection.
template <int NV>
__device__ __forceinline__ void topk_softmax_token(const RouteParams& p, int tok, int lane) {
    float v[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int e = lane + 32 * i;
        v[i] = e < p.E ? __ldcg(p.logits + static_cast<size_t>(tok) * p.E + e) : -INFINITY;
    }
    float my_v = 0.0f, top_v = 0.0f;
    int my_e = 0;
    for (int s = 0; s < p.top_k; ++s) {
        float bv = -INFINITY;
        int be = 0x7FFFFFFF;
#pragma unroll
        for (int i = 0; i < NV; ++i)
            if (v[i] > bv) { bv = v[i]; be = lane + 32 * i; }
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) {
            const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, m);
            const int oe = __shfl_xor_sync(0xFFFFFFFFu, be, m);
            if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
        }
        if (s == 0) top_v = bv;
        if (lane == s) { my_v = bv; my_e = be; }
        if ((be & 31) == lane) {
#pragma unroll
            for (int i = 0; i < NV; ++i)
                if (i == (be >> 5)) v[i] = -INFINITY;
        }
    }
    // softmax over the k selected values: exp(v - max), summed in selection order
    const float ex = lane < p.top_k ? expf(__fsub_rn(my_v, top_v)) : 0.0f;
    float sum = 0.0f;
    for (int s = 0; s < p.top_k; ++s) sum = __fadd_rn(sum, __shfl_sync(0xFFFFFFFFu, ex, s));
    if (lane < p.top_k) {
        p.ids[static_cast<size_t>(tok) * p.top_k + lane] = my_e;
        p.scores[static_cast<size_t>(tok) * p.top_k + lane] = __fdiv_rn(ex, sum);
    }
}

__global__ void __launch_bounds__(256)
moe_route_kernel(const RouteParams p) {
    extern __shared__ int32_t s_dyn[];  // phase 3: [El + 1] job offsets, [m] local experts, [El] + [1 or 8][El] counts
    __shared__ float s_part[8][8];
    __shared__ int s_flag;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n_gate = p.ids_in ? 0 : p.E;
    const int n_rows = n_gate + (p.shg_w ? 1 : 0);
    const int r = blockIdx.x, tile = blockIdx.y, t0 = tile * 8;
    const int n_tiles = gridDim.y;
    // scheduled early (programmatic dependent launch): wait for the producer of x
    grid_launch_dependents();
    grid_dependency_wait();

    // ---- phase 1: this CTA's row against the tile's tokens
    if (r < n_rows) {
        const __half* wrow = r < n_gate ? p.gate_w + static_cast<size_t>(r) * p.H : p.shg_w;
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
        for (int k = tid * 8; k < p.H; k += 2048) {
            const uint4 wv = *reinterpret_cast<const uint4*>(wrow + k);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int tok = min(t0 + j, p.T - 1);
                const uint4 xv = *reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(tok) * p.H + k);
                acc[j] = dot8(wv, xv, acc[j]);
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float a = acc[j];
#pragma unroll
            for (int m = 16; m > 0; m >>= 1) a = __fadd_rn(a, __shfl_xor_sync(0xFFFFFFFFu, a, m));
            if (lane == 0) s_part[warp][j] = a;
        }
        __syncthreads();
        if (tid < 8 && t0 + tid < p.T) {
            float a = s_part[0][tid];
#pragma unroll
            for (int w = 1; w < 8; ++w) a = __fadd_rn(a, s_part[w][tid]);
            const float v = round_through_half(a);
            if (r < n_gate) p.logits[static_cast<size_t>(t0 + tid) * p.E + r] = v;
            else p.slog[t0 + tid] = v;
        }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        int32_t* ctr = p.counter + 1 + tile;
        const int prev = atomicAdd(ctr, 1);
        const int last = prev == static_cast<int>(gridDim.x) - 1;
        if (last) *ctr = 0;
        s_flag = last;
    }
    __syncthreads();
    if (!s_flag) return;
    __threadfence();

    // ---- phase 2: top-k and softmax for the tile's tokens, one warp per token
    const int tok = t0 + warp;
    if (!p.ids_in && tok < p.T) {
        if (p.E <= 256) topk_softmax_token<8>(p, tok, lane);     // the common expert counts
        else topk_softmax_token<kMaxExpertsPerLane>(p, tok, lane);
    }
    if (!p.jobs) return;
    __syncthreads();
    if (n_tiles > 1) {   // with a single tile its last CTA is the launch's last CTA
        __threadfence();
        if (tid == 0) {
            const int prev = atomicAdd(p.counter, 1);
            const int last = prev == n_tiles - 1;
            if (last) *p.counter = 0;
            s_flag = last;
        }
        __syncthreads();
        if (!s_flag) return;
        __threadfence();
    }

    // ---- phase 3: rows -> jobs.  Rows are counted per expert with shared-memory
    // atomics (per expert, and beyond 128 rows per expert and eighth of the rows) and the
    // counts turned into job offsets; then thread e fills in the headers of expert e's jobs,
    // and the rows are walked in ascending order, 32 at a time, giving each row its rank
    // among the rows of its expert: rows of earlier ranges (a prefix of the counts) + rows
    // seen so far in this range (a running count) + lanes before it in the group of 32
    // (lanes of one expert find each other with a warp match).  So jobs ascend by expert
    // and rows ascend inside a job -- the stable order moe.build_groups produces --
    // whatever order the atomics ran in.
    const int32_t* row_ids = p.ids_in ? p.ids_in : p.ids;
    const int m = p.T * p.top_k, El = p.e_hi - p.e_lo, R = p.R;
    int32_t* s_off = s_dyn;            // [El + 1]
    int32_t* s_loc = s_dyn + El + 1;   // [m] local expert of each row, -1 if another rank's
    int32_t* s_cnt = s_loc + m;        // [El] rows of each expert
    int32_t* s_run = s_cnt + El;       // [ranges][El] rows of each expert in (then: before) each range
    // Beyond 128 rows the rows are cut into eight contiguous ranges, one per warp, of a
    // multiple of 32 rows; up to 128 rows one warp walks them all (measured: the set-up of
    // the ranges costs small batches more than the shorter walk saves).
    const int n_ranges = m > 128 ? 8 : 1;
    const int per_warp = n_ranges == 1 ? ((m + 31) & ~31) : (((m + 255) >> 8) << 5);
    for (int e = tid; e <= El; e += blockDim.x) s_off[e] = 0;
    for (int e = tid; e < n_ranges * El; e += blockDim.x) s_run[e] = 0;
    __syncthreads();
    for (int i = tid; i < m; i += blockDim.x) {
        const int e = __ldcg(row_ids + i);
        const int loc = (e >= p.e_lo && e < p.e_hi) ? e - p.e_lo : -1;
        s_loc[i] = loc;
        if (loc >= 0) {
            atomicAdd(&s_off[loc + 1], 1);
            if (n_ranges > 1) atomicAdd(&s_run[(i / per_warp) * El + loc], 1);
        }
    }
    __syncthreads();
    // counts -> job offsets: exclusive prefix sum of ceil(count / R) over the experts.
    // Thread t owns a run of consecutive experts; runs are combined with a warp scan and
    // a scan of the eight warp totals (R is 8 or 16: the division is a shift).
    {
        __shared__ int s_warp_total[8];
        const int rshift = R == 8 ? 3 : 4;
        const int per = (El + 255) / 256;                 // experts per thread (<= 4)
        const int e_first = tid * per;
        int local[4], sum = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int e = e_first + k;
            const int cnt = (k < per && e < El) ? s_off[e + 1] : 0;
            if (k < per && e < El) s_cnt[e] = cnt;
            local[k] = (cnt + R - 1) >> rshift;
            sum += local[k];
        }
        int incl = sum;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int up = __shfl_up_sync(0xFFFFFFFFu, incl, d);
            if (lane >= d) incl += up;
        }
        if (lane == 31) s_warp_total[warp] = incl;
        __syncthreads();
        int base = 0;
        for (int w = 0; w < warp; ++w) base += s_warp_total[w];
        int run = base + incl - sum;                      // exclusive prefix of this thread's run
        __syncthreads();                                   // counts are read before they are overwritten
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int e = e_first + k;
            if (k < per && e < El) {
                run += local[k];
                s_off[e + 1] = run;
            }
        }
    }
    __syncthreads();
    const int total = s_off[El];
    const int rshift = R == 8 ? 3 : 4, rmask = R - 1;
    // job headers: expert and row count of every job of expert e
    for (int e = tid; e < El; e += blockDim.x) {
        const int base = s_off[e], njobs_e = s_off[e + 1] - base, cnt = s_cnt[e];
        for (int jj = 0; jj < njobs_e; ++jj) {
            const int j = base + jj;
            if (j < p.njobs_cap) {
                p.jobs[j].expert = e;
                p.jobs[j].nrows = min(R, cnt - (jj << rshift));
            }
        }
    }
    // an expert's rows before each range: exclusive prefix over the ranges
    if (n_ranges > 1) {
        for (int e = tid; e < El; e += blockDim.x) {
            int before = 0;
#pragma unroll
            for (int w = 0; w < 8; ++w) {
                const int here = s_run[w * El + e];
                s_run[w * El + e] = before;
                before += here;
            }
        }
        __syncthreads();
    }
    // rows, in ascending order inside every range: a warp walks its range 32 rows at a time
    if (warp < n_ranges) {
        int32_t* const run = s_run + warp * El;
        const int i_end = min(m, (warp + 1) * per_warp);
        for (int i0 = warp * per_warp; i0 < i_end; i0 += 32) {
            const int i = i0 + lane;
            const int e = i < i_end ? s_loc[i] : -1;
            // lanes holding rows of the same expert (rows of other ranks' experts and lanes
            // past the end match among themselves and are skipped)
            const unsigned same = __match_any_sync(0xFFFFFFFFu, e);
            if (e >= 0) {
                const int k = run[e] + __popc(same & ((1u << lane) - 1u));
                const int j = s_off[e] + (k >> rshift);
                if (j < p.njobs_cap) p.jobs[j].rows[k & rmask] = i;
            }
            __syncwarp();
            if (e >= 0 && lane == 31 - __clz(same)) run[e] += __popc(same);
            __syncwarp();
        }
    }
    for (int j = total + tid; j < p.njobs_cap; j += blockDim.x) {
        p.jobs[j].expert = 0;
        p.jobs[j].nrows = 0;
    }
}

}  // namespace

size_t route_shared_bytes(int T, int top_k, int e_lo, int e_hi) {
    const size_t m = static_cast<size_t>(T) * top_k;
    return ((m > 128 ? 10 : 3) * static_cast<size_t>(e_hi - e_lo) + 1 + m) * sizeof(int32_t);
}

cudaError_t launch_moe_route(const RouteParams& p, cudaStream_t st) {
    const int n_rows = (p.ids_in ? 0 : p.E) + (p.shg_w ? 1 : 0);
    const dim3 grid(n_rows > 0 ? n_rows : 1, (p.T + 7) / 8);
    const size_t smem = route_shared_bytes(p.T, p.top_k, p.e_lo, p.e_hi);
    static SmemLimit limit;
    if (smem > 48 * 1024) {
        const cudaError_t e = limit.ensure(moe_route_kernel, smem);
        if (e != cudaSuccess) return e;
    }
    return launch_dependent(moe_route_kernel, grid, dim3(256), smem, st, p);
}

}  // namespace escha
