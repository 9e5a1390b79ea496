// Row bookkeeping and elementwise stages of the routed-expert path
// (escha_mlx/moe.py:30-83 build_groups; escha_mlx/models/qwen3_5_moe.py:207-253
// _expert_path of the reference).  Everything is device-resident with static
// shapes -- no host synchronisation, CUDA-graph capturable -- like the
// reference's build_groups.
#include "common.cuh"
#include "kernels.h"

namespace escha {

// ---------------------------------------------------------------------------
// group_rows: rows (token, slot) -> RowJobs, one job per (expert, up to R rows).
// Thread e owns expert e and scans the row list twice (count, then emit), so
// rows stay in ascending order inside an expert -- the stable order
// moe.build_groups produces -- without any atomics.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
group_rows_kernel(const int32_t* __restrict__ row_expert, int m, int E, int R,
                  RowJob* __restrict__ jobs, int njobs_cap, int32_t* __restrict__ njobs_out) {
    extern __shared__ int32_t s_off[];  // [E + 1] job offsets
    const int tid = threadIdx.x;
    for (int e = tid; e < E; e += blockDim.x) {
        int c = 0;
        for (int i = 0; i < m; ++i) c += (row_expert[i] == e);
        s_off[e + 1] = (c + R - 1) / R;
    }
    if (tid == 0) s_off[0] = 0;
    __syncthreads();
    if (tid == 0)
        for (int e = 0; e < E; ++e) s_off[e + 1] += s_off[e];
    __syncthreads();
    const int total = s_off[E];
    if (tid == 0 && njobs_out) *njobs_out = total < njobs_cap ? total : njobs_cap;
    for (int e = tid; e < E; e += blockDim.x) {
        int k = 0;
        const int base = s_off[e];
        for (int i = 0; i < m; ++i) {
            if (row_expert[i] != e) continue;
            const int j = base + k / R;
            if (j < njobs_cap) {
                jobs[j].rows[k % R] = i;
                if (k % R == 0) jobs[j].expert = e;
                jobs[j].nrows = k % R + 1;  // ascending k: the last write is the count
            }
            ++k;
        }
    }
    for (int j = total + tid; j < njobs_cap; j += blockDim.x) {
        jobs[j].expert = 0;
        jobs[j].nrows = 0;
    }
}

// (rows_idx, group_expert) of moe.build_groups -> RowJobs.  Group g holds R
// slots; slots equal to n_rows are padding; expert -1 marks groups past the end.
// A group wider than 16 rows becomes ceil(R/16) jobs.
__global__ void jobs_from_groups_kernel(const int32_t* __restrict__ rows_idx,
                                        const int32_t* __restrict__ group_expert, int n_groups,
                                        int R, int n_rows, int per_group, int rows_per_job,
                                        RowJob* __restrict__ jobs) {
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= n_groups * per_group) return;
    const int g = j / per_group, sub = j - g * per_group;
    const int e = group_expert[g];
    RowJob jb;
    jb.expert = e < 0 ? 0 : e;
    jb.nrows = 0;
    if (e >= 0) {
        const int lo = sub * rows_per_job, hi = min(R, lo + rows_per_job);
        for (int s = lo; s < hi; ++s) {
            const int r = rows_idx[g * R + s];
            if (r < n_rows) jb.rows[jb.nrows++] = r;
        }
    }
    for (int s = jb.nrows; s < 16; ++s) jb.rows[s] = 0;
    jobs[j] = jb;
}

// ---------------------------------------------------------------------------
// SwiGLU on the fp16-rounded merged gate/up output (ref.py:296-301):
//   s = f16( g / (1 + exp(-g)) ) computed in f32,   h = f16( s * u )
// ---------------------------------------------------------------------------
__global__ void swiglu_kernel(const __half* __restrict__ gate, const __half* __restrict__ up,
                              int M, int I, long stride, __half* __restrict__ h) {
    grid_launch_dependents();
    grid_dependency_wait();
    const long idx = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= static_cast<long>(M) * I) return;
    const long r = idx / I, i = idx - r * I;
    const float g = __half2float(gate[r * stride + i]);
    const __half s = __float2half_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))));
    h[idx] = __hmul(s, up[r * stride + i]);
}

// ---------------------------------------------------------------------------
// Fixed slot-order combine (models/qwen3_5_moe.py:227-253):
//   y[t, c] = f16( sum_{s=0..top_k-1} f32(d16[t*top_k+s, c]) * f32(f16(score[t, s])) )
// summed in ascending slot order -- never a scatter-add.
// ---------------------------------------------------------------------------
__global__ void moe_combine_kernel(const __half* __restrict__ d16, const float* __restrict__ scores,
                                   int T, int top_k, int H, __half* __restrict__ y) {
    const long idx = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= static_cast<long>(T) * H) return;
    const long t = idx / H, c = idx - t * H;
    float acc = 0.0f;
    for (int s = 0; s < top_k; ++s) {
        const long r = t * top_k + s;
        const float w16 = __half2float(__float2half_rn(scores[r]));
        const float contrib = __fmul_rn(__half2float(d16[r * H + c]), w16);
        acc = __fadd_rn(acc, contrib);  // starts from +0 like a sum reduction
    }
    y[idx] = __float2half_rn(acc);
}

cudaError_t launch_group_rows(const int32_t* row_expert, int m, int E, int R, RowJob* jobs,
                              int njobs_cap, int32_t* njobs_out, cudaStream_t st) {
    const int threads = E >= 1024 ? 1024 : ((E + 31) / 32) * 32;
    group_rows_kernel<<<1, threads, (E + 1) * sizeof(int32_t), st>>>(row_expert, m, E, R, jobs,
                                                                     njobs_cap, njobs_out);
    return cudaGetLastError();
}

cudaError_t launch_jobs_from_groups(const int32_t* rows_idx, const int32_t* group_expert,
                                    int n_groups, int R, int n_rows, int rows_per_job,
                                    RowJob* jobs, cudaStream_t st) {
    const int per_group = (R + rows_per_job - 1) / rows_per_job;
    const int n = n_groups * per_group;
    jobs_from_groups_kernel<<<(n + 127) / 128, 128, 0, st>>>(rows_idx, group_expert, n_groups, R,
                                                            n_rows, per_group, rows_per_job, jobs);
    return cudaGetLastError();
}

cudaError_t launch_swiglu(const __half* gate, const __half* up, int M, int I, long stride,
                          __half* h, cudaStream_t st) {
    const long n = static_cast<long>(M) * I;
    return launch_chained(swiglu_kernel, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0, st,
                          gate, up, M, I, stride, h);
}

cudaError_t launch_moe_combine(const __half* d16, const float* scores, int T, int top_k, int H,
                               __half* y, cudaStream_t st) {
    const long n = static_cast<long>(T) * H;
    moe_combine_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, st>>>(d16, scores, T,
                                                                               top_k, H, y);
    return cudaGetLastError();
}

}  // namespace escha
