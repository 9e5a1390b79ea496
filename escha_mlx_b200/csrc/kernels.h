// Internal launcher declarations shared by the .cu files and the C-ABI layer.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

namespace escha {

// Dynamic shared memory limit of one kernel, raised at most once per device and size.  The
// launchers keep one of these per kernel instantiation; check and update happen under its
// lock, so host threads launching on different streams cannot leave the attribute below the
// size another thread has recorded.
struct SmemLimit {
    std::mutex mu;
    size_t have[64] = {0};
    template <class Kernel>
    cudaError_t ensure(Kernel kernel, size_t smem) {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        std::lock_guard<std::mutex> lock(mu);
        if (dev >= 0 && dev < 64 && smem <= have[dev]) return cudaSuccess;
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem));
        if (e == cudaSuccess && dev >= 0 && dev < 64) have[dev] = smem;
        return e;
    }
};


// One unit of row work for the tensor-core GEMV: up to 16 rows that share one
// code stream (one expert).  Built on the device by the grouping kernel for the
// MoE path; implicit (rows z*R .. z*R+R-1, expert 0) for a dense linear.
struct RowJob {
    int32_t expert;
    int32_t nrows;
    int32_t rows[16];
};

constexpr int kMaxProblems = 8;
constexpr int kMaxPeers = 7;   // other GPUs of an 8-GPU node

// One projection inside a (possibly multi-projection) launch.  All projections
// of a launch share the input rows; each has its own stream, vectors, output and,
// in the persistent kernel, its own rate and input width.
struct GemvProblem {
    const uint32_t* code;   // [E?, TK, TN, 8K]
    const __half* x;        // this projection's own input rows, or nullptr for the shared ones
    const float* rin;      // [E?, IC]; read only when the input transform is fused
    const float* rout;      // nullptr -> write f32 mid; else [E?, OC] and write f16 y
    void* out;              // f32 [M, OC] or f16 [M, OC]
    int OC;
    int ocb0;               // index of this projection's first 128-channel block in the grid
    int splits;             // split-K factor of this projection (<= GemvMmaParams::splits)
    // Filled in by the launcher: rate and input width of this projection (the launch-wide
    // K / IC when the caller left them 0), its first index in the launch's item list, and how
    // many consecutive output blocks one item covers (they share one staging of the rows).
    int K, IC, item0, opi;
    // ceil(2^40 / d) for d = splits and d = output-block groups: item index -> (job, group,
    // split) without integer division in the kernel (exact for indices below 2^24)
    unsigned long long magic_s, magic_g;
    int ngroups;
    int bbase, brem;        // input blocks per split: bbase, the first brem splits one more
    // Output placement.  out_ld = elements between output rows (0: OC), out_col0 = this
    // projection's first column inside a row.  peer[0..npeer) are the SAME buffer mapped
    // from other GPUs: the epilogue stores its block there too, so that a split-N shard
    // lands in every rank's gathered [M, OC_total] row without a separate all-gather.
    int out_ld, out_col0, npeer;
    void* peer[kMaxPeers];
};

enum GemvInput : int {
    kInputTransformed = 0,  // x is xh = f16(H128(x * rin) * RS), ready for the product
    kInputRaw = 1,          // x is the raw f16 activation; the kernel applies rin, H128, RS
    kInputSwiglu = 2,       // raw input is f16(f16(silu(x)) * x_up); then as kInputRaw
};

// How a launch uses programmatic dependent launch (the next kernel of a stream is
// scheduled while the previous one drains).
enum GemvPdl : int {
    kPdlOff = 0,        // ordinary stream order
    kPdlWaitFirst = 1,  // early scheduling only: every thread waits for the previous kernel first
    kPdlPrefetch = 2,   // dense launches also stream weights before that wait
};

struct GemvMmaParams {
    GemvProblem prob[kMaxProblems];
    int nprob;
    int total_ocb;            // grid.x
    const __half* x;          // [*, x_stride]
    const __half* x_up;       // second operand for kInputSwiglu
    long x_stride;            // elements between consecutive rows of x / x_up
    int x_row_div;            // output row r reads input row r / x_row_div (top_k for the
                              // first expert leg, where rows are (token, slot) pairs); >= 1
    const RowJob* jobs;       // nullptr -> dense implicit jobs
    float* part;              // split-K partials (unused when splits == 1)
    int32_t* counters;        // one per (job, output block); zero on entry, zero on exit
    int M, IC, K;
    int splits;               // grid.y: the largest per-projection split factor
    int rows_per_job;         // 8 or 16
    int njobs;                // grid.z
    int input;                // GemvInput
    int xcb;                  // activation blocks staged per chunk (set by the launcher)
    int ocb_group;            // output blocks per CTA in the one-CTA-per-block kernel (launcher)
    int pdl;                  // GemvPdl (set by the launcher)
    // Persistent kernel only (set by the launcher): length of the item list, code-ring depth
    // and slot size in words, rows an activation buffer holds.
    int total_items, nstages, slot_words, xrows;
    // Two int32 in the caller's workspace (zero on entry, zero on exit): the next item index
    // beyond the first wave, and the number of CTAs that ran out of items.  nullptr: items
    // are taken by block stride instead.
    int32_t* sched;
    // Tries (of about a microsecond) a bounded wait makes before it gives up.
    uint32_t wait_limit;
    // Test hook: the producer announces its copies but does not issue them, so the decode
    // warps' bounded waits run out and the kernel reports it through the status word.
    int test_stall;
    float rs;
    // codebook constants 0x8FFF8FFF / 0x3B603B60, passed as run-time values so the
    // decode's (p & mask) ^ x stays a single three-input logic instruction
    uint32_t hash_mask, hash_xor;
    // 2^k multipliers {2, 4, 16, 32, 64, 128}: shifts issued as multiplies (see common.cuh)
    uint32_t mul2, mul4, mul16, mul32, mul64, mul128;
};

// Router + grouping launch (route.cu).
struct RouteParams {
    const __half* x;         // [T, H]
    const __half* gate_w;    // [E, H]; unused when ids_in is given
    const __half* shg_w;     // [H] shared expert's gate vector, or nullptr
    const int32_t* ids_in;   // [T, top_k] routing decided by the caller, or nullptr
    int T, H, E, top_k;
    int e_lo, e_hi;          // this rank's experts; rows of other experts get no job
    int R;                   // rows per job (8 or 16)
    int32_t* ids;            // out [T, top_k] (unused with ids_in)
    float* scores;           // out [T, top_k] (unused with ids_in)
    float* slog;             // out [T] f32(f16(x . shg_w)) (unused without shg_w)
    float* logits;           // scratch [T, E] f32 (unused with ids_in)
    RowJob* jobs;            // out [njobs_cap], or nullptr to skip the grouping
    int njobs_cap;
    int32_t* counter;        // one int32, zero on entry, zero on exit
};

enum Q8Input : int { kQ8InputPlain = 0, kQ8InputSwiglu = 1 };
enum Q8Store : int { kQ8StorePlain = 0, kQ8StoreGatedAdd = 1 };

// int8 linear launch (w8a16_mma.cu).
struct Q8Params {
    const __half* x;          // [M, Kd], or the merged gate/up rows [M, 2 Kd] for kQ8InputSwiglu
    const int8_t* w8;         // [N, Kd]
    const __half* scale;      // [N]
    __half* y;                // [M, N]
    int M, N, Kd;
    int input, epilogue;
    // kQ8StoreGatedAdd only:
    const __half* d16;        // [M * top_k, N] expert outputs, (token, slot) rows token-major;
                              // with ids: [ranks, M * top_k, N], row r taken from its owner's copy
    const int32_t* ids;       // [M * top_k] routed expert of each row, or nullptr
    int experts_per_rank;     // owner of row r = ids[r] / experts_per_rank
    const float* scores;      // [M * top_k]
    const float* gate_logit;  // [M]
    int top_k;
    // several linears of one input in one launch (plain input and store only): nseg > 0 makes
    // blockIdx.x pick its segment from blk0 (16-row blocks before each segment, ascending)
    int nseg;
    const int8_t* seg_w8[4];
    const __half* seg_scale[4];
    __half* seg_y[4];
    int seg_N[4];
    int blk0[5];
};

cudaError_t launch_lut_init(__half* lut, cudaStream_t st);
cudaError_t launch_decode_tiles(const uint32_t* code, int K, int IC, int OC, const __half* lut,
                                __half* w, cudaStream_t st);
cudaError_t launch_scaled_had_many(const __half* rows, const __half* up, int n,
                                   const float* const* rins, __half* const* outs, int M, int dim,
                                   float rs, cudaStream_t st);
cudaError_t launch_scaled_had(bool output, const void* src0, const float* vec0, __half* out0,
                              int dim0, const void* src1, const float* vec1, __half* out1,
                              int dim1, const int32_t* row_expert, int M, float rs,
                              cudaStream_t st);
cudaError_t launch_gemv_ref(const __half* xh, const uint32_t* code, const int32_t* row_expert,
                            const int32_t* row_map, int slots, const __half* lut, float* out,
                            float* part, int M, int IC, int OC, int K, int splits,
                            cudaStream_t st);
cudaError_t launch_gemv_mma(const GemvMmaParams& p, cudaStream_t st);
// The persistent form of the same kernel (gemv_stream.cu); launch_gemv_mma routes to it
// unless ESCHA_B200_GEMV_KERNEL=grid.
cudaError_t launch_gemv_stream(const GemvMmaParams& p, cudaStream_t st);
// Status word of the persistent kernel: nonzero after a bounded wait gave up; cleared on read.
cudaError_t gemv_stream_status(int* host_status);
// Test hook: from now on launches make their producers announce copies without issuing
// them and give every bounded wait `limit` tries (0 restores normal operation).
void gemv_stream_test_stall(int on, unsigned limit);
// the current values of that hook (limit: the default when the hook is off)
void gemv_test_hooks(int* stall, unsigned* limit);
// Status word of the one-CTA-per-block kernel (gemv_mma.cu), same convention.
cudaError_t gemv_mma_status(int* host_status);
cudaError_t launch_group_rows(const int32_t* row_expert, int m, int E, int R, RowJob* jobs,
                              int njobs_cap, int32_t* njobs_out, cudaStream_t st);
cudaError_t launch_jobs_from_groups(const int32_t* rows_idx, const int32_t* group_expert,
                                    int n_groups, int R, int n_rows, int rows_per_job,
                                    RowJob* jobs, cudaStream_t st);
cudaError_t launch_swiglu(const __half* gate, const __half* up, int M, int I, long stride,
                          __half* h, cudaStream_t st);
cudaError_t launch_moe_combine(const __half* d16, const float* scores, int T, int top_k, int H,
                               __half* y, cudaStream_t st);
cudaError_t launch_had128(const float* x, float* out, long nblocks, cudaStream_t st);
cudaError_t launch_w8a16(const __half* x, const int8_t* w8, const __half* scale, __half* y, int M,
                         int N, int Kd, cudaStream_t st);
cudaError_t launch_q8_embed(const int64_t* ids, const int8_t* w8, const __half* scale, __half* out,
                            int rows, int N, int Kd, cudaStream_t st);
size_t gemv_mma_part_floats(int njobs, int splits, int total_ocb, int rows_per_job);

// Used by the entry point that carries its own scratch (noalloc.cu): record an
// error message for escha_last_error(), and launch the dense single-projection
// GEMV with explicit counter / partial pointers.  Returns an ESCHA_* code.
void set_last_error(const char* msg);
int coded_gemv_with_scratch(const void* xh, const void* code, const float* rout, int M, int IC,
                            int OC, int K, int splits, float rs, int32_t* counters, float* part,
                            void* out, void* stream);

// Prefill coded GEMM on tcgen05 (gemm_tc.cu): out[split][M][OC] f32 partial products.
struct GemmTcParams {
    const uint32_t* code;   // [IC/16, OC/16, 8K]
    const __half* xh;       // [M, IC] transformed activations
    float* out;             // [splits, M, OC]
    // splits == 1 and rout given: the epilogue runs the output transform itself and writes
    // y16 = f16((H128(mid) * rs) * rout) instead of the f32 plane
    const float* rout;      // [OC] or nullptr
    __half* y16;            // [M, OC]
    float rs;
    int M, IC, OC, K, splits;
    uint32_t hash_mask, hash_xor;
    uint32_t mul2, mul4, mul16, mul32, mul64, mul128;
    // Up to two more projections of the same IC and K in the same launch (Q/K/V), each with its
    // own activations (tensor map), code, outputs; column blocks from cb0 on belong to it.
    // Only the tensor-memory kernel reads these.
    struct More {
        const uint32_t* code;
        float* out;
        const float* rout;
        __half* y16;
        int OC, cb0;
    };
    int nproj;      // 0 or 1: just the projection above
    More more[2];
    // set by the launcher: tries of about a microsecond every bounded wait gets, and the test
    // hook that announces the weight copies without issuing them (so that the waits run out)
    uint32_t wait_limit;
    int test_stall;
};
cudaError_t launch_gemm_tc(const GemmTcParams& p, cudaStream_t st);
cudaError_t launch_planes_out(const float* planes, const float* rout, __half* y, int M, int OC,
                              int splits, float rs, cudaStream_t st);
cudaError_t launch_planes_out_many(int n, const float* const* planes, const float* const* routs,
                                   __half* const* ys, const int* OCs, int M, int splits, float rs,
                                   cudaStream_t st);
cudaError_t launch_sum_planes(const float* planes, float* mid, size_t n, int splits, cudaStream_t st);
cudaError_t gemm_tc_status(int* host_status);
void gemm_tcm_test_stall(int on, unsigned limit);
// the same product with the decoded weights handed over through tensor memory (gemm_tcm.cu)
bool gemm_tcm_supports(const GemmTcParams& p);
bool gemm_tcm_cluster_sum(int IC, int splits);
// whether launch_gemm_tc would take the tensor-memory kernel at all (environment switch)
bool gemm_tc_uses_tmem();
cudaError_t launch_gemm_tcm(const GemmTcParams& p, cudaStream_t st);
// the same for p.nproj projections; xh_more[i] are the activations of p.more[i]
cudaError_t launch_gemm_tcm_many(const GemmTcParams& p, const __half* const* xh_more, cudaStream_t st);
cudaError_t gemm_tcm_status(int* host_status);

// Cross-GPU barrier over peer-mapped flag words (peer.cu).
struct PeerBarrierParams {
    int32_t* local;              // this GPU's flags: [nranks] arrivals, [nranks] epoch, [nranks+1] status
    int32_t* peer[kMaxPeers + 1];  // every rank's flags (index = rank; own entry unused)
    int rank, nranks;
};
cudaError_t launch_peer_barrier(const PeerBarrierParams& p, cudaStream_t st);
// Test hook: polls a barrier launch makes before it gives up (0 restores the default).
void peer_barrier_poll_limit(unsigned polls);

cudaError_t launch_moe_route(const RouteParams& p, cudaStream_t st);
size_t route_shared_bytes(int T, int top_k, int e_lo, int e_hi);
bool w8a16_mma_supports(int N, int Kd);
cudaError_t launch_w8a16_mma(const Q8Params& p, cudaStream_t st);

}  // namespace escha
