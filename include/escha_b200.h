/*
 * escha_b200.h -- C ABI of libescha_b200.so: the escha coded-projection hot
 * path (trellis-coded 2/3-bit weight decode fused into GEMV / small-batch GEMM /
 * expert GEMV, plus the scaled 128-block Hadamard transforms) for NVIDIA B200
 * (sm_100a).
 *
 * The reference project (EschaLabs/escha-mlx) has no compiled plugin ABI: its
 * boundary for this path is the Python function surface of escha_mlx/msl.py,
 * whose functions each launch one Metal kernel.  Every entry point below
 * replaces one of those launches; the comment gives the reference file:line.
 *
 * Conventions
 *  - All pointers are DEVICE pointers owned by the caller, 16-byte aligned,
 *    dense row-major.  The library allocates nothing.  Its only device state
 *    are two status words (raised if a bounded wait inside a kernel ever gives
 *    up) and the static scratch of escha_coded_gemv_static.
 *  - Half-precision buffers are IEEE binary16 (declared void*).
 *  - `stream` is a cudaStream_t passed as void* (NULL = default stream).  Calls
 *    only enqueue work; they never synchronise.
 *  - Return value: ESCHA_OK, or a negative code; escha_last_error() returns a
 *    thread-local description of the most recent failure on this thread.
 *    Arguments are validated on the host before any launch; the kernels
 *    themselves do no bounds checks (as in the reference, dense.py:202-209).
 *  - Code streams are uint32 [TK, TN, 8K] (dense) or [E, TK, TN, 8K]
 *    (E-stacked), TK = IC/16, TN = OC/16, K in {2, 3}: the reference's int16
 *    [.., 16K] export viewed as little-endian uint32 (msl.py:1398-1401).
 */
#ifndef ESCHA_B200_H
#define ESCHA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ESCHA_OK 0
#define ESCHA_EINVAL (-1) /* contract violation; nothing was launched */
#define ESCHA_ECUDA (-2)  /* a CUDA runtime call failed */

#define ESCHA_ABI_VERSION 1

int escha_version(void);
const char *escha_last_error(void);

/* Fill a 65,536-entry binary16 table lut[state] = decode(state) on the device.
 * Replaces ref.cba_lut()/msl._lut_array (ref.py:37-48, msl.py:1074-1076): the
 * table the *_lut kernel variants read instead of hashing. */
int escha_lut_init(void *lut, void *stream);

/* code [TK,TN,8K] -> w [IC,OC] binary16, bit-exact to ref.reconstruct.
 * lut == NULL selects the integer-hash decode, otherwise the table decode.
 * Replaces msl.decode_tiles (msl.py:1404-1421; kernel source :183-202).
 * IC and OC must be multiples of 16. */
int escha_decode_tiles(const void *code, int K, int IC, int OC, const void *lut, void *w,
                       void *stream);

/* out = f16( H128( f32(rows) * rin[e] ) * rs ),  rows [M,IC] binary16.
 * row_expert == NULL: rin is [IC]; else rin is [E,IC] and row r uses
 * rin[row_expert[r]].  Replaces msl.scaled_had / dense_scaled_had
 * (msl.py:1029-1047, :1481-1483; kernel source :875-916). */
int escha_scaled_had(const void *rows, const float *rin, const int32_t *row_expert, int M, int IC,
                     float rs, void *out, void *stream);

/* out = f16( (H128(mid) * rs) * rout[e] ),  mid [M,OC] f32.
 * Replaces msl.scaled_had_out / dense_scaled_had_out
 * (msl.py:1050-1067, :1486-1488; kernel source :919-949). */
int escha_scaled_had_out(const float *mid, const float *rout, const int32_t *row_expert, int M,
                         int OC, float rs, void *out, void *stream);

/* Two dense input transforms of the same rows in one launch.
 * Replaces msl.dense_scaled_had_pair (msl.py:1491-1504). */
int escha_scaled_had_pair(const void *rows, const float *rin0, const float *rin1, int M, int IC,
                          float rs, void *out0, void *out1, void *stream);

/* One to four dense input transforms of the same rows in one launch, each with its own
 * scale vector: rins[i] f32 [IC] -> outs[i] f16 [M, IC].  With `up` non-null the rows are the
 * gate half of a SwiGLU MLP and the transformed input is f16(f16(silu(rows)) * up)
 * (ref.py:296-301), i.e. SwiGLU fused into the down projection's input transform as in
 * _FusedMLP (models/qwen3_5.py:63-198); msl.dense_scaled_had_pair (msl.py:1491-1504) is the
 * n = 2 case.  rins / outs are HOST arrays of n device pointers. */
int escha_scaled_had_many(const void *rows, const void *up, int n, const float *const *rins,
                          void *const *outs, int M, int IC, float rs, void *stream);

/* Two dense output transforms in one launch (equal row counts).
 * Replaces msl.dense_scaled_had_out_pair (msl.py:1507-1527). */
int escha_scaled_had_out_pair(const float *mid0, const float *mid1, const float *rout0,
                              const float *rout1, int M, int OC0, int OC1, float rs, void *out0,
                              void *out1, void *stream);

/* out = H128(x) on nblocks contiguous 128-float blocks, unnormalised, f32 in
 * and out.  Replaces moe.had_blocks, i.e. mx.hadamard_transform(scale=1.0)
 * (escha_mlx/moe.py:19-27); bit-identical to ref.h128 (ref.py:204-218). */
int escha_had128(const float *x, long nblocks, float *out, void *stream);

/* int8-weight linear  y = f16( f32(x) @ f32( f16( f32(w8) * f32(scale) ) )^T ):
 * x [M,Kd] binary16, w8 [N,Kd] int8, scale [N] binary16, y [M,N] binary16,
 * Kd a multiple of 16.  Replaces EschaQ8Linear's mx.quantized_matmul call
 * (escha_mlx/quant.py:129-143) and follows ref.w8a16 (ref.py:308-311). */
int escha_w8a16(const void *x, const void *w8, const void *scale, int M, int N, int Kd, void *y,
                void *stream);

/* Up to four int8-weight linears of the SAME input rows in one launch: y[i] =
 * escha_w8a16(x, w8[i], scale[i]) for i < n, each bit-identical to its own call
 * (an output channel's sum does not depend on which launch computes it).  w8,
 * scale, N and y are HOST tables of n entries; N[i] multiples of 16, Kd a
 * multiple of 64.  The reference issues one mx.quantized_matmul per
 * EschaQ8Linear (escha_mlx/quant.py:129-143); q/k/v of an attention block read
 * the same rows, and at decode batch sizes each launch costs more than its
 * bytes. */
int escha_w8a16_many(const void *x, int n, const void *const *w8, const void *const *scale,
                     const int *N, int Kd, int M, void *const *y, void *stream);

/* Embedding lookup in an int8 table with one binary16 scale per row:
 *   out[r,:] = f16( f32(w8[ids[r],:]) * f32(scale[ids[r]]) ),  ids int64 [rows],
 * w8 [N,Kd] int8, out [rows,Kd] binary16, Kd a multiple of 16.  Replaces
 * EschaQ8Embedding's mx.dequantize of gathered rows (escha_mlx/quant.py:249-262). */
int escha_q8_embed(const int64_t *ids, const void *w8, const void *scale, int rows, int N, int Kd,
                   void *out, void *stream);

/* Per-row coded GEMV in the reference kernels' exact accumulation order
 * (bit-identical to them for a given input):
 *     mid[r,:] = f32(xh[r,:]) @ f32(decode(code[row_expert[r]]))      f32 [M,OC]
 * Replaces msl.moe_gemv / dense_gemv incl. the split-K variant
 * (msl.py:1424-1478, :1530-1538; kernel sources :205-435) and, through
 * row_map, the row-blocked forms msl.moe_gemm_rows / dense_gemm_rows[_direct]
 * (msl.py:1366-1395, :1785-1841), whose per-(row, channel) order is the same.
 *  row_expert NULL -> dense stream.   lut NULL -> hash decode.
 *  row_map NULL -> slots == M and slot s is row s; else row_map[slots] gives the
 *    row of each slot and entries >= M are padding (skipped).  splits must be 1
 *    with a row_map.
 *  splits > 1 must divide IC/16; part must then hold splits*M*OC floats and the
 *    partials are summed in ascending split order. */
int escha_gemv_ref(const void *xh, const void *code, const int32_t *row_expert,
                   const int32_t *row_map, int slots, const void *lut, int M, int IC, int OC,
                   int K, int splits, float *part, float *mid, void *stream);

/* Workspace the tensor-core GEMV needs for a given launch shape, in bytes: a
 * fixed 1 MiB counter region followed by the split-K partials (0 when
 * splits <= 1).  The caller allocates it once, zero-filled; every launch leaves
 * the counter region zero again, so one workspace serves launches of any shape
 * as long as they do not overlap on the GPU.  njobs = number of row groups
 * (escha_coded_gemv: (M + rows_per_job - 1) / rows_per_job). */
size_t escha_coded_gemv_workspace_bytes(int njobs, int OC, int splits, int rows_per_job);

/* Split policy: how many ways the kernel splits the input dimension so that the
 * grid fills the GPU (sm_count <= 0 queries the current device).  Depends only
 * on the shape and njobs, never on data, so results are reproducible. */
int escha_coded_gemv_splits(int IC, int OC, int njobs, int sm_count);

/* Tensor-core coded GEMV / small-batch GEMM for a dense stream (M >= 1 rows,
 * any M: rows are processed 8 or 16 per decode).
 *   rout == NULL: out is f32 mid [M,OC]                (msl.dense_gemv,
 *                                                        dense_gemm_rows[_direct])
 *   rout != NULL: out is binary16 y = f16((H128(mid)*rs)*rout)
 *                                                       (msl.dense_gemm_rows_direct_out,
 *                                                        msl.py:1844-1870)
 * Same product as escha_gemv_ref with a different (fixed) summation order:
 * tolerance-equal to it, bit-reproducible run to run for fixed (shape, splits).
 * splits <= 0 selects escha_coded_gemv_splits(). */
int escha_coded_gemv(const void *xh, const void *code, const float *rout, int M, int IC, int OC,
                     int K, int splits, float rs, void *workspace, size_t workspace_bytes,
                     void *out, void *stream);

/* escha_coded_gemv for callers that cannot allocate device memory and so have no
 * workspace to pass: a plugin inside a host runtime that owns all device memory
 * (a server with a pre-sized arena, a fixed memory map), a callback that must
 * not re-enter the host allocator, a loop that cannot take cudaMalloc's
 * device-wide synchronisation.  This entry point has no counterpart in the
 * reference.  Same arguments and results as escha_coded_gemv (bit-identical for
 * equal splits) minus the workspace: the split-K scratch is a static device
 * array inside the library (8 MiB of partials + 64 KiB of counters, held by every
 * GPU that loads the library until the process exits).  It allocates nothing.
 *  - Limits: 1 <= M <= 16 and splits * (OC/128) * (M <= 8 ? 8 : 16) * 512 bytes
 *    <= 8 MiB; anything larger returns ESCHA_EINVAL with a message.
 *  - The array is shared by all calls on a device and keeps the last call's
 *    contents: calls that can overlap on the GPU race; order them on one stream.
 *  - The first call on each device does a one-time set-up (resolves the array's
 *    address, clears its counters): make it before any stream capture. */
int escha_coded_gemv_static(const void *xh, const void *code, const float *rout, int M, int IC,
                            int OC, int K, int splits, float rs, void *out, void *stream);

/* General form of the tensor-core kernel: nproj (1..4) projections of the SAME
 * rows in one launch, with the transforms around the product optionally fused.
 * Replaces, per launch, one of the reference's pair/fused dispatches:
 * msl.dense_gemm_pair[_out] (msl.py:1873-1950) for gate/up and K/V, preceded by
 * msl.dense_scaled_had[_pair] (msl.py:1481-1504) when the input transform is
 * fused, and the SwiGLU stage (models/qwen3_5_moe.py:221-223) for a down
 * projection.  Every fusion is bit-identical to running the stages separately.
 *   input_mode 0: x is xh, already transformed.
 *              1: x is the raw binary16 activation; the kernel computes
 *                 xh = f16(H128(x * rin[i]) * rs) per projection i.
 *              2: as 1 on h = f16(f16(silu(x)) * x_up)  (x = gate, x_up = up).
 *   x_proj: NULL, or a host array of nproj row pointers: a non-NULL entry gives
 *     that projection its own input rows (mode 0: each projection has its own
 *     xh because each has its own rin); NULL entries use x.
 *   x_stride: elements between rows of x (and x_up); <= 0 means IC.
 *   x_row_div: output row r reads input row r / x_row_div (<= 1: the same row).
 *     With (token, slot) rows laid out token-major, top_k here replaces the
 *     xf[row_token] gather of models/qwen3_5_moe.py:112-114.
 *   code/rin/rout/out/OC: host arrays of nproj entries.  rin[i] is [IC] (or
 *     [E,IC] with jobs) and only read for input_mode != 0; rout[i] NULL makes
 *     out[i] f32 mid [M,OC[i]], otherwise out[i] is binary16 [M,OC[i]].
 *   jobs NULL: dense streams, rows 0..M-1 (njobs/rows_per_job/E ignored).
 *   jobs given: E-stacked streams indexed by each job's expert.
 *   splits: host array of nproj split factors (NULL or an entry <= 0 selects
 *     escha_coded_gemv_splits(IC, OC[i], 1)); each projection keeps the factor
 *     it has when launched alone, so a joint launch changes no output bit.
 *   workspace: escha_coded_gemv_workspace_bytes(njobs, sum(OC), max(splits),
 *     rows_per_job). */
int escha_coded_projections(const void *x, const void *const *x_proj, const void *x_up,
                            long x_stride, int x_row_div, int input_mode,
                            int nproj, const void *const *code, const float *const *rin,
                            const float *const *rout, void *const *out, const int *OC,
                            const void *jobs, int njobs, int rows_per_job, int M, int E, int IC,
                            int K, const int *splits, float rs, void *workspace,
                            size_t workspace_bytes, void *stream);

/* ---- routed experts (E-stacked streams) ---------------------------------- */

/* A row job: up to 16 rows that read the same expert's stream.  Plain int32
 * record, ESCHA_ROW_JOB_INTS words: {expert, nrows, rows[16]}. */
#define ESCHA_ROW_JOB_INTS 18

/* Upper bound on the number of jobs escha_moe_group_rows can emit for m rows
 * over E experts with R rows per job: (m + min(m,E)*(R-1)) / R. */
int escha_moe_jobs_bound(int m, int E, int R);

/* Group m (token, slot) rows by expert into row jobs of at most R rows
 * (R = 8 or 16), rows ascending inside an expert; jobs past the last real one
 * get nrows = 0.  jobs must hold njobs_cap records; njobs_out (optional) gets
 * the real count.  Device-resident replacement for moe.build_groups
 * (escha_mlx/moe.py:30-78) -- same stable order, no padding rows. */
int escha_moe_group_rows(const int32_t *row_expert, int m, int E, int R, void *jobs,
                         int njobs_cap, int32_t *njobs_out, void *stream);

/* Convert the (rows_idx [n_groups*R], group_expert [n_groups]) form that
 * moe.build_groups returns (padding slots == n_rows, expert -1 past the end)
 * into row jobs; emits n_groups * ceil(R / rows_per_job) records. */
int escha_jobs_from_groups(const int32_t *rows_idx, const int32_t *group_expert, int n_groups,
                           int R, int n_rows, int rows_per_job, void *jobs, void *stream);

/* Tensor-core expert GEMV over row jobs: for every job, rows read
 * code[job.expert]; rout (if given) is [E,OC] and indexed by job.expert.
 * xh is [M,IC], out is [M,OC] (f32 mid, or binary16 y when rout != NULL); rows
 * no job names are left untouched.  Replaces msl.moe_gemv with a row_expert
 * and msl.moe_gemm_rows (msl.py:1366-1395, :1424-1478).  splits must be >= 1
 * (use escha_coded_gemv_splits with the expected job count); workspace as
 * escha_coded_gemv_workspace_bytes(njobs, OC, splits, rows_per_job). */
int escha_coded_gemv_jobs(const void *xh, const void *code, const float *rout, const void *jobs,
                          int njobs, int rows_per_job, int M, int E, int IC, int OC, int K,
                          int splits, float rs, void *workspace, size_t workspace_bytes, void *out,
                          void *stream);

/* h[r,i] = f16( f16(silu(g)) * u ), g = gate[r*stride+i], u = up[r*stride+i]
 * (binary16; 2-byte aligned pointers suffice).  For the merged [M,2I] layout
 * pass gate = gu, up = gu + I, stride = 2I; for two separate [M,I] tensors
 * stride = I.  Replaces the elementwise stage at models/qwen3_5_moe.py:221-223
 * (ref.swiglu, ref.py:296-301). */
int escha_swiglu(const void *gate, const void *up, int M, int I, long stride, void *h,
                 void *stream);

/* y[t,:] = f16( sum over slots s, ascending, of f32(d16[t*top_k+s,:]) *
 * f32(f16(scores[t*top_k+s])) ) -- the fixed-order combine at
 * models/qwen3_5_moe.py:227-253 (never a scatter-add). */
int escha_moe_combine(const void *d16, const float *scores, int T, int top_k, int H, void *y,
                      void *stream);

/* The MoE block's router and row grouping in one launch.  Replaces, for x [T,H]
 * binary16: the gate linear + top-k + softmax of EschaSparseMoeBlock.__call__
 * (models/qwen3_5_moe.py:255-262; ref.py:326-331: f32 logits rounded once through
 * binary16, k largest with ties to the lower expert index, softmax over those k),
 * the shared expert's gate logit f32(f16(x . shg_w)) (models/qwen3_5_moe.py:268),
 * and moe.build_groups (moe.py:30-83) as RowJobs for escha_coded_gemv_jobs /
 * escha_coded_projections.
 *   gate_w [E,H] binary16, shg_w [H] binary16 or NULL (then no gate logit).
 *   ids_in NULL: ids [T,top_k] int32 and scores [T,top_k] f32 are written;
 *     logits_scratch is T*E floats of scratch.  ids_in given (routing decided by
 *     the caller): gate_w/ids/scores/logits_scratch are ignored.
 *   jobs NULL skips the grouping; otherwise rows (t*top_k+s) whose expert lies in
 *     [e_lo, e_hi) -- this rank's shard under expert parallelism, [0,E) otherwise
 *     -- are grouped under the local expert index e - e_lo, rows_per_job (8 or 16)
 *     per job, njobs_cap >= escha_moe_jobs_bound(T*top_k, e_hi-e_lo, rows_per_job).
 *   workspace: the zero-initialised split-K workspace (>= 1 MiB); its last counter
 *     is used and left zero.
 * Limits: E <= 1024, top_k <= 16, H a multiple of 8. */
int escha_moe_route(const void *x, const void *gate_w, const void *shg_w, const int32_t *ids_in,
                    int T, int H, int E, int top_k, int e_lo, int e_hi, int rows_per_job,
                    int32_t *ids, float *scores, float *shared_gate_logit, float *logits_scratch,
                    void *jobs, int njobs_cap, void *workspace, size_t workspace_bytes,
                    void *stream);

/* The MoE block's tail in one launch (models/qwen3_5_moe.py:227-273; ref.py:333-349):
 *   hh      = f16( (g * sigmoid(g)) * u ),  g, u = gu[t, :I], gu[t, I:]   (f32 math)
 *   sh      = w8a16(hh, w8, scale)                       shared expert's down linear
 *   routed  = f16( sum over slots s ascending of f32(d16[t*top_k+s,:]) * f32(f16(scores)) )
 *   out[t,:] = f16( f32(routed) + f32(sh) * sigmoid(shared_gate_logit[t]) )
 * gu [T,2I] binary16 (the shared expert's gate and up outputs side by side),
 * w8 [H,I] int8, scale [H] binary16, d16 [T*top_k,H] binary16, out [T,H] binary16.
 * Expert parallel (no reference counterpart): with ids [T*top_k] given, d16 is the
 * all-gathered [ranks, T*top_k, H] buffer and row r is read from the copy of rank
 * ids[r] / experts_per_rank, the one that computed it; rows a rank does not own are
 * never read, so they need not be initialised.  ids NULL: a single [T*top_k,H] buffer.
 * H a multiple of 16, I a multiple of 64. */
int escha_moe_shared_finish(const void *gu, const void *w8, const void *scale, const void *d16,
                            const int32_t *ids, int experts_per_rank, const float *scores,
                            const float *shared_gate_logit, int T, int top_k, int H, int I,
                            void *out, void *stream);

/* escha_coded_projections with the all-gather that follows it under multi-GPU
 * sharding fused into the kernel's epilogue (no counterpart in the reference, which
 * is single-device).  Arguments as escha_coded_projections, plus: each output out[i]
 * is a gathered buffer of rows of out_ld[i] elements in which this rank's OC[i]
 * columns start at out_col0[i]; peer_out (host table of nproj*npeers device
 * pointers, peer g of projection i at [i*npeers+g]) holds the same buffer of every
 * other GPU, mapped into this process (CUDA IPC / symmetric memory).  The epilogue
 * stores each 128-channel block of each output row into out[i] and into every peer
 * with plain stores over NVLink, then fences system-wide.
 *   split-N tensor parallelism (dense streams): out_ld = OC_total, out_col0 = rank's
 *     first column -- every rank ends up with the whole row;
 *   expert parallelism (row jobs): out_ld = OC, out_col0 = 0 -- a rank's jobs cover
 *     only the rows of its experts, rows are disjoint across ranks, and every rank
 *     ends up with all rows.
 * Follow the launch with escha_peer_barrier on every rank before anyone reads its
 * buffer, and do not overwrite a buffer until a later barrier has passed
 * (double-buffer across steps).  npeers <= 7; out_ld, out_col0 multiples of 8. */
int escha_coded_projections_gather(const void *x, const void *const *x_proj, const void *x_up,
                                   long x_stride, int x_row_div, int input_mode, int nproj,
                                   const void *const *code, const float *const *rin,
                                   const float *const *rout, void *const *out, const int *OC,
                                   const void *jobs, int njobs, int rows_per_job, int M, int E,
                                   int IC, int K, const int *splits, float rs, void *workspace,
                                   size_t workspace_bytes, void *const *peer_out, int npeers,
                                   const int *out_ld, const int *out_col0, void *stream);

/* Barrier between the GPUs of a node over peer-mapped flag words (no reference
 * counterpart).  local_flags: this rank's nranks+2 int32 words, zero-initialised
 * once, in memory the other ranks can write; peer_flags: host array of nranks
 * device pointers, entry r = rank r's flag words mapped here (own entry ignored).
 * One small kernel per rank: it announces a new epoch to every peer (release,
 * system scope, after a system-wide fence) and polls until every peer has
 * announced it.  The poll is bounded (about two seconds); if a peer never arrives
 * word nranks+1 of local_flags is set to 1 and the kernel returns.  Ranks must run
 * on different GPUs.  Identical launch every time: CUDA-graph replayable. */
int escha_peer_barrier(int32_t *local_flags, int32_t *const *peer_flags, int rank, int nranks,
                       void *stream);

/* Prefill form of the coded product on the tcgen05 tensor cores, for tens to
 * hundreds of rows:  mid[r,:] = f32(xh[r,:]) @ f32(decode(code)),  f32 [M,OC].
 * Replaces msl.dense_gemm_mat and the row-blocked msl.dense_gemm_rows at prefill
 * sizes (msl.py:1608-1782, :1785-1841): every weight is decoded once per 256 rows
 * into tensor memory as binary16 (the A operand of tcgen05.mma; into a shared-memory
 * ring with ESCHA_B200_TC_WEIGHTS=smem) and contracted with fp32 accumulators in
 * tensor memory.  Reassociated like dense_gemm_mat, deterministic:
 * tolerance-equal to escha_gemv_ref, bit-reproducible for fixed (shape, splits).
 *   xh [M,IC] binary16 (already input-transformed), code [IC/16, OC/16, 8K].
 *   rout == NULL: out is f32 mid [M,OC];  rout != NULL: out is binary16
 *     y = f16((H128(mid)*rs)*rout), the split-order sum and the output transform
 *     (msl.dense_scaled_had_out, ref.py:226-228) running as one second kernel.
 *     With splits == 1 the transform runs in the GEMM's own epilogue instead, and with
 *     2..4 splits the splits of an output block run as a thread-block cluster that sums
 *     them in split order through distributed shared memory and transforms (same bits).
 *   splits <= 0 selects escha_coded_gemm_tc_splits().  `planes` is scratch of
 *     splits*M*OC floats, needed when splits > 1. */
int escha_coded_gemm_tc(const void *xh, const void *code, const float *rout, int M, int IC, int OC,
                        int K, int splits, float rs, float *planes, void *out, void *stream);

/* Split policy of escha_coded_gemm_tc (shape only; sm_count <= 0 queries the device). */
int escha_coded_gemm_tc_splits(int IC, int OC, int sm_count);

/* 1 if escha_coded_gemm_tc with these arguments will use the `planes` scratch, 0 if it sums its
 * splits inside the kernel (or is unsplit): lets a caller skip the allocation.  The reference's
 * matrix-unit GEMM has no split scratch (msl.py:1608-1782 accumulates in one threadgroup). */
int escha_coded_gemm_tc_needs_planes(int IC, int splits, int has_rout);

/* One to three prefill projections of equal IC and K in ONE tcgen05 launch (Q/K/V), each with
 * its own transformed activations xhs[i] f16 [M, IC], code, transform vector routs[i] f32 [OCs[i]]
 * (required) and f16 output outs[i] [M, OCs[i]].  splits <= 0 picks the policy value for the
 * summed width; with splits > 1, planes[i] is an f32 workspace of splits * M * OCs[i].
 * The reference dispatches the pair form of this (dense_gemm_pair_out, msl.py:1880-1950) for
 * gate/up and K/V; here it also removes two launches whose fixed cost exceeds their work.
 * xhs, codes, routs, planes, outs are HOST arrays of n device pointers, OCs a host int array. */
int escha_coded_gemm_tc_many(int n, const void *const *xhs, const void *const *codes,
                             const float *const *routs, int M, int IC, const int *OCs, int K,
                             int splits, float rs, float *const *planes, void *const *outs,
                             void *stream);

/* 0 if no tensor-core GEMM launch on the current device has given up a bounded wait
 * since the library was loaded; synchronises the device.  For tests and diagnostics. */
int escha_coded_gemm_tc_status(void);

/* escha_coded_projections[_gather] for projections of DIFFERENT rates: Ks[i] in {2, 3} is
 * projection i's bits per weight; up to 8 projections of the same input rows and IC share the
 * launch (with npeers == 0, peer_out / out_ld / out_col0 may be NULL).  Every projection keeps
 * the split factor it has when launched alone, so a joint launch changes no output bit.  The
 * reference fuses the projections that share an input at module level (_FusedAttention q/k/v,
 * _FusedMLP gate/up, escha_mlx/models/qwen3_5.py:63-198; pair kernels msl.py:1880-1950) but
 * needs one kernel name per rate; here one persistent launch walks a work list over all of
 * them, so e.g. 2-bit attention projections and 3-bit MLP projections of one hidden state
 * cost one ramp-up and one tail. */
int escha_coded_projections_mixed(const void *x, const void *const *x_proj, const void *x_up,
                                  long x_stride, int x_row_div, int input_mode, int nproj,
                                  const void *const *code, const float *const *rin,
                                  const float *const *rout, void *const *out, const int *OC,
                                  const int *Ks, const void *jobs, int njobs, int rows_per_job,
                                  int M, int E, int IC, const int *splits, float rs,
                                  void *workspace, size_t workspace_bytes,
                                  void *const *peer_out, int npeers, const int *out_ld,
                                  const int *out_col0, void *stream);

/* 0 if no coded GEMV launch (escha_coded_gemv, escha_coded_projections[_gather],
 * escha_coded_gemv_jobs, escha_coded_gemv_static) on the current device has given up a
 * bounded wait since the last call; reading clears it; synchronises the device.  The
 * reference's kernels cannot report such a condition (msl.py launches have no status);
 * here every wait inside a kernel is bounded and a kernel that gives up returns, leaves
 * its outputs undefined and raises this word.  After a nonzero status zero the first
 * 1 MiB of the workspace the launch used before using it again. */
int escha_coded_gemv_status(void);

/* Test hook for the status path above, no counterpart in the reference.  on != 0: from
 * now on GEMV launches announce their weight copies without issuing them and give every
 * bounded wait `limit` tries of about a microsecond, so the waits run out, the kernel
 * returns and escha_coded_gemv_status() reports it; nothing faults and the device stays
 * usable.  on == 0 restores normal operation. */
void escha_debug_gemv_stall(int on, unsigned limit);

/* The same hook for the tensor-memory prefill GEMM (escha_coded_gemm_tc[_many] in its
 * default form): weight copies are announced and not issued, every bounded wait of the
 * kernel gets `limit` tries of about a microsecond, all roles run out of patience, meet at
 * the CTA barrier, free their tensor memory and return; escha_coded_gemm_tc_status()
 * reports it (that word is not cleared by reading: use a process of its own). */
void escha_debug_gemm_tc_stall(int on, unsigned limit);

/* Test hook, no counterpart in the reference: the number of polls (about 100 ns apart) an
 * escha_peer_barrier launch makes for a peer before it gives up, raises word nranks+1 of
 * local_flags (see escha_peer_barrier) and returns; 0 restores the default
 * (about two seconds).  Lets a test watch the barrier give up on a peer that never arrives. */
void escha_debug_peer_poll_limit(unsigned polls);

#ifdef __cplusplus
}
#endif
#endif /* ESCHA_B200_H */
