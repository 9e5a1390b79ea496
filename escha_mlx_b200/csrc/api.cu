// extern "C" boundary of libescha_b200.so: argument validation, error
// reporting and dispatch to the kernel launchers.  Declarations and the
// reference call each one replaces are in include/escha_b200.h.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>

#include "../../include/escha_b200.h"
#include "kernels.h"

namespace {

thread_local std::string g_err;

int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_err = buf;
    return code;
}

int cuda_result(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return ESCHA_OK;
    return fail(ESCHA_ECUDA, "%s: %s", what, cudaGetErrorString(e));
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

#define REQUIRE_PTR(p)                                                                  \
    do {                                                                                \
        if ((p) == nullptr) return fail(ESCHA_EINVAL, "%s: %s is NULL", __func__, #p);  \
        if (!aligned16(p)) return fail(ESCHA_EINVAL, "%s: %s is not 16-byte aligned", __func__, #p); \
    } while (0)
#define OPTIONAL_PTR(p)                                                                 \
    do {                                                                                \
        if ((p) != nullptr && !aligned16(p))                                            \
            return fail(ESCHA_EINVAL, "%s: %s is not 16-byte aligned", __func__, #p);   \
    } while (0)
#define REQUIRE(cond, ...)                                   \
    do {                                                     \
        if (!(cond)) return fail(ESCHA_EINVAL, __VA_ARGS__); \
    } while (0)

int check_shape(const char* fn, int K, int IC, int OC, int mult) {
    if (K != 2 && K != 3)
        return fail(ESCHA_EINVAL, "%s: K=%d; this runtime implements K in [2, 3]", fn, K);
    if (IC <= 0 || OC <= 0 || IC % mult || OC % mult)
        return fail(ESCHA_EINVAL, "%s: dimensions must be positive multiples of %d, got %dx%d", fn,
                    mult, IC, OC);
    return ESCHA_OK;
}

cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }

// The workspace starts with a fixed-size counter region (one int32 per (job,
// output block)); split-K partials follow it.  Keeping the boundary fixed means
// memory that ever holds partials is never read as a counter, so the "counters
// are zero between launches" invariant survives launches of different shapes
// sharing one workspace.
constexpr size_t kCounterBytes = size_t(1) << 20;
constexpr size_t kMaxCounters = kCounterBytes / sizeof(int32_t);
// escha_moe_route's counters (one per tile of 8 tokens + one) at the end of the region
constexpr size_t kRouteTiles = 4096;
constexpr size_t kRouteCounters = kRouteTiles + 1;
// the persistent GEMV's two scheduling words sit just below them
constexpr size_t kSchedCounters = 2;
constexpr size_t kSchedIndex = kMaxCounters - kRouteCounters - kSchedCounters;

}  // namespace

namespace escha {

void set_last_error(const char* msg) { g_err = msg; }

int coded_gemv_with_scratch(const void* xh, const void* code, const float* rout, int M, int IC,
                            int OC, int K, int splits, float rs, int32_t* counters, float* part,
                            void* out, void* stream) {
    if (int rc = check_shape(__func__, K, IC, OC, 128)) return rc;
    REQUIRE(M >= 1 && M <= 16, "%s: M=%d outside [1, 16]", __func__, M);
    REQUIRE(splits >= 1 && splits <= IC / 128, "%s: splits=%d outside [1, %d]", __func__, splits,
            IC / 128);
    REQUIRE_PTR(xh);
    REQUIRE_PTR(code);
    REQUIRE_PTR(out);
    OPTIONAL_PTR(rout);
    REQUIRE_PTR(counters);
    REQUIRE_PTR(part);
    GemvMmaParams p{};
    p.prob[0].code = static_cast<const uint32_t*>(code);
    p.prob[0].rout = rout;
    p.prob[0].out = out;
    p.prob[0].OC = OC;
    p.prob[0].ocb0 = 0;
    p.prob[0].splits = splits;
    p.nprob = 1;
    p.total_ocb = OC / 128;
    p.x = static_cast<const __half*>(xh);
    p.x_stride = IC;
    p.x_row_div = 1;
    p.M = M; p.IC = IC; p.K = K;
    p.splits = splits;
    p.rows_per_job = M <= 8 ? 8 : 16;
    p.njobs = 1;
    p.input = kInputTransformed;
    p.rs = rs;
    p.hash_mask = 0x8FFF8FFFu;
    p.hash_xor = 0x3B603B60u;
    p.mul2 = 2u; p.mul4 = 4u; p.mul16 = 16u; p.mul32 = 32u; p.mul64 = 64u; p.mul128 = 128u;
    p.counters = counters;
    p.part = part;
    return cuda_result(launch_gemv_mma(p, as_stream(stream)), "escha_coded_gemv_static");
}

}  // namespace escha

extern "C" {

int escha_version(void) { return ESCHA_ABI_VERSION; }

const char* escha_last_error(void) { return g_err.c_str(); }

int escha_lut_init(void* lut, void* stream) {
    REQUIRE_PTR(lut);
    return cuda_result(escha::launch_lut_init(static_cast<__half*>(lut), as_stream(stream)),
                       "escha_lut_init");
}

int escha_decode_tiles(const void* code, int K, int IC, int OC, const void* lut, void* w,
                       void* stream) {
    if (int rc = check_shape(__func__, K, IC, OC, 16)) return rc;
    REQUIRE_PTR(code);
    REQUIRE_PTR(w);
    OPTIONAL_PTR(lut);
    REQUIRE(IC / 16 <= 65535, "%s: IC=%d exceeds the launch grid", __func__, IC);
    return cuda_result(
        escha::launch_decode_tiles(static_cast<const uint32_t*>(code), K, IC, OC,
                                   static_cast<const __half*>(lut), static_cast<__half*>(w),
                                   as_stream(stream)),
        "escha_decode_tiles");
}

int escha_scaled_had(const void* rows, const float* rin, const int32_t* row_expert, int M, int IC,
                     float rs, void* out, void* stream) {
    REQUIRE(M >= 1, "%s: needs at least one row, got M=%d", __func__, M);
    REQUIRE(IC > 0 && IC % 128 == 0, "%s: Hadamard dimension must be divisible by 128, got %d",
            __func__, IC);
    REQUIRE_PTR(rows);
    REQUIRE_PTR(rin);
    REQUIRE_PTR(out);
    return cuda_result(
        escha::launch_scaled_had(false, rows, rin, static_cast<__half*>(out), IC, nullptr, nullptr,
                                 nullptr, 0, row_expert, M, rs, as_stream(stream)),
        "escha_scaled_had");
}

int escha_scaled_had_out(const float* mid, const float* rout, const int32_t* row_expert, int M,
                         int OC, float rs, void* out, void* stream) {
    REQUIRE(M >= 1, "%s: needs at least one row, got M=%d", __func__, M);
    REQUIRE(OC > 0 && OC % 128 == 0, "%s: Hadamard dimension must be divisible by 128, got %d",
            __func__, OC);
    REQUIRE_PTR(mid);
    REQUIRE_PTR(rout);
    REQUIRE_PTR(out);
    return cuda_result(
        escha::launch_scaled_had(true, mid, rout, static_cast<__half*>(out), OC, nullptr, nullptr,
                                 nullptr, 0, row_expert, M, rs, as_stream(stream)),
        "escha_scaled_had_out");
}

int escha_scaled_had_pair(const void* rows, const float* rin0, const float* rin1, int M, int IC,
                          float rs, void* out0, void* out1, void* stream) {
    REQUIRE(M >= 1, "%s: needs at least one row, got M=%d", __func__, M);
    REQUIRE(IC > 0 && IC % 128 == 0, "%s: Hadamard dimension must be divisible by 128, got %d",
            __func__, IC);
    REQUIRE_PTR(rows);
    REQUIRE_PTR(rin0);
    REQUIRE_PTR(rin1);
    REQUIRE_PTR(out0);
    REQUIRE_PTR(out1);
    return cuda_result(
        escha::launch_scaled_had(false, rows, rin0, static_cast<__half*>(out0), IC, rows, rin1,
                                 static_cast<__half*>(out1), IC, nullptr, M, rs, as_stream(stream)),
        "escha_scaled_had_pair");
}

int escha_scaled_had_many(const void* rows, const void* up, int n, const float* const* rins,
                          void* const* outs, int M, int IC, float rs, void* stream) {
    REQUIRE(M >= 1, "%s: needs at least one row, got M=%d", __func__, M);
    REQUIRE(IC > 0 && IC % 128 == 0, "%s: Hadamard dimension must be divisible by 128, got %d",
            __func__, IC);
    REQUIRE(n >= 1 && n <= 4, "%s: one to four transforms per launch, got %d", __func__, n);
    REQUIRE_PTR(rows);
    OPTIONAL_PTR(up);
    // host-side tables: any alignment; the device pointers inside them are checked below
    REQUIRE(rins && outs, "%s: NULL argument table", __func__);
    __half* o[4] = {nullptr, nullptr, nullptr, nullptr};
    for (int i = 0; i < n; ++i) {
        REQUIRE(rins[i] != nullptr && outs[i] != nullptr, "%s: transform %d has a null pointer",
                __func__, i);
        REQUIRE(aligned16(rins[i]) && aligned16(outs[i]),
                "%s: transform %d has a pointer that is not 16-byte aligned", __func__, i);
        o[i] = static_cast<__half*>(outs[i]);
    }
    return cuda_result(
        escha::launch_scaled_had_many(static_cast<const __half*>(rows), static_cast<const __half*>(up),
                                      n, rins, o, M, IC, rs, as_stream(stream)),
        "escha_scaled_had_many");
}

int escha_scaled_had_out_pair(const float* mid0, const float* mid1, const float* rout0,
                              const float* rout1, int M, int OC0, int OC1, float rs, void* out0,
                              void* out1, void* stream) {
    REQUIRE(M >= 1, "%s: needs at least one row, got M=%d", __func__, M);
    REQUIRE(OC0 > 0 && OC0 % 128 == 0 && OC1 > 0 && OC1 % 128 == 0,
            "%s: Hadamard dimensions must be divisible by 128, got %d and %d", __func__, OC0, OC1);
    REQUIRE_PTR(mid0);
    REQUIRE_PTR(mid1);
    REQUIRE_PTR(rout0);
    REQUIRE_PTR(rout1);
    REQUIRE_PTR(out0);
    REQUIRE_PTR(out1);
    return cuda_result(
        escha::launch_scaled_had(true, mid0, rout0, static_cast<__half*>(out0), OC0, mid1, rout1,
                                 static_cast<__half*>(out1), OC1, nullptr, M, rs, as_stream(stream)),
        "escha_scaled_had_out_pair");
}

int escha_had128(const float* x, long nblocks, float* out, void* stream) {
    REQUIRE(nblocks >= 1, "%s: needs at least one 128-block, got %ld", __func__, nblocks);
    REQUIRE_PTR(x);
    REQUIRE_PTR(out);
    return cuda_result(escha::launch_had128(x, out, nblocks, as_stream(stream)), "escha_had128");
}

int escha_w8a16(const void* x, const void* w8, const void* scale, int M, int N, int Kd, void* y,
                void* stream) {
    REQUIRE(M >= 1 && N >= 1, "%s: empty input (M=%d N=%d)", __func__, M, N);
    REQUIRE(Kd >= 16 && Kd % 16 == 0, "%s: input width must be a positive multiple of 16, got %d",
            __func__, Kd);
    REQUIRE_PTR(x);
    REQUIRE_PTR(w8);
    REQUIRE(scale != nullptr && y != nullptr, "%s: NULL pointer", __func__);
    REQUIRE((M + 7) / 8 <= 65535, "%s: M=%d exceeds the launch grid", __func__, M);
    if (escha::w8a16_mma_supports(N, Kd)) {
        escha::Q8Params q{};
        q.x = static_cast<const __half*>(x);
        q.w8 = static_cast<const int8_t*>(w8);
        q.scale = static_cast<const __half*>(scale);
        q.y = static_cast<__half*>(y);
        q.M = M; q.N = N; q.Kd = Kd;
        q.input = escha::kQ8InputPlain;
        q.epilogue = escha::kQ8StorePlain;
        return cuda_result(escha::launch_w8a16_mma(q, as_stream(stream)), "escha_w8a16");
    }
    return cuda_result(
        escha::launch_w8a16(static_cast<const __half*>(x), static_cast<const int8_t*>(w8),
                            static_cast<const __half*>(scale), static_cast<__half*>(y), M, N, Kd,
                            as_stream(stream)),
        "escha_w8a16");
}

int escha_w8a16_many(const void* x, int n, const void* const* w8, const void* const* scale,
                     const int* N, int Kd, int M, void* const* y, void* stream) {
    REQUIRE(n >= 1 && n <= 4, "%s: 1..4 linears per launch, got %d", __func__, n);
    REQUIRE(M >= 1, "%s: needs at least one row, got M=%d", __func__, M);
    REQUIRE(Kd >= 64 && Kd % 64 == 0, "%s: input width must be a positive multiple of 64, got %d",
            __func__, Kd);
    REQUIRE_PTR(x);
    REQUIRE(w8 != nullptr && scale != nullptr && N != nullptr && y != nullptr,
            "%s: NULL table", __func__);
    REQUIRE((M + 7) / 8 <= 65535, "%s: M=%d exceeds the launch grid", __func__, M);
    escha::Q8Params q{};
    q.x = static_cast<const __half*>(x);
    q.M = M; q.Kd = Kd;
    q.input = escha::kQ8InputPlain;
    q.epilogue = escha::kQ8StorePlain;
    q.nseg = n;
    int blocks = 0;
    for (int i = 0; i < n; ++i) {
        REQUIRE(N[i] >= 16 && N[i] % 16 == 0,
                "%s: output widths must be positive multiples of 16, got N[%d]=%d", __func__, i, N[i]);
        REQUIRE(w8[i] != nullptr && scale[i] != nullptr && y[i] != nullptr,
                "%s: NULL pointer in table entry %d", __func__, i);
        REQUIRE((reinterpret_cast<uintptr_t>(w8[i]) & 15u) == 0,
                "%s: w8[%d] must be 16-byte aligned", __func__, i);
        q.seg_w8[i] = static_cast<const int8_t*>(w8[i]);
        q.seg_scale[i] = static_cast<const __half*>(scale[i]);
        q.seg_y[i] = static_cast<__half*>(y[i]);
        q.seg_N[i] = N[i];
        q.blk0[i] = blocks;
        blocks += N[i] / 16;
    }
    q.blk0[n] = blocks;
    q.w8 = q.seg_w8[0]; q.scale = q.seg_scale[0]; q.y = q.seg_y[0]; q.N = q.seg_N[0];
    return cuda_result(escha::launch_w8a16_mma(q, as_stream(stream)), "escha_w8a16_many");
}

int escha_q8_embed(const int64_t* ids, const void* w8, const void* scale, int rows, int N, int Kd,
                   void* out, void* stream) {
    REQUIRE(rows >= 1 && N >= 1, "%s: empty input (rows=%d N=%d)", __func__, rows, N);
    REQUIRE(Kd >= 16 && Kd % 16 == 0, "%s: row width must be a positive multiple of 16, got %d",
            __func__, Kd);
    REQUIRE(ids != nullptr && scale != nullptr, "%s: NULL pointer", __func__);
    REQUIRE_PTR(w8);
    REQUIRE_PTR(out);
    return cuda_result(
        escha::launch_q8_embed(ids, static_cast<const int8_t*>(w8), static_cast<const __half*>(scale),
                               static_cast<__half*>(out), rows, N, Kd, as_stream(stream)),
        "escha_q8_embed");
}

int escha_gemv_ref(const void* xh, const void* code, const int32_t* row_expert,
                   const int32_t* row_map, int slots, const void* lut, int M, int IC, int OC,
                   int K, int splits, float* part, float* mid, void* stream) {
    if (int rc = check_shape(__func__, K, IC, OC, 128)) return rc;
    REQUIRE(M >= 1, "%s: needs at least one row, got M=%d", __func__, M);
    REQUIRE_PTR(xh);
    REQUIRE_PTR(code);
    REQUIRE_PTR(mid);
    OPTIONAL_PTR(lut);
    if (splits < 1) splits = 1;
    REQUIRE((IC / 16) % splits == 0, "%s: splits=%d does not divide IC/16=%d", __func__, splits,
            IC / 16);
    if (row_map) {
        REQUIRE(splits == 1, "%s: a row_map requires splits == 1", __func__);
        REQUIRE(slots >= 1, "%s: row_map needs slots >= 1", __func__);
    } else {
        slots = M;
    }
    REQUIRE(slots <= 65535 && splits <= 65535, "%s: %d slots exceed the launch grid", __func__,
            slots);
    if (splits > 1) REQUIRE_PTR(part);
    return cuda_result(
        escha::launch_gemv_ref(static_cast<const __half*>(xh), static_cast<const uint32_t*>(code),
                               row_expert, row_map, slots, static_cast<const __half*>(lut), mid,
                               part, M, IC, OC, K, splits, as_stream(stream)),
        "escha_gemv_ref");
}

size_t escha_coded_gemv_workspace_bytes(int njobs, int OC, int splits, int rows_per_job) {
    if (njobs < 1 || OC < 128 || rows_per_job < 1) return 0;
    if (splits <= 1) return 0;
    return kCounterBytes + escha::gemv_mma_part_floats(njobs, splits, OC / 128, rows_per_job) * sizeof(float);
}

int escha_coded_gemv_splits(int IC, int OC, int njobs, int sm_count) {
    if (IC < 128 || OC < 128) return 1;
    if (sm_count <= 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            sm_count = 148;
    }
    if (njobs < 1) njobs = 1;
    const int nblk = IC / 128;
    const long units = static_cast<long>(OC / 128) * njobs;   // (row job, output block) pairs
    static const bool grid_kernel = [] {
        const char* v = std::getenv("ESCHA_B200_GEMV_KERNEL");
        return v == nullptr || std::strcmp(v, "stream") != 0;
    }();
    if (grid_kernel) {
        // One CTA per (output block, split), one wave: fill the GPU's resident-CTA slots
        // (three CTAs of the kernel fit on an SM) without exceeding them, at least two
        // 128-channel blocks per split.  Measured on the dense 27B-class shapes this beats
        // "two CTAs per SM" by 7 to 20 percent per projection.  Depends on the shape only.
        static const int min_blocks_grid = [] { const char* v = std::getenv("ESCHA_B200_SPLIT_MIN_BLOCKS"); return v && *v ? std::atoi(v) : 2; }();
        const long smax = nblk >= min_blocks_grid ? nblk / min_blocks_grid : 1;
        long s = 3L * sm_count / units;
        if (s > smax) s = smax;
        if (s < 1) s = 1;
        return static_cast<int>(s);
    }
    // The persistent kernel keeps three CTAs per SM busy from a list of items; the list
    // should be several times longer than the CTA count so that the CTAs finish together,
    // while an item should still hold a few 128-channel blocks so that its fixed work
    // (staging the rows, publishing a partial) stays small.  Depends on the shape only.
    static const int per_slot = [] { const char* v = std::getenv("ESCHA_B200_SPLIT_ITEMS"); return v && *v ? std::atoi(v) : 4; }();
    static const int min_blocks = [] { const char* v = std::getenv("ESCHA_B200_SPLIT_MIN_BLOCKS"); return v && *v ? std::atoi(v) : 4; }();
    const long want = static_cast<long>(per_slot) * 3L * sm_count;
    long s = (want + units - 1) / units;
    const long smax = nblk >= min_blocks ? nblk / min_blocks : 1;
    if (s > smax) s = smax;
    if (s < 1) s = 1;
    return static_cast<int>(s);
}

}  // extern "C"

namespace {
int coded_projections_impl(const char* fn, const void* x, const void* const* x_proj, const void* x_up,
                           long x_stride, int x_row_div, int input_mode,
                           int nproj, const void* const* code, const float* const* rin,
                           const float* const* rout, void* const* out, const int* OC,
                           const void* jobs, int njobs, int rows_per_job, int M, int E, int IC,
                           int K, const int* splits, float rs, void* workspace,
                           size_t workspace_bytes, void* stream,
                           void* const* peer_out, int npeers, const int* out_ld, const int* out_col0,
                           const int* Ks = nullptr) {
    REQUIRE(npeers >= 0 && npeers <= escha::kMaxPeers, "%s: npeers=%d outside [0, %d]", fn,
            npeers, escha::kMaxPeers);
    if (npeers > 0) REQUIRE(peer_out != nullptr, "%s: peer_out is NULL", fn);
    REQUIRE(nproj >= 1 && nproj <= escha::kMaxProblems, "%s: nproj=%d outside [1, %d]", fn,
            nproj, escha::kMaxProblems);
    REQUIRE(code && rout && out && OC, "%s: NULL projection table", fn);
    REQUIRE(input_mode >= 0 && input_mode <= 2, "%s: unknown input mode %d", fn, input_mode);
    REQUIRE(M >= 1, "%s: needs at least one row, got M=%d", fn, M);
    REQUIRE(E >= 1, "%s: needs at least one expert stream, got E=%d", fn, E);
    REQUIRE_PTR(x);
    if (input_mode == escha::kInputSwiglu) REQUIRE_PTR(x_up);
    if (x_stride <= 0) x_stride = IC;
    REQUIRE(x_stride >= IC && x_stride % 8 == 0, "%s: row stride %ld must be >= IC=%d and a multiple of 8",
            fn, x_stride, IC);
    escha::GemvMmaParams p{};
    int total_ocb = 0;
    for (int i = 0; i < nproj; ++i) {
        if (int rc = check_shape(fn, Ks ? Ks[i] : K, IC, OC[i], 128)) return rc;
        p.prob[i].K = Ks ? Ks[i] : K;
        REQUIRE_PTR(code[i]);
        REQUIRE_PTR(out[i]);
        OPTIONAL_PTR(rout[i]);
        if (input_mode != escha::kInputTransformed) {
            REQUIRE(rin != nullptr, "%s: a fused input transform needs rin", fn);
            REQUIRE_PTR(rin[i]);
        }
        p.prob[i].code = static_cast<const uint32_t*>(code[i]);
        if (x_proj && x_proj[i]) {
            REQUIRE_PTR(x_proj[i]);
            p.prob[i].x = static_cast<const __half*>(x_proj[i]);
        }
        p.prob[i].rin =input_mode != escha::kInputTransformed ? rin[i] : nullptr;
        p.prob[i].rout = rout[i];
        p.prob[i].out = out[i];
        p.prob[i].OC = OC[i];
        p.prob[i].ocb0 = total_ocb;
        total_ocb += OC[i] / 128;
        p.prob[i].out_ld = out_ld ? out_ld[i] : 0;
        p.prob[i].out_col0 = out_col0 ? out_col0[i] : 0;
        if (p.prob[i].out_ld) {
            REQUIRE(p.prob[i].out_ld >= p.prob[i].out_col0 + OC[i] && p.prob[i].out_ld % 8 == 0 &&
                        p.prob[i].out_col0 % 8 == 0 && p.prob[i].out_col0 >= 0,
                    "%s: output row of %d elements cannot hold %d columns at offset %d", fn,
                    p.prob[i].out_ld, OC[i], p.prob[i].out_col0);
        } else {
            REQUIRE(p.prob[i].out_col0 == 0, "%s: out_col0 needs out_ld", fn);
        }
        p.prob[i].npeer = npeers;
        for (int g = 0; g < npeers; ++g) {
            void* pp = peer_out[static_cast<size_t>(i) * npeers + g];
            REQUIRE_PTR(pp);
            p.prob[i].peer[g] = pp;
        }
    }
    p.nprob = nproj;
    p.total_ocb = total_ocb;
    if (jobs) {
        REQUIRE_PTR(jobs);
        REQUIRE(rows_per_job == 8 || rows_per_job == 16, "%s: rows per job must be 8 or 16, got %d",
                fn, rows_per_job);
        REQUIRE(njobs >= 1, "%s: njobs=%d", fn, njobs);
    } else {
        rows_per_job = M <= 8 ? 8 : 16;
        njobs = (M + rows_per_job - 1) / rows_per_job;
    }
    REQUIRE(njobs <= 65535, "%s: %d row jobs exceed the launch grid", fn, njobs);
    int smax = 1;
    for (int i = 0; i < nproj; ++i) {
        int si = splits ? splits[i] : 0;
        if (si <= 0) {
            REQUIRE(jobs == nullptr, "%s: with row jobs pass the split factor explicitly", fn);
            si = escha_coded_gemv_splits(IC, OC[i], 1, 0);
        }
        REQUIRE(si <= IC / 128 && si <= 65535, "%s: splits=%d exceeds the %d input blocks", fn,
                si, IC / 128);
        p.prob[i].splits = si;
        if (si > smax) smax = si;
    }
    p.x = static_cast<const __half*>(x);
    p.x_up = static_cast<const __half*>(x_up);
    p.x_stride = x_stride;
    p.x_row_div = x_row_div < 1 ? 1 : x_row_div;
    p.hash_mask = 0x8FFF8FFFu;
    p.hash_xor = 0x3B603B60u;
    p.mul2 = 2u; p.mul4 = 4u; p.mul16 = 16u; p.mul32 = 32u; p.mul64 = 64u; p.mul128 = 128u;
    p.jobs = static_cast<const escha::RowJob*>(jobs);
    p.M = M; p.IC = IC; p.K = K;
    p.splits = smax;
    p.rows_per_job = rows_per_job;
    p.njobs = njobs;
    p.input = input_mode;
    p.rs = rs;
    if (smax > 1) {
        const size_t need =
            escha_coded_gemv_workspace_bytes(njobs, total_ocb * 128, smax, rows_per_job);
        REQUIRE_PTR(workspace);
        REQUIRE(workspace_bytes >= need, "%s: workspace of %zu bytes is smaller than the %zu needed",
                fn, workspace_bytes, need);
        // the tail of the counter region belongs to escha_moe_route
        REQUIRE(static_cast<size_t>(njobs) * total_ocb <= kSchedIndex,
                "%s: %d jobs x %d output blocks exceed the %zu split-K counters", fn, njobs,
                total_ocb, kMaxCounters);
        p.counters = static_cast<int32_t*>(workspace);
        p.part = reinterpret_cast<float*>(static_cast<char*>(workspace) + kCounterBytes);
    }
    // with a workspace the persistent kernel hands items out through a counter in it
    if (workspace != nullptr && workspace_bytes >= kCounterBytes) {
        REQUIRE_PTR(workspace);
        p.sched = static_cast<int32_t*>(workspace) + kSchedIndex;
    }
    return cuda_result(escha::launch_gemv_mma(p, as_stream(stream)), fn);
}
}  // namespace

extern "C" {

int escha_coded_projections(const void* x, const void* const* x_proj, const void* x_up,
                            long x_stride, int x_row_div, int input_mode,
                            int nproj, const void* const* code, const float* const* rin,
                            const float* const* rout, void* const* out, const int* OC,
                            const void* jobs, int njobs, int rows_per_job, int M, int E, int IC,
                            int K, const int* splits, float rs, void* workspace,
                            size_t workspace_bytes, void* stream) {
    return coded_projections_impl(__func__, x, x_proj, x_up, x_stride, x_row_div, input_mode, nproj,
                                  code, rin, rout, out, OC, jobs, njobs, rows_per_job, M, E, IC, K,
                                  splits, rs, workspace, workspace_bytes, stream, nullptr, 0, nullptr,
                                  nullptr);
}

int escha_coded_projections_gather(const void* x, const void* const* x_proj, const void* x_up,
                                   long x_stride, int x_row_div, int input_mode,
                                   int nproj, const void* const* code, const float* const* rin,
                                   const float* const* rout, void* const* out, const int* OC,
                                   const void* jobs, int njobs, int rows_per_job, int M, int E,
                                   int IC, int K, const int* splits, float rs,
                                   void* workspace, size_t workspace_bytes,
                                   void* const* peer_out, int npeers, const int* out_ld,
                                   const int* out_col0, void* stream) {
    REQUIRE(out_ld != nullptr && out_col0 != nullptr, "%s: out_ld and out_col0 are required", __func__);
    return coded_projections_impl(__func__, x, x_proj, x_up, x_stride, x_row_div, input_mode, nproj,
                                  code, rin, rout, out, OC, jobs, njobs, rows_per_job, M, E, IC, K,
                                  splits, rs, workspace, workspace_bytes, stream, peer_out, npeers,
                                  out_ld, out_col0);
}

int escha_coded_projections_mixed(const void* x, const void* const* x_proj, const void* x_up,
                                  long x_stride, int x_row_div, int input_mode,
                                  int nproj, const void* const* code, const float* const* rin,
                                  const float* const* rout, void* const* out, const int* OC,
                                  const int* Ks, const void* jobs, int njobs, int rows_per_job,
                                  int M, int E, int IC, const int* splits, float rs,
                                  void* workspace, size_t workspace_bytes,
                                  void* const* peer_out, int npeers, const int* out_ld,
                                  const int* out_col0, void* stream) {
    REQUIRE(Ks != nullptr, "%s: Ks is NULL", __func__);
    if (npeers > 0) REQUIRE(out_ld != nullptr && out_col0 != nullptr,
                            "%s: out_ld and out_col0 are required with peers", __func__);
    return coded_projections_impl(__func__, x, x_proj, x_up, x_stride, x_row_div, input_mode, nproj,
                                  code, rin, rout, out, OC, jobs, njobs, rows_per_job, M, E, IC,
                                  Ks[0], splits, rs, workspace, workspace_bytes, stream, peer_out,
                                  npeers, out_ld, out_col0, Ks);
}

int escha_peer_barrier(int32_t* local_flags, int32_t* const* peer_flags, int rank, int nranks,
                       void* stream) {
    REQUIRE(nranks >= 2 && nranks <= escha::kMaxPeers + 1, "%s: nranks=%d outside [2, %d]", __func__,
            nranks, escha::kMaxPeers + 1);
    REQUIRE(rank >= 0 && rank < nranks, "%s: rank %d outside [0, %d)", __func__, rank, nranks);
    REQUIRE(local_flags != nullptr && peer_flags != nullptr, "%s: NULL flags", __func__);
    escha::PeerBarrierParams p{};
    p.local = local_flags;
    for (int g = 0; g < nranks; ++g) {
        if (g != rank) REQUIRE(peer_flags[g] != nullptr, "%s: peer %d has no flags", __func__, g);
        p.peer[g] = peer_flags[g];
    }
    p.rank = rank;
    p.nranks = nranks;
    return cuda_result(escha::launch_peer_barrier(p, as_stream(stream)), __func__);
}

int escha_coded_gemv(const void* xh, const void* code, const float* rout, int M, int IC, int OC,
                     int K, int splits, float rs, void* workspace, size_t workspace_bytes,
                     void* out, void* stream) {
    return escha_coded_projections(xh, nullptr, nullptr, IC, 1, escha::kInputTransformed, 1, &code,
                                   nullptr,
                                   &rout, &out, &OC, nullptr, 0, 0, M, 1, IC, K, &splits, rs,
                                   workspace, workspace_bytes, stream);
}

int escha_moe_jobs_bound(int m, int E, int R) {
    if (m < 1 || E < 1 || R < 1) return 0;
    const long hit = m < E ? m : E;
    return static_cast<int>((m + hit * (R - 1)) / R);
}

int escha_moe_group_rows(const int32_t* row_expert, int m, int E, int R, void* jobs,
                         int njobs_cap, int32_t* njobs_out, void* stream) {
    REQUIRE(m >= 1 && E >= 1, "%s: needs m >= 1 and E >= 1, got m=%d E=%d", __func__, m, E);
    REQUIRE(R == 8 || R == 16, "%s: rows per job must be 8 or 16, got %d", __func__, R);
    REQUIRE(E <= 12000, "%s: E=%d exceeds the grouping kernel's shared memory", __func__, E);
    REQUIRE_PTR(row_expert);
    REQUIRE_PTR(jobs);
    REQUIRE(njobs_cap >= escha_moe_jobs_bound(m, E, R),
            "%s: njobs_cap=%d is below the bound %d for m=%d E=%d R=%d", __func__, njobs_cap,
            escha_moe_jobs_bound(m, E, R), m, E, R);
    return cuda_result(escha::launch_group_rows(row_expert, m, E, R,
                                                static_cast<escha::RowJob*>(jobs), njobs_cap,
                                                njobs_out, as_stream(stream)),
                       "escha_moe_group_rows");
}

int escha_jobs_from_groups(const int32_t* rows_idx, const int32_t* group_expert, int n_groups,
                           int R, int n_rows, int rows_per_job, void* jobs, void* stream) {
    REQUIRE(n_groups >= 1 && R >= 1 && n_rows >= 1, "%s: empty grouping (n_groups=%d R=%d n_rows=%d)",
            __func__, n_groups, R, n_rows);
    REQUIRE(rows_per_job == 8 || rows_per_job == 16, "%s: rows per job must be 8 or 16, got %d",
            __func__, rows_per_job);
    REQUIRE_PTR(rows_idx);
    REQUIRE_PTR(group_expert);
    REQUIRE_PTR(jobs);
    return cuda_result(
        escha::launch_jobs_from_groups(rows_idx, group_expert, n_groups, R, n_rows, rows_per_job,
                                       static_cast<escha::RowJob*>(jobs), as_stream(stream)),
        "escha_jobs_from_groups");
}

int escha_coded_gemv_jobs(const void* xh, const void* code, const float* rout, const void* jobs,
                          int njobs, int rows_per_job, int M, int E, int IC, int OC, int K,
                          int splits, float rs, void* workspace, size_t workspace_bytes, void* out,
                          void* stream) {
    REQUIRE(jobs != nullptr, "%s: jobs is NULL", __func__);
    REQUIRE(splits >= 1, "%s: splits=%d; pass the policy's value explicitly", __func__, splits);
    return escha_coded_projections(xh, nullptr, nullptr, IC, 1, escha::kInputTransformed, 1, &code,
                                   nullptr,
                                   &rout, &out, &OC, jobs, njobs, rows_per_job, M, E, IC, K,
                                   &splits, rs, workspace, workspace_bytes, stream);
}

int escha_swiglu(const void* gate, const void* up, int M, int I, long stride, void* h,
                 void* stream) {
    REQUIRE(M >= 1 && I >= 1, "%s: empty input (M=%d I=%d)", __func__, M, I);
    REQUIRE(stride >= I, "%s: row stride %ld is below I=%d", __func__, stride, I);
    if (gate == nullptr || up == nullptr || h == nullptr)
        return fail(ESCHA_EINVAL, "%s: NULL pointer", __func__);
    return cuda_result(escha::launch_swiglu(static_cast<const __half*>(gate),
                                            static_cast<const __half*>(up), M, I, stride,
                                            static_cast<__half*>(h), as_stream(stream)),
                       "escha_swiglu");
}

int escha_moe_combine(const void* d16, const float* scores, int T, int top_k, int H, void* y,
                      void* stream) {
    REQUIRE(T >= 1 && top_k >= 1 && H >= 1, "%s: empty input (T=%d top_k=%d H=%d)", __func__, T,
            top_k, H);
    REQUIRE_PTR(d16);
    REQUIRE_PTR(scores);
    REQUIRE_PTR(y);
    return cuda_result(escha::launch_moe_combine(static_cast<const __half*>(d16), scores, T, top_k,
                                                 H, static_cast<__half*>(y), as_stream(stream)),
                       "escha_moe_combine");
}

int escha_moe_route(const void* x, const void* gate_w, const void* shg_w, const int32_t* ids_in,
                    int T, int H, int E, int top_k, int e_lo, int e_hi, int rows_per_job,
                    int32_t* ids, float* scores, float* shared_gate_logit, float* logits_scratch,
                    void* jobs, int njobs_cap, void* workspace, size_t workspace_bytes,
                    void* stream) {
    REQUIRE(T >= 1 && E >= 1 && top_k >= 1, "%s: empty input (T=%d E=%d top_k=%d)", __func__, T, E,
            top_k);
    REQUIRE(H >= 8 && H % 8 == 0, "%s: hidden size must be a positive multiple of 8, got %d",
            __func__, H);
    REQUIRE(top_k <= 16 && top_k <= E, "%s: top_k=%d outside [1, min(16, E)]", __func__, top_k);
    REQUIRE(E <= 1024, "%s: E=%d exceeds 1024", __func__, E);
    REQUIRE(static_cast<size_t>((T + 7) / 8) <= kRouteTiles, "%s: T=%d exceeds %zu tokens", __func__,
            T, kRouteTiles * 8);
    REQUIRE(0 <= e_lo && e_lo < e_hi && e_hi <= E, "%s: expert range [%d, %d) outside [0, %d)",
            __func__, e_lo, e_hi, E);
    REQUIRE_PTR(x);
    if (ids_in == nullptr) {
        REQUIRE_PTR(gate_w);
        REQUIRE(ids && scores && logits_scratch,
                "%s: ids, scores and logits_scratch are required when ids_in is NULL", __func__);
    }
    if (shg_w) REQUIRE(shared_gate_logit != nullptr, "%s: shared_gate_logit is NULL", __func__);
    if (jobs) {
        REQUIRE(rows_per_job == 8 || rows_per_job == 16, "%s: rows per job must be 8 or 16, got %d",
                __func__, rows_per_job);
        REQUIRE(njobs_cap >= escha_moe_jobs_bound(T * top_k, e_hi - e_lo, rows_per_job),
                "%s: njobs_cap=%d is below the bound %d", __func__, njobs_cap,
                escha_moe_jobs_bound(T * top_k, e_hi - e_lo, rows_per_job));
        REQUIRE(escha::route_shared_bytes(T, top_k, e_lo, e_hi) <= 200 * 1024,
                "%s: %d rows exceed the grouping phase's shared memory", __func__, T * top_k);
    }
    REQUIRE_PTR(workspace);
    REQUIRE(workspace_bytes >= kCounterBytes, "%s: workspace of %zu bytes is smaller than the %zu "
            "counter region", __func__, workspace_bytes, kCounterBytes);
    escha::RouteParams p{};
    p.x = static_cast<const __half*>(x);
    p.gate_w = static_cast<const __half*>(gate_w);
    p.shg_w = static_cast<const __half*>(shg_w);
    p.ids_in = ids_in;
    p.T = T; p.H = H; p.E = E; p.top_k = top_k;
    p.e_lo = e_lo; p.e_hi = e_hi;
    p.R = rows_per_job;
    p.ids = ids; p.scores = scores; p.slog = shared_gate_logit; p.logits = logits_scratch;
    p.jobs = static_cast<escha::RowJob*>(jobs);
    p.njobs_cap = njobs_cap;
    p.counter = static_cast<int32_t*>(workspace) + (kMaxCounters - kRouteCounters);
    return cuda_result(escha::launch_moe_route(p, as_stream(stream)), "escha_moe_route");
}

int escha_moe_shared_finish(const void* gu, const void* w8, const void* scale, const void* d16,
                            const int32_t* ids, int experts_per_rank, const float* scores,
                            const float* shared_gate_logit, int T, int top_k, int H, int I,
                            void* out, void* stream) {
    if (ids) REQUIRE(experts_per_rank >= 1, "%s: experts_per_rank=%d with ids given", __func__,
                     experts_per_rank);
    REQUIRE(T >= 1 && top_k >= 1, "%s: empty input (T=%d top_k=%d)", __func__, T, top_k);
    REQUIRE(escha::w8a16_mma_supports(H, I), "%s: needs H %% 16 == 0 and I %% 64 == 0, got H=%d I=%d",
            __func__, H, I);
    REQUIRE_PTR(gu);
    REQUIRE_PTR(w8);
    REQUIRE_PTR(d16);
    REQUIRE_PTR(out);
    REQUIRE(scale && scores && shared_gate_logit, "%s: NULL pointer", __func__);
    REQUIRE((T + 31) / 32 <= 65535, "%s: T=%d exceeds the launch grid", __func__, T);
    escha::Q8Params q{};
    q.x = static_cast<const __half*>(gu);
    q.w8 = static_cast<const int8_t*>(w8);
    q.scale = static_cast<const __half*>(scale);
    q.y = static_cast<__half*>(out);
    q.M = T; q.N = H; q.Kd = I;
    q.input = escha::kQ8InputSwiglu;
    q.epilogue = escha::kQ8StoreGatedAdd;
    q.d16 = static_cast<const __half*>(d16);
    q.ids = ids;
    q.experts_per_rank = experts_per_rank;
    q.scores = scores;
    q.gate_logit = shared_gate_logit;
    q.top_k = top_k;
    return cuda_result(escha::launch_w8a16_mma(q, as_stream(stream)), "escha_moe_shared_finish");
}

int escha_coded_gemm_tc_splits(int IC, int OC, int sm_count) {
    if (IC < 128 || OC < 128) return 1;
    if (sm_count <= 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            sm_count = 148;
    }
    // one CTA per SM (a CTA holds most of an SM's shared memory): as many splits as keep
    // the grid within one wave, at least four 64-channel chunks per split
    long s = sm_count / (OC / 128);
    const long smax = IC / 256;
    if (s > smax) s = smax;
    if (s < 1) s = 1;
    return static_cast<int>(s);
}

int escha_coded_gemm_tc(const void* xh, const void* code, const float* rout, int M, int IC, int OC,
                        int K, int splits, float rs, float* planes, void* out, void* stream) {
    if (int rc = check_shape(__func__, K, IC, OC, 128)) return rc;
    REQUIRE(M >= 1, "%s: needs at least one row, got M=%d", __func__, M);
    REQUIRE_PTR(xh);
    REQUIRE_PTR(code);
    REQUIRE_PTR(out);
    OPTIONAL_PTR(rout);
    if (splits <= 0) splits = escha_coded_gemm_tc_splits(IC, OC, 0);
    REQUIRE(splits <= IC / 64 && splits <= 65535, "%s: splits=%d exceeds the %d 64-channel chunks",
            __func__, splits, IC / 64);
    REQUIRE((M + 255) / 256 <= 65535, "%s: M=%d exceeds the launch grid", __func__, M);
    // transform inside the GEMM's epilogue: unsplit, or split with the split-order sum done by a
    // cluster of CTAs inside the kernel
    static const bool cluster_sums = [] {
        const char* v = std::getenv("ESCHA_B200_TC_CLUSTER_SUM");
        return v == nullptr || std::strcmp(v, "0") != 0;
    }();
    const bool fused_out = rout != nullptr &&
        (splits == 1 || (cluster_sums && escha::gemm_tc_uses_tmem() && escha::gemm_tcm_cluster_sum(IC, splits)));
    const bool need_planes = splits > 1 && !fused_out;
    if (need_planes) REQUIRE_PTR(planes);
    escha::GemmTcParams p{};
    p.code = static_cast<const uint32_t*>(code);
    p.xh = static_cast<const __half*>(xh);
    p.out = need_planes ? planes : static_cast<float*>(out);
    if (fused_out) {
        p.out = nullptr;
        p.rout = rout;
        p.y16 = static_cast<__half*>(out);
        p.rs = rs;
    }
    p.M = M; p.IC = IC; p.OC = OC; p.K = K; p.splits = splits;
    p.hash_mask = 0x8FFF8FFFu;
    p.hash_xor = 0x3B603B60u;
    p.mul2 = 2u; p.mul4 = 4u; p.mul16 = 16u; p.mul32 = 32u; p.mul64 = 64u; p.mul128 = 128u;
    cudaError_t e = escha::launch_gemm_tc(p, as_stream(stream));
    if (e == cudaSuccess && rout != nullptr && !fused_out)
        e = escha::launch_planes_out(planes, rout, static_cast<__half*>(out), M, OC, splits, rs,
                                     as_stream(stream));
    else if (e == cudaSuccess && need_planes)
        e = escha::launch_sum_planes(planes, static_cast<float*>(out), static_cast<size_t>(M) * OC,
                                     splits, as_stream(stream));
    return cuda_result(e, "escha_coded_gemm_tc");
}

int escha_coded_gemm_tc_needs_planes(int IC, int splits, int has_rout) {
    if (splits <= 1) return 0;
    static const bool cluster_sums = [] {
        const char* v = std::getenv("ESCHA_B200_TC_CLUSTER_SUM");
        return v == nullptr || std::strcmp(v, "0") != 0;
    }();
    const bool fused_out = has_rout && cluster_sums && escha::gemm_tc_uses_tmem() &&
                           escha::gemm_tcm_cluster_sum(IC, splits);
    return fused_out ? 0 : 1;
}

int escha_coded_gemm_tc_many(int n, const void* const* xhs, const void* const* codes,
                             const float* const* routs, int M, int IC, const int* OCs, int K,
                             int splits, float rs, float* const* planes, void* const* outs,
                             void* stream) {
    REQUIRE(n >= 1 && n <= 3, "%s: one to three projections per launch, got %d", __func__, n);
    // host-side tables: any alignment; the device pointers inside them are checked below
    REQUIRE(xhs && codes && routs && OCs && outs, "%s: NULL argument table", __func__);
    REQUIRE(M >= 1, "%s: needs at least one row, got M=%d", __func__, M);
    REQUIRE((M + 255) / 256 <= 65535, "%s: M=%d exceeds the launch grid", __func__, M);
    int oc_total = 0;
    for (int i = 0; i < n; ++i) {
        if (int rc = check_shape(__func__, K, IC, OCs[i], 128)) return rc;
        REQUIRE(xhs[i] != nullptr && codes[i] != nullptr && routs[i] != nullptr && outs[i] != nullptr,
                "%s: projection %d has a null pointer", __func__, i);
        REQUIRE(aligned16(xhs[i]) && aligned16(codes[i]) && aligned16(routs[i]) && aligned16(outs[i]),
                "%s: projection %d has a pointer that is not 16-byte aligned", __func__, i);
        oc_total += OCs[i];
    }
    if (splits <= 0) splits = escha_coded_gemm_tc_splits(IC, oc_total, 0);
    REQUIRE(splits <= IC / 128 && splits <= 65535, "%s: splits=%d exceeds the %d 128-channel stages",
            __func__, splits, IC / 128);
    static const bool cluster_sums = [] {
        const char* v = std::getenv("ESCHA_B200_TC_CLUSTER_SUM");
        return v == nullptr || std::strcmp(v, "0") != 0;
    }();
    const bool fused_out = splits == 1 || (cluster_sums && escha::gemm_tcm_cluster_sum(IC, splits));
    if (!fused_out) {
        REQUIRE(planes != nullptr, "%s: planes table is NULL", __func__);
        for (int i = 0; i < n; ++i)
            REQUIRE(planes[i] != nullptr, "%s: projection %d needs a plane workspace", __func__, i);
    }
    escha::GemmTcParams p{};
    p.code = static_cast<const uint32_t*>(codes[0]);
    p.xh = static_cast<const __half*>(xhs[0]);
    p.out = fused_out ? nullptr : planes[0];
    p.rout = fused_out ? routs[0] : nullptr;
    p.y16 = fused_out ? static_cast<__half*>(outs[0]) : nullptr;
    p.rs = rs;
    p.M = M; p.IC = IC; p.OC = OCs[0]; p.K = K; p.splits = splits;
    p.hash_mask = 0x8FFF8FFFu;
    p.hash_xor = 0x3B603B60u;
    p.mul2 = 2u; p.mul4 = 4u; p.mul16 = 16u; p.mul32 = 32u; p.mul64 = 64u; p.mul128 = 128u;
    p.nproj = n;
    const __half* xh_more[2] = {nullptr, nullptr};
    int cb = OCs[0] / 128;
    for (int i = 1; i < n; ++i) {
        escha::GemmTcParams::More& m = p.more[i - 1];
        m.code = static_cast<const uint32_t*>(codes[i]);
        m.out = fused_out ? nullptr : planes[i];
        m.rout = fused_out ? routs[i] : nullptr;
        m.y16 = fused_out ? static_cast<__half*>(outs[i]) : nullptr;
        m.OC = OCs[i];
        m.cb0 = cb;
        cb += OCs[i] / 128;
        xh_more[i - 1] = static_cast<const __half*>(xhs[i]);
    }
    cudaError_t e = escha::launch_gemm_tcm_many(p, xh_more, as_stream(stream));
    // measured on the 27B-class Q/K/V group: one plane-sum launch for all projections is 1.3%
    // faster per layer step up to 128 rows and 1% slower at 256, where each sum is large
    const bool one_sum_launch = M <= 128;
    for (int i = 0; i < n && e == cudaSuccess && !fused_out && !one_sum_launch; ++i)
        e = escha::launch_planes_out(planes[i], routs[i], static_cast<__half*>(outs[i]), M, OCs[i],
                                     splits, rs, as_stream(stream));
    if (e == cudaSuccess && !fused_out && one_sum_launch) {
        __half* ys[3] = {nullptr, nullptr, nullptr};
        for (int i = 0; i < n; ++i) ys[i] = static_cast<__half*>(outs[i]);
        e = escha::launch_planes_out_many(n, planes, routs, ys, OCs, M, splits, rs, as_stream(stream));
    }
    return cuda_result(e, "escha_coded_gemm_tc_many");
}

int escha_coded_gemv_status(void) {
    int a = 0, b = 0;
    if (escha::gemv_stream_status(&a) != cudaSuccess || escha::gemv_mma_status(&b) != cudaSuccess) return -1;
    return a ? a : b;
}

void escha_debug_gemv_stall(int on, unsigned limit) { escha::gemv_stream_test_stall(on, limit); }

void escha_debug_peer_poll_limit(unsigned polls) { escha::peer_barrier_poll_limit(polls); }

void escha_debug_gemm_tc_stall(int on, unsigned limit) { escha::gemm_tcm_test_stall(on, limit); }

int escha_coded_gemm_tc_status(void) {
    int st = 0;
    if (escha::gemm_tc_status(&st) != cudaSuccess) return -1;
    return st;
}

}  // extern "C"
