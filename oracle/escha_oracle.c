/*
 * escha_oracle.c -- CPU restatement of the escha coded-projection path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA kernels are
 * compared against and the CPU baseline the benchmark reports beside the GPU
 * numbers.  Nothing in the product package may call it.
 *
 * Every function restates one function of the reference project
 * (EschaLabs/escha-mlx); the citation beside it is the reference file and line
 * range it follows.  Parity of this restatement is pinned: it reproduces the
 * reference's committed golden vectors (tests/data/codec, tests/data/qwen3_5)
 * bit-exactly for decode and within the reference's own tolerance for the
 * linear goldens, and it reproduces outputs of the reference's NumPy module
 * escha_mlx/ref.py run on seeded inputs (fixtures under tests/golden/).
 *
 * All half-precision values cross this interface as raw IEEE binary16 bit
 * patterns in uint16_t.  Plain C99 + OpenMP; no dependencies.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ESC_RS 0.088388347648f /* escha_mlx/ref.py:30 -- pinned f32 literal */

/* ------------------------------------------------------------------------ */
/* binary16 <-> binary32, round-to-nearest-even, no hardware dependence      */
/* ------------------------------------------------------------------------ */

static inline float esc_h2f(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: normalise */
            int e = -1;
            do {
                man <<= 1;
                e++;
            } while (!(man & 0x400u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

static inline uint16_t esc_f2h(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    uint32_t ax = x & 0x7FFFFFFFu;
    if (ax >= 0x7F800000u) /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | ((ax > 0x7F800000u) ? (0x200u | ((ax >> 13) & 0x3FFu)) : 0u));
    if (ax >= 0x477FF000u) /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7C00u);
    if (ax < 0x33000001u) /* <= 2^-25 rounds to zero (tie goes to even = 0) */
        return sign;
    int32_t e = (int32_t)(ax >> 23) - 127;
    uint32_t man = (ax & 0x7FFFFFu) | 0x800000u;
    uint32_t shift;
    uint32_t base;
    if (e < -14) { /* subnormal half */
        shift = (uint32_t)(13 + (-14 - e));
        base = 0;
    } else {
        shift = 13;
        base = ((uint32_t)(e + 15) << 10) - 0x400u; /* implicit bit adds back 0x400 */
    }
    uint32_t q = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u)))
        q++;
    return (uint16_t)(sign | (base + q));
}

void esc_f16_to_f32(const uint16_t *h, float *f, long n)
{
    for (long i = 0; i < n; i++)
        f[i] = esc_h2f(h[i]);
}

void esc_f32_to_f16(const float *f, uint16_t *h, long n)
{
    for (long i = 0; i < n; i++)
        h[i] = esc_f2h(f[i]);
}

/* ------------------------------------------------------------------------ */
/* codebook -- escha_mlx/ref.py:37-48 (cba_lut), escha_mlx/msl.py:34-41       */
/* ------------------------------------------------------------------------ */

static inline uint16_t esc_cba_decode(uint32_t state)
{
    uint32_t r = ((state * 0xCBAC1FEDu) & 0x8FFF8FFFu) ^ 0x3B603B60u;
    float lo = esc_h2f((uint16_t)(r & 0xFFFFu));
    float hi = esc_h2f((uint16_t)(r >> 16));
    /* both addends are binary16 with exponents within 3 of each other, so the
       binary32 sum is exact and the conversion below is the single RNE rounding
       a binary16 adder performs. */
    return esc_f2h(lo + hi);
}

static uint16_t g_lut[65536];
static int g_lut_ready = 0;

static void esc_lut_ensure(void)
{
    if (g_lut_ready)
        return;
#ifdef _OPENMP
#pragma omp critical(esc_lut)
#endif
    {
        if (!g_lut_ready) {
            for (uint32_t s = 0; s < 65536u; s++)
                g_lut[s] = esc_cba_decode(s);
            g_lut_ready = 1;
        }
    }
}

void esc_cba_lut(uint16_t *lut)
{
    esc_lut_ensure();
    memcpy(lut, g_lut, sizeof(g_lut));
}

/* ------------------------------------------------------------------------ */
/* window extraction -- escha_mlx/ref.py:64-93 (decode8_k2, decode8_k3)       */
/* ------------------------------------------------------------------------ */

static inline void esc_states_k2(const uint32_t *w, int lane, uint32_t *s)
{
    uint32_t t_off = (uint32_t)lane * 8u;
    uint32_t i1 = t_off >> 4;
    uint32_t i0 = (i1 + 15u) & 15u;
    uint64_t merged = ((uint64_t)w[i0] << 32) | (uint64_t)w[i1];
    uint32_t shift = ((~t_off) & 8u) << 1;
    uint32_t wv = (uint32_t)(merged >> shift);
    for (int j = 0; j < 8; j++)
        s[j] = (wv >> (2 * (7 - j))) & 0xFFFFu;
}

static inline void esc_states_k3(const uint32_t *w, int lane, uint32_t *s)
{
    uint32_t t_off = (uint32_t)lane * 8u;
    uint32_t b1 = (t_off + 257u) * 3u;
    uint32_t b0 = b1 - 16u;
    uint32_t b2 = b1 + 21u;
    uint32_t i0 = b0 >> 5;
    uint32_t i2 = (b2 - 1u) >> 5;
    uint32_t s2 = ((i2 + 1u) << 5) - b2;
    uint64_t merged = ((uint64_t)w[i0 % 24u] << 32) | (uint64_t)w[i2 % 24u];
    uint32_t w7 = (uint32_t)(merged >> s2);
    uint32_t w3 = (uint32_t)(merged >> (s2 + 12u));
    s[0] = (w3 >> 9) & 0xFFFFu;
    s[1] = (w3 >> 6) & 0xFFFFu;
    s[2] = (w3 >> 3) & 0xFFFFu;
    s[3] = w3 & 0xFFFFu;
    s[4] = (w7 >> 9) & 0xFFFFu;
    s[5] = (w7 >> 6) & 0xFFFFu;
    s[6] = (w7 >> 3) & 0xFFFFu;
    s[7] = w7 & 0xFFFFu;
}

static inline void esc_states(const uint32_t *w, int lane, int K, uint32_t *s)
{
    if (K == 2)
        esc_states_k2(w, lane, s);
    else
        esc_states_k3(w, lane, s);
}

/* escha_mlx/ref.py:96-111 (lane_positions): value j of lane L sits at
   (row, col) of the 16x16 tile. */
static inline void esc_lane_pos(int lane, int j, int *row, int *col)
{
    int l0 = lane & ~4;
    int c_off = (lane >> 2) & 1;
    int fi = j >> 1;
    *row = (lane & 3) * 2 + (j & 1) + (fi & 1) * 8;
    *col = 2 * ((l0 >> 3) + (j >= 4 ? 4 : 0)) + c_off;
}

/* states only (for tests of the window walk): out [tiles][32][8] u16 */
void esc_tile_states(const uint32_t *code, long tiles, int K, uint16_t *out)
{
    int wpt = 8 * K;
    for (long t = 0; t < tiles; t++)
        for (int lane = 0; lane < 32; lane++) {
            uint32_t s[8];
            esc_states(code + t * wpt, lane, K, s);
            for (int j = 0; j < 8; j++)
                out[(t * 32 + lane) * 8 + j] = (uint16_t)s[j];
        }
}

/* ------------------------------------------------------------------------ */
/* reconstruct -- escha_mlx/ref.py:114-134, 173-197; msl.py:183-202           */
/* code [TK][TN][8K] u32 -> w [IC][OC] binary16                               */
/* ------------------------------------------------------------------------ */

void esc_reconstruct(const uint32_t *code, int IC, int OC, int K, uint16_t *w)
{
    esc_lut_ensure();
    int tk = IC / 16, tn = OC / 16, wpt = 8 * K;
#ifdef _OPENMP
#pragma omp parallel for schedule(static)
#endif
    for (int kt = 0; kt < tk; kt++) {
        for (int nt = 0; nt < tn; nt++) {
            const uint32_t *wp = code + ((size_t)kt * tn + nt) * wpt;
            for (int lane = 0; lane < 32; lane++) {
                uint32_t s[8];
                esc_states(wp, lane, K, s);
                for (int j = 0; j < 8; j++) {
                    int r, c;
                    esc_lane_pos(lane, j, &r, &c);
                    w[((size_t)kt * 16 + r) * OC + (size_t)nt * 16 + c] = g_lut[s[j]];
                }
            }
        }
    }
}

/* ------------------------------------------------------------------------ */
/* transforms -- escha_mlx/ref.py:204-228; msl.py:875-949                      */
/* ------------------------------------------------------------------------ */

/* in-place unnormalised 128-point Sylvester WHT: stage h pairs i with i^h,
   a+b to the low index, a-b to the high index (ref.py:210-217). */
static inline void esc_h128_block(float *v)
{
    for (int h = 1; h < 128; h <<= 1)
        for (int i = 0; i < 128; i += 2 * h)
            for (int j = i; j < i + h; j++) {
                float a = v[j], b = v[j + h];
                v[j] = a + b;
                v[j + h] = a - b;
            }
}

void esc_h128(float *x, long rows, int n)
{
    for (long r = 0; r < rows; r++)
        for (int b = 0; b < n / 128; b++)
            esc_h128_block(x + r * n + b * 128);
}

/* xh = f16( H128( f32(x) * rin ) * RS ); rin is [IC] (row_expert NULL) or
   [E][IC] gathered by row_expert (ref.py:221-223; msl.py:895-916). */
void esc_input_transform(const uint16_t *x, const float *rin, const int32_t *row_expert,
                         int M, int IC, uint16_t *xh)
{
#ifdef _OPENMP
#pragma omp parallel for schedule(static) if (M * (long)IC > 65536)
#endif
    for (int r = 0; r < M; r++) {
        const float *rv = rin + (row_expert ? (size_t)row_expert[r] * IC : 0);
        for (int b = 0; b < IC / 128; b++) {
            float v[128];
            for (int i = 0; i < 128; i++)
                v[i] = esc_h2f(x[(size_t)r * IC + b * 128 + i]) * rv[b * 128 + i];
            esc_h128_block(v);
            for (int i = 0; i < 128; i++)
                xh[(size_t)r * IC + b * 128 + i] = esc_f2h(v[i] * ESC_RS);
        }
    }
}

/* y = f16( (H128(mid) * RS) * rout ), two separate f32 multiplies in that
   order (ref.py:226-228; msl.py:946-948). */
void esc_output_transform(const float *mid, const float *rout, const int32_t *row_expert,
                          int M, int OC, uint16_t *y)
{
#ifdef _OPENMP
#pragma omp parallel for schedule(static) if (M * (long)OC > 65536)
#endif
    for (int r = 0; r < M; r++) {
        const float *rv = rout + (row_expert ? (size_t)row_expert[r] * OC : 0);
        for (int b = 0; b < OC / 128; b++) {
            float v[128];
            memcpy(v, mid + (size_t)r * OC + b * 128, sizeof(v));
            esc_h128_block(v);
            for (int i = 0; i < 128; i++) {
                float scaled = v[i] * ESC_RS;
                float weighted = scaled * rv[b * 128 + i];
                y[(size_t)r * OC + b * 128 + i] = esc_f2h(weighted);
            }
        }
    }
}

/* ------------------------------------------------------------------------ */
/* coded GEMV in the reference kernels' accumulation order                    */
/* escha_mlx/msl.py:205-308 (direct GEMV), :389-435 (staged), :438-506 and     */
/* :688-872 (row-blocked: same per-(row, channel) order)                       */
/*                                                                            */
/* mid[r, :] = f32(xh[r, :]) @ f32(decode(code[row_expert[r]])), f32           */
/* accumulate: kt ascending; inside a tile lane L adds its values j=0..3 into  */
/* acc0 (column col) and j=4..7 into acc1 (column col+8); the four lanes that  */
/* share a column are then combined as (L + L^1) + (L^2 + L^3).               */
/* code is [E][TK][TN][8K] (row_expert given) or [TK][TN][8K].                */
/* ------------------------------------------------------------------------ */

void esc_gemv_ref_order(const uint16_t *xh, const uint32_t *code, const int32_t *row_expert,
                        int M, int IC, int OC, int K, float *mid)
{
    esc_lut_ensure();
    int tk = IC / 16, tn = OC / 16, wpt = 8 * K;
    size_t estride = (size_t)tk * tn * wpt;
    long units = (long)M * tn;
#ifdef _OPENMP
#pragma omp parallel for schedule(static)
#endif
    for (long u = 0; u < units; u++) {
        int r = (int)(u / tn), nt = (int)(u % tn);
        const uint32_t *base = code + (row_expert ? (size_t)row_expert[r] * estride : 0);
        float xf[16];
        float acc0[32], acc1[32];
        for (int l = 0; l < 32; l++)
            acc0[l] = acc1[l] = 0.0f;
        for (int kt = 0; kt < tk; kt++) {
            const uint32_t *wp = base + ((size_t)kt * tn + nt) * wpt;
            for (int i = 0; i < 16; i++)
                xf[i] = esc_h2f(xh[(size_t)r * IC + kt * 16 + i]);
            for (int lane = 0; lane < 32; lane++) {
                uint32_t s[8];
                esc_states(wp, lane, K, s);
                int xrow = (lane & 3) * 2;
                float x0 = xf[xrow], x1 = xf[xrow + 1], x8 = xf[xrow + 8], x9 = xf[xrow + 9];
                float a0 = acc0[lane], a1 = acc1[lane];
                a0 += x0 * esc_h2f(g_lut[s[0]]);
                a0 += x1 * esc_h2f(g_lut[s[1]]);
                a0 += x8 * esc_h2f(g_lut[s[2]]);
                a0 += x9 * esc_h2f(g_lut[s[3]]);
                a1 += x0 * esc_h2f(g_lut[s[4]]);
                a1 += x1 * esc_h2f(g_lut[s[5]]);
                a1 += x8 * esc_h2f(g_lut[s[6]]);
                a1 += x9 * esc_h2f(g_lut[s[7]]);
                acc0[lane] = a0;
                acc1[lane] = a1;
            }
        }
        for (int q = 0; q < 8; q++) { /* quad q = lanes 4q..4q+3 */
            int lane = 4 * q;
            float s0 = (acc0[lane] + acc0[lane + 1]) + (acc0[lane + 2] + acc0[lane + 3]);
            float s1 = (acc1[lane] + acc1[lane + 1]) + (acc1[lane + 2] + acc1[lane + 3]);
            int l0 = lane & ~4, c_off = (lane >> 2) & 1;
            int col = 2 * (l0 >> 3) + c_off;
            mid[(size_t)r * OC + nt * 16 + col] = s0;
            mid[(size_t)r * OC + nt * 16 + col + 8] = s1;
        }
    }
}

/* Same product with binary64 accumulation of the reference-decoded weights:
   the tolerance oracle (tests/test_splitk.py:127-144 in the reference). */
void esc_gemv_f64(const uint16_t *xh, const uint32_t *code, const int32_t *row_expert,
                  int M, int IC, int OC, int K, double *out)
{
    esc_lut_ensure();
    int tk = IC / 16, tn = OC / 16, wpt = 8 * K;
    size_t estride = (size_t)tk * tn * wpt;
    long units = (long)M * tn;
#ifdef _OPENMP
#pragma omp parallel for schedule(static)
#endif
    for (long u = 0; u < units; u++) {
        int r = (int)(u / tn), nt = (int)(u % tn);
        const uint32_t *base = code + (row_expert ? (size_t)row_expert[r] * estride : 0);
        double acc[16];
        for (int c = 0; c < 16; c++)
            acc[c] = 0.0;
        for (int kt = 0; kt < tk; kt++) {
            const uint32_t *wp = base + ((size_t)kt * tn + nt) * wpt;
            double tile[16][16];
            for (int lane = 0; lane < 32; lane++) {
                uint32_t s[8];
                esc_states(wp, lane, K, s);
                for (int j = 0; j < 8; j++) {
                    int rr, cc;
                    esc_lane_pos(lane, j, &rr, &cc);
                    tile[rr][cc] = (double)esc_h2f(g_lut[s[j]]);
                }
            }
            for (int i = 0; i < 16; i++) {
                double xv = (double)esc_h2f(xh[(size_t)r * IC + kt * 16 + i]);
                for (int c = 0; c < 16; c++)
                    acc[c] += xv * tile[i][c];
            }
        }
        for (int c = 0; c < 16; c++)
            out[(size_t)r * OC + nt * 16 + c] = acc[c];
    }
}

/* ------------------------------------------------------------------------ */
/* full linear -- escha_mlx/ref.py:231-293 (expert_linear, dense_linear)       */
/* with the production kernels' accumulation order for the product.           */
/* scratch-free for the caller: allocates xh/mid internally.                  */
/* bias (binary16 [OC]) may be NULL; added as f16(f32(y)+f32(bias)).          */
/* ------------------------------------------------------------------------ */

int esc_linear(const uint16_t *x, const uint32_t *code, const float *rin, const float *rout,
               const int32_t *row_expert, const uint16_t *bias, int M, int IC, int OC, int K,
               uint16_t *y)
{
    uint16_t *xh = (uint16_t *)malloc((size_t)M * IC * sizeof(uint16_t));
    float *mid = (float *)malloc((size_t)M * OC * sizeof(float));
    if (!xh || !mid) {
        free(xh);
        free(mid);
        return -1;
    }
    esc_input_transform(x, rin, row_expert, M, IC, xh);
    esc_gemv_ref_order(xh, code, row_expert, M, IC, OC, K, mid);
    esc_output_transform(mid, rout, row_expert, M, OC, y);
    if (bias)
        for (long i = 0; i < (long)M * OC; i++)
            y[i] = esc_f2h(esc_h2f(y[i]) + esc_h2f(bias[i % OC]));
    free(xh);
    free(mid);
    return 0;
}

/* ------------------------------------------------------------------------ */
/* SwiGLU -- escha_mlx/ref.py:296-301; models/qwen3_5_moe.py:221-223           */
/* gu [M][2I] binary16 (gate first) -> h [M][I]:                              */
/*   s = f16( g / (1 + exp(-g)) ) in f32, h = f16( f32(s) * f32(u) )          */
/* ------------------------------------------------------------------------ */

void esc_swiglu(const uint16_t *gu, int M, int I, uint16_t *h)
{
    for (int r = 0; r < M; r++)
        for (int i = 0; i < I; i++) {
            float g = esc_h2f(gu[(size_t)r * 2 * I + i]);
            float u = esc_h2f(gu[(size_t)r * 2 * I + I + i]);
            uint16_t s16 = esc_f2h(g / (1.0f + expf(-g)));
            h[(size_t)r * I + i] = esc_f2h(esc_h2f(s16) * u);
        }
}

/* ------------------------------------------------------------------------ */
/* int8 linear -- escha_mlx/ref.py:308-311 (w8a16)                             */
/* y = f16( f32(x) @ f32( f16( f32(w8) * f32(scale) ) )^T ), w8 [N][Kd],       */
/* scale binary16 [N] widened by the caller to f32.                           */
/* ------------------------------------------------------------------------ */

void esc_w8a16(const uint16_t *x, const int8_t *w8, const float *scale, int M, int N, int Kd,
               uint16_t *y)
{
#ifdef _OPENMP
#pragma omp parallel for schedule(static)
#endif
    for (int n = 0; n < N; n++) {
        float sc = scale[n];
        for (int r = 0; r < M; r++) {
            float acc = 0.0f;
            for (int k = 0; k < Kd; k++) {
                float wf = esc_h2f(esc_f2h((float)w8[(size_t)n * Kd + k] * sc));
                acc += esc_h2f(x[(size_t)r * Kd + k]) * wf;
            }
            y[(size_t)r * N + n] = esc_f2h(acc);
        }
    }
}

/* ------------------------------------------------------------------------ */
/* routed-expert path of the MoE block                                        */
/* escha_mlx/models/qwen3_5_moe.py:207-253 (_expert_path); ref.py:333-342      */
/* x [T][H] binary16, ids [T][top_k], scores [T][top_k] f32.                   */
/* rows are token-major; combine is a fixed slot-order f32 sum; the result is  */
/* rounded to binary16 (y16 [T][H]).                                           */
/* gu: code [E][H/16][2I/16][8Kg], rin [E][H], rout [E][2I];                   */
/* dn: code [E][I/16][H/16][8Kd],  rin [E][I], rout [E][H].                    */
/* ------------------------------------------------------------------------ */

int esc_moe_routed(const uint16_t *x, const int32_t *ids, const float *scores, int T, int top_k,
                   int H, int I, const uint32_t *gu_code, const float *gu_rin,
                   const float *gu_rout, int Kg, const uint32_t *dn_code, const float *dn_rin,
                   const float *dn_rout, int Kd, uint16_t *y16)
{
    int m = T * top_k;
    uint16_t *rows = (uint16_t *)malloc((size_t)m * H * 2);
    uint16_t *gu16 = (uint16_t *)malloc((size_t)m * 2 * I * 2);
    uint16_t *h = (uint16_t *)malloc((size_t)m * I * 2);
    uint16_t *d16 = (uint16_t *)malloc((size_t)m * H * 2);
    if (!rows || !gu16 || !h || !d16) {
        free(rows);
        free(gu16);
        free(h);
        free(d16);
        return -1;
    }
    for (int r = 0; r < m; r++)
        memcpy(rows + (size_t)r * H, x + (size_t)(r / top_k) * H, (size_t)H * 2);
    esc_linear(rows, gu_code, gu_rin, gu_rout, ids, NULL, m, H, 2 * I, Kg, gu16);
    esc_swiglu(gu16, m, I, h);
    esc_linear(h, dn_code, dn_rin, dn_rout, ids, NULL, m, I, H, Kd, d16);
    for (int t = 0; t < T; t++)
        for (int c = 0; c < H; c++) {
            float acc = 0.0f;
            for (int s = 0; s < top_k; s++) {
                int r = t * top_k + s;
                float w16 = esc_h2f(esc_f2h(scores[r]));
                float contrib = esc_h2f(d16[(size_t)r * H + c]) * w16;
                acc = acc + contrib; /* starts from +0 like a sum reduction */
            }
            y16[(size_t)t * H + c] = esc_f2h(acc);
        }
    free(rows);
    free(gu16);
    free(h);
    free(d16);
    return 0;
}

/* ------------------------------------------------------------------------ */
/* shared expert + final add -- models/qwen3_5_moe.py:267-272; ref.py:343-349  */
/* out = f16( f32(y16) + sh * sigmoid(shg) )                                   */
/*   g,u = w8a16(x, gate/up) as f32; hh = f16( g*sigmoid(g) * u );             */
/*   sh = f32(w8a16(hh, down)); shg = f32(f16( x @ shg_w^T )).                 */
/* ------------------------------------------------------------------------ */

int esc_moe_shared_add(const uint16_t *x, const uint16_t *y16, int T, int H, int I,
                       const int8_t *g_w8, const float *g_sc, const int8_t *u_w8,
                       const float *u_sc, const int8_t *d_w8, const float *d_sc,
                       const uint16_t *shg_w, uint16_t *out)
{
    uint16_t *g = (uint16_t *)malloc((size_t)T * I * 2);
    uint16_t *u = (uint16_t *)malloc((size_t)T * I * 2);
    uint16_t *hh = (uint16_t *)malloc((size_t)T * I * 2);
    uint16_t *sh = (uint16_t *)malloc((size_t)T * H * 2);
    if (!g || !u || !hh || !sh) {
        free(g);
        free(u);
        free(hh);
        free(sh);
        return -1;
    }
    esc_w8a16(x, g_w8, g_sc, T, I, H, g);
    esc_w8a16(x, u_w8, u_sc, T, I, H, u);
    for (long i = 0; i < (long)T * I; i++) {
        float gf = esc_h2f(g[i]), uf = esc_h2f(u[i]);
        float sig = 1.0f / (1.0f + expf(-gf));
        hh[i] = esc_f2h((gf * sig) * uf);
    }
    esc_w8a16(hh, d_w8, d_sc, T, H, I, sh);
    for (int t = 0; t < T; t++) {
        float acc = 0.0f;
        for (int k = 0; k < H; k++)
            acc += esc_h2f(x[(size_t)t * H + k]) * esc_h2f(shg_w[k]);
        float shg = esc_h2f(esc_f2h(acc));
        float sgate = 1.0f / (1.0f + expf(-shg));
        for (int c = 0; c < H; c++)
            out[(size_t)t * H + c] =
                esc_f2h(esc_h2f(y16[(size_t)t * H + c]) + esc_h2f(sh[(size_t)t * H + c]) * sgate);
    }
    free(g);
    free(u);
    free(hh);
    free(sh);
    return 0;
}

/* ------------------------------------------------------------------------ */
/* row grouping -- escha_mlx/moe.py:30-83 (build_groups, n_groups_bound)       */
/* stable sort of rows by expert, each expert padded to a multiple of R.      */
/* rows_idx [n_groups*R] (padding = m), group_expert [n_groups] (-1 past end) */
/* ------------------------------------------------------------------------ */

void esc_build_groups(const int32_t *row_expert, int m, int E, int R, int n_groups,
                      int32_t *rows_idx, int32_t *group_expert)
{
    int32_t *counts = (int32_t *)calloc((size_t)E, sizeof(int32_t));
    int32_t *fill = (int32_t *)calloc((size_t)E, sizeof(int32_t));
    int32_t *dst_start = (int32_t *)calloc((size_t)E, sizeof(int32_t));
    for (int i = 0; i < m; i++)
        counts[row_expert[i]]++;
    int acc = 0;
    for (int e = 0; e < E; e++) {
        dst_start[e] = acc;
        acc += ((counts[e] + R - 1) / R) * R;
    }
    int total_groups = acc / R;
    for (int i = 0; i < n_groups * R; i++)
        rows_idx[i] = m;
    for (int g = 0; g < n_groups; g++)
        group_expert[g] = -1;
    for (int i = 0; i < m; i++) { /* ascending i within an expert = stable */
        int e = row_expert[i];
        rows_idx[dst_start[e] + fill[e]++] = i;
    }
    for (int e = 0; e < E; e++)
        for (int g = dst_start[e] / R; g < (dst_start[e] + ((counts[e] + R - 1) / R) * R) / R; g++)
            if (g < n_groups && g < total_groups)
                group_expert[g] = e;
    free(counts);
    free(fill);
    free(dst_start);
}

int esc_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void esc_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0)
        omp_set_num_threads(n);
#else
    (void)n;
#endif
}
