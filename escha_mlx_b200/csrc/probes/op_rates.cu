// Per-instruction issue rates (a standalone program, not part of the library): lane-operations
// per clock and SM on sm_100a for the integer, multiply and half-precision instructions the
// trellis decode is made of, alone and in pairs that show which share a pipe; inline PTX, eight
// independent dependent chains per thread, 64 warps per SM.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o op_rates op_rates.cu
#include <cstdio>
#include <cstdint>
#include <cuda_fp16.h>

#define CH 8
#define OP1(NAME, ASM)                                                                     \
__global__ void __launch_bounds__(256) k_##NAME(uint32_t seed, uint32_t c1, uint32_t c2, int iters, uint32_t* out) { \
    uint32_t r[CH];                                                                        \
    for (int i = 0; i < CH; ++i) r[i] = seed * (threadIdx.x + 1 + i * 977);               \
    for (int it = 0; it < iters; ++it) {                                                   \
        _Pragma("unroll") for (int u = 0; u < 4; ++u)                                      \
        _Pragma("unroll") for (int i = 0; i < CH; ++i) { ASM }                             \
    }                                                                                      \
    uint32_t a = 0; for (int i = 0; i < CH; ++i) a ^= r[i];                                \
    out[blockIdx.x * blockDim.x + threadIdx.x] = a;                                        \
}

OP1(prmt,    asm volatile("prmt.b32 %0, %0, %1, 0x4421;" : "+r"(r[i]) : "r"(c1));)
OP1(prmt0,   asm volatile("prmt.b32 %0, %0, 0, 0x4421;" : "+r"(r[i]));)
OP1(shr,     asm volatile("shr.u32 %0, %0, 2;" : "+r"(r[i]));)
OP1(shl,     asm volatile("shl.b32 %0, %0, 2;" : "+r"(r[i]));)
OP1(shf,     asm volatile("shf.r.wrap.b32 %0, %0, %1, 3;" : "+r"(r[i]) : "r"(c1));)
OP1(lop3,    asm volatile("lop3.b32 %0, %0, 0x8FFF8FFF, 0x3B603B60, 0x6A;" : "+r"(r[i]));)
OP1(and_,    asm volatile("and.b32 %0, %0, %1;" : "+r"(r[i]) : "r"(c1));)
OP1(imad,    asm volatile("mul.lo.u32 %0, %0, 0xCBAC1FED;" : "+r"(r[i]));)
OP1(imadr,   asm volatile("mad.lo.u32 %0, %0, %1, %2;" : "+r"(r[i]) : "r"(c1), "r"(c2));)
OP1(mulp2r,  asm volatile("mul.lo.u32 %0, %0, %1;" : "+r"(r[i]) : "r"(c2));)
OP1(mulhi,   asm volatile("mul.hi.u32 %0, %0, %1;" : "+r"(r[i]) : "r"(c1));)
OP1(iadd,    asm volatile("add.u32 %0, %0, %1;" : "+r"(r[i]) : "r"(c1));)
OP1(dp2a,    asm volatile("dp2a.lo.u32.u32 %0, %0, %1, %2;" : "+r"(r[i]) : "r"(c1), "r"(c2));)
OP1(dp4a,    asm volatile("dp4a.u32.u32 %0, %0, %1, %2;" : "+r"(r[i]) : "r"(c1), "r"(c2));)
OP1(bfe,     asm volatile("bfe.u32 %0, %0, 6, 16;" : "+r"(r[i]));)
OP1(bfi,     asm volatile("bfi.b32 %0, %0, %1, 8, 16;" : "+r"(r[i]) : "r"(c1));)
OP1(hadd2,   asm volatile("add.rn.f16x2 %0, %0, %1;" : "+r"(r[i]) : "r"(c1));)
OP1(hfma2,   asm volatile("fma.rn.f16x2 %0, %0, %1, %2;" : "+r"(r[i]) : "r"(c1), "r"(c2));)
OP1(ffma,    asm volatile("fma.rn.f32 %0, %0, %1, %2;" : "+r"(r[i]) : "r"(c1), "r"(c2));)
OP1(mul16,   asm volatile("{.reg .u16 lo, hi; mov.b32 {lo,hi}, %0; mul.wide.u16 %0, lo, hi;}" : "+r"(r[i]));)
OP1(mul16c,  asm volatile("{.reg .u16 lo, hi; mov.b32 {lo,hi}, %0; mul.wide.u16 %0, hi, 0x1FED;}" : "+r"(r[i]));)
OP1(cvt16,   asm volatile("{.reg .u16 lo; cvt.u16.u32 lo, %0; cvt.u32.u16 %0, lo; add.u32 %0, %0, %1;}" : "+r"(r[i]) : "r"(c1));)
OP1(hadd2sel, { __half2 h = *reinterpret_cast<__half2*>(&r[i]); __half2 s = __hadd2(__low2half2(h), __high2half2(h)); r[i] = *reinterpret_cast<uint32_t*>(&s) ^ c1; })
OP1(vshr,    asm volatile("vshr.u32.u32.u32.clamp %0, %0, %1;" : "+r"(r[i]) : "r"(c2));)
OP1(popc,    asm volatile("popc.b32 %0, %0;" : "+r"(r[i]));)
OP1(imnmx,   asm volatile("min.u32 %0, %0, %1;" : "+r"(r[i]) : "r"(c1));)
// pairs to probe pipe sharing
OP1(prmt_imad, asm volatile("prmt.b32 %0, %0, %1, 0x4421; mul.lo.u32 %0, %0, 0xCBAC1FED;" : "+r"(r[i]) : "r"(c1));)
OP1(prmt_lop3, asm volatile("prmt.b32 %0, %0, %1, 0x4421; lop3.b32 %0, %0, 0x8FFF8FFF, 0x3B603B60, 0x6A;" : "+r"(r[i]) : "r"(c1));)
OP1(prmt_hadd2, asm volatile("prmt.b32 %0, %0, %1, 0x4421; add.rn.f16x2 %0, %0, %1;" : "+r"(r[i]) : "r"(c1));)
OP1(imad_hadd2, asm volatile("mul.lo.u32 %0, %0, 0xCBAC1FED; add.rn.f16x2 %0, %0, %1;" : "+r"(r[i]) : "r"(c1));)
OP1(prmt_dp2a, asm volatile("prmt.b32 %0, %0, %1, 0x4421; dp2a.lo.u32.u32 %0, %0, %1, %2;" : "+r"(r[i]) : "r"(c1), "r"(c2));)
OP1(imad_dp2a, asm volatile("mul.lo.u32 %0, %0, 0xCBAC1FED; dp2a.lo.u32.u32 %0, %0, %1, %2;" : "+r"(r[i]) : "r"(c1), "r"(c2));)
OP1(imad_ffma, asm volatile("mul.lo.u32 %0, %0, 0xCBAC1FED; fma.rn.f32 %0, %0, %1, %2;" : "+r"(r[i]) : "r"(c1), "r"(c2));)
OP1(hadd2_ffma, asm volatile("add.rn.f16x2 %0, %0, %1; fma.rn.f32 %0, %0, %1, %2;" : "+r"(r[i]) : "r"(c1), "r"(c2));)
OP1(shl_prmt, asm volatile("shl.b32 %0, %0, 2; prmt.b32 %0, %0, %1, 0x4421;" : "+r"(r[i]) : "r"(c1));)
OP1(full4, asm volatile("prmt.b32 %0, %0, %1, 0x4421; mul.lo.u32 %0, %0, 0xCBAC1FED; lop3.b32 %0, %0, 0x8FFF8FFF, 0x3B603B60, 0x6A; add.rn.f16x2 %0, %0, %1;" : "+r"(r[i]) : "r"(c1));)

template <typename F>
void run(const char* name, F kern, int nops, int sms, double ghz_nominal) {
    const int iters = 4000, blocks = sms * 8;
    uint32_t* out; cudaMalloc(&out, blocks * 256 * 4);
    kern<<<blocks, 256>>>(3, 0x01000001u, 4u, 10, out);
    cudaEvent_t a, b; cudaEventCreate(&a); cudaEventCreate(&b);
    cudaEventRecord(a);
    kern<<<blocks, 256>>>(12345, 0x01000001u, 4u, iters, out);
    cudaEventRecord(b); cudaEventSynchronize(b);
    float ms; cudaEventElapsedTime(&ms, a, b);
    double laneops = (double)blocks * 256 * iters * 4 * CH * nops;
    printf("%-12s %8.3f ms  %7.1f lane-ops/clk/SM @%.3fGHz (x%d ops)\n", name, ms,
           laneops / (ms * 1e-3) / sms / (ghz_nominal * 1e9), ghz_nominal, nops);
    cudaFree(out);
}

int main() {
    cudaDeviceProp p; cudaGetDeviceProperties(&p, 0);
    int sms = p.multiProcessorCount; double ghz = p.clockRate / 1e6;
    printf("%s sms=%d nominal %.3f GHz\n", p.name, sms, ghz);
#define R(N, n) run(#N, k_##N, n, sms, ghz)
    R(ffma,1); R(ffma,1); R(prmt,1); R(prmt0,1); R(shr,1); R(shl,1); R(shf,1); R(lop3,1); R(and_,1); R(iadd,1);
    R(imad,1); R(imadr,1); R(mulp2r,1); R(mulhi,1); R(dp2a,1); R(dp4a,1); R(bfe,1); R(bfi,1);
    R(hadd2,1); R(hfma2,1); R(hadd2sel,1); R(mul16,1); R(mul16c,1); R(cvt16,1); R(vshr,1); R(popc,1); R(imnmx,1);
    R(prmt_imad,2); R(prmt_lop3,2); R(prmt_hadd2,2); R(imad_hadd2,2); R(prmt_dp2a,2); R(imad_dp2a,2);
    R(imad_ffma,2); R(hadd2_ffma,2); R(shl_prmt,2); R(full4,4);
    return 0;
}
