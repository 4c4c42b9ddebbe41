// Checks round_pair_f16 (rllama_b200/csrc/round_f16.h) on the device against the plain conversions:
//  - the mixed-precision widening (add.rn.f32.f16 with -0) equals __half2float for all 65536 f16 bit patterns;
//  - the packed rounding equals __float2half_rn followed by __half2float for 2^26 f32 bit patterns spread over every
//    sign, exponent and leading mantissa bits (low bits from a hash), and for their negatives.
// Prints the two mismatch counts; exit status 0 when both are zero. Built and run by tests/test_gpu_ops.py.
#include <cstdio>
#include "round_f16.h"

__global__ void all_halves(unsigned long long* bad) {
    const unsigned i = blockIdx.x * blockDim.x + threadIdx.x;   // 0..65535
    const unsigned short hb = (unsigned short)i;
    float w;
    asm("add.rn.f32.f16 %0, %1, %2;" : "=f"(w) : "h"(hb), "f"(-0.0f));
    const float ref = __half2float(__ushort_as_half(hb));
    const bool both_nan = (ref != ref) && (w != w);
    if (!both_nan && __float_as_uint(w) != __float_as_uint(ref)) atomicAdd(bad, 1ull);
}

__global__ void pairs(unsigned long long n, unsigned long long* bad) {
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    for (unsigned long long i = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x; i < n; i += stride) {
        const uint32_t u = (uint32_t)(i << 6) ^ (uint32_t)((i * 0x9E3779B97F4A7C15ull) >> 58);
        float a = __uint_as_float(u), b = __uint_as_float(u ^ 0x80000000u);
        const float ra = __half2float(__float2half_rn(a)), rb = __half2float(__float2half_rn(b));
        round_pair_f16(a, b);
        const bool oka = (ra != ra && a != a) || __float_as_uint(a) == __float_as_uint(ra);
        const bool okb = (rb != rb && b != b) || __float_as_uint(b) == __float_as_uint(rb);
        if (!oka || !okb) atomicAdd(bad, 1ull);
    }
}

int main() {
    unsigned long long *bad = nullptr, h[2] = {0, 0};
    if (cudaMalloc(&bad, 16) != cudaSuccess) { printf("no device\n"); return 2; }
    cudaMemset(bad, 0, 16);
    all_halves<<<256, 256>>>(bad);
    pairs<<<148 * 8, 256>>>(1ull << 26, bad + 1);
    const cudaError_t e = cudaDeviceSynchronize();
    cudaMemcpy(h, bad, 16, cudaMemcpyDeviceToHost);
    printf("status: %s; widening mismatches: %llu; rounding mismatches: %llu\n", cudaGetErrorString(e), h[0], h[1]);
    return (e != cudaSuccess || h[0] || h[1]) ? 1 : 0;
}
