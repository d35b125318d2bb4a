// Benchmark support kernels: synthetic fp16 fill and a read-bandwidth probe.
#include <cuda_fp16.h>
#include <stdint.h>

namespace vteb {

__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

}  // namespace vteb

// Element pair (2i, 2i+1) gets the two Box-Muller normals of hash(seed, i).
extern "C" __global__ void vteb_fill_normal_f16_kernel(
    __half* __restrict__ dst, unsigned long long n, unsigned long long seed,
    float sigma, float outlier_prob, float outlier_scale)
{
    const unsigned long long pairs = (n + 1) / 2;
    for (unsigned long long i = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x; i < pairs;
         i += (unsigned long long)gridDim.x * blockDim.x) {
        const uint64_t h = vteb::mix64(seed * 0xD1342543DE82EF95ull + i);
        const uint64_t h2 = vteb::mix64(h);
        const float u1 = ((uint32_t)(h >> 40) + 1.0f) * (1.0f / 16777217.0f);   // (0, 1)
        const float u2 = (uint32_t)(h & 0xFFFFFF) * (1.0f / 16777216.0f);       // [0, 1)
        const float r = sqrtf(-2.0f * __logf(u1)) * sigma;
        float s, c;
        __sincosf(6.283185307179586f * u2, &s, &c);
        float a = r * c, b = r * s;
        if (outlier_prob > 0.f) {
            if ((uint32_t)(h2 & 0xFFFFFF) * (1.0f / 16777216.0f) < outlier_prob) a *= outlier_scale;
            if ((uint32_t)((h2 >> 24) & 0xFFFFFF) * (1.0f / 16777216.0f) < outlier_prob) b *= outlier_scale;
        }
        if (2 * i + 1 < n) {
            *reinterpret_cast<__half2*>(dst + 2 * i) = __floats2half2_rn(a, b);
        } else {
            dst[2 * i] = __float2half(a);
        }
    }
}

// Each CTA streams a contiguous slice with 128-bit loads, several in flight per
// thread, and leaves an XOR checksum so the loads cannot be dropped.
extern "C" __global__ void __launch_bounds__(512) vteb_read_bandwidth_kernel(
    const uint4* __restrict__ src, unsigned long long n_vec, unsigned* __restrict__ sink)
{
    const unsigned long long per_cta = (n_vec + gridDim.x - 1) / gridDim.x;
    const unsigned long long lo = blockIdx.x * per_cta;
    const unsigned long long hi = (lo + per_cta < n_vec) ? lo + per_cta : n_vec;
    uint4 acc = make_uint4(0, 0, 0, 0);
    unsigned long long i = lo + threadIdx.x;
    for (; i + 3ull * blockDim.x < hi; i += 4ull * blockDim.x) {
        const uint4 a = __ldg(src + i), b = __ldg(src + i + blockDim.x);
        const uint4 c = __ldg(src + i + 2ull * blockDim.x), d = __ldg(src + i + 3ull * blockDim.x);
        acc.x ^= a.x ^ b.x ^ c.x ^ d.x; acc.y ^= a.y ^ b.y ^ c.y ^ d.y;
        acc.z ^= a.z ^ b.z ^ c.z ^ d.z; acc.w ^= a.w ^ b.w ^ c.w ^ d.w;
    }
    for (; i < hi; i += blockDim.x) {
        const uint4 a = __ldg(src + i);
        acc.x ^= a.x; acc.y ^= a.y; acc.z ^= a.z; acc.w ^= a.w;
    }
    unsigned v = acc.x ^ acc.y ^ acc.z ^ acc.w;
    for (int off = 16; off > 0; off >>= 1) v ^= __shfl_xor_sync(0xffffffffu, v, off);
    if ((threadIdx.x & 31) == 0) atomicXor(sink + blockIdx.x, v);
}
