// Counter-based Gaussian noise for sharded rollouts: element i of step t is a pure function of
// (seed, t, i), so a rank that owns systems [b0, b1) draws exactly the values a single-GPU run draws
// for those systems, whatever the number of ranks. The reference draws torch.randn_like per step
// (archs/meanflow_painn8.py:302-310), whose stream depends on how the batch is split.
//   x = seed*C1 + step*C2 + index (64-bit, wrapping); x = splitmix64 finaliser(x)
//   u1 = (bits 40..63 + 1) / 2^24 in (0, 1], u2 = bits 16..39 / 2^24 in [0, 1)
//   z = sqrt(-2 ln u1) * cos(2 pi u2)                       (Box-Muller, float32)
// ld_b200.sharding.counter_noise_torch is the same arithmetic in torch integer ops (CPU or CUDA).
#include "common.cuh"

namespace {

__device__ __forceinline__ unsigned long long mix64(unsigned long long x) {
  x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull;
  x ^= x >> 27; x *= 0x94D049BB133111EBull;
  x ^= x >> 31;
  return x;
}

__global__ void counter_noise_kernel(float* __restrict__ out, const float* __restrict__ base, float scale,
                                     unsigned long long first, long long count, unsigned long long seed,
                                     unsigned long long step) {
  const unsigned long long key = seed * 0x9E3779B97F4A7C15ull + step * 0xBF58476D1CE4E5B9ull;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x) {
    const unsigned long long x = mix64(key + first + (unsigned long long)i);
    const float u1 = (float)((x >> 40) + 1ull) * (1.0f / 16777216.0f);
    const float u2 = (float)((x >> 16) & 0xFFFFFFull) * (1.0f / 16777216.0f);
    const float z = sqrtf(-2.0f * logf(u1)) * cosf(6.283185307179586f * u2);
    out[i] = base != nullptr ? fmaf(scale, z, base[i]) : scale * z;
  }
}

}  // namespace

// out[i] = base[i] + scale * z(seed, step, first_element + i) for i in [0, count); base may be NULL (then out = scale*z).
extern "C" int ld_counter_noise(float* out, const float* base, float scale, long long first_element, long long count,
                                unsigned long long seed, unsigned long long step, void* stream) {
  if (count < 0 || first_element < 0) return LD_ERR_SHAPE;
  if (count == 0) return LD_OK;
  long long blocks = ld_cdiv(count, 256);
  if (blocks > 148LL * 8) blocks = 148LL * 8;
  counter_noise_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(out, base, scale, (unsigned long long)first_element, count,
                                                                      seed, step);
  LD_LAUNCH_CHECK();
  return LD_OK;
}
