// Edge radial encodings as a standalone operator: r[rows, 3] (or r[rows] for the scalar form) -> out[rows, n].
//   kind 0  cos/sin pairs of archs/meanflow_painn8.py:25-35
//   kind 1  Gaussian basis x cosine cutoff (asked for by the benchmark configs; not in the reference)
//   kind 2  radial_encode_edge of archs/diffuser_atoms5.py:25-30: cos(m*pi*sqrt(|r|^2/rmax)) * relu(1 - |r|^2/rmax)
//   kind 3  radial_encode of managan/layers_common.py:122-126: cos(pi*m*r) for a scalar r (rmax unused)
//   kind 4  radial_encode_8 of managan/jacobi_radenc.py:27-33 (n = 8, 8x9 coefficient matrix)
// The fused message kernels evaluate kinds 0, 1 and 4 in place (tp_math.h); this entry point exists for callers that
// want the encoding itself (older archs feed it to their own layers). One thread per output element; the kernel is
// bound by its 4*n bytes of output per row.
#include "common.cuh"
#include "tp_math.h"

namespace {

__global__ void radial_encode_kernel(int kind, const float* __restrict__ r, long long rows, int n, float rmax,
                                     float pi_over_rmax, const float* __restrict__ coeff, float* __restrict__ out) {
  __shared__ float s_cheb[72];
  if (kind == 4) {
    if (threadIdx.x < 8) ld_poly8_to_chebyshev(coeff + threadIdx.x * 9, s_cheb + threadIdx.x * 9);
    __syncthreads();
  }
  const long long total = rows * n;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / n;
    const int m = (int)(i - row * n);
    float v;
    if (kind == 3) {
      const float npi = (float)m * 3.14159265358979323846f;   // float32(pi) * m, as torch.pi * arange(n) evaluates
      v = cosf(npi * r[row]);
    } else {
      const float x = r[row * 3], y = r[row * 3 + 1], z = r[row * 3 + 2];
      const float sq = x * x + y * y + z * z;
      if (kind == 2) {
        const float xs = sq / rmax;
        const float npi = (float)m * 3.14159265358979323846f;
        v = cosf(npi * sqrtf(xs)) * fmaxf(1.f - xs, 0.f);
      } else if (kind == 4) {
        const float zz = sqrtf(sq) / rmax;
        const float t = 2.f * zz - 1.f, t2 = 2.f * t;
        const float* c = s_cheb + m * 9;
        float b1 = 0.f, b2 = 0.f;
        for (int k = 8; k >= 1; k--) { const float b0 = fmaf(t2, b1, c[k] - b2); b2 = b1; b1 = b0; }
        v = (fmaf(t, b1, c[0]) - b2) * fmaxf(1.f - zz, 0.f);
      } else {
        v = radial_feature(kind, m, n, sqrtf(sq), rmax, pi_over_rmax);
      }
    }
    out[i] = v;
  }
}

}  // namespace

extern "C" int ld_radial_encode(int kind, const float* r, long long rows, int n, float rmax, const float* coeff, float* out,
                                void* stream) {
  if (kind < 0 || kind > 4 || rows < 0 || n <= 0) return LD_ERR_SHAPE;
  if (kind != 3 && !(rmax > 0.f)) return LD_ERR_SHAPE;
  if (kind == 4 && (n != 8 || coeff == nullptr)) { ld_set_last_message("radial encode: the polynomial basis needs n = 8 and its 8x9 coefficients"); return LD_ERR_SHAPE; }
  if (rows == 0) return LD_OK;
  const long long total = rows * n;
  long long blocks = ld_cdiv(total, 256);
  if (blocks > 148LL * 16) blocks = 148LL * 16;
  const float pi_over_rmax = kind == 3 ? 0.f : (float)(3.14159265358979323846 / (double)rmax);
  radial_encode_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(kind, r, rows, n, rmax, pi_over_rmax, coeff, out);
  LD_LAUNCH_CHECK();
  return LD_OK;
}
