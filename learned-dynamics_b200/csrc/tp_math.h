// Per-channel arithmetic of the l<=2 Cartesian tensor products ("Bee" / "Cow" sets) and of the
// radial encodings, written once for device and host. The host build exists so that the index
// conventions can be checked on a CPU against the reference's einsum definitions
// (managan/codegen_tensor_products.py:235-249 for Bee, :279-288 for Cow) without a GPU.
//
// Operand naming follows the reference: l_0, l_1[x], l_2[x][y] (row-major 3x3), same for r.
// Output order of the Bee set: 000,110,220,011,101,121,211,022,202,112,222,111,212.
#pragma once
#include <math.h>

#if defined(__CUDACC__)
#define LD_HD __host__ __device__ __forceinline__
#else
#define LD_HD static inline
#endif

struct BeeOut {
  float y000, y110, y220;
  float y011[3], y101[3], y121[3], y211[3];
  float y022[9], y202[9], y112[9], y222[9];
  float y111[3], y212[9];
};

LD_HD void ld_cross(const float* a, const float* b, float* c) {
  c[0] = a[1] * b[2] - a[2] * b[1];
  c[1] = a[2] * b[0] - a[0] * b[2];
  c[2] = a[0] * b[1] - a[1] * b[0];
}

LD_HD void bee_fwd_point(float l0, const float* l1, const float* l2, float r0, const float* r1, const float* r2,
                         BeeOut* o) {
  o->y000 = l0 * r0;
  o->y110 = l1[0] * r1[0] + l1[1] * r1[1] + l1[2] * r1[2];
  float s = 0.f;
  for (int k = 0; k < 9; k++) s += l2[k] * r2[k];
  o->y220 = s;
  for (int x = 0; x < 3; x++) {
    o->y011[x] = l0 * r1[x];
    o->y101[x] = l1[x] * r0;
    // 121: l_x r_yx -> y
    o->y121[x] = l1[0] * r2[x * 3 + 0] + l1[1] * r2[x * 3 + 1] + l1[2] * r2[x * 3 + 2];
    // 211: l_xy r_y -> x
    o->y211[x] = l2[x * 3 + 0] * r1[0] + l2[x * 3 + 1] * r1[1] + l2[x * 3 + 2] * r1[2];
  }
  for (int k = 0; k < 9; k++) {
    o->y022[k] = l0 * r2[k];
    o->y202[k] = l2[k] * r0;
  }
  for (int x = 0; x < 3; x++)
    for (int y = 0; y < 3; y++) {
      o->y112[x * 3 + y] = l1[x] * r1[y];
      // 222: l_xy r_zy -> xz
      o->y222[x * 3 + y] = l2[x * 3 + 0] * r2[y * 3 + 0] + l2[x * 3 + 1] * r2[y * 3 + 1] + l2[x * 3 + 2] * r2[y * 3 + 2];
    }
  // 111: l_x r_y eps_xyz -> z  (cross product)
  ld_cross(l1, r1, o->y111);
  // 212: l_xy r_z eps_yzw -> xw  (row-wise cross product)
  for (int x = 0; x < 3; x++) ld_cross(l2 + 3 * x, r1, o->y212 + 3 * x);
}

// Adjoint with respect to the left operands, given the right operands and all 13 output grads.
LD_HD void bee_bwl_point(float r0, const float* r1, const float* r2, const BeeOut* g, float* dl0, float* dl1, float* dl2) {
  float a = g->y000 * r0;
  for (int x = 0; x < 3; x++) a += g->y011[x] * r1[x];
  for (int k = 0; k < 9; k++) a += g->y022[k] * r2[k];
  *dl0 = a;
  float c[3];
  ld_cross(r1, g->y111, c);
  for (int x = 0; x < 3; x++) {
    float v = g->y110 * r1[x] + g->y101[x] * r0 + c[x];
    for (int y = 0; y < 3; y++) v += g->y121[y] * r2[y * 3 + x] + g->y112[x * 3 + y] * r1[y];
    dl1[x] = v;
  }
  for (int x = 0; x < 3; x++) {
    float cc[3];
    ld_cross(r1, g->y212 + 3 * x, cc);
    for (int y = 0; y < 3; y++) {
      float v = g->y220 * r2[x * 3 + y] + g->y211[x] * r1[y] + g->y202[x * 3 + y] * r0 + cc[y];
      for (int z = 0; z < 3; z++) v += g->y222[x * 3 + z] * r2[z * 3 + y];
      dl2[x * 3 + y] = v;
    }
  }
}

// Adjoint with respect to the right operands, given the left operands and all 13 output grads.
LD_HD void bee_bwr_point(float l0, const float* l1, const float* l2, const BeeOut* g, float* dr0, float* dr1, float* dr2) {
  float a = g->y000 * l0;
  for (int x = 0; x < 3; x++) a += g->y101[x] * l1[x];
  for (int k = 0; k < 9; k++) a += g->y202[k] * l2[k];
  *dr0 = a;
  float c[3];
  ld_cross(g->y111, l1, c);
  float c2[3] = {0.f, 0.f, 0.f};
  for (int x = 0; x < 3; x++) {
    float t[3];
    ld_cross(g->y212 + 3 * x, l2 + 3 * x, t);
    c2[0] += t[0]; c2[1] += t[1]; c2[2] += t[2];
  }
  for (int y = 0; y < 3; y++) {
    float v = g->y110 * l1[y] + g->y011[y] * l0 + c[y] + c2[y];
    for (int x = 0; x < 3; x++) v += g->y211[x] * l2[x * 3 + y] + g->y112[x * 3 + y] * l1[x];
    dr1[y] = v;
  }
  for (int z = 0; z < 3; z++)
    for (int y = 0; y < 3; y++) {
      float v = g->y220 * l2[z * 3 + y] + g->y121[z] * l1[y] + g->y022[z * 3 + y] * l0;
      for (int x = 0; x < 3; x++) v += g->y222[x * 3 + z] * l2[x * 3 + y];
      dr2[z * 3 + y] = v;
    }
}

// ---- radial encodings -------------------------------------------------------------------------
// kind 0: PaiNN cos/sin (archs/meanflow_painn8.py:25-35): hn=(n+1)/2 cosines then n-hn sines,
//         wavenumber (pi/rmax)*(1 + m/2) (integer division).
// kind 1: Gaussian basis x cosine cutoff (asked for by the benchmark configs, not in the
//         reference): centres mu_m = m*rmax/(n-1), width rmax/(n-1),
//         exp(-0.5*((d-mu)/width)^2) * 0.5*(cos(pi*d/rmax)+1) for d<rmax else 0.
// pi_over_rmax is float(pi/rmax) evaluated in double by the host, as torch does for the scalar.
LD_HD float radial_feature(int kind, int m, int n, float d, float rmax, float pi_over_rmax) {
  const float pi = 3.14159265358979323846f;
  if (kind == 0) {
    const int hn = (n + 1) / 2;
    if (m < hn) {
      float coef = pi_over_rmax * (float)(1 + m / 2);
      return cosf(coef * d);
    }
    float coef = pi_over_rmax * (float)(1 + (m - hn) / 2);
    return sinf(coef * d);
  }
  float width = n > 1 ? rmax / (float)(n - 1) : rmax;
  float mu = (float)m * width;
  float u = (d - mu) / width;
  float env = d < rmax ? 0.5f * (cosf(pi * d / rmax) + 1.0f) : 0.f;
  return expf(-0.5f * u * u) * env;
}

LD_HD float silu_f(float x) { return x / (1.0f + expf(-x)); }

// Polynomial radial basis of managan/jacobi_radenc.py:27-33: enc[m] = env * sum_p coeff[m][p] z^p for an 8x9
// coefficient matrix (the shifted Jacobi(1,0) polynomials there), z in [0, 1]. The monomial coefficients reach 2.7e4
// with alternating signs, so a float32 power sum loses four digits to cancellation (the reference's own float32
// evaluation is 2.4e-4 off the exact value of a basis function of size 1). Here each polynomial is re-expressed once,
// in double, in the Chebyshev basis of t = 2z - 1 (coefficients of order 1) and evaluated per edge by Clenshaw's
// recurrence in float32: error about 2e-6 of a basis function of size 8, at 16 FMAs per function.
LD_HD void ld_poly8_to_chebyshev(const float* a, float* c) {
  double p[10], q[10];
  for (int n = 0; n < 10; n++) p[n] = 0.0;
  p[0] = (double)a[8];
  for (int k = 7; k >= 0; k--) {
    // q = p * z with z = (t + 1) / 2;  t T_0 = T_1,  t T_n = (T_{n+1} + T_{n-1}) / 2
    for (int n = 0; n < 10; n++) q[n] = 0.0;
    q[1] += p[0];
    for (int n = 1; n < 9; n++) { q[n + 1] += 0.5 * p[n]; q[n - 1] += 0.5 * p[n]; }
    for (int n = 0; n < 10; n++) p[n] = 0.5 * (q[n] + p[n]);
    p[0] += (double)a[k];
  }
  for (int n = 0; n < 9; n++) c[n] = (float)p[n];
}

// one polynomial of the Chebyshev form: t = 2z - 1, t2 = 2t, c its nine coefficients
LD_HD float ld_cheb9(float t, float t2, const float* c) {
  float b1 = 0.f, b2 = 0.f;
  for (int k = 8; k >= 1; k--) {
    const float b0 = fmaf(t2, b1, c[k] - b2);
    b2 = b1; b1 = b0;
  }
  return fmaf(t, b1, c[0]) - b2;
}

LD_HD void ld_radial_cheb8(float z, float env, const float* cheb, float* enc) {
  const float t = 2.f * z - 1.f, t2 = 2.f * t;
  for (int m = 0; m < 8; m++) {
    const float* c = cheb + m * 9;
    float b1 = 0.f, b2 = 0.f;
    for (int k = 8; k >= 1; k--) {
      const float b0 = fmaf(t2, b1, c[k] - b2);
      b2 = b1; b1 = b0;
    }
    enc[m] = (fmaf(t, b1, c[0]) - b2) * env;
  }
}
