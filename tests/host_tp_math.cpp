// Test harness: exposes the host build of csrc/tp_math.h so the per-channel product formulas and
// their adjoints can be checked on a CPU against einsum + autograd.
#include "tp_math.h"
extern "C" {
void host_bee_fwd(const float* l0, const float* l1, const float* l2, const float* r0, const float* r1, const float* r2,
                  int n, float* out /* n*63 */) {
  for (int i = 0; i < n; i++) {
    BeeOut o;
    bee_fwd_point(l0[i], l1 + 3 * i, l2 + 9 * i, r0[i], r1 + 3 * i, r2 + 9 * i, &o);
    const float* p = (const float*)&o;
    for (int k = 0; k < 63; k++) out[i * 63 + k] = p[k];
  }
}
void host_bee_bw(int left, const float* o0, const float* o1, const float* o2, const float* g /* n*63 */, int n, float* d /* n*13 */) {
  for (int i = 0; i < n; i++) {
    BeeOut go;
    float* p = (float*)&go;
    for (int k = 0; k < 63; k++) p[k] = g[i * 63 + k];
    if (left) bee_bwl_point(o0[i], o1 + 3 * i, o2 + 9 * i, &go, d + 13 * i, d + 13 * i + 1, d + 13 * i + 4);
    else bee_bwr_point(o0[i], o1 + 3 * i, o2 + 9 * i, &go, d + 13 * i, d + 13 * i + 1, d + 13 * i + 4);
  }
}
void host_radial(int kind, int n, float rmax, const float* d, int count, float* out) {
  const float pr = (float)(3.14159265358979323846 / (double)rmax);
  for (int i = 0; i < count; i++)
    for (int m = 0; m < n; m++) out[i * n + m] = radial_feature(kind, m, n, d[i], rmax, pr);
}
}
