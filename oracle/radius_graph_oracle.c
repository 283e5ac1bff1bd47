/* TEST INFRASTRUCTURE ONLY - never linked or called by the product path.
 *
 * Brute-force O(N^2) CPU restatement of the reference's radius-graph membership rule
 * (extensions/neighbour_grid/neighbour_grid_kern.cu:39-48 wrap and minimum image, :57-93 cell
 * assignment, :95-150 predicate `self.index != other.index && dot(delta,delta) <= r0sq`;
 * extensions/neighbour_grid/neighbour_grid.cpp:78-82 `ndiv = ceil(box/cutoff)`, :180-194 edge
 * order system-major then node). The reference's `dot` leaves FMA contraction to the compiler, so
 * this file fixes the canonical form d2 = fmaf(dz,dz, fmaf(dy,dy, dx*dx)) that the CUDA kernels
 * use too. Build with -ffp-contract=off so nothing else is fused.
 *
 * mode 0: every pair with d2 <= rc^2 (exact).
 * mode 1: additionally require the two particles' cells (reference grid) to be within the
 *         3x3x3 window, reproducing the pairs the reference misses when box/cutoff is not an
 *         integer.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

static float wrap_pos(float x, float box) {
  float h = 0.5f * box;
  return remainderf(x - h, box) + h;
}

static int periodic_cell(float p, float box, int ndiv) {
  float t = (float)ndiv * p;
  int c = (int)(t / box);
  c %= ndiv;
  if (c < 0) c += ndiv;
  return c;
}

static int cells_adjacent(int a, int b, int ndiv) {
  int d = a - b;
  d %= ndiv;
  if (d < 0) d += ndiv;
  return d == 0 || d == 1 || d == ndiv - 1;
}

static float torch_mod_wrap(float d, float box) {
  float h = 0.5f * box;
  float t = d + h;
  float m = fmodf(t, box);
  if (m != 0.f && m < 0.f) m = m + box;
  return m - h;
}

/* Returns the number of directed edges; writes up to `capacity` of them ordered by (system, i, j).
 * src/dst are global node ids b*N+i. shift packs three signed bytes; rij is [E,3]. Any output
 * pointer may be NULL. */
long long oracle_radius_graph(const float* pos, int batch, int nodes, int periodic, float cutoff,
                              const float* box, int mode, long long capacity, int32_t* src, int32_t* dst,
                              int32_t* shift, float* rij, int32_t* degree) {
  const float rc2 = cutoff * cutoff;
  long long e = 0;
  int nd[3] = {1, 1, 1};
  if (periodic && mode == 1)
    for (int a = 0; a < 3; a++) nd[a] = (int)ceilf(box[a] / cutoff);
  float* p = (float*)malloc(sizeof(float) * 3 * (size_t)(nodes > 0 ? nodes : 1));
  int* cell = (int*)malloc(sizeof(int) * 3 * (size_t)(nodes > 0 ? nodes : 1));
  for (int b = 0; b < batch; b++) {
    const float* x = pos + (size_t)b * nodes * 3;
    for (int i = 0; i < nodes; i++)
      for (int a = 0; a < 3; a++) {
        float v = x[i * 3 + a];
        if (periodic) {
          v = wrap_pos(v, box[a]);
          cell[i * 3 + a] = (mode == 1) ? periodic_cell(v, box[a], nd[a]) : 0;
        }
        p[i * 3 + a] = v;
      }
    for (int i = 0; i < nodes; i++) {
      int deg = 0;
      for (int j = 0; j < nodes; j++) {
        if (i == j) continue;
        float dx = p[i * 3 + 0] - p[j * 3 + 0];
        float dy = p[i * 3 + 1] - p[j * 3 + 1];
        float dz = p[i * 3 + 2] - p[j * 3 + 2];
        if (periodic) {
          dx = remainderf(dx, box[0]);
          dy = remainderf(dy, box[1]);
          dz = remainderf(dz, box[2]);
        }
        float d2 = fmaf(dz, dz, fmaf(dy, dy, dx * dx));
        if (!(d2 <= rc2)) continue;
        if (periodic && mode == 1) {
          if (!(cells_adjacent(cell[i * 3], cell[j * 3], nd[0]) && cells_adjacent(cell[i * 3 + 1], cell[j * 3 + 1], nd[1]) &&
                cells_adjacent(cell[i * 3 + 2], cell[j * 3 + 2], nd[2])))
            continue;
        }
        if (e < capacity) {
          if (src) src[e] = b * nodes + i;
          if (dst) dst[e] = b * nodes + j;
          float d[3];
          int s[3] = {0, 0, 0};
          for (int a = 0; a < 3; a++) {
            d[a] = x[j * 3 + a] - x[i * 3 + a];
            if (periodic) {
              float h = 0.5f * box[a];
              float t = d[a] + h;
              s[a] = -(int)floorf(t / box[a]);
              d[a] = torch_mod_wrap(d[a], box[a]);
            }
          }
          if (shift) shift[e] = (s[0] & 0xff) | ((s[1] & 0xff) << 8) | ((s[2] & 0xff) << 16);
          if (rij) { rij[e * 3] = d[0]; rij[e * 3 + 1] = d[1]; rij[e * 3 + 2] = d[2]; }
        }
        e++;
        deg++;
      }
      if (degree) degree[b * nodes + i] = deg;
    }
  }
  free(p);
  free(cell);
  return e;
}
