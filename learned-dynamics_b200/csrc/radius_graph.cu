// Cell-list radius graph for batches of independent systems (periodic or open boundaries).
//
// Replaces the reference's extensions/neighbour_grid (neighbour_grid_kern.cu:57-150, 334-352 and
// neighbour_grid.cpp:59-103, 170-195). Differences in design, not in result:
//   * no per-call cudaMalloc / device sync: the caller owns one workspace;
//   * cells are filled with warp-aggregated atomics and then sorted by particle index, so the
//     edge order is deterministic (the reference's order depends on atomic arrival);
//   * two passes (count, prefix sum, fill) write a CSR directly: no padded [B,N,neighboursmax]
//     intermediate and no per-node capacity;
//   * one warp per particle tests 32 candidates per step and writes compacted, coalesced runs.
//
// Membership predicate (float32, fixed operation order so a CPU restatement is bit-exact):
//   periodic: p = remainderf(x - box/2, box) + box/2 for both particles,
//             d = remainderf(p_i - p_j, box) per axis
//   open:     d = x_i - x_j
//   edge  <=> i != j  and  fmaf(dz,dz, fmaf(dy,dy, dx*dx)) <= cutoff*cutoff
#include "common.cuh"
#include <math.h>

namespace {

struct GridDesc {
  float ox, oy, oz;     // origin of cell (0,0,0)
  float sx, sy, sz;     // open: cells per unit length; periodic: unused
  int nx, ny, nz;       // cells per axis
  int pad0, pad1, pad2;
};

struct GraphParams {
  int batch, nodes;
  int periodic;         // 1: periodic box, 0: open
  int mode;             // 0 exact, 1 reference-compatible cell grid (periodic only)
  float cutoff, rc2;
  float bx, by, bz;     // periodic box
  int nx, ny, nz;       // periodic cell grid
  int cells_cap;        // cells reserved per system
};

__device__ __forceinline__ bool finite3(float x, float y, float z) {
  return isfinite(x) && isfinite(y) && isfinite(z);
}

__device__ __forceinline__ float wrap_pos(float x, float box) {
  // same form as the reference's assignParticlesToCells: boxwrap(x - h) + h
  float h = __fmul_rn(0.5f, box);
  return __fadd_rn(remainderf(__fsub_rn(x, h), box), h);
}

__device__ __forceinline__ int periodic_cell(float p, float box, int ndiv) {
  // (int)(ndiv*pos/box) % ndiv with explicit rounding at every step
  int c = (int)__fdiv_rn(__fmul_rn((float)ndiv, p), box);
  c %= ndiv;
  if (c < 0) c += ndiv;
  return c;
}

__device__ __forceinline__ int open_cell(float x, float origin, float scale, int ndiv) {
  int c = (int)__fmul_rn(__fsub_rn(x, origin), scale);
  return min(max(c, 0), ndiv - 1);
}

// One block per system. Open boundary: bounding box -> cell grid with edge >= cutoff*(1+1e-5).
__global__ void grid_setup_kernel(const float* __restrict__ pos, GraphParams P, GridDesc* __restrict__ desc,
                                  int* __restrict__ status) {
  const int b = blockIdx.x;
  __shared__ float red[6][32];
  __shared__ int bad;
  if (threadIdx.x == 0) bad = 0;
  __syncthreads();
  float lo[3] = {INFINITY, INFINITY, INFINITY}, hi[3] = {-INFINITY, -INFINITY, -INFINITY};
  int mybad = 0;
  for (int i = threadIdx.x; i < P.nodes; i += blockDim.x) {
    const float* p = pos + ((size_t)b * P.nodes + i) * 3;
    float x = p[0], y = p[1], z = p[2];
    if (finite3(x, y, z)) {
      lo[0] = fminf(lo[0], x); hi[0] = fmaxf(hi[0], x);
      lo[1] = fminf(lo[1], y); hi[1] = fmaxf(hi[1], y);
      lo[2] = fminf(lo[2], z); hi[2] = fmaxf(hi[2], z);
    } else {
      mybad = 1;
    }
  }
  if (mybad) bad = 1;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
  for (int a = 0; a < 3; a++) {
    for (int d = 16; d > 0; d >>= 1) {
      lo[a] = fminf(lo[a], __shfl_xor_sync(0xffffffffu, lo[a], d));
      hi[a] = fmaxf(hi[a], __shfl_xor_sync(0xffffffffu, hi[a], d));
    }
    if (lane == 0) { red[a][w] = lo[a]; red[3 + a][w] = hi[a]; }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (bad) atomicOr(status, LD_FLAG_NONFINITE);
    GridDesc g;
    g.pad0 = g.pad1 = g.pad2 = 0;
    if (P.periodic) {
      g.ox = g.oy = g.oz = 0.f;
      g.sx = g.sy = g.sz = 0.f;
      g.nx = P.nx; g.ny = P.ny; g.nz = P.nz;
    } else {
      const int nw = blockDim.x >> 5;
      float mn[3], mx[3];
      for (int a = 0; a < 3; a++) {
        mn[a] = INFINITY; mx[a] = -INFINITY;
        for (int k = 0; k < nw; k++) { mn[a] = fminf(mn[a], red[a][k]); mx[a] = fmaxf(mx[a], red[3 + a][k]); }
        if (!(mn[a] <= mx[a])) { mn[a] = 0.f; mx[a] = 0.f; }  // no finite particle
      }
      const float edge = P.cutoff * 1.00001f;
      int nd[3];
      float ext[3];
      for (int a = 0; a < 3; a++) {
        ext[a] = mx[a] - mn[a];
        float q = floorf(ext[a] / edge);
        nd[a] = (int)fminf(fmaxf(q, 1.f), 1024.f);
      }
      double prod = (double)nd[0] * nd[1] * nd[2];
      if (prod > (double)P.cells_cap) {
        float f = cbrtf((float)((double)P.cells_cap / prod));
        for (int a = 0; a < 3; a++) nd[a] = max(1, (int)floorf(nd[a] * f));
        // coarsening one axis at a time keeps every cell edge >= cutoff
        while ((long long)nd[0] * nd[1] * nd[2] > P.cells_cap) {
          int a = (nd[0] >= nd[1] && nd[0] >= nd[2]) ? 0 : (nd[1] >= nd[2] ? 1 : 2);
          nd[a] = max(1, nd[a] - 1);
        }
      }
      g.ox = mn[0]; g.oy = mn[1]; g.oz = mn[2];
      g.sx = ext[0] > 0.f ? (float)nd[0] / ext[0] : 0.f;
      g.sy = ext[1] > 0.f ? (float)nd[1] / ext[1] : 0.f;
      g.sz = ext[2] > 0.f ? (float)nd[2] / ext[2] : 0.f;
      g.nx = nd[0]; g.ny = nd[1]; g.nz = nd[2];
    }
    desc[b] = g;
  }
}

__device__ __forceinline__ int cell_of(const GraphParams& P, const GridDesc& g, float x, float y, float z,
                                       float* px, float* py, float* pz) {
  if (!finite3(x, y, z)) { *px = x; *py = y; *pz = z; return 0; }
  int cx, cy, cz;
  if (P.periodic) {
    x = wrap_pos(x, P.bx); y = wrap_pos(y, P.by); z = wrap_pos(z, P.bz);
    cx = periodic_cell(x, P.bx, g.nx); cy = periodic_cell(y, P.by, g.ny); cz = periodic_cell(z, P.bz, g.nz);
  } else {
    cx = open_cell(x, g.ox, g.sx, g.nx); cy = open_cell(y, g.oy, g.sy, g.ny); cz = open_cell(z, g.oz, g.sz, g.nz);
  }
  *px = x; *py = y; *pz = z;
  return (cx * g.ny + cy) * g.nz + cz;
}

// Pass 1 (FILL=false): count particles per cell. Pass 2 (FILL=true): place them, warp-aggregated.
template <bool FILL>
__global__ void bin_kernel(const float* __restrict__ pos, GraphParams P, const GridDesc* __restrict__ desc,
                           int* __restrict__ cell_count, const int* __restrict__ cell_start,
                           int* __restrict__ cell_cursor, float4* __restrict__ binned, int* __restrict__ binned_cell) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int total = P.batch * P.nodes;
  const bool active = i < total;
  int gcell = -1;
  float x = 0.f, y = 0.f, z = 0.f;
  int local = 0;
  if (active) {
    const int b = i / P.nodes;
    local = i - b * P.nodes;
    const GridDesc g = desc[b];
    const float* p = pos + (size_t)i * 3;
    int c = cell_of(P, g, p[0], p[1], p[2], &x, &y, &z);
    gcell = b * P.cells_cap + c;
  }
  const unsigned amask = __ballot_sync(0xffffffffu, active);
  if (!active) return;
  const unsigned peers = __match_any_sync(amask, gcell);
  const int lane = threadIdx.x & 31;
  const int leader = __ffs(peers) - 1;
  const int rank = __popc(peers & ((1u << lane) - 1));
  if (!FILL) {
    if (lane == leader) atomicAdd(&cell_count[gcell], __popc(peers));
  } else {
    int base = 0;
    if (lane == leader) base = atomicAdd(&cell_cursor[gcell], __popc(peers));
    base = __shfl_sync(peers, base, leader);
    const int slot = cell_start[gcell] + base + rank;
    binned[slot] = make_float4(x, y, z, __int_as_float(local));
    binned_cell[slot] = gcell;
  }
}

// Deterministic order inside every cell: ascending particle index (rank by counting).
__global__ void cell_sort_kernel(const float4* __restrict__ binned, const int* __restrict__ binned_cell,
                                 const int* __restrict__ cell_start, int total,
                                 float4* __restrict__ sorted, int* __restrict__ sorted_cell) {
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= total) return;
  const int c = binned_cell[s];
  const int lo = cell_start[c], hi = cell_start[c + 1];
  const float4 me = binned[s];
  const int my = __float_as_int(me.w);
  int rank = 0;
  for (int k = lo; k < hi; k++) rank += (__float_as_int(binned[k].w) < my) ? 1 : 0;
  sorted[lo + rank] = me;
  sorted_cell[lo + rank] = c;
}

__device__ __forceinline__ float torch_mod_wrap(float d, float box) {
  // ((d + 0.5*box) % box) - 0.5*box with torch's floor-mod for floats
  float h = __fmul_rn(0.5f, box);
  float t = __fadd_rn(d, h);
  float m = fmodf(t, box);
  if (m != 0.f && m < 0.f) m = __fadd_rn(m, box);
  return __fsub_rn(m, h);
}

constexpr int NB_WARPS = 8;

// minimum image of a difference of two wrapped coordinates, d in [-box, box]. Bit-identical to
// remainderf(d, box) there: the quotient is -1, 0 or +1 (ties at +-box/2 go to the even quotient 0)
// and d -+ box is exact (Sterbenz), so two compares replace the library routine.
__device__ __forceinline__ float min_image(float d, float box, float half) {
  if (d > half) return __fsub_rn(d, box);
  if (d < -half) return __fadd_rn(d, box);
  return d;
}

// ((d + 0.5*box) % box) - 0.5*box with torch's floor-mod; fast exact paths for |d + box/2| < 2*box
__device__ __forceinline__ float torch_mod_wrap_fast(float d, float box, float half) {
  const float t = __fadd_rn(d, half);
  float m;
  if (t >= 0.f && t < box) m = t;                                   // fmod(t, box) = t
  else if (t >= box && t < __fadd_rn(box, box)) m = __fsub_rn(t, box);   // exact
  else if (t < 0.f && t > -box) m = __fadd_rn(t, box);              // fmod = t (negative) then + box, as torch does
  else {
    m = fmodf(t, box);
    if (m != 0.f && m < 0.f) m = __fadd_rn(m, box);
  }
  return __fsub_rn(m, half);
}

// One warp per particle (in cell order). FILL=false: degree per node. FILL=true: write the edges.
// Candidates: the 3x3 neighbouring cell columns in (x, y); along z the cells cz-1, cz, cz+1 are
// consecutive in the cell-sorted particle array, so each column is one contiguous run (two when it
// wraps around the box): at most 18 runs, walked 32 candidates at a time.
template <bool FILL>
__global__ void __launch_bounds__(NB_WARPS * 32)
neighbour_kernel(const float* __restrict__ pos, GraphParams P, const GridDesc* __restrict__ desc,
                 const int* __restrict__ cell_start, const float4* __restrict__ sorted,
                 const int* __restrict__ sorted_cell, int* __restrict__ degree, const int* __restrict__ row_ptr,
                 long long capacity, int* __restrict__ src, int* __restrict__ dst, int* __restrict__ shift,
                 float* __restrict__ rij, int* __restrict__ status) {
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int s = blockIdx.x * NB_WARPS + w;
  const int total = P.batch * P.nodes;
  if (s >= total) return;
  const float4 me = sorted[s];
  const int idx = __float_as_int(me.w);
  const int gcell = sorted_cell[s];
  const int b = gcell / P.cells_cap;
  const int lc = gcell - b * P.cells_cap;
  const GridDesc g = desc[b];
  const int cz = lc % g.nz;
  const int cy = (lc / g.nz) % g.ny;
  const int cx = lc / (g.nz * g.ny);
  const float hx = __fmul_rn(0.5f, P.bx), hy = __fmul_rn(0.5f, P.by), hz = __fmul_rn(0.5f, P.bz);

  // lanes 0..8: (dx, dy) column, first run; lanes 16..24: same column, second run (z wrap-around)
  int run_start = 0, run_len = 0;
  {
    const int col = lane & 15;
    const bool second = lane >= 16;
    if (col < 9) {
      const int dx = col / 3 - 1, dy = col % 3 - 1;
      int ncx = cx + dx, ncy = cy + dy;
      bool ok = true;
      int z_lo, z_hi;  // inclusive range of cz offsets handled by this run, in unwrapped cell units
      if (P.periodic) {
        // with fewer than 3 cells on an axis the offsets {-1,0,1} would visit a cell twice
        if (g.nx < 3) ok = ok && (dx >= 0) && (dx < g.nx);
        if (g.ny < 3) ok = ok && (dy >= 0) && (dy < g.ny);
        ncx = (ncx + g.nx) % g.nx; ncy = (ncy + g.ny) % g.ny;
        if (g.nz < 3) { z_lo = 0; z_hi = g.nz - 1; ok = ok && !second; }   // the whole column, once
        else {
          const int lo = cz - 1, hi = cz + 1;
          if (lo >= 0 && hi < g.nz) { z_lo = lo; z_hi = hi; ok = ok && !second; }
          else if (lo < 0) { if (!second) { z_lo = 0; z_hi = hi; } else { z_lo = g.nz - 1; z_hi = g.nz - 1; } }
          else { if (!second) { z_lo = lo; z_hi = g.nz - 1; } else { z_lo = 0; z_hi = 0; } }
        }
      } else {
        ok = ncx >= 0 && ncx < g.nx && ncy >= 0 && ncy < g.ny && !second;
        z_lo = max(cz - 1, 0); z_hi = min(cz + 1, g.nz - 1);
      }
      if (ok) {
        const int base_cell = b * P.cells_cap + (ncx * g.ny + ncy) * g.nz;
        run_start = cell_start[base_cell + z_lo];
        run_len = cell_start[base_cell + z_hi + 1] - run_start;
      }
    }
  }

  const int node = b * P.nodes + idx;
  long long base = 0;
  float xi = 0.f, yi = 0.f, zi = 0.f;
  if (FILL) {
    base = row_ptr[node];
    const float* p = pos + (size_t)node * 3;
    xi = p[0]; yi = p[1]; zi = p[2];
  }
  int found = 0;
  unsigned live = __ballot_sync(0xffffffffu, run_len > 0);
  while (live) {
    const int r = __ffs(live) - 1;
    live &= live - 1;
    const int rs = __shfl_sync(0xffffffffu, run_start, r);
    const int rl = __shfl_sync(0xffffffffu, run_len, r);
    for (int k0 = 0; k0 < rl; k0 += 32) {
      const int k = k0 + lane;
      bool hit = false;
      int jdx = 0;
      if (k < rl) {
        const float4 q = __ldg(&sorted[rs + k]);
        jdx = __float_as_int(q.w);
        float dx = __fsub_rn(me.x, q.x), dy = __fsub_rn(me.y, q.y), dz = __fsub_rn(me.z, q.z);
        if (P.periodic) { dx = min_image(dx, P.bx, hx); dy = min_image(dy, P.by, hy); dz = min_image(dz, P.bz, hz); }
        const float d2 = __fmaf_rn(dz, dz, __fmaf_rn(dy, dy, __fmul_rn(dx, dx)));
        hit = (jdx != idx) && (d2 <= P.rc2);
      }
      const unsigned bal = __ballot_sync(0xffffffffu, hit);
      if (FILL) {
        if (hit) {
          const long long e = base + found + __popc(bal & ((1u << lane) - 1));
          if (e < capacity) {
            const int nj = b * P.nodes + jdx;
            src[e] = node;
            dst[e] = nj;
            if (rij != nullptr || shift != nullptr) {
              const float* pj = pos + (size_t)nj * 3;
              float ddx = __fsub_rn(__ldg(pj), xi), ddy = __fsub_rn(__ldg(pj + 1), yi), ddz = __fsub_rn(__ldg(pj + 2), zi);
              if (shift != nullptr) {
                int sx = 0, sy = 0, sz = 0;
                if (P.periodic) {
                  sx = -(int)floorf(__fdiv_rn(__fadd_rn(ddx, hx), P.bx));
                  sy = -(int)floorf(__fdiv_rn(__fadd_rn(ddy, hy), P.by));
                  sz = -(int)floorf(__fdiv_rn(__fadd_rn(ddz, hz), P.bz));
                }
                shift[e] = (sx & 0xff) | ((sy & 0xff) << 8) | ((sz & 0xff) << 16);
                // three signed bytes: positions more than 127 box lengths apart do not fit
                if ((abs(sx) > 127 || abs(sy) > 127 || abs(sz) > 127) && status != nullptr) atomicOr(status, LD_FLAG_OVERFLOW);
              }
              if (rij != nullptr) {
                if (P.periodic) {
                  ddx = torch_mod_wrap_fast(ddx, P.bx, hx); ddy = torch_mod_wrap_fast(ddy, P.by, hy);
                  ddz = torch_mod_wrap_fast(ddz, P.bz, hz);
                }
                rij[e * 3 + 0] = ddx; rij[e * 3 + 1] = ddy; rij[e * 3 + 2] = ddz;
              }
            }
          }
        }
      }
      found += __popc(bal);
    }
  }
  if (!FILL) {
    if (lane == 0) degree[node] = found;
  } else {
    if (lane == 0 && base + found > capacity) atomicOr(status, LD_FLAG_CAPACITY);
  }
}

__global__ void edge_counts_kernel(const int* __restrict__ row_ptr, int batch, int nodes, int* __restrict__ edge_counts) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < batch) edge_counts[b] = row_ptr[(size_t)(b + 1) * nodes];
}

struct Workspace {
  GridDesc* desc;
  int* cell_count;   // [ncells_total + 1]
  int* cell_start;   // [ncells_total + 1]
  int* cell_cursor;  // [ncells_total]
  float4* binned;    // [Nt]
  float4* sorted;    // [Nt]
  int* binned_cell;  // [Nt]
  int* sorted_cell;  // [Nt]
  int* degree;       // [Nt + 1]
  int* scan;         // scratch for the prefix sums
  size_t bytes;
};

int plan(const GraphParams& P, void* base, Workspace* w) {
  const size_t Nt = (size_t)P.batch * P.nodes;
  const size_t nc = (size_t)P.batch * P.cells_cap;
  size_t off = 0;
  auto take = [&](size_t bytes) { size_t o = off; off = ld_align_up(off + bytes, 256); return o; };
  char* p = (char*)base;
  w->desc = (GridDesc*)(p + take(sizeof(GridDesc) * (size_t)P.batch));
  w->cell_count = (int*)(p + take(4 * (nc + 1)));
  w->cell_start = (int*)(p + take(4 * (nc + 1)));
  w->cell_cursor = (int*)(p + take(4 * nc));
  w->binned = (float4*)(p + take(16 * Nt));
  w->sorted = (float4*)(p + take(16 * Nt));
  w->binned_cell = (int*)(p + take(4 * Nt));
  w->sorted_cell = (int*)(p + take(4 * Nt));
  w->degree = (int*)(p + take(4 * (Nt + 1)));
  size_t scan_ints = ld_scan_scratch_ints((long long)(nc > Nt ? nc : Nt) + 1);
  w->scan = (int*)(p + take(4 * scan_ints));
  w->bytes = off;
  return LD_OK;
}

int make_params(int batch, int nodes, int periodic, float cutoff, const float* box, int mode, int open_cells_cap,
                GraphParams* P) {
  if (batch < 0 || nodes < 0 || !(cutoff > 0.f) || !isfinite(cutoff)) {
    ld_set_last_message("radius graph: batch, nodes must be >= 0 and cutoff > 0");
    return LD_ERR_SHAPE;
  }
  if ((long long)batch * nodes > 0x7fffffffLL - 1) { ld_set_last_message("radius graph: too many nodes"); return LD_ERR_SHAPE; }
  P->batch = batch; P->nodes = nodes; P->periodic = periodic ? 1 : 0; P->mode = mode;
  P->cutoff = cutoff; P->rc2 = cutoff * cutoff;
  P->bx = P->by = P->bz = 0.f; P->nx = P->ny = P->nz = 1;
  if (periodic) {
    if (box == nullptr) { ld_set_last_message("radius graph: periodic boundary needs a box"); return LD_ERR_SHAPE; }
    P->bx = box[0]; P->by = box[1]; P->bz = box[2];
    int nd[3];
    for (int a = 0; a < 3; a++) {
      if (!(box[a] > 0.f) || !isfinite(box[a])) { ld_set_last_message("radius graph: box must be positive"); return LD_ERR_SHAPE; }
      // same admissibility rule as the reference (neighbour_grid.cpp:78-82): ceil(box/cutoff) >= 3
      int ceil_div = (int)ceilf(box[a] / cutoff);
      if (ceil_div < 3) { ld_set_last_message("box dimension must be greater than 3*cutoff"); return LD_ERR_BOX_TOO_SMALL; }
      if (mode == 1) {
        nd[a] = ceil_div;  // reference grid: cell edge may be < cutoff, pairs two cells apart are missed
      } else {
        // cell edge >= cutoff with a margin for the float32 rounding of the cell index: (int)(n*p/box) is off by up to
        // about n*1.2e-7 cells, so the margin grows with the number of cells per axis (n <= 1024)
        float est = box[a] / cutoff;
        if (est > 1024.f) est = 1024.f;
        nd[a] = (int)floorf(box[a] / (cutoff * (1.00001f + 4.f * est * 1.1920929e-7f)));
        if (nd[a] < 1) nd[a] = 1;
      }
      if (nd[a] > 1024) nd[a] = 1024;
    }
    P->nx = nd[0]; P->ny = nd[1]; P->nz = nd[2];
    long long nc = (long long)nd[0] * nd[1] * nd[2];
    if (nc * (long long)(batch > 0 ? batch : 1) > 0x3fffffffLL) { ld_set_last_message("radius graph: too many cells"); return LD_ERR_SHAPE; }
    P->cells_cap = (int)nc;
  } else {
    if (mode == 1) { ld_set_last_message("radius graph: reference-compatible mode is periodic only"); return LD_ERR_SHAPE; }
    int cap = open_cells_cap > 0 ? open_cells_cap : (nodes < 64 ? 64 : (nodes > 4096 ? 4096 : nodes));
    P->cells_cap = cap;
  }
  return LD_OK;
}

}  // namespace

namespace {
// sum of the degrees in 64 bits; more than INT_MAX edges cannot be addressed by the int32 row offsets
__global__ void degree_overflow_kernel(const int* __restrict__ degree, int Nt, int* status) {
  __shared__ unsigned long long s_sum;
  if (threadIdx.x == 0) s_sum = 0ull;
  __syncthreads();
  unsigned long long t = 0ull;
  for (int i = threadIdx.x; i < Nt; i += blockDim.x) t += (unsigned long long)degree[i];
  atomicAdd(&s_sum, t);
  __syncthreads();
  if (threadIdx.x == 0 && s_sum > 0x7fffffffull && status != nullptr) atomicOr(status, LD_FLAG_OVERFLOW);
}

__global__ void capacity_flag_kernel(const int* __restrict__ row_ptr, int Nt, int* status) {
  if (status != nullptr && row_ptr[Nt] > 0) atomicOr(status, LD_FLAG_CAPACITY);
}
}  // namespace

extern "C" int ld_radius_graph_workspace_size(int batch, int nodes, int periodic, float cutoff, const float* box,
                                              int mode, int open_cells_cap, size_t* bytes) {
  GraphParams P;
  int rc = make_params(batch, nodes, periodic, cutoff, box, mode, open_cells_cap, &P);
  if (rc != LD_OK) return rc;
  Workspace w;
  plan(P, nullptr, &w);
  *bytes = w.bytes;
  return LD_OK;
}

// Counts neighbours: writes row_ptr[Nt+1] (exclusive prefix over global node id b*N+i) and the
// cumulative per-system edge counts edge_counts[B]. Leaves the sorted cells in the workspace for
// ld_radius_graph_fill. status_dev: one int32 on the device, OR-ed with LD_FLAG_* bits.
extern "C" int ld_radius_graph_count(const float* pos, int batch, int nodes, int periodic, float cutoff,
                                     const float* box, int mode, int open_cells_cap, void* workspace,
                                     size_t workspace_bytes, int* row_ptr, int* edge_counts, int* status_dev,
                                     void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  GraphParams P;
  int rc = make_params(batch, nodes, periodic, cutoff, box, mode, open_cells_cap, &P);
  if (rc != LD_OK) return rc;
  Workspace w;
  plan(P, workspace, &w);
  if (workspace == nullptr || workspace_bytes < w.bytes) { ld_set_last_message("radius graph: workspace too small"); return LD_ERR_WORKSPACE; }
  const int Nt = batch * nodes;
  if (Nt == 0) {
    if (batch > 0 && edge_counts) LD_CUDA_TRY(cudaMemsetAsync(edge_counts, 0, 4 * (size_t)batch, stream));
    LD_CUDA_TRY(cudaMemsetAsync(row_ptr, 0, 4, stream));
    return LD_OK;
  }
  const size_t nc = (size_t)batch * P.cells_cap;
  LD_CUDA_TRY(cudaMemsetAsync(w.cell_count, 0, 4 * (nc + 1), stream));
  LD_CUDA_TRY(cudaMemsetAsync(w.cell_cursor, 0, 4 * nc, stream));
  grid_setup_kernel<<<batch, 256, 0, stream>>>(pos, P, w.desc, status_dev);
  LD_LAUNCH_CHECK();
  const int nb = ld_cdiv(Nt, 256);
  bin_kernel<false><<<nb, 256, 0, stream>>>(pos, P, w.desc, w.cell_count, nullptr, nullptr, nullptr, nullptr);
  LD_LAUNCH_CHECK();
  rc = ld_scan_exclusive(w.cell_count, w.cell_start, (long long)nc, w.scan, stream);
  if (rc != LD_OK) return rc;
  bin_kernel<true><<<nb, 256, 0, stream>>>(pos, P, w.desc, nullptr, w.cell_start, w.cell_cursor, w.binned, w.binned_cell);
  LD_LAUNCH_CHECK();
  cell_sort_kernel<<<nb, 256, 0, stream>>>(w.binned, w.binned_cell, w.cell_start, Nt, w.sorted, w.sorted_cell);
  LD_LAUNCH_CHECK();
  neighbour_kernel<false><<<ld_cdiv(Nt, NB_WARPS), NB_WARPS * 32, 0, stream>>>(
      pos, P, w.desc, w.cell_start, w.sorted, w.sorted_cell, w.degree, nullptr, 0, nullptr, nullptr, nullptr, nullptr,
      status_dev);
  LD_LAUNCH_CHECK();
  rc = ld_scan_exclusive(w.degree, row_ptr, (long long)Nt, w.scan, stream);
  if (rc != LD_OK) return rc;
  // row_ptr is int32: only problems whose edge count could pass 2^31-1 pay for the 64-bit check of the degree sum
  if ((long long)Nt * (nodes - 1) > 0x7fffffffLL) {
    degree_overflow_kernel<<<1, 256, 0, stream>>>(w.degree, Nt, status_dev);
    LD_LAUNCH_CHECK();
  }
  if (edge_counts != nullptr) {
    edge_counts_kernel<<<ld_cdiv(batch, 256), 256, 0, stream>>>(row_ptr, batch, nodes, edge_counts);
    LD_LAUNCH_CHECK();
  }
  return LD_OK;
}

// Writes the edges counted by ld_radius_graph_count (same arguments, same workspace contents).
// src/dst hold global node ids, src ascending. shift (optional) packs the lattice shift as three
// signed bytes (x | y<<8 | z<<16) with r_ij = x_j - x_i + shift*box. rij (optional) is the wrapped
// displacement [capacity,3] in the reference's boxwrap form (managan/graph_layers.py:62-66).
// If row_ptr[Nt] > capacity nothing is written past capacity and LD_FLAG_CAPACITY is raised.
extern "C" int ld_radius_graph_fill(const float* pos, int batch, int nodes, int periodic, float cutoff, const float* box,
                                    int mode, int open_cells_cap, void* workspace, size_t workspace_bytes,
                                    const int* row_ptr, long long capacity, int* src, int* dst, int* shift, float* rij,
                                    int* status_dev, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  GraphParams P;
  int rc = make_params(batch, nodes, periodic, cutoff, box, mode, open_cells_cap, &P);
  if (rc != LD_OK) return rc;
  Workspace w;
  plan(P, workspace, &w);
  if (workspace == nullptr || workspace_bytes < w.bytes) { ld_set_last_message("radius graph: workspace too small"); return LD_ERR_WORKSPACE; }
  const int Nt = batch * nodes;
  if (Nt == 0) return LD_OK;
  if (capacity <= 0) {   // nothing can be written: still report edges that do not fit
    capacity_flag_kernel<<<1, 1, 0, stream>>>(row_ptr, Nt, status_dev);
    LD_LAUNCH_CHECK();
    return LD_OK;
  }
  neighbour_kernel<true><<<ld_cdiv(Nt, NB_WARPS), NB_WARPS * 32, 0, stream>>>(
      pos, P, w.desc, w.cell_start, w.sorted, w.sorted_cell, nullptr, row_ptr, capacity, src, dst, shift, rij, status_dev);
  LD_LAUNCH_CHECK();
  return LD_OK;
}

// ---------------------------------------------------------------------------------------------
// Allocation-free graph build.
//
// Some hosts of this library may not create device memory at the point where they need a
// neighbour graph: a simulation engine that calls into a plugin from inside its time-step loop
// with a fixed memory budget, a service whose allocator is frozen after start-up, or code that
// runs between other stream-ordered work where an allocation would synchronise the device. For
// them the scratch space of the build lives in the library image itself: a fixed array in device
// memory that every GPU loading this library holds until the process exits.
//
// The array's name below is only a host-side handle. Kernels must be given its device address,
// which is looked up once per device (with that device current) by cudaGetSymbolAddress.
// ---------------------------------------------------------------------------------------------
#include <mutex>

#define LD_NOALLOC_SCRATCH_BYTES (8u << 20)   /* 8 MiB: about 130k nodes in total */
static __device__ __align__(256) unsigned char g_noalloc_scratch[LD_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int LD_MAX_DEVICES = 64;
void* g_noalloc_addr[LD_MAX_DEVICES] = {nullptr};
std::mutex g_noalloc_mutex;

// device address of the scratch array on the current device; set-up happens on the first call per device
int noalloc_scratch_address(void** out) {
  int dev = -1;
  LD_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= LD_MAX_DEVICES) { ld_set_last_message("allocation-free build: device index out of range"); return LD_ERR_UNSUPPORTED; }
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_addr[dev] == nullptr) {
    void* p = nullptr;
    LD_CUDA_TRY(cudaGetSymbolAddress(&p, g_noalloc_scratch));
    if (p == nullptr) { ld_set_last_message("allocation-free build: scratch symbol has no device address"); return LD_ERR_CUDA; }
    g_noalloc_addr[dev] = p;
  }
  *out = g_noalloc_addr[dev];
  return LD_OK;
}
}  // namespace

// Radius graph without any device allocation: count + fill in one call, scratch in a fixed 8 MiB
// array inside the library. Arguments as ld_radius_graph_count / ld_radius_graph_fill; the caller
// still owns row_ptr[batch*nodes+1], edge_counts[batch], the edge arrays of `capacity` entries
// (shift and rij optional) and status_dev. Edges beyond `capacity` are not written and raise
// LD_FLAG_CAPACITY in *status_dev.
//  * Problems whose scratch need exceeds the array are refused with LD_ERR_WORKSPACE (nothing is
//    launched); ld_radius_graph_workspace_size tells the need in advance.
//  * The first call on each device looks up the array's device address (a host-side runtime call);
//    make that first call before starting any stream capture.
//  * All calls on a device share the one array and it keeps the previous call's contents; the
//    counters that must start at zero are cleared by this call. Two builds that overlap in time on
//    the same device (different streams or threads) race on it: serialise them.
//  * Calls no cudaMalloc, cudaFree or other allocating routine.
extern "C" int ld_radius_graph_build_noalloc(const float* pos, int batch, int nodes, int periodic, float cutoff,
                                             const float* box, int mode, int open_cells_cap, int* row_ptr,
                                             int* edge_counts, long long capacity, int* src, int* dst, int* shift,
                                             float* rij, int* status_dev, void* stream) {
  size_t need = 0;
  int rc = ld_radius_graph_workspace_size(batch, nodes, periodic, cutoff, box, mode, open_cells_cap, &need);
  if (rc != LD_OK) return rc;
  if (need > (size_t)LD_NOALLOC_SCRATCH_BYTES) {
    ld_set_last_message("allocation-free build: problem needs more than the 8 MiB built-in scratch; use ld_radius_graph_count/_fill with a caller workspace");
    return LD_ERR_WORKSPACE;
  }
  void* scratch = nullptr;
  rc = noalloc_scratch_address(&scratch);
  if (rc != LD_OK) return rc;
  rc = ld_radius_graph_count(pos, batch, nodes, periodic, cutoff, box, mode, open_cells_cap, scratch,
                             (size_t)LD_NOALLOC_SCRATCH_BYTES, row_ptr, edge_counts, status_dev, stream);
  if (rc != LD_OK) return rc;
  return ld_radius_graph_fill(pos, batch, nodes, periodic, cutoff, box, mode, open_cells_cap, scratch,
                              (size_t)LD_NOALLOC_SCRATCH_BYTES, row_ptr, capacity, src, dst, shift, rij, status_dev, stream);
}
