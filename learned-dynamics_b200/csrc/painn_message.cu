// PaiNN message step, FP32 path: radial encoding -> distance MLP -> product with the neighbour's
// activation -> vector/scalar messages -> sum over each source node's edges, in ONE kernel.
// Restates Message.forward of the reference (archs/meanflow_painn8.py:77-100) without any
// edge-sized tensor in HBM:
//   D_e   = mlp_dist(radial_encode(r_e))                      (per edge, three dense layers)
//   P_e   = D_e * A[dst_e],  A = mlp_actv(x_a) (per NODE: the reference evaluates mlp_actv on
//           x_a[dst] per edge, which is the same rows repeated; ld_mlp3_rows computes A once)
//   dir_e = r_e / sqrt(eps + |r_e|^2)
//   m_v   = x_v[dst]*P0 + cross(x_v[dst], dir)*P1 + dir*P2 ;  m_a = P3
//   out_v[i] = sum_{e: src_e = i} m_v ,  out_a[i] = sum m_a       (+ optional residual)
// A block walks a contiguous, node-aligned range of the CSR, 32 edges per tile; sums for the
// current source node live in registers and every node is written exactly once (no atomics,
// fixed summation order).
#include "common.cuh"
#include "mlp_tile.cuh"

namespace {

struct MlpWeights {
  const float* W1t; const float* b1;
  const float* W2t; const float* b2;
  const float* W3t; const float* b3;
  int k0, n1, n2, n3;
};

__host__ __device__ inline int max4(int a, int b, int c, int d) {
  int m = a > b ? a : b; m = m > c ? m : c; return m > d ? m : d;
}

// dynamic shared memory: buf0[32*maxdim] | buf1[32*maxdim (+pad for row-major)] | wstage[2*KC*maxN]
struct SmemPlan {
  int maxdim, maxn, ldo;
  size_t buf_floats, stage_floats;
  __host__ __device__ SmemPlan(const MlpWeights& m) {
    maxdim = max4(m.k0, m.n1, m.n2, m.n3);
    maxn = max4(0, m.n1, m.n2, m.n3);
    ldo = m.n3 + 1;  // row-major output stride (odd: conflict-free column walks)
    size_t a = (size_t)MT_ROWS * maxdim, b = (size_t)MT_ROWS * ldo;
    buf_floats = ((a > b ? a : b) + 3) / 4 * 4;
    stage_floats = (size_t)2 * MT_KC * maxn;
  }
  __host__ __device__ size_t bytes() const { return (2 * buf_floats + stage_floats) * 4 + 1024; }
};

template <int NCOL>
__device__ __forceinline__ void run_mlp3(const MlpWeights& m, int act, float* buf0, float* buf1, int ldo, float* wstage) {
  mt_tile_linear<NCOL, false>(buf0, m.k0, m.W1t, m.b1, m.n1, act, buf1, 0, wstage);
  mt_tile_linear<NCOL, false>(buf1, m.n1, m.W2t, m.b2, m.n2, act, buf0, 0, wstage);
  mt_tile_linear<NCOL, true>(buf0, m.n2, m.W3t, m.b3, m.n3, LD_ACT_NONE, buf1, ldo, wstage);
}

// out[r, :] = W3 act(W2 act(W1 x[r] + b1) + b2) + b3 (+ Wd x[r] when Wdt != nullptr)
template <int NCOL>
__global__ void __launch_bounds__(MT_THREADS, 1)
mlp3_rows_kernel(const float* __restrict__ x, long long rows, MlpWeights m, int act, const float* __restrict__ Wdt,
                 float* __restrict__ out) {
  extern __shared__ __align__(16) float smem[];
  const SmemPlan plan(m);
  float* buf0 = smem;
  float* buf1 = buf0 + plan.buf_floats;
  float* wstage = buf1 + plan.buf_floats;
  const int tid = threadIdx.x;
  const long long ntiles = (rows + MT_ROWS - 1) / MT_ROWS;
  for (long long t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const long long r0 = t * MT_ROWS;
    for (int idx = tid; idx < MT_ROWS * m.k0; idx += MT_THREADS) {
      const int r = idx & (MT_ROWS - 1), k = idx >> 5;
      buf0[k * MT_ROWS + r] = (r0 + r < rows) ? x[(r0 + r) * m.k0 + k] : 0.f;
    }
    __syncthreads();
    run_mlp3<NCOL>(m, act, buf0, buf1, plan.ldo, wstage);
    if (Wdt != nullptr) {
      // direct linear term: reload x (buf0 was overwritten by layer 2) and accumulate
      for (int idx = tid; idx < MT_ROWS * m.k0; idx += MT_THREADS) {
        const int r = idx & (MT_ROWS - 1), k = idx >> 5;
        buf0[k * MT_ROWS + r] = (r0 + r < rows) ? x[(r0 + r) * m.k0 + k] : 0.f;
      }
      __syncthreads();
      for (int idx = tid; idx < MT_ROWS * m.n3; idx += MT_THREADS) {
        const int r = idx / m.n3, c = idx - r * m.n3;
        float a = 0.f;
        for (int k = 0; k < m.k0; k++) a = fmaf(buf0[k * MT_ROWS + r], Wdt[(size_t)k * m.n3 + c], a);
        buf1[(size_t)r * plan.ldo + c] += a;
      }
      __syncthreads();
    }
    for (int idx = tid; idx < MT_ROWS * m.n3; idx += MT_THREADS) {
      const int r = idx / m.n3, c = idx - r * m.n3;
      if (r0 + r < rows) out[(r0 + r) * m.n3 + c] = buf1[(size_t)r * plan.ldo + c];
    }
    __syncthreads();
  }
}

struct MessageParams {
  const int* row_ptr;   // [Nt+1]
  const int* dst;       // [E]
  const float* rij;     // [E,3]
  int Nt, n, n_rbf, radial_kind;
  float rmax, pi_over_rmax, eps;
  const float* actv;    // [Nt, 4n]
  const float* x_v;     // [Nt, n, 3]
  const float* res_a;   // optional [Nt, n]
  const float* res_v;   // optional [Nt, n, 3]
  float* out_a;         // [Nt, n]
  float* out_v;         // [Nt, n, 3]
  long long* edge_counter;  // optional: += edges processed (for throughput accounting)
};

constexpr int MSG_MAX_OUT = 2;  // outputs per thread: 4n <= 512

__device__ __forceinline__ int lower_bound_row(const int* __restrict__ row_ptr, int lo, int hi, long long target) {
  // first v in [lo, hi] with row_ptr[v] >= target
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if ((long long)row_ptr[mid] < target) lo = mid + 1; else hi = mid;
  }
  return lo;
}


// first node v in [0, Nt] with row_ptr[v] + v >= target (work = edges + nodes before v)
__device__ __forceinline__ int work_lower_bound(const int* __restrict__ row_ptr, int Nt, long long target) {
  int lo = 0, hi = Nt;
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if ((long long)row_ptr[mid] + mid < target) lo = mid + 1; else hi = mid;
  }
  return lo;
}

template <int NCOL>
__global__ void __launch_bounds__(MT_THREADS, 1)
painn_message_kernel(MessageParams P, MlpWeights m) {
  extern __shared__ __align__(16) float smem[];
  const SmemPlan plan(m);
  float* buf0 = smem;
  float* buf1 = buf0 + plan.buf_floats;
  float* wstage = buf1 + plan.buf_floats;
  __shared__ float s_dir[MT_ROWS][3];
  __shared__ float s_dist[MT_ROWS];
  __shared__ int s_dst[MT_ROWS];
  __shared__ int s_src[MT_ROWS];

  const int tid = threadIdx.x;
  const int n = P.n;
  const long long E = P.row_ptr[P.Nt];
  // node-aligned share for this block, balanced over edges + nodes (nodes without edges still
  // have to be written)
  long long per = (E + P.Nt + gridDim.x - 1) / gridDim.x;
  if (per < MT_ROWS) per = MT_ROWS;
  const int n_begin = blockIdx.x == 0 ? 0 : work_lower_bound(P.row_ptr, P.Nt, per * blockIdx.x);
  const int n_end = blockIdx.x == gridDim.x - 1 ? P.Nt : work_lower_bound(P.row_ptr, P.Nt, per * (blockIdx.x + 1));
  if (n_begin >= n_end) return;
  const long long e_begin = P.row_ptr[n_begin], e_end = P.row_ptr[n_end];

  // this thread's outputs: o < 3n -> vector element (c = o/3, k = o%3); else scalar channel o-3n
  float acc[MSG_MAX_OUT];
  int oc[MSG_MAX_OUT], ok_[MSG_MAX_OUT];
  bool oact[MSG_MAX_OUT];
#pragma unroll
  for (int q = 0; q < MSG_MAX_OUT; q++) {
    const int o = tid + MT_THREADS * q;
    oact[q] = o < 4 * n;
    acc[q] = 0.f;
    if (o < 3 * n) { oc[q] = o / 3; ok_[q] = o % 3; } else { oc[q] = o - 3 * n; ok_[q] = 3; }
  }
  int cur = n_begin;  // node whose sum is being accumulated

  auto flush_until = [&](int next) {
    // write node `cur`, zero-fill nodes (cur, next), continue with `next`
    for (int v = cur; v < next; v++) {
#pragma unroll
      for (int q = 0; q < MSG_MAX_OUT; q++) {
        if (!oact[q]) continue;
        float val = (v == cur) ? acc[q] : 0.f;
        if (ok_[q] < 3) {
          const size_t off = ((size_t)v * n + oc[q]) * 3 + ok_[q];
          if (P.res_v != nullptr) val += P.res_v[off];
          P.out_v[off] = val;
        } else {
          const size_t off = (size_t)v * n + oc[q];
          if (P.res_a != nullptr) val += P.res_a[off];
          P.out_a[off] = val;
        }
      }
    }
#pragma unroll
    for (int q = 0; q < MSG_MAX_OUT; q++) acc[q] = 0.f;
    cur = next;
  };

  for (long long e0 = e_begin; e0 < e_end; e0 += MT_ROWS) {
    const int cnt = (int)((e_end - e0) < MT_ROWS ? (e_end - e0) : MT_ROWS);
    if (tid < MT_ROWS) {
      float dx = 0.f, dy = 0.f, dz = 0.f;
      int j = 0, s = -1;
      if (tid < cnt) {
        const long long e = e0 + tid;
        dx = P.rij[e * 3]; dy = P.rij[e * 3 + 1]; dz = P.rij[e * 3 + 2];
        j = P.dst[e];
        s = lower_bound_row(P.row_ptr, n_begin, n_end, e + 1) - 1;  // row_ptr[s] <= e < row_ptr[s+1]
      }
      const float r2 = dx * dx + dy * dy + dz * dz;
      const float inv = 1.0f / sqrtf(P.eps + r2);
      s_dir[tid][0] = dx * inv; s_dir[tid][1] = dy * inv; s_dir[tid][2] = dz * inv;
      s_dist[tid] = sqrtf(r2);
      s_dst[tid] = j;
      s_src[tid] = s;
    }
    __syncthreads();
    for (int idx = tid; idx < MT_ROWS * P.n_rbf; idx += MT_THREADS) {
      const int r = idx & (MT_ROWS - 1), k = idx >> 5;
      buf0[k * MT_ROWS + r] = r < cnt ? radial_feature(P.radial_kind, k, P.n_rbf, s_dist[r], P.rmax, P.pi_over_rmax) : 0.f;
    }
    __syncthreads();
    run_mlp3<NCOL>(m, LD_ACT_SILU, buf0, buf1, plan.ldo, wstage);
    // buf1: D[e][4n] row-major, stride ldo
    for (int e = 0; e < cnt; e++) {
      const int s = s_src[e];
      if (s != cur) flush_until(s);
      const int j = s_dst[e];
      const float* Aj = P.actv + (size_t)j * 4 * n;
      const float* De = buf1 + (size_t)e * plan.ldo;
#pragma unroll
      for (int q = 0; q < MSG_MAX_OUT; q++) {
        if (!oact[q]) continue;
        const int c = oc[q];
        if (ok_[q] < 3) {
          const int k = ok_[q], k1 = (k + 1) % 3, k2 = (k + 2) % 3;
          const float* xv = P.x_v + ((size_t)j * n + c) * 3;
          const float p0 = De[c] * __ldg(Aj + c);
          const float p1 = De[n + c] * __ldg(Aj + n + c);
          const float p2 = De[2 * n + c] * __ldg(Aj + 2 * n + c);
          const float xk = __ldg(xv + k), xk1 = __ldg(xv + k1), xk2 = __ldg(xv + k2);
          const float cr = xk1 * s_dir[e][k2] - xk2 * s_dir[e][k1];  // cross(x_v, dir)_k
          acc[q] += xk * p0 + cr * p1 + s_dir[e][k] * p2;
        } else {
          acc[q] += De[3 * n + c] * __ldg(Aj + 3 * n + c);
        }
      }
    }
    __syncthreads();  // buf1 and s_* are rewritten by the next tile
  }
  flush_until(n_end);
  if (P.edge_counter != nullptr && tid == 0) atomicAdd((unsigned long long*)P.edge_counter, (unsigned long long)(e_end - e_begin));
}

int check_mlp(const MlpWeights& m, int* ncol) {
  const int dims[3] = {m.n1, m.n2, m.n3};
  int mx = 0;
  for (int i = 0; i < 3; i++) {
    if (dims[i] <= 0 || dims[i] % 8 != 0) { ld_set_last_message("mlp: layer widths must be positive multiples of 8"); return LD_ERR_UNSUPPORTED; }
    if (dims[i] > mx) mx = dims[i];
  }
  if (m.k0 <= 0 || m.k0 > 512 || mx > 512) { ld_set_last_message("mlp (FP32 path): widths above 512 are not supported"); return LD_ERR_UNSUPPORTED; }
  *ncol = mx > 256 ? 2 : 1;
  const uintptr_t al = (uintptr_t)m.W1t | (uintptr_t)m.W2t | (uintptr_t)m.W3t;
  if (al % 16 != 0) { ld_set_last_message("mlp: packed weights must be 16-byte aligned"); return LD_ERR_SHAPE; }
  return LD_OK;
}

template <typename K>
int set_smem(K kernel, size_t bytes) {
  if (bytes > 227 * 1024) { ld_set_last_message("mlp: shared-memory plan exceeds 227 KB"); return LD_ERR_UNSUPPORTED; }
  LD_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  return LD_OK;
}

int sm_count() {
  int dev = 0, n = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  return n > 0 ? n : 148;
}

}  // namespace

// Three dense layers on `rows` rows. Weights are passed transposed ("packed"): Wkt is [in][out]
// contiguous, i.e. nn.Linear.weight.t().contiguous(). act: 0 none, 1 SiLU, 2 LeakyReLU(0.1),
// applied after layers 1 and 2. Wdt (optional, [k0][n3]) adds a direct linear term x*Wd.
extern "C" int ld_mlp3_rows(const float* x, long long rows, int k0, const float* W1t, const float* b1, int n1,
                            const float* W2t, const float* b2, int n2, const float* W3t, const float* b3, int n3, int act,
                            const float* Wdt, float* out, void* stream) {
  if (rows < 0) return LD_ERR_SHAPE;
  MlpWeights m{W1t, b1, W2t, b2, W3t, b3, k0, n1, n2, n3};
  int ncol = 1;
  int rc = check_mlp(m, &ncol);
  if (rc != LD_OK) return rc;
  if (rows == 0) return LD_OK;
  const SmemPlan plan(m);
  const size_t smem = plan.bytes();
  const long long ntiles = (rows + MT_ROWS - 1) / MT_ROWS;
  const int grid = (int)(ntiles < sm_count() ? ntiles : sm_count());
  if (ncol == 1) {
    rc = set_smem(mlp3_rows_kernel<1>, smem); if (rc != LD_OK) return rc;
    mlp3_rows_kernel<1><<<grid, MT_THREADS, smem, (cudaStream_t)stream>>>(x, rows, m, act, Wdt, out);
  } else {
    rc = set_smem(mlp3_rows_kernel<2>, smem); if (rc != LD_OK) return rc;
    mlp3_rows_kernel<2><<<grid, MT_THREADS, smem, (cudaStream_t)stream>>>(x, rows, m, act, Wdt, out);
  }
  LD_LAUNCH_CHECK();
  return LD_OK;
}

// Fused PaiNN message (FP32). Graph in CSR form sorted by source (row_ptr[Nt+1], dst[E], rij[E,3]).
// Distance MLP: n_rbf -> 4n -> 4n -> 4n, SiLU, packed weights. actv = mlp_actv(x_a) [Nt,4n].
// radial_kind 0: cos/sin encoding of the reference (then n_rbf is the reference's n);
// radial_kind 1: Gaussian basis with cosine cutoff. res_a/res_v optional residual inputs.
// edge_counter: optional device int64, incremented by the number of edges processed.
extern "C" int ld_painn_message_f32(const int* row_ptr, const int* dst, const float* rij, int Nt, int n, int n_rbf,
                                    int radial_kind, float rmax, float eps, const float* W1t, const float* b1,
                                    const float* W2t, const float* b2, const float* W3t, const float* b3, const float* actv,
                                    const float* x_v, const float* res_a, const float* res_v, float* out_a, float* out_v,
                                    long long* edge_counter, void* stream) {
  if (Nt < 0 || n <= 0 || n_rbf <= 0) return LD_ERR_SHAPE;
  if (4 * n > MT_THREADS * MSG_MAX_OUT) { ld_set_last_message("painn message (FP32 path): n above 128 is not supported"); return LD_ERR_UNSUPPORTED; }
  MlpWeights m{W1t, b1, W2t, b2, W3t, b3, n_rbf, 4 * n, 4 * n, 4 * n};
  int ncol = 1;
  int rc = check_mlp(m, &ncol);
  if (rc != LD_OK) return rc;
  if (Nt == 0) return LD_OK;
  MessageParams P;
  P.row_ptr = row_ptr; P.dst = dst; P.rij = rij; P.Nt = Nt; P.n = n; P.n_rbf = n_rbf; P.radial_kind = radial_kind;
  P.rmax = rmax; P.pi_over_rmax = (float)(3.14159265358979323846 / (double)rmax); P.eps = eps;
  P.actv = actv; P.x_v = x_v; P.res_a = res_a; P.res_v = res_v; P.out_a = out_a; P.out_v = out_v;
  P.edge_counter = edge_counter;
  const SmemPlan plan(m);
  const size_t smem = plan.bytes();
  const int grid = sm_count();
  if (ncol == 1) {
    rc = set_smem(painn_message_kernel<1>, smem); if (rc != LD_OK) return rc;
    painn_message_kernel<1><<<grid, MT_THREADS, smem, (cudaStream_t)stream>>>(P, m);
  } else {
    rc = set_smem(painn_message_kernel<2>, smem); if (rc != LD_OK) return rc;
    painn_message_kernel<2><<<grid, MT_THREADS, smem, (cudaStream_t)stream>>>(P, m);
  }
  LD_LAUNCH_CHECK();
  return LD_OK;
}
