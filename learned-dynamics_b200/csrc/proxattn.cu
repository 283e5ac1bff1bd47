// Dense proximity attention without a normalising reduction:
//   out[z,m,:] = sum_n w(m,n) * (q_m . k_n) * v_n,   w(m,n) = r0sq / (r0sq + dist2(x_m, y_n)),
// dist2 = |x_m - y_n|^2 in open space, or sum_a (1 - cos(2 pi R_a / L_a)) L_a^2 / (2 pi^2) in a periodic box,
// with r0sq taken per head (head = z mod heads), and its gradients with respect to Q, K, V, X and Y.
//
// Replaces the reference's Triton kernels _fwd_kernel, _bwd_kernel_kvy and _bwd_kernel_qx of
// managan/triton_kernels/proxattn.py:30-236 and proxattn_periodic.py (same structure with the box), whose
// defining math is refimpl_proxattn (proxattn.py:9-27, proxattn_periodic.py:9-28).
//
// FP32 throughout (the Triton kernels take their dot products in TF32; these kernels match the einsum
// definition to FP32 rounding). A block owns a tile of 64 rows and walks the other index in tiles of 64:
//   forward / dQ,dX : rows = queries m, walked index = keys n
//   dK,dV,dY        : rows = keys n,    walked index = queries m
// Each step is two kinds of small matrix products out of shared memory: "NT" (64 x 64 scores from two
// row tiles, contraction over the feature dimension) and "NN" (64 x dim accumulator += 64 x 64 weights times
// a row tile). Rows past N are zero-filled on load, which makes every one of their contributions zero, so
// only the final stores are masked.
#include <cuda_runtime.h>
#include "common.cuh"

namespace {

constexpr int PT = 64;          // tile edge in both indices
constexpr int PA_THREADS = 256; // thread (ty, tx) = (tid / 16, tid % 16) owns rows 4 ty .. 4 ty + 3
constexpr int PLD = PT + 4;     // row pitch of a 64 x 64 weight tile in shared memory

struct PaBox { float lx, ly, lz; };

template <int D>
__device__ __forceinline__ void pa_load_tile(float* __restrict__ s, const float* __restrict__ g, int row0, int N) {
  constexpr int LD = D + 4, V4 = D / 4;
  for (int idx = threadIdx.x; idx < PT * V4; idx += PA_THREADS) {
    const int r = idx / V4, c = idx % V4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (row0 + r < N) v = __ldg(reinterpret_cast<const float4*>(g + (size_t)(row0 + r) * D) + c);
    *reinterpret_cast<float4*>(s + r * LD + 4 * c) = v;
  }
}

// positions of a row tile. Open space: [64][3] coordinates. Periodic: [64][6] = (cos, sin) of 2 pi x_a / L_a per
// axis, so that the pair loop gets cos and sin of the angle difference from four multiply-adds per axis
// instead of two transcendental calls.
template <bool PER>
__device__ __forceinline__ void pa_load_pos(float* __restrict__ s, const float* __restrict__ g, int row0, int N, const PaBox& box) {
  for (int idx = threadIdx.x; idx < PT * 3; idx += PA_THREADS) {
    const float v = (row0 + idx / 3 < N) ? __ldg(g + (size_t)row0 * 3 + idx) : 0.f;
    if (PER) {
      const int a = idx % 3;
      const float L = a == 0 ? box.lx : (a == 1 ? box.ly : box.lz);
      float sn, cs;
      sincosf(6.283185307179586f * v / L, &sn, &cs);
      s[(idx / 3) * 6 + 2 * a] = cs;
      s[(idx / 3) * 6 + 2 * a + 1] = sn;
    } else {
      s[idx] = v;
    }
  }
}

// acc[i][j] = sum_d A[4 ty + i][d] * B[tx + 16 j][d]
template <int D>
__device__ __forceinline__ void pa_gemm_nt(const float* __restrict__ sA, const float* __restrict__ sB, float (&acc)[4][4]) {
  constexpr int LD = D + 4;
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
#pragma unroll 2
  for (int d = 0; d < D; d += 4) {
    float4 a[4], b[4];
#pragma unroll
    for (int i = 0; i < 4; i++) a[i] = *reinterpret_cast<const float4*>(sA + (ty * 4 + i) * LD + d);
#pragma unroll
    for (int j = 0; j < 4; j++) b[j] = *reinterpret_cast<const float4*>(sB + (tx + 16 * j) * LD + d);
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int j = 0; j < 4; j++) {
        float t = acc[i][j];
        t = fmaf(a[i].x, b[j].x, t);
        t = fmaf(a[i].y, b[j].y, t);
        t = fmaf(a[i].z, b[j].z, t);
        t = fmaf(a[i].w, b[j].w, t);
        acc[i][j] = t;
      }
  }
}

// acc[i][c] += sum_n P[4 ty + i][n] * B[n][tx + 16 c]
template <int D>
__device__ __forceinline__ void pa_gemm_nn(const float* __restrict__ sP, const float* __restrict__ sB, float (&acc)[4][D / 16]) {
  constexpr int LD = D + 4, CPT = D / 16;
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
#pragma unroll 2
  for (int n = 0; n < PT; n += 4) {
    float p[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const float4 t = *reinterpret_cast<const float4*>(sP + (ty * 4 + i) * PLD + n);
      p[i][0] = t.x; p[i][1] = t.y; p[i][2] = t.z; p[i][3] = t.w;
    }
#pragma unroll
    for (int nn = 0; nn < 4; nn++) {
      float b[CPT];
#pragma unroll
      for (int c = 0; c < CPT; c++) b[c] = sB[(n + nn) * LD + tx + 16 * c];
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int c = 0; c < CPT; c++) acc[i][c] = fmaf(p[i][nn], b[c], acc[i][c]);
    }
  }
}

// weight of a pair and the gradient of dist2 with respect to R = x - y (x, y: rows of the position tiles)
template <bool PER>
__device__ __forceinline__ float pa_pair(const float* x, const float* y, float r0sq, const PaBox& box, float (&gv)[3]) {
  float dd = 0.f;
  const float L[3] = {box.lx, box.ly, box.lz};
#pragma unroll
  for (int a = 0; a < 3; a++) {
    if (PER) {
      const float cx = x[2 * a], sx = x[2 * a + 1], cy = y[2 * a], sy = y[2 * a + 1];
      const float cs = fmaf(cx, cy, sx * sy), sn = fmaf(sx, cy, -cx * sy);   // cos, sin of 2 pi (x_a - y_a) / L_a
      dd = fmaf(1.f - cs, L[a] * L[a] * 0.05066059182116889f, dd);           // L^2 / (2 pi^2)
      gv[a] = sn * (L[a] * 0.3183098861837907f);                             // L / pi
    } else {
      const float R = x[a] - y[a];
      dd = fmaf(R, R, dd);
      gv[a] = 2.f * R;
    }
  }
  return r0sq / (r0sq + dd);
}

template <int D>
__device__ __forceinline__ void pa_store_rows(float* __restrict__ g, int row0, int N, const float (&acc)[4][D / 16]) {
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int r = row0 + ty * 4 + i;
    if (r < N) {
#pragma unroll
      for (int c = 0; c < D / 16; c++) g[(size_t)r * D + tx + 16 * c] = acc[i][c];
    }
  }
}

// sum of a per-row 3-vector over the 16 threads that share the row, stored by tx == 0
__device__ __forceinline__ void pa_store_pos_grad(float* __restrict__ g, int row0, int N, float (&d)[4][3]) {
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int a = 0; a < 3; a++) {
      float v = d[i][a];
#pragma unroll
      for (int o = 8; o >= 1; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      const int r = row0 + ty * 4 + i;
      if (tx == 0 && r < N) g[(size_t)r * 3 + a] = v;
    }
}

struct PaArgs {
  const float *Q, *K, *V, *X, *Y, *r0sq, *dO;
  float *out, *dQ, *dK, *dV, *dX, *dY;
  int heads, N;
  PaBox box;
};

// out = (w o Q K^T) V; block = (query tile, z)
template <int D, bool PER>
__global__ void __launch_bounds__(PA_THREADS) proxattn_fwd_kernel(PaArgs p) {
  constexpr int LD = D + 4, CPT = D / 16, PS = PER ? 6 : 3;
  extern __shared__ __align__(16) float smem[];
  float *sQ = smem, *sK = sQ + PT * LD, *sV = sK + PT * LD, *sP = sV + PT * LD, *sX = sP + PT * PLD, *sY = sX + PT * 6;
  const int z = blockIdx.y, m0 = blockIdx.x * PT, N = p.N;
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  const size_t zf = (size_t)z * N * D, zp = (size_t)z * N * 3;
  const float r0sq = __ldg(p.r0sq + z % p.heads);
  pa_load_tile<D>(sQ, p.Q + zf, m0, N);
  pa_load_pos<PER>(sX, p.X + zp, m0, N, p.box);
  float acc[4][CPT];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int c = 0; c < CPT; c++) acc[i][c] = 0.f;
  for (int n0 = 0; n0 < N; n0 += PT) {
    __syncthreads();
    pa_load_tile<D>(sK, p.K + zf, n0, N);
    pa_load_tile<D>(sV, p.V + zf, n0, N);
    pa_load_pos<PER>(sY, p.Y + zp, n0, N, p.box);
    __syncthreads();
    float s[4][4], gv[3];
    pa_gemm_nt<D>(sQ, sK, s);
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const float w = pa_pair<PER>(sX + (ty * 4 + i) * PS, sY + (tx + 16 * j) * PS, r0sq, p.box, gv);
        sP[(ty * 4 + i) * PLD + tx + 16 * j] = w * s[i][j];
      }
    __syncthreads();
    pa_gemm_nn<D>(sP, sV, acc);
  }
  pa_store_rows<D>(p.out + zf, m0, N, acc);
}

// dQ = (w o dO V^T) K, dX_m = sum_n s g dw/ddist2 * d dist2 / dR; block = (query tile, z)
template <int D, bool PER>
__global__ void __launch_bounds__(PA_THREADS) proxattn_bwd_qx_kernel(PaArgs p) {
  constexpr int LD = D + 4, CPT = D / 16, PS = PER ? 6 : 3;
  extern __shared__ __align__(16) float smem[];
  float *sQ = smem, *sG = sQ + PT * LD, *sK = sG + PT * LD, *sV = sK + PT * LD, *sP = sV + PT * LD, *sX = sP + PT * PLD,
        *sY = sX + PT * 6;
  const int z = blockIdx.y, m0 = blockIdx.x * PT, N = p.N;
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  const size_t zf = (size_t)z * N * D, zp = (size_t)z * N * 3;
  const float r0sq = __ldg(p.r0sq + z % p.heads), inv_r0sq = 1.f / r0sq;
  pa_load_tile<D>(sQ, p.Q + zf, m0, N);
  pa_load_tile<D>(sG, p.dO + zf, m0, N);
  pa_load_pos<PER>(sX, p.X + zp, m0, N, p.box);
  float dq[4][CPT], dx[4][3];
#pragma unroll
  for (int i = 0; i < 4; i++) {
#pragma unroll
    for (int c = 0; c < CPT; c++) dq[i][c] = 0.f;
    dx[i][0] = dx[i][1] = dx[i][2] = 0.f;
  }
  for (int n0 = 0; n0 < N; n0 += PT) {
    __syncthreads();
    pa_load_tile<D>(sK, p.K + zf, n0, N);
    pa_load_tile<D>(sV, p.V + zf, n0, N);
    pa_load_pos<PER>(sY, p.Y + zp, n0, N, p.box);
    __syncthreads();
    float s[4][4], g[4][4], gv[3];
    pa_gemm_nt<D>(sQ, sK, s);
    pa_gemm_nt<D>(sG, sV, g);
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const float w = pa_pair<PER>(sX + (ty * 4 + i) * PS, sY + (tx + 16 * j) * PS, r0sq, p.box, gv);
        sP[(ty * 4 + i) * PLD + tx + 16 * j] = w * g[i][j];
        const float coef = -s[i][j] * g[i][j] * w * w * inv_r0sq;
#pragma unroll
        for (int a = 0; a < 3; a++) dx[i][a] = fmaf(coef, gv[a], dx[i][a]);
      }
    __syncthreads();
    pa_gemm_nn<D>(sP, sK, dq);
  }
  pa_store_rows<D>(p.dQ + zf, m0, N, dq);
  pa_store_pos_grad(p.dX + zp, m0, N, dx);
}

// dV = (w o Q K^T)^T dO, dK = (w o dO V^T)^T Q, dY_n = -sum_m (...); block = (key tile, z)
template <int D, bool PER>
__global__ void __launch_bounds__(PA_THREADS) proxattn_bwd_kvy_kernel(PaArgs p) {
  constexpr int LD = D + 4, CPT = D / 16, PS = PER ? 6 : 3;
  extern __shared__ __align__(16) float smem[];
  float *sK = smem, *sV = sK + PT * LD, *sQ = sV + PT * LD, *sG = sQ + PT * LD, *sP = sG + PT * LD, *sP2 = sP + PT * PLD,
        *sY = sP2 + PT * PLD, *sX = sY + PT * 6;
  const int z = blockIdx.y, n0 = blockIdx.x * PT, N = p.N;
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  const size_t zf = (size_t)z * N * D, zp = (size_t)z * N * 3;
  const float r0sq = __ldg(p.r0sq + z % p.heads), inv_r0sq = 1.f / r0sq;
  pa_load_tile<D>(sK, p.K + zf, n0, N);
  pa_load_tile<D>(sV, p.V + zf, n0, N);
  pa_load_pos<PER>(sY, p.Y + zp, n0, N, p.box);
  float dk[4][CPT], dv[4][CPT], dy[4][3];
#pragma unroll
  for (int i = 0; i < 4; i++) {
#pragma unroll
    for (int c = 0; c < CPT; c++) dk[i][c] = dv[i][c] = 0.f;
    dy[i][0] = dy[i][1] = dy[i][2] = 0.f;
  }
  for (int m0 = 0; m0 < N; m0 += PT) {
    __syncthreads();
    pa_load_tile<D>(sQ, p.Q + zf, m0, N);
    pa_load_tile<D>(sG, p.dO + zf, m0, N);
    pa_load_pos<PER>(sX, p.X + zp, m0, N, p.box);
    __syncthreads();
    float st[4][4], gt[4][4], gv[3];   // transposed tiles: [key][query]
    pa_gemm_nt<D>(sK, sQ, st);
    pa_gemm_nt<D>(sV, sG, gt);
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const float w = pa_pair<PER>(sX + (tx + 16 * j) * PS, sY + (ty * 4 + i) * PS, r0sq, p.box, gv);
        sP[(ty * 4 + i) * PLD + tx + 16 * j] = w * st[i][j];
        sP2[(ty * 4 + i) * PLD + tx + 16 * j] = w * gt[i][j];
        const float coef = st[i][j] * gt[i][j] * w * w * inv_r0sq;   // sign: d dist2 / dy = -d dist2 / dR
#pragma unroll
        for (int a = 0; a < 3; a++) dy[i][a] = fmaf(coef, gv[a], dy[i][a]);
      }
    __syncthreads();
    pa_gemm_nn<D>(sP, sG, dv);
    pa_gemm_nn<D>(sP2, sQ, dk);
  }
  pa_store_rows<D>(p.dV + zf, n0, N, dv);
  pa_store_rows<D>(p.dK + zf, n0, N, dk);
  pa_store_pos_grad(p.dY + zp, n0, N, dy);
}

template <int D>
constexpr size_t pa_smem(int feature_tiles, int weight_tiles) {
  return sizeof(float) * ((size_t)feature_tiles * PT * (D + 4) + (size_t)weight_tiles * PT * PLD + 2 * PT * 6);
}

template <int D, bool PER>
int pa_launch(const PaArgs& a, int Z, int which, cudaStream_t st) {
  const dim3 grid((a.N + PT - 1) / PT, Z);
  if (which == 0) {
    constexpr size_t sm = pa_smem<D>(3, 1);
    LD_CUDA_TRY(cudaFuncSetAttribute(proxattn_fwd_kernel<D, PER>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm));
    proxattn_fwd_kernel<D, PER><<<grid, PA_THREADS, sm, st>>>(a);
  } else if (which == 1) {
    constexpr size_t sm = pa_smem<D>(4, 1);
    LD_CUDA_TRY(cudaFuncSetAttribute(proxattn_bwd_qx_kernel<D, PER>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm));
    proxattn_bwd_qx_kernel<D, PER><<<grid, PA_THREADS, sm, st>>>(a);
  } else {
    constexpr size_t sm = pa_smem<D>(4, 2);
    LD_CUDA_TRY(cudaFuncSetAttribute(proxattn_bwd_kvy_kernel<D, PER>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm));
    proxattn_bwd_kvy_kernel<D, PER><<<grid, PA_THREADS, sm, st>>>(a);
  }
  LD_LAUNCH_CHECK();
  return LD_OK;
}

template <bool PER>
int pa_dispatch(const PaArgs& a, int Z, int dim, int which, cudaStream_t st) {
  switch (dim) {
    case 16: return pa_launch<16, PER>(a, Z, which, st);
    case 32: return pa_launch<32, PER>(a, Z, which, st);
    case 64: return pa_launch<64, PER>(a, Z, which, st);
    case 128: return pa_launch<128, PER>(a, Z, which, st);
  }
  ld_set_last_message("proximity attention: dim must be 16, 32, 64 or 128");
  return LD_ERR_UNSUPPORTED;
}

int pa_check(int heads, int Z, int N, int periodic, float lx, float ly, float lz) {
  if (heads <= 0 || Z < 0 || N < 0 || Z % heads != 0 || Z > 65535) return LD_ERR_SHAPE;
  if (periodic && !(lx > 0.f && ly > 0.f && lz > 0.f)) return LD_ERR_SHAPE;
  return LD_OK;
}

}  // namespace

extern "C" int ld_proxattn_fwd(const float* Q, const float* K, const float* V, const float* X, const float* Y, const float* r0sq,
                               int heads, int Z, int N, int dim, int periodic, float box_x, float box_y, float box_z, float* out,
                               void* stream) {
  const int rc = pa_check(heads, Z, N, periodic, box_x, box_y, box_z);
  if (rc != LD_OK) return rc;
  if (Z == 0 || N == 0) return LD_OK;
  PaArgs a{};
  a.Q = Q; a.K = K; a.V = V; a.X = X; a.Y = Y; a.r0sq = r0sq; a.out = out; a.heads = heads; a.N = N;
  a.box = PaBox{box_x, box_y, box_z};
  return periodic ? pa_dispatch<true>(a, Z, dim, 0, (cudaStream_t)stream) : pa_dispatch<false>(a, Z, dim, 0, (cudaStream_t)stream);
}

extern "C" int ld_proxattn_bwd(const float* Q, const float* K, const float* V, const float* X, const float* Y, const float* r0sq,
                               int heads, int Z, int N, int dim, int periodic, float box_x, float box_y, float box_z,
                               const float* d_out, float* dQ, float* dK, float* dV, float* dX, float* dY, void* stream) {
  int rc = pa_check(heads, Z, N, periodic, box_x, box_y, box_z);
  if (rc != LD_OK) return rc;
  if (Z == 0 || N == 0) return LD_OK;
  PaArgs a{};
  a.Q = Q; a.K = K; a.V = V; a.X = X; a.Y = Y; a.r0sq = r0sq; a.dO = d_out; a.heads = heads; a.N = N;
  a.dQ = dQ; a.dK = dK; a.dV = dV; a.dX = dX; a.dY = dY;
  a.box = PaBox{box_x, box_y, box_z};
  cudaStream_t st = (cudaStream_t)stream;
  rc = periodic ? pa_dispatch<true>(a, Z, dim, 2, st) : pa_dispatch<false>(a, Z, dim, 2, st);
  if (rc != LD_OK) return rc;
  return periodic ? pa_dispatch<true>(a, Z, dim, 1, st) : pa_dispatch<false>(a, Z, dim, 1, st);
}
