// Dense-weight l<=2 tensor products ("Ant16": y_o[b,o,.] = sum_{l,r} P[o,l,r] * (left[b,l,.] (x) x[b,r,.]))
// and the bare channel-wise product of two tensors with trailing-index contraction.
//
// Replaces the generated kernels ant16_{o0,o1,o2,oc}{,_backward,_backleft,_wtsback} of
// extensions/codegen_tensops/codegen_tensops_kern.cu:1341-3797 (einsum definitions:
// managan/codegen_tensor_products.py:112-133) and the einsum of TensorProdBare
// (managan/tensor_products.py:91-108).
//
// Factorisation used here. With U[b,(o,l),J] = sum_r P[o,l,r] x[b,r,J] (a tensor_linear with the weight
// P viewed as [(o l), r]) every Ant16 direction is one of three small contractions with the constant
// coupling c[I,J,K] in {0,+1,-1} of the product (I, J, K = flattened spatial indices of left, x, y):
//   forward   y[b,o,K]     = sum_l sum_{IJ} c * left[b,l,I] * U[b,o,l,J]          (ld_ant16_contract_left)
//   backward  dU[b,o,l,J]  = sum_{IK} c * left[b,l,I] * dy[b,o,K]  -> dx = tensor_linear(dU, P^T)   (ld_ant16_expand)
//   backleft  dleft[b,l,I] = sum_o sum_{JK} c * U[b,o,l,J] * dy[b,o,K]            (ld_ant16_contract_out)
//   wtsback   dP[(o,l),r]  = sum_b sum_J dU[b,(o,l),J] * x[b,r,J]                 (tensor_linear weight gradient)
// The two GEMM-shaped steps run on the library's own linear kernels; this file holds the three
// coupling contractions, one template instance per product.
#include <cuda_runtime.h>
#include "common.cuh"

namespace {

// product ids in the reference's fixed order 000,110,220,011,101,121,211,022,202,112,222,111,212
enum { A000 = 0, A110, A220, A011, A101, A121, A211, A022, A202, A112, A222, A111, A212, A_COUNT };

__host__ __device__ constexpr int ipow3(int r) { return r == 0 ? 1 : (r == 1 ? 3 : 9); }
__host__ __device__ constexpr int rank_l(int p) {
  return (p == A000 || p == A011 || p == A022) ? 0 : ((p == A110 || p == A101 || p == A121 || p == A112 || p == A111) ? 1 : 2);
}
__host__ __device__ constexpr int rank_r(int p) {
  return (p == A000 || p == A101 || p == A202) ? 0 : ((p == A110 || p == A011 || p == A211 || p == A112 || p == A111 || p == A212) ? 1 : 2);
}
__host__ __device__ constexpr int rank_o(int p) {
  return (p == A000 || p == A110 || p == A220) ? 0 : ((p == A011 || p == A101 || p == A121 || p == A211 || p == A111) ? 1 : 2);
}
__host__ __device__ constexpr int eps3(int i, int j, int k) { return (i - j) * (j - k) * (k - i) / 2; }

// One coupling term for loop indices (a, b, c, d) in [0,3)^4; sign 0 = no term. Every product uses a
// subset of the four loops (the others must be 0).
struct Term { int I, J, K, s; };
template <int P>
__host__ __device__ constexpr Term term(int a, int b, int c, int d) {
  const bool z1 = (b == 0 && c == 0 && d == 0), z2 = (c == 0 && d == 0), z3 = (d == 0);
  switch (P) {
    case A000: return {0, 0, 0, (a == 0 && z1) ? 1 : 0};
    case A110: return {a, a, 0, z1 ? 1 : 0};
    case A220: return {3 * a + b, 3 * a + b, 0, z2 ? 1 : 0};
    case A011: return {0, a, a, z1 ? 1 : 0};
    case A101: return {a, 0, a, z1 ? 1 : 0};
    case A121: return {a, 3 * b + a, b, z2 ? 1 : 0};          // l_x r_yx -> y
    case A211: return {3 * a + b, b, a, z2 ? 1 : 0};          // l_xy r_y -> x
    case A022: return {0, 3 * a + b, 3 * a + b, z2 ? 1 : 0};
    case A202: return {3 * a + b, 0, 3 * a + b, z2 ? 1 : 0};
    case A112: return {a, b, 3 * a + b, z2 ? 1 : 0};
    case A222: return {3 * a + b, 3 * c + b, 3 * a + c, z3 ? 1 : 0};   // l_xy r_zy -> xz
    case A111: return {a, b, c, z3 ? eps3(a, b, c) : 0};               // l_x r_y eps_xyz -> z
    case A212: return {3 * a + b, c, 3 * a + d, eps3(b, c, d)};        // l_xy r_z eps_yzw -> xw
  }
  return {0, 0, 0, 0};
}

// out[K] += sum c * Lv[I] * Rv[J]   (MODE 0);  out[J] += sum c * Lv[I] * Ov[K] (MODE 1);  out[I] += sum c * Rv[J] * Ov[K] (MODE 2)
template <int P, int MODE>
__device__ __forceinline__ void couple(const float* Lv, const float* Rv, const float* Ov, float* out) {
#pragma unroll
  for (int a = 0; a < 3; a++)
#pragma unroll
    for (int b = 0; b < 3; b++)
#pragma unroll
      for (int c = 0; c < 3; c++)
#pragma unroll
        for (int d = 0; d < 3; d++) {
          const Term t = term<P>(a, b, c, d);
          if (t.s != 0) {
            const float sg = (float)t.s;
            if (MODE == 0) out[t.K] = fmaf(sg * Lv[t.I], Rv[t.J], out[t.K]);
            if (MODE == 1) out[t.J] = fmaf(sg * Lv[t.I], Ov[t.K], out[t.J]);
            if (MODE == 2) out[t.I] = fmaf(sg * Rv[t.J], Ov[t.K], out[t.I]);
          }
        }
}

template <int N>
__device__ __forceinline__ void load_vec(const float* __restrict__ p, float* v) {
#pragma unroll
  for (int i = 0; i < N; i++) v[i] = __ldg(p + i);
}

// y[b,o,:] (+)= sum_l couple(left[b,l,:], U[b,o,l,:]); thread = (b, o), o fastest
template <int P>
__global__ void __launch_bounds__(256) contract_left_kernel(const float* __restrict__ left, const float* __restrict__ U,
                                                            long long rows, int dim_o, int dim_l, float* __restrict__ y,
                                                            int accumulate) {
  constexpr int SL = ipow3(rank_l(P)), SR = ipow3(rank_r(P)), SO = ipow3(rank_o(P));
  const long long total = rows * dim_o;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const long long b = idx / dim_o;
    float acc[SO];
#pragma unroll
    for (int k = 0; k < SO; k++) acc[k] = 0.f;
    const float* lp = left + b * dim_l * SL;
    const float* up = U + idx * dim_l * SR;
    for (int l = 0; l < dim_l; l++) {
      float Lv[SL], Rv[SR];
      load_vec<SL>(lp + l * SL, Lv);
      load_vec<SR>(up + l * SR, Rv);
      couple<P, 0>(Lv, Rv, nullptr, acc);
    }
#pragma unroll
    for (int k = 0; k < SO; k++) y[idx * SO + k] = accumulate ? y[idx * SO + k] + acc[k] : acc[k];
  }
}

// dU[b,o,l,:] = couple(left[b,l,:], dy[b,o,:]); thread = (b, o, l), l fastest
template <int P>
__global__ void __launch_bounds__(256) expand_kernel(const float* __restrict__ left, const float* __restrict__ dy, long long rows,
                                                     int dim_o, int dim_l, float* __restrict__ dU) {
  constexpr int SL = ipow3(rank_l(P)), SR = ipow3(rank_r(P)), SO = ipow3(rank_o(P));
  const long long total = rows * dim_o * dim_l;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const int l = (int)(idx % dim_l);
    const long long bo = idx / dim_l, b = bo / dim_o;
    float Lv[SL], Ov[SO], out[SR];
    load_vec<SL>(left + (b * dim_l + l) * SL, Lv);
    load_vec<SO>(dy + bo * SO, Ov);
#pragma unroll
    for (int j = 0; j < SR; j++) out[j] = 0.f;
    couple<P, 1>(Lv, nullptr, Ov, out);
#pragma unroll
    for (int j = 0; j < SR; j++) dU[idx * SR + j] = out[j];
  }
}

// dleft[b,l,:] = sum_o couple(U[b,o,l,:], dy[b,o,:]); thread = (b, l), l fastest
template <int P>
__global__ void __launch_bounds__(256) contract_out_kernel(const float* __restrict__ U, const float* __restrict__ dy, long long rows,
                                                           int dim_o, int dim_l, float* __restrict__ dleft) {
  constexpr int SL = ipow3(rank_l(P)), SR = ipow3(rank_r(P)), SO = ipow3(rank_o(P));
  const long long total = rows * dim_l;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const int l = (int)(idx % dim_l);
    const long long b = idx / dim_l;
    float acc[SL];
#pragma unroll
    for (int i = 0; i < SL; i++) acc[i] = 0.f;
    for (int o = 0; o < dim_o; o++) {
      float Rv[SR], Ov[SO];
      load_vec<SR>(U + ((b * dim_o + o) * dim_l + l) * SR, Rv);
      load_vec<SO>(dy + (b * dim_o + o) * SO, Ov);
      couple<P, 2>(nullptr, Rv, Ov, acc);
    }
#pragma unroll
    for (int i = 0; i < SL; i++) dleft[idx * SL + i] = acc[i];
  }
}

int grid_for(long long total) {
  long long blocks = (total + 255) / 256;
  const long long cap = 148LL * 32;
  return (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

template <int P>
int launch_mode(int mode, const float* a, const float* b, long long rows, int dim_o, int dim_l, float* out, int accumulate,
                cudaStream_t st) {
  if (mode == 0) contract_left_kernel<P><<<grid_for(rows * dim_o), 256, 0, st>>>(a, b, rows, dim_o, dim_l, out, accumulate);
  else if (mode == 1) expand_kernel<P><<<grid_for(rows * dim_o * dim_l), 256, 0, st>>>(a, b, rows, dim_o, dim_l, out);
  else contract_out_kernel<P><<<grid_for(rows * dim_l), 256, 0, st>>>(a, b, rows, dim_o, dim_l, out);
  LD_LAUNCH_CHECK();
  return LD_OK;
}

int dispatch(int product, int mode, const float* a, const float* b, long long rows, int dim_o, int dim_l, float* out,
             int accumulate, cudaStream_t st) {
  switch (product) {
#define LD_CASE(P) case P: return launch_mode<P>(mode, a, b, rows, dim_o, dim_l, out, accumulate, st);
    LD_CASE(A000) LD_CASE(A110) LD_CASE(A220) LD_CASE(A011) LD_CASE(A101) LD_CASE(A121) LD_CASE(A211)
    LD_CASE(A022) LD_CASE(A202) LD_CASE(A112) LD_CASE(A222) LD_CASE(A111) LD_CASE(A212)
#undef LD_CASE
  }
  ld_set_last_message("ant16: product id out of range (0..12)");
  return LD_ERR_SHAPE;
}

int check_dims(long long rows, int dim_o, int dim_l) {
  if (rows < 0 || dim_o <= 0 || dim_l <= 0) {
    ld_set_last_message("ant16: negative row count or non-positive channel count");
    return LD_ERR_SHAPE;
  }
  return LD_OK;
}

// ---- bare channel-wise product with trailing-index contraction --------------------------------------
// y[.., keep_l + keep_r] = sum_c x_l[.., keep_l + c] * x_r[.., keep_r + c], ranks <= 2.
// MODE 0: forward; 1: dl[keep_l + c] = sum_{keep_r} dy * x_r; 2: dr[keep_r + c] = sum_{keep_l} dy * x_l.
template <int MODE>
__global__ void __launch_bounds__(256) bare_prod_kernel(const float* __restrict__ A, const float* __restrict__ B, long long n,
                                                        int nkl, int nkr, int nc, float* __restrict__ out) {
  // sizes (powers of 3): nkl = 3^(kept left indices), nkr = 3^(kept right indices), nc = 3^(contracted indices)
  const int SL = nkl * nc, SR = nkr * nc, SO = nkl * nkr;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < n; idx += (long long)gridDim.x * blockDim.x) {
    if (MODE == 0) {
      const float* xl = A + idx * SL;
      const float* xr = B + idx * SR;
      for (int i = 0; i < nkl; i++)
        for (int j = 0; j < nkr; j++) {
          float s = 0.f;
          for (int c = 0; c < nc; c++) s = fmaf(__ldg(xl + i * nc + c), __ldg(xr + j * nc + c), s);
          out[idx * SO + i * nkr + j] = s;
        }
    } else if (MODE == 1) {
      const float* dy = A + idx * SO;
      const float* xr = B + idx * SR;
      for (int i = 0; i < nkl; i++)
        for (int c = 0; c < nc; c++) {
          float s = 0.f;
          for (int j = 0; j < nkr; j++) s = fmaf(__ldg(dy + i * nkr + j), __ldg(xr + j * nc + c), s);
          out[idx * SL + i * nc + c] = s;
        }
    } else {
      const float* dy = A + idx * SO;
      const float* xl = B + idx * SL;
      for (int j = 0; j < nkr; j++)
        for (int c = 0; c < nc; c++) {
          float s = 0.f;
          for (int i = 0; i < nkl; i++) s = fmaf(__ldg(dy + i * nkr + j), __ldg(xl + i * nc + c), s);
          out[idx * SR + j * nc + c] = s;
        }
    }
  }
}

}  // namespace

extern "C" {

int ld_ant16_contract_left(int product, const float* left, const float* U, long long rows, int dim_o, int dim_l, float* y,
                           int accumulate, void* stream) {
  if (int e = check_dims(rows, dim_o, dim_l)) return e;
  if (rows == 0) return LD_OK;
  return dispatch(product, 0, left, U, rows, dim_o, dim_l, y, accumulate, (cudaStream_t)stream);
}

int ld_ant16_expand(int product, const float* left, const float* dy, long long rows, int dim_o, int dim_l, float* dU,
                    void* stream) {
  if (int e = check_dims(rows, dim_o, dim_l)) return e;
  if (rows == 0) return LD_OK;
  return dispatch(product, 1, left, dy, rows, dim_o, dim_l, dU, 0, (cudaStream_t)stream);
}

int ld_ant16_contract_out(int product, const float* U, const float* dy, long long rows, int dim_o, int dim_l, float* dleft,
                          void* stream) {
  if (int e = check_dims(rows, dim_o, dim_l)) return e;
  if (rows == 0) return LD_OK;
  return dispatch(product, 2, U, dy, rows, dim_o, dim_l, dleft, 0, (cudaStream_t)stream);
}

int ld_tensor_prod_bare(int mode, int inds_l, int inds_r, int inds_o, const float* a, const float* b, long long n, float* out,
                        void* stream) {
  const int twice = inds_l + inds_r - inds_o;
  if (inds_l < 0 || inds_l > 2 || inds_r < 0 || inds_r > 2 || inds_o < 0 || twice < 0 || (twice & 1) || twice / 2 > inds_l ||
      twice / 2 > inds_r || mode < 0 || mode > 2 || n < 0) {
    ld_set_last_message("tensor_prod_bare: ranks must be 0..2 with (inds_l + inds_r - inds_o) / 2 contractions in range");
    return LD_ERR_SHAPE;
  }
  if (n == 0) return LD_OK;
  const int c = twice / 2;
  const int nkl = ipow3(inds_l - c), nkr = ipow3(inds_r - c), nc = ipow3(c);
  cudaStream_t st = (cudaStream_t)stream;
  const int grid = grid_for(n);
  if (mode == 0) bare_prod_kernel<0><<<grid, 256, 0, st>>>(a, b, n, nkl, nkr, nc, out);
  else if (mode == 1) bare_prod_kernel<1><<<grid, 256, 0, st>>>(a, b, n, nkl, nkr, nc, out);
  else bare_prod_kernel<2><<<grid, 256, 0, st>>>(a, b, n, nkl, nkr, nc, out);
  LD_LAUNCH_CHECK();
  return LD_OK;
}

}  // extern "C"
