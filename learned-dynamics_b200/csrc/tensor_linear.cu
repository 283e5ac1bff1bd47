// Channel mixing for rank-0/1/2 Cartesian tensors, FP32 SIMT path:
//   y[r, o, s] = sum_i W[o, i] * x[r, i, s],   s in [0, 3^inds)
// Replaces tensorLinearKern / tensorLinearBackwardKern of the reference
// (extensions/tensor_ops/tensor_ops_kern.cu:6-71; autograd glue tensor_ops.cpp:31-170).
// The reference gives one warp to each (output channel, row); here a block computes a
// 64-output x (rows*3^inds) tile from shared memory, so W is read once per 16..64 rows instead
// of once per row. W may be strided (the backward pass uses it transposed); x and y are
// contiguous. This path keeps full FP32 products and accumulation (1e-5 parity); the tensor-core
// path for large row counts lives in gemm_tc.cu.
#include "common.cuh"

namespace {

constexpr int TL_TO = 64;   // outputs per block
constexpr int TL_KC = 16;   // input channels per shared-memory step

template <int S, int CPT>
__global__ void __launch_bounds__(256)
tensor_linear_kernel(const float* __restrict__ W, long long sw0, long long sw1, const float* __restrict__ x,
                     float* __restrict__ y, long long rows, int I, int O) {
  constexpr int C = 16 * CPT;       // columns (row, s) per block
  static_assert(C % S == 0, "tile must hold whole rows");
  constexpr int TR = C / S;         // rows per block
  __shared__ __align__(16) float Ws[TL_KC][TL_TO];
  __shared__ float Xs[TL_KC][C];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const long long r0 = (long long)blockIdx.x * TR;
  const int o0 = blockIdx.y * TL_TO;
  float acc[4][CPT];
#pragma unroll
  for (int u = 0; u < 4; u++)
#pragma unroll
    for (int j = 0; j < CPT; j++) acc[u][j] = 0.f;

  for (int i0 = 0; i0 < I; i0 += TL_KC) {
    for (int idx = tid; idx < TL_KC * TL_TO; idx += 256) {
      const int kc = idx % TL_KC, o = idx / TL_KC;
      float v = 0.f;
      if (i0 + kc < I && o0 + o < O) v = W[(long long)(o0 + o) * sw0 + (long long)(i0 + kc) * sw1];
      Ws[kc][o] = v;
    }
    for (int idx = tid; idx < TR * TL_KC * S; idx += 256) {
      const int rl = idx / (TL_KC * S), rem = idx % (TL_KC * S);
      const int kc = rem / S, s = rem % S;
      float v = 0.f;
      if (r0 + rl < rows && i0 + kc < I) v = x[((r0 + rl) * I + i0) * S + rem];
      Xs[kc][rl * S + s] = v;
    }
    __syncthreads();
#pragma unroll
    for (int kc = 0; kc < TL_KC; kc++) {
      const float4 a = *reinterpret_cast<const float4*>(&Ws[kc][ty * 4]);
      float b[CPT];
#pragma unroll
      for (int j = 0; j < CPT; j++) b[j] = Xs[kc][tx + 16 * j];
#pragma unroll
      for (int j = 0; j < CPT; j++) {
        acc[0][j] = fmaf(a.x, b[j], acc[0][j]);
        acc[1][j] = fmaf(a.y, b[j], acc[1][j]);
        acc[2][j] = fmaf(a.z, b[j], acc[2][j]);
        acc[3][j] = fmaf(a.w, b[j], acc[3][j]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int j = 0; j < CPT; j++) {
    const int c = tx + 16 * j;
    const int rl = c / S, s = c % S;
    const long long r = r0 + rl;
    if (r >= rows) continue;
#pragma unroll
    for (int u = 0; u < 4; u++) {
      const int o = o0 + ty * 4 + u;
      if (o < O) y[(r * O + o) * S + s] = acc[u][j];
    }
  }
}

// dW[o, i] = sum_{r, s} dy[r, o, s] * x[r, i, s]. Block = 64 x 64 tile of dW over one slice of rows.
// nsplit > 1: partial[z][o][i] written, summed afterwards in fixed order (no atomics).
template <int S>
__global__ void __launch_bounds__(256)
tensor_linear_dw_kernel(const float* __restrict__ dy, const float* __restrict__ x, float* __restrict__ out,
                        long long rows, int I, int O, long long rows_per_split) {
  constexpr int RK = (S == 1) ? 16 : (S == 3 ? 8 : 2);  // rows per step
  constexpr int KC = RK * S;
  __shared__ __align__(16) float As[KC][64];
  __shared__ __align__(16) float Bs[KC][64];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int o0 = blockIdx.y * 64, i0 = blockIdx.x * 64;
  const long long rbeg = (long long)blockIdx.z * rows_per_split;
  const long long rend = (rbeg + rows_per_split < rows) ? rbeg + rows_per_split : rows;
  float acc[4][4];
#pragma unroll
  for (int u = 0; u < 4; u++)
#pragma unroll
    for (int v = 0; v < 4; v++) acc[u][v] = 0.f;
  for (long long r0 = rbeg; r0 < rend; r0 += RK) {
    for (int idx = tid; idx < RK * 64 * S; idx += 256) {
      const int rl = idx / (64 * S), rem = idx % (64 * S);
      const int ch = rem / S, s = rem % S;
      float a = 0.f, b = 0.f;
      if (r0 + rl < rend) {
        if (o0 + ch < O) a = dy[((r0 + rl) * O + o0 + ch) * S + s];
        if (i0 + ch < I) b = x[((r0 + rl) * I + i0 + ch) * S + s];
      }
      As[rl * S + s][ch] = a;
      Bs[rl * S + s][ch] = b;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < KC; k++) {
      const float4 a = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
      const float4 b = *reinterpret_cast<const float4*>(&Bs[k][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int u = 0; u < 4; u++)
#pragma unroll
        for (int v = 0; v < 4; v++) acc[u][v] = fmaf(av[u], bv[v], acc[u][v]);
    }
    __syncthreads();
  }
  float* dst = out + (size_t)blockIdx.z * O * I;
#pragma unroll
  for (int u = 0; u < 4; u++)
#pragma unroll
    for (int v = 0; v < 4; v++) {
      const int o = o0 + ty * 4 + u, i = i0 + tx * 4 + v;
      if (o < O && i < I) dst[(size_t)o * I + i] = acc[u][v];
    }
}

__global__ void sum_partials_kernel(const float* __restrict__ partial, int nsplit, size_t n, float* __restrict__ out) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float a = 0.f;
    for (int z = 0; z < nsplit; z++) a += partial[(size_t)z * n + i];
    out[i] = a;
  }
}

int dw_splits(long long rows, int I, int O) {
  long long tiles = (long long)ld_cdiv(I, 64) * ld_cdiv(O, 64);
  long long want = (148 * 2 + tiles - 1) / tiles;
  long long maxs = (rows + 255) / 256;
  if (want > maxs) want = maxs;
  if (want < 1) want = 1;
  if (want > 64) want = 64;
  return (int)want;
}

}  // namespace

// inds in {0,1,2}. W[o,i] at W + o*sw0 + i*sw1 (element strides). x:[rows, I, 3^inds], y:[rows, O, 3^inds].
extern "C" int ld_tensor_linear(int inds, const float* W, long long sw0, long long sw1, const float* x, float* y,
                                long long rows, int dim_in, int dim_out, void* stream) {
  if (inds < 0 || inds > 2) { ld_set_last_message("tensor_linear supports up to 2 tensor indices"); return LD_ERR_UNSUPPORTED; }
  if (rows < 0 || dim_in < 0 || dim_out < 0) return LD_ERR_SHAPE;
  if (rows == 0 || dim_out == 0) return LD_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int gy = ld_cdiv(dim_out, TL_TO);
  if (inds == 0) {
    dim3 g((unsigned)((rows + 63) / 64), gy);
    tensor_linear_kernel<1, 4><<<g, 256, 0, st>>>(W, sw0, sw1, x, y, rows, dim_in, dim_out);
  } else if (inds == 1) {
    dim3 g((unsigned)((rows + 31) / 32), gy);
    tensor_linear_kernel<3, 6><<<g, 256, 0, st>>>(W, sw0, sw1, x, y, rows, dim_in, dim_out);
  } else {
    dim3 g((unsigned)((rows + 15) / 16), gy);
    tensor_linear_kernel<9, 9><<<g, 256, 0, st>>>(W, sw0, sw1, x, y, rows, dim_in, dim_out);
  }
  LD_LAUNCH_CHECK();
  return LD_OK;
}

extern "C" int ld_tensor_linear_dw_workspace(int inds, long long rows, int dim_in, int dim_out, size_t* bytes) {
  if (inds < 0 || inds > 2 || rows < 0) return LD_ERR_SHAPE;
  int ns = dw_splits(rows, dim_in, dim_out);
  *bytes = ns > 1 ? (size_t)ns * dim_in * dim_out * 4 : 0;
  return LD_OK;
}

// dW[o,i] (contiguous [dim_out, dim_in]) = sum_{r,s} dy[r,o,s] x[r,i,s]
extern "C" int ld_tensor_linear_dw(int inds, const float* dy, const float* x, float* dW, long long rows, int dim_in,
                                   int dim_out, void* workspace, size_t workspace_bytes, void* stream) {
  if (inds < 0 || inds > 2) return LD_ERR_UNSUPPORTED;
  if (rows < 0 || dim_in < 0 || dim_out < 0) return LD_ERR_SHAPE;
  if (dim_in == 0 || dim_out == 0) return LD_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (rows == 0) { LD_CUDA_TRY(cudaMemsetAsync(dW, 0, (size_t)dim_in * dim_out * 4, st)); return LD_OK; }
  const int ns = dw_splits(rows, dim_in, dim_out);
  const size_t need = ns > 1 ? (size_t)ns * dim_in * dim_out * 4 : 0;
  if (need > workspace_bytes || (need > 0 && workspace == nullptr)) return LD_ERR_WORKSPACE;
  float* out = ns > 1 ? (float*)workspace : dW;
  const long long per = (rows + ns - 1) / ns;
  dim3 g(ld_cdiv(dim_in, 64), ld_cdiv(dim_out, 64), ns);
  if (inds == 0) tensor_linear_dw_kernel<1><<<g, 256, 0, st>>>(dy, x, out, rows, dim_in, dim_out, per);
  else if (inds == 1) tensor_linear_dw_kernel<3><<<g, 256, 0, st>>>(dy, x, out, rows, dim_in, dim_out, per);
  else tensor_linear_dw_kernel<9><<<g, 256, 0, st>>>(dy, x, out, rows, dim_in, dim_out, per);
  LD_LAUNCH_CHECK();
  if (ns > 1) {
    const size_t n = (size_t)dim_in * dim_out;
    sum_partials_kernel<<<ld_cdiv((long long)n, 256), 256, 0, st>>>((const float*)workspace, ns, n, dW);
    LD_LAUNCH_CHECK();
  }
  return LD_OK;
}
