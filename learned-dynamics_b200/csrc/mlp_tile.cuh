// A 32-row tile of a dense layer kept entirely in shared memory (FP32 SIMT path).
// Shared by the per-node MLP kernel and the fused PaiNN message kernel: the three layers of an
// MLP run back to back on the same 32 rows (edges or nodes) without touching HBM in between.
//
// Layouts. Activations are "k-major": h[k][32] (32 consecutive floats = the 32 rows of the
// tile), so that for a fixed k all 32 values are fetched with eight broadcast 16-byte loads.
// Weights are passed pre-transposed, Wt[K][N] (nn.Linear stores [N][K]); a K-chunk of Wt is a
// contiguous slab that is staged with 16-byte cp.async copies, double buffered.
// Thread mapping (256 threads): warp w owns columns [w*N/8, (w+1)*N/8); lane owns up to NCOL of
// them (lane, lane+32) and all 32 rows: 32*NCOL accumulators, operand reuse 32x for weights.
#pragma once
#include <cuda_runtime.h>
#include "tp_math.h"

constexpr int MT_ROWS = 32;     // rows per tile
constexpr int MT_KC = 16;       // K-chunk staged per step
constexpr int MT_THREADS = 256;

enum { LD_ACT_NONE = 0, LD_ACT_SILU = 1, LD_ACT_LEAKY01 = 2 };

__device__ __forceinline__ float mt_act(float v, int act) {
  if (act == LD_ACT_SILU) return silu_f(v);
  if (act == LD_ACT_LEAKY01) return v > 0.f ? v : 0.1f * v;
  return v;
}

__device__ __forceinline__ void mt_cp_async16(void* smem, const void* gmem) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void mt_cp_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void mt_cp_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// Stage rows [k0, k0+kc) of Wt (row length N floats, N % 4 == 0) into dst[kc][N].
__device__ __forceinline__ void mt_stage_weights(float* dst, const float* __restrict__ Wt, int N, int k0, int kc) {
  const int vec_per_row = N >> 2;
  const int total = kc * vec_per_row;
  const float* src = Wt + (size_t)k0 * N;
  for (int i = threadIdx.x; i < total; i += MT_THREADS) mt_cp_async16(dst + 4 * i, src + 4 * i);
}

// hout = act(hin * Wt + bias) for one 32-row tile.
//   hin  : shared, k-major [K][ldh] (ldh >= 32, multiple of 4; default 32)
//   hout : shared; ROW_MAJOR_OUT ? [32][ldo] : k-major [N][32]
//   wstage : shared, 2 * MT_KC * N floats
// Requires N % 8 == 0 and N <= 256 * NCOL. Ends with __syncthreads().
template <int NCOL, bool ROW_MAJOR_OUT>
__device__ void mt_tile_linear(const float* hin, int K, const float* __restrict__ Wt, const float* __restrict__ bias, int N,
                               int act, float* hout, int ldo, float* wstage, int ldh = MT_ROWS) {
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cpw = N >> 3;  // columns per warp
  int col[NCOL];
  bool valid[NCOL];
#pragma unroll
  for (int j = 0; j < NCOL; j++) {
    valid[j] = lane + 32 * j < cpw;
    col[j] = w * cpw + (valid[j] ? lane + 32 * j : 0);
  }
  float acc[NCOL][MT_ROWS];
#pragma unroll
  for (int j = 0; j < NCOL; j++)
#pragma unroll
    for (int e = 0; e < MT_ROWS; e++) acc[j][e] = 0.f;

  const int nchunks = (K + MT_KC - 1) / MT_KC;
  mt_stage_weights(wstage, Wt, N, 0, min(MT_KC, K));
  mt_cp_commit();
  for (int ch = 0; ch < nchunks; ch++) {
    const int k0 = ch * MT_KC;
    const int kc = min(MT_KC, K - k0);
    float* cur = wstage + (ch & 1) * MT_KC * N;
    if (ch + 1 < nchunks) {
      mt_stage_weights(wstage + ((ch + 1) & 1) * MT_KC * N, Wt, N, k0 + MT_KC, min(MT_KC, K - k0 - MT_KC));
      mt_cp_commit();
      mt_cp_wait<1>();
    } else {
      mt_cp_wait<0>();
    }
    __syncthreads();
    for (int kk = 0; kk < kc; kk++) {
      float a[MT_ROWS];
      const float4* ap = reinterpret_cast<const float4*>(hin + (size_t)(k0 + kk) * ldh);
#pragma unroll
      for (int q = 0; q < MT_ROWS / 4; q++) {
        const float4 v = ap[q];
        a[4 * q] = v.x; a[4 * q + 1] = v.y; a[4 * q + 2] = v.z; a[4 * q + 3] = v.w;
      }
#pragma unroll
      for (int j = 0; j < NCOL; j++) {
        const float b = cur[kk * N + col[j]];
#pragma unroll
        for (int e = 0; e < MT_ROWS; e++) acc[j][e] = fmaf(a[e], b, acc[j][e]);
      }
    }
    __syncthreads();  // everyone is done with `cur` before it is overwritten two steps later
  }
#pragma unroll
  for (int j = 0; j < NCOL; j++) {
    if (!valid[j]) continue;
    const float bv = bias != nullptr ? bias[col[j]] : 0.f;
    if (ROW_MAJOR_OUT) {
#pragma unroll
      for (int e = 0; e < MT_ROWS; e++) hout[(size_t)e * ldo + col[j]] = mt_act(acc[j][e] + bv, act);
    } else {
      float4* op = reinterpret_cast<float4*>(hout + (size_t)col[j] * MT_ROWS);
      // rotate the 16-byte pieces by lane so that the eight lanes of a store phase hit different banks
#pragma unroll
      for (int q = 0; q < MT_ROWS / 4; q++) {
        const int qq = (q + lane) & 7;
        float4 v;
        // register arrays need compile-time indices: select with a small switch
        float t[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
          float s = 0.f;
#pragma unroll
          for (int z = 0; z < MT_ROWS / 4; z++) s = (z == qq) ? acc[j][4 * z + u] : s;
          t[u] = mt_act(s + bv, act);
        }
        v.x = t[0]; v.y = t[1]; v.z = t[2]; v.w = t[3];
        op[qq] = v;
      }
    }
  }
  __syncthreads();
}
