// Channel-wise l<=2 Cartesian tensor products and their adjoints (the "Bee" and "Cow" sets).
// Replaces bee_fwd/bwl/bwr and cow_o0/o1 fwd/bwl/bwr of the reference's generated
// extensions/codegen_tensops (codegen_tensops_kern.cu:3800-4394, wrappers codegen_tensops.cpp:1519-1979).
// One thread per (row, channel); a warp covers 32 consecutive channels, so its loads of the
// rank-1 / rank-2 operands touch 96 / 288 consecutive floats (every fetched sector is used).
// These ops are HBM bound: 26 floats in, 63 out per (row, channel) for the forward Bee set.
#include "common.cuh"
#include <cuda_bf16.h>
#include "tp_math.h"

namespace {

__device__ __forceinline__ void ld3(const float* p, size_t i, float* v) { v[0] = p[i * 3]; v[1] = p[i * 3 + 1]; v[2] = p[i * 3 + 2]; }
__device__ __forceinline__ void ld9(const float* p, size_t i, float* v) {
#pragma unroll
  for (int k = 0; k < 9; k++) v[k] = p[i * 9 + k];
}
__device__ __forceinline__ void st3(float* p, size_t i, const float* v) { p[i * 3] = v[0]; p[i * 3 + 1] = v[1]; p[i * 3 + 2] = v[2]; }
__device__ __forceinline__ void st9(float* p, size_t i, const float* v) {
#pragma unroll
  for (int k = 0; k < 9; k++) p[i * 9 + k] = v[k];
}

struct BeePtrs { float* y[13]; };
struct BeeGrads { const float* g[13]; };

__global__ void bee_fwd_kernel(const float* __restrict__ l0, const float* __restrict__ l1, const float* __restrict__ l2,
                               const float* __restrict__ r0, const float* __restrict__ r1, const float* __restrict__ r2,
                               BeePtrs out, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float a1[3], a2[9], b1[3], b2[9];
    ld3(l1, i, a1); ld9(l2, i, a2); ld3(r1, i, b1); ld9(r2, i, b2);
    BeeOut o;
    bee_fwd_point(l0[i], a1, a2, r0[i], b1, b2, &o);
    out.y[0][i] = o.y000; out.y[1][i] = o.y110; out.y[2][i] = o.y220;
    st3(out.y[3], i, o.y011); st3(out.y[4], i, o.y101); st3(out.y[5], i, o.y121); st3(out.y[6], i, o.y211);
    st9(out.y[7], i, o.y022); st9(out.y[8], i, o.y202); st9(out.y[9], i, o.y112); st9(out.y[10], i, o.y222);
    st3(out.y[11], i, o.y111); st9(out.y[12], i, o.y212);
  }
}

__device__ __forceinline__ void load_grads(const BeeGrads& G, size_t i, BeeOut* g) {
  g->y000 = G.g[0][i]; g->y110 = G.g[1][i]; g->y220 = G.g[2][i];
  ld3(G.g[3], i, g->y011); ld3(G.g[4], i, g->y101); ld3(G.g[5], i, g->y121); ld3(G.g[6], i, g->y211);
  ld9(G.g[7], i, g->y022); ld9(G.g[8], i, g->y202); ld9(G.g[9], i, g->y112); ld9(G.g[10], i, g->y222);
  ld3(G.g[11], i, g->y111); ld9(G.g[12], i, g->y212);
}

// LEFT=true: d/dl given r ; LEFT=false: d/dr given l
template <bool LEFT>
__global__ void bee_bw_kernel(const float* __restrict__ o0, const float* __restrict__ o1, const float* __restrict__ o2,
                              BeeGrads G, float* __restrict__ d0, float* __restrict__ d1, float* __restrict__ d2, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float b1[3], b2[9];
    ld3(o1, i, b1); ld9(o2, i, b2);
    BeeOut g;
    load_grads(G, i, &g);
    float r0v, r1v[3], r2v[9];
    if (LEFT) bee_bwl_point(o0[i], b1, b2, &g, &r0v, r1v, r2v);
    else bee_bwr_point(o0[i], b1, b2, &g, &r0v, r1v, r2v);
    d0[i] = r0v; st3(d1, i, r1v); st9(d2, i, r2v);
  }
}

// ---- Cow sets (l <= 1) ---------------------------------------------------------------------------
__global__ void cow_o0_fwd_kernel(const float* __restrict__ l0, const float* __restrict__ l1, const float* __restrict__ r0,
                                  const float* __restrict__ r1, float* __restrict__ y000, float* __restrict__ y110, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float a[3], b[3];
    ld3(l1, i, a); ld3(r1, i, b);
    y000[i] = l0[i] * r0[i];
    y110[i] = a[0] * b[0] + a[1] * b[1] + a[2] * b[2];
  }
}

// adjoint of cow_o0 w.r.t. one side given the other side's operands (the set is symmetric)
__global__ void cow_o0_bw_kernel(const float* __restrict__ o0, const float* __restrict__ o1, const float* __restrict__ g000,
                                 const float* __restrict__ g110, float* __restrict__ d0, float* __restrict__ d1, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float b[3];
    ld3(o1, i, b);
    const float g1 = g110[i];
    d0[i] = g000[i] * o0[i];
    float v[3] = {g1 * b[0], g1 * b[1], g1 * b[2]};
    st3(d1, i, v);
  }
}

__global__ void cow_o1_fwd_kernel(const float* __restrict__ l0, const float* __restrict__ l1, const float* __restrict__ r0,
                                  const float* __restrict__ r1, float* __restrict__ y011, float* __restrict__ y101,
                                  float* __restrict__ y111, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float a[3], b[3], c[3];
    ld3(l1, i, a); ld3(r1, i, b);
    const float a0 = l0[i], b0 = r0[i];
    float u[3] = {a0 * b[0], a0 * b[1], a0 * b[2]};
    float v[3] = {a[0] * b0, a[1] * b0, a[2] * b0};
    ld_cross(a, b, c);
    st3(y011, i, u); st3(y101, i, v); st3(y111, i, c);
  }
}

// LEFT=true: (dl_0, dl_1) from (r_0, r_1); LEFT=false: (dr_0, dr_1) from (l_0, l_1)
template <bool LEFT>
__global__ void cow_o1_bw_kernel(const float* __restrict__ o0, const float* __restrict__ o1, const float* __restrict__ g011,
                                 const float* __restrict__ g101, const float* __restrict__ g111, float* __restrict__ d0,
                                 float* __restrict__ d1, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float b[3], ga[3], gb[3], gc[3], c[3];
    ld3(o1, i, b); ld3(g011, i, ga); ld3(g101, i, gb); ld3(g111, i, gc);
    const float b0 = o0[i];
    float s, v[3];
    if (LEFT) {
      // y011 = l0 r1 ; y101 = l1 r0 ; y111 = l1 x r1
      s = ga[0] * b[0] + ga[1] * b[1] + ga[2] * b[2];
      ld_cross(b, gc, c);
      for (int k = 0; k < 3; k++) v[k] = gb[k] * b0 + c[k];
    } else {
      s = gb[0] * b[0] + gb[1] * b[1] + gb[2] * b[2];
      ld_cross(gc, b, c);
      for (int k = 0; k < 3; k++) v[k] = ga[k] * b0 + c[k];
    }
    d0[i] = s;
    st3(d1, i, v);
  }
}

inline int grid_for(size_t n) {
  size_t b = (n + 255) / 256;
  const size_t cap = 148 * 32;
  return (int)(b < cap ? (b ? b : 1) : cap);
}

// Node-local products of SelfTensProds (archs/diffuser_atoms15.py:59-95) in the layout its Y maps want as ONE
// channel mixing per rank: left and right operands come from one linear per rank with 2*chan outputs
// (lr[row][0:chan] = left, [chan:2chan] = right), the 13 products are written concatenated,
//   P_a[row][3*chan]      = (000 | 110 | 220)
//   P_v[row][5*chan][3]   = (011 | 101 | 121 | 211 | 111)
//   P_d[row][5*chan][3][3] = (022 | 202 | 112 | 222 | 212).
// A warp owns (row, 32 channels). Rank-1/2 operands and results have a stride of 3 or 9 floats per channel; they
// pass through a per-warp shared-memory buffer so that every global access of the warp is a contiguous 128 bytes
// (strides 3 and 9 are coprime with the 32 banks: no conflicts).
constexpr int SP_WARPS = 4;

template <int S>
__device__ __forceinline__ void sp_load(const float* __restrict__ g, float* wbuf, int lane, float* v) {
#pragma unroll
  for (int j = 0; j < S; j++) wbuf[lane + 32 * j] = __ldg(g + lane + 32 * j);
  __syncwarp();
#pragma unroll
  for (int s = 0; s < S; s++) v[s] = wbuf[lane * S + s];
  __syncwarp();
}
template <int S, typename OT>
__device__ __forceinline__ void sp_store(OT* __restrict__ g, float* wbuf, int lane, const float* v) {
#pragma unroll
  for (int s = 0; s < S; s++) wbuf[lane * S + s] = v[s];
  __syncwarp();
#pragma unroll
  for (int j = 0; j < S; j++) g[lane + 32 * j] = (OT)wbuf[lane + 32 * j];
  __syncwarp();
}

// CM: lr1 / lr2 are component-major, [rows][3][2*chan] and [rows][9][2*chan] (lanes read consecutive addresses)
template <typename OT, bool CM>
__global__ void __launch_bounds__(SP_WARPS * 32)
bee_self_products_kernel(const float* __restrict__ lr0, const float* __restrict__ lr1, const float* __restrict__ lr2,
                         long long rows, int C, float* __restrict__ P_a, OT* __restrict__ P_v, OT* __restrict__ P_d) {
  __shared__ float s_buf[SP_WARPS][288];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  float* wbuf = s_buf[w];
  const int groups = C >> 5;
  const long long items = rows * groups;
  for (long long it = (long long)blockIdx.x * SP_WARPS + w; it < items; it += (long long)gridDim.x * SP_WARPS) {
    const long long row = it / groups;
    const int c0 = (int)(it - row * groups) * 32;
    const size_t in = (size_t)row * 2 * C + c0;     // left operand of channel c0 (right: + C)
    float l1[3], l2[9], r1[3], r2[9];
    const float l0 = __ldg(lr0 + in + lane), r0 = __ldg(lr0 + in + C + lane);
    if (CM) {
      const float* p1 = lr1 + (size_t)row * 3 * 2 * C + c0 + lane;
      const float* p2 = lr2 + (size_t)row * 9 * 2 * C + c0 + lane;
#pragma unroll
      for (int x = 0; x < 3; x++) { l1[x] = __ldg(p1 + (size_t)x * 2 * C); r1[x] = __ldg(p1 + (size_t)x * 2 * C + C); }
#pragma unroll
      for (int x = 0; x < 9; x++) { l2[x] = __ldg(p2 + (size_t)x * 2 * C); r2[x] = __ldg(p2 + (size_t)x * 2 * C + C); }
    } else {
      sp_load<3>(lr1 + in * 3, wbuf, lane, l1);
      sp_load<3>(lr1 + (in + C) * 3, wbuf, lane, r1);
      sp_load<9>(lr2 + in * 9, wbuf, lane, l2);
      sp_load<9>(lr2 + (in + C) * 9, wbuf, lane, r2);
    }
    BeeOut o;
    bee_fwd_point(l0, l1, l2, r0, r1, r2, &o);
    float* pa = P_a + (size_t)row * 3 * C + c0 + lane;
    pa[0] = o.y000; pa[C] = o.y110; pa[2 * C] = o.y220;
    if (sizeof(OT) == 2) {
      // BF16 outputs are component-major, [row][3 | 9][5*chan]: lanes are consecutive addresses, no staging needed
      OT* pv = P_v + (size_t)row * 3 * 5 * C + c0 + lane;
      OT* pd = P_d + (size_t)row * 9 * 5 * C + c0 + lane;
      const float* vs[5] = {o.y011, o.y101, o.y121, o.y211, o.y111};
      const float* ds[5] = {o.y022, o.y202, o.y112, o.y222, o.y212};
#pragma unroll
      for (int q = 0; q < 5; q++) {
#pragma unroll
        for (int x = 0; x < 3; x++) pv[(size_t)x * 5 * C + q * C] = (OT)vs[q][x];
#pragma unroll
        for (int x = 0; x < 9; x++) pd[(size_t)x * 5 * C + q * C] = (OT)ds[q][x];
      }
    } else {
      OT* pv = P_v + ((size_t)row * 5 * C + c0) * 3;
      sp_store<3>(pv, wbuf, lane, o.y011);
      sp_store<3>(pv + (size_t)C * 3, wbuf, lane, o.y101);
      sp_store<3>(pv + (size_t)2 * C * 3, wbuf, lane, o.y121);
      sp_store<3>(pv + (size_t)3 * C * 3, wbuf, lane, o.y211);
      sp_store<3>(pv + (size_t)4 * C * 3, wbuf, lane, o.y111);
      OT* pd = P_d + ((size_t)row * 5 * C + c0) * 9;
      sp_store<9>(pd, wbuf, lane, o.y022);
      sp_store<9>(pd + (size_t)C * 9, wbuf, lane, o.y202);
      sp_store<9>(pd + (size_t)2 * C * 9, wbuf, lane, o.y112);
      sp_store<9>(pd + (size_t)3 * C * 9, wbuf, lane, o.y222);
      sp_store<9>(pd + (size_t)4 * C * 9, wbuf, lane, o.y212);
    }
  }
}

}  // namespace

// lr0 [rows][2*chan], lr1 [rows][2*chan][3], lr2 [rows][2*chan][3][3]: left operands in channels [0, chan), right in
// [chan, 2*chan). Outputs as described at bee_self_products_kernel. chan a multiple of 32.
// out_bf16: P_v and P_d are BF16 and component-major, [rows][3][5*chan] and [rows][9][5*chan] (the input form of
// ld_linear_bf16_tc_in16); P_a stays FP32.
// ld_bee_self_products_cm: lr1 / lr2 component-major, [rows][3][2*chan] and [rows][9][2*chan]; BF16 outputs only.
static int self_products_launch(const float* lr0, const float* lr1, const float* lr2, long long rows, int chan, float* P_a,
                                void* P_v, void* P_d, int out_bf16, int in_cm, void* stream) {
  if (rows < 0 || chan <= 0) return LD_ERR_SHAPE;
  if (chan % 32 != 0) { ld_set_last_message("bee self products: chan must be a multiple of 32"); return LD_ERR_UNSUPPORTED; }
  if (rows == 0) return LD_OK;
  const long long items = rows * (chan / 32);
  long long blocks = (items + SP_WARPS - 1) / SP_WARPS;
  if (blocks > 148LL * 16) blocks = 148LL * 16;
  if (in_cm && !out_bf16) { ld_set_last_message("bee self products: component-major inputs come with BF16 outputs"); return LD_ERR_UNSUPPORTED; }
  if (in_cm)
    bee_self_products_kernel<__nv_bfloat16, true><<<(unsigned)blocks, SP_WARPS * 32, 0, (cudaStream_t)stream>>>(
        lr0, lr1, lr2, rows, chan, P_a, (__nv_bfloat16*)P_v, (__nv_bfloat16*)P_d);
  else if (out_bf16)
    bee_self_products_kernel<__nv_bfloat16, false><<<(unsigned)blocks, SP_WARPS * 32, 0, (cudaStream_t)stream>>>(
        lr0, lr1, lr2, rows, chan, P_a, (__nv_bfloat16*)P_v, (__nv_bfloat16*)P_d);
  else
    bee_self_products_kernel<float, false><<<(unsigned)blocks, SP_WARPS * 32, 0, (cudaStream_t)stream>>>(lr0, lr1, lr2, rows, chan, P_a,
                                                                                                         (float*)P_v, (float*)P_d);
  LD_LAUNCH_CHECK();
  return LD_OK;
}

extern "C" int ld_bee_self_products(const float* lr0, const float* lr1, const float* lr2, long long rows, int chan, float* P_a,
                                    void* P_v, void* P_d, int out_bf16, void* stream) {
  return self_products_launch(lr0, lr1, lr2, rows, chan, P_a, P_v, P_d, out_bf16, 0, stream);
}

extern "C" int ld_bee_self_products_cm(const float* lr0, const float* lr1, const float* lr2, long long rows, int chan, float* P_a,
                                       void* P_v, void* P_d, void* stream) {
  return self_products_launch(lr0, lr1, lr2, rows, chan, P_a, P_v, P_d, 1, 1, stream);
}

// rows*chan elements per rank-0 operand; operands are contiguous [rows, chan, (3,)^l] float32.
extern "C" int ld_bee_fwd(const float* l0, const float* l1, const float* l2, const float* r0, const float* r1,
                          const float* r2, long long rows, int chan, float* const* out13, void* stream) {
  if (rows < 0 || chan < 0) return LD_ERR_SHAPE;
  const size_t n = (size_t)rows * chan;
  if (n == 0) return LD_OK;
  BeePtrs P;
  for (int k = 0; k < 13; k++) P.y[k] = out13[k];
  bee_fwd_kernel<<<grid_for(n), 256, 0, (cudaStream_t)stream>>>(l0, l1, l2, r0, r1, r2, P, n);
  LD_LAUNCH_CHECK();
  return LD_OK;
}

// left != 0: gradients of the left operands from (r_0,r_1,r_2); else of the right operands from (l_0,l_1,l_2)
extern "C" int ld_bee_bw(int left, const float* o0, const float* o1, const float* o2, const float* const* grads13,
                         long long rows, int chan, float* d0, float* d1, float* d2, void* stream) {
  if (rows < 0 || chan < 0) return LD_ERR_SHAPE;
  const size_t n = (size_t)rows * chan;
  if (n == 0) return LD_OK;
  BeeGrads G;
  for (int k = 0; k < 13; k++) G.g[k] = grads13[k];
  if (left) bee_bw_kernel<true><<<grid_for(n), 256, 0, (cudaStream_t)stream>>>(o0, o1, o2, G, d0, d1, d2, n);
  else bee_bw_kernel<false><<<grid_for(n), 256, 0, (cudaStream_t)stream>>>(o0, o1, o2, G, d0, d1, d2, n);
  LD_LAUNCH_CHECK();
  return LD_OK;
}

extern "C" int ld_cow_o0_fwd(const float* l0, const float* l1, const float* r0, const float* r1, long long rows, int chan,
                             float* y000, float* y110, void* stream) {
  if (rows < 0 || chan < 0) return LD_ERR_SHAPE;
  const size_t n = (size_t)rows * chan;
  if (n == 0) return LD_OK;
  cow_o0_fwd_kernel<<<grid_for(n), 256, 0, (cudaStream_t)stream>>>(l0, l1, r0, r1, y000, y110, n);
  LD_LAUNCH_CHECK();
  return LD_OK;
}

extern "C" int ld_cow_o0_bw(const float* o0, const float* o1, const float* g000, const float* g110, long long rows, int chan,
                            float* d0, float* d1, void* stream) {
  if (rows < 0 || chan < 0) return LD_ERR_SHAPE;
  const size_t n = (size_t)rows * chan;
  if (n == 0) return LD_OK;
  cow_o0_bw_kernel<<<grid_for(n), 256, 0, (cudaStream_t)stream>>>(o0, o1, g000, g110, d0, d1, n);
  LD_LAUNCH_CHECK();
  return LD_OK;
}

extern "C" int ld_cow_o1_fwd(const float* l0, const float* l1, const float* r0, const float* r1, long long rows, int chan,
                             float* y011, float* y101, float* y111, void* stream) {
  if (rows < 0 || chan < 0) return LD_ERR_SHAPE;
  const size_t n = (size_t)rows * chan;
  if (n == 0) return LD_OK;
  cow_o1_fwd_kernel<<<grid_for(n), 256, 0, (cudaStream_t)stream>>>(l0, l1, r0, r1, y011, y101, y111, n);
  LD_LAUNCH_CHECK();
  return LD_OK;
}

extern "C" int ld_cow_o1_bw(int left, const float* o0, const float* o1, const float* g011, const float* g101,
                            const float* g111, long long rows, int chan, float* d0, float* d1, void* stream) {
  if (rows < 0 || chan < 0) return LD_ERR_SHAPE;
  const size_t n = (size_t)rows * chan;
  if (n == 0) return LD_OK;
  if (left) cow_o1_bw_kernel<true><<<grid_for(n), 256, 0, (cudaStream_t)stream>>>(o0, o1, g011, g101, g111, d0, d1, n);
  else cow_o1_bw_kernel<false><<<grid_for(n), 256, 0, (cudaStream_t)stream>>>(o0, o1, g011, g101, g111, d0, d1, n);
  LD_LAUNCH_CHECK();
  return LD_OK;
}
