// l<=2 ("Bee") message layer, fused: Messages.forward of the reference
// (archs/diffuser_atoms15.py:227-253) without edge-sized tensors in HBM.
//
//   phi_a = lin_enc(radial_encode_8(r_ij))                      (managan/jacobi_radenc.py:27-33)
//   rhat  = tens_sigmoid(1, r_ij * 7/r0)                        (managan/tensor_products.py:167-182)
//   phi_v = phi_a (x) rhat,  phi_d = phi_a (x) rhat (x) rhat
//   y_k   = Bee(L0(x_a)[dst], L1(x_v)[dst], L2(x_d)[dst]; phi_a, phi_v, phi_d)   13 products / channel
//   psi_a = Y_000 y_000 + Y_110 y_110 + Y_220 y_220 ; psi_a += mlp_a(psi_a)      per edge
//   psi_v = sum of five Y_k y_k (rank 1), psi_d = sum of five Y_k y_k (rank 2)   per edge
//   B_*   = 0.1 * sum over the edges of each source node
//
// The rank-1 and rank-2 outputs are linear in the products, and the edge sum is linear, so the
// ten products are summed per node first (ld_bee_messages_vd_f32: one thread per channel, sixty
// accumulators in registers, one write per node) and the Y maps then run once per NODE as an
// ordinary channel mixing over 5*chan inputs. Only the scalar output has a per-edge non-linearity
// (mlp_a); ld_bee_messages_scalar_f32 keeps that per edge, in 32-edge tiles in shared memory.
// Both kernels walk node-aligned slices of the CSR; no atomics, fixed summation order.
#include "common.cuh"
#include "mlp_tile.cuh"
#include "tp_math.h"
#include <cuda_bf16.h>
#include "tc05.cuh"

namespace {

__device__ __forceinline__ float bm_ld(const float* p, size_t i) { return __ldg(p + i); }
__device__ __forceinline__ float bm_ld(const __nv_bfloat16* p, size_t i) { return __bfloat162float(p[i]); }


constexpr int BM_TILE = 32;  // edges staged per step (scalar kernel: the rows of its MLP tile)
constexpr int BV_TILE = 128;  // edges staged per step in the product-sum kernel (two block barriers per step)

struct BeeEdgeParams {
  const int* row_ptr; const int* dst; const float* rij;
  int Nt, chan;
  float r0;
  const float* L0; const float* L1; const float* L2;   // [Nt,chan], [Nt,chan,3], [Nt,chan,9]
  const float* enc_w; const float* enc_b;               // lin_enc: [chan,8], [chan]
  const float* jacobi;                                  // [8][9] polynomial coefficients
  int seg_nodes;                                        // nodes per scheduling segment (0: the whole range at once)
  int* next_node;                                       // product-sum kernel: zeroed counter its blocks draw nodes from
};

// first node v in [lo, hi] whose preceding work (edges + nodes) reaches target
__device__ __forceinline__ int bm_work_lower_bound(const int* __restrict__ row_ptr, int lo, int hi, long long target) {
  const long long base = (long long)row_ptr[lo] + lo;
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if ((long long)row_ptr[mid] + mid - base < target) lo = mid + 1; else hi = mid;
  }
  return lo;
}

// this block's slice of the node range [lo, hi), balanced over edges + nodes
__device__ __forceinline__ void bm_block_range(const int* __restrict__ row_ptr, int lo, int hi, int* n_begin, int* n_end) {
  const long long work = ((long long)row_ptr[hi] - row_ptr[lo]) + (hi - lo);
  long long per = (work + gridDim.x - 1) / gridDim.x;
  if (per < 1) per = 1;
  *n_begin = blockIdx.x == 0 ? lo : bm_work_lower_bound(row_ptr, lo, hi, per * blockIdx.x);
  *n_end = blockIdx.x == gridDim.x - 1 ? hi : bm_work_lower_bound(row_ptr, lo, hi, per * (blockIdx.x + 1));
}

// per-edge geometry shared by all channels: rhat[3] and the eight radial features
struct __align__(16) EdgeGeom { float enc[8]; float rhat[3]; float pad; };   // 48 bytes: three 16-byte shared-memory loads

__device__ __forceinline__ void edge_geometry(const float* __restrict__ rij, long long e, float r0,
                                              const float* __restrict__ jac, EdgeGeom* g) {
  const float x = rij[e * 3], y = rij[e * 3 + 1], z = rij[e * 3 + 2];
  const float d = sqrtf(x * x + y * y + z * z);
  const float zz = d / r0;
  const float env = fmaxf(1.f - zz, 0.f);
  ld_radial_cheb8(zz, env, jac, g->enc);
  const float s = 7.f / r0;
  const float ux = x * s, uy = y * s, uz = z * s;
  const float inv = 1.0f / sqrtf(1.f + ux * ux + uy * uy + uz * uz);
  g->rhat[0] = ux * inv; g->rhat[1] = uy * inv; g->rhat[2] = uz * inv;
}

// the right-hand operands of one channel: phi_a scalar, phi_v = phi_a rhat, phi_d = phi_a rhat rhat^T
__device__ __forceinline__ void edge_phi(const EdgeGeom& g, const float* w8, float bias, float* pa, float* pv, float* pd) {
  float a = bias;
#pragma unroll
  for (int m = 0; m < 8; m++) a = fmaf(g.enc[m], w8[m], a);
  *pa = a;
#pragma unroll
  for (int k = 0; k < 3; k++) pv[k] = a * g.rhat[k];
#pragma unroll
  for (int x = 0; x < 3; x++)
#pragma unroll
    for (int y = 0; y < 3; y++) pd[x * 3 + y] = a * g.rhat[x] * g.rhat[y];
}


// ---- rank-1 / rank-2 products summed per node --------------------------------------------------
// S_v[node][k][c][3], k over (011,101,121,211,111); S_d[node][k][c][9], k over (022,202,112,222,212):
// the layouts a channel mixing with 5*chan inputs expects. Thread = channel; a block walks its nodes
// and stages the geometry of up to 32 edges at a time in shared memory.
// CC: the channel count as a compile-time constant (0: taken from the parameters)
template <typename FT, bool PACKED, int CC>
__global__ void __launch_bounds__(128, 4)   // four blocks per SM: at most 128 registers
bee_vd_kernel(BeeEdgeParams P, float* __restrict__ S_v, float* __restrict__ S_d, float scale, int out_bf16_) {
  const int out_bf16 = CC > 0 ? 1 : out_bf16_;   // the instance with a constant width is the tensor-core path's: BF16 sums
  const FT* __restrict__ F0 = reinterpret_cast<const FT*>(P.L0);
  const FT* __restrict__ F1 = reinterpret_cast<const FT*>(P.L1);
  const FT* __restrict__ F2 = reinterpret_cast<const FT*>(P.L2);
  __shared__ EdgeGeom s_geom[BV_TILE];
  __shared__ int s_dst[BV_TILE];
  __shared__ float s_jac[72];
  if (threadIdx.x < 8) ld_poly8_to_chebyshev(P.jacobi + threadIdx.x * 9, s_jac + threadIdx.x * 9);   // Chebyshev form of the radial polynomials
  __syncthreads();
  const int C = CC > 0 ? CC : P.chan;
  // The blocks draw nodes one at a time from a counter: a node's sums are formed by one block in the order of its edge
  // list, so the result does not depend on which block took it. All blocks work at the front of the node range,
  // so the neighbour rows they gather (a node's neighbours are nearby nodes) stay resident in L2, and no block is left
  // with more than one node while others are idle. The next node is asked for while the present one is processed.
  __shared__ int s_node[2];
  int drawn = 0;
  if (threadIdx.x == 0) drawn = atomicAdd(P.next_node, 1);
  const bool one_group = C <= (int)blockDim.x;
  float w8[8], wb = 0.f;
  {
    const bool cok0 = (int)threadIdx.x < C;
#pragma unroll
    for (int m = 0; m < 8; m++) w8[m] = cok0 ? P.enc_w[threadIdx.x * 8 + m] : 0.f;
    if (cok0) wb = P.enc_b[threadIdx.x];
  }
  for (int it = 0;; it++) {
  if (threadIdx.x == 0) s_node[it & 1] = drawn;
  __syncthreads();   // (a slot is rewritten two nodes later, behind the barrier of the node in between)
  const int v = s_node[it & 1];
  if (v >= P.Nt) break;
  if (threadIdx.x == 0) drawn = atomicAdd(P.next_node, 1);
  for (int c0 = 0; c0 < C; c0 += blockDim.x) {   // channel groups (one pass when chan <= 128)
    const int c = c0 + threadIdx.x;
    const bool cok = c < C;
    if (!one_group) {
#pragma unroll
      for (int m = 0; m < 8; m++) w8[m] = cok ? P.enc_w[c * 8 + m] : 0.f;
      wb = cok ? P.enc_b[c] : 0.f;
    }
    {
      // av = (011, 101, 121, 211, 111), ad = (022, 202, 112, 222, 212). Two of the sixty sums need no work per edge: 111
      // (l1 cross phi_v) is the antisymmetric part of 112 (l1 phi_v^T) and is formed from its sums after the loop, and
      // 022 (l0 phi_d, phi_d = pa rhat rhat^T) is symmetric, so only its upper triangle is accumulated
      float av[15], ad[45];
#pragma unroll
      for (int i = 0; i < 15; i++) av[i] = 0.f;
#pragma unroll
      for (int i = 0; i < 45; i++) ad[i] = 0.f;
      const int e_lo = P.row_ptr[v], e_hi = P.row_ptr[v + 1];
      for (int eb = e_lo; eb < e_hi; eb += BV_TILE) {
        const int cnt = min(BV_TILE, e_hi - eb);
        __syncthreads();  // previous tile's readers are done
        constexpr int UNR = 4;  // neighbour rows in flight per thread
        // the edge list of the step is padded to whole batches with edges of weight zero (they read the row of the
        // step's first neighbour), so that the batches below need neither bounds checks nor clamped indices
        const int cnt_pad = (cnt + UNR - 1) & ~(UNR - 1);
        if (threadIdx.x < cnt) {
          edge_geometry(P.rij, (long long)eb + threadIdx.x, P.r0, s_jac, &s_geom[threadIdx.x]);
          s_geom[threadIdx.x].pad = 1.f;
          s_dst[threadIdx.x] = P.dst[eb + threadIdx.x];
        } else if (threadIdx.x < cnt_pad) {
          EdgeGeom z;
#pragma unroll
          for (int m = 0; m < 8; m++) z.enc[m] = 0.f;
          z.rhat[0] = z.rhat[1] = z.rhat[2] = 0.f; z.pad = 0.f;
          s_geom[threadIdx.x] = z;
          s_dst[threadIdx.x] = P.dst[eb];
        }
        __syncthreads();
        if (cok) {
          for (int tb = 0; tb < cnt_pad; tb += UNR) {
            uint32_t raw[UNR][8];
            if (PACKED) {
#pragma unroll
              for (int u = 0; u < UNR; u++)
                tc::ldg_raw8(reinterpret_cast<const __nv_bfloat16*>(P.L0) + ((size_t)s_dst[tb + u] * C + c) * 16, raw[u]);
            }
#pragma unroll
            for (int u = 0; u < UNR; u++) {
              const int t = tb + u;
              const size_t j = (size_t)s_dst[t] * C + c;
              float l1[3], l2[9], pa;
              float l0;
              if (PACKED) {
                l0 = tc::bf16_at(raw[u], 0);
#pragma unroll
                for (int k = 0; k < 3; k++) l1[k] = tc::bf16_at(raw[u], 1 + k);
#pragma unroll
                for (int k = 0; k < 9; k++) l2[k] = tc::bf16_at(raw[u], 4 + k);
              } else {
                l0 = bm_ld(F0, j);
#pragma unroll
                for (int k = 0; k < 3; k++) l1[k] = bm_ld(F1, j * 3 + k);
#pragma unroll
                for (int k = 0; k < 9; k++) l2[k] = bm_ld(F2, j * 9 + k);
              }
              // phi_a = pa, phi_v = pa * rhat, phi_d = pa * rhat rhat^T: every product is a short
              // expression in l, rhat and pa (e.g. 222: l_xy phi_zy = pa (l_x . rhat) rhat_z), about 90 operations for
              // the 60 sums instead of 150 for general right operands
              const float4* gp = reinterpret_cast<const float4*>(&s_geom[t]);
              const float4 e0 = gp[0], e1 = gp[1], rr = gp[2];
              pa = wb;
              pa = fmaf(e0.x, w8[0], pa); pa = fmaf(e0.y, w8[1], pa); pa = fmaf(e0.z, w8[2], pa); pa = fmaf(e0.w, w8[3], pa);
              pa = fmaf(e1.x, w8[4], pa); pa = fmaf(e1.y, w8[5], pa); pa = fmaf(e1.z, w8[6], pa); pa = fmaf(e1.w, w8[7], pa);
              pa *= rr.w;   // 1 for an edge, 0 for the padding of the last batch: every product below carries pa as a factor
              const float rh[3] = {rr.x, rr.y, rr.z};
              // with rp = pa * rhat no separately scaled copy of l is needed: most products are single FMAs of an
              // element of l with rhat, rp or pa straight into the running sums
              const float rp[3] = {pa * rh[0], pa * rh[1], pa * rh[2]};
              const float d1 = l1[0] * rh[0] + l1[1] * rh[1] + l1[2] * rh[2];
              float m2[3], t0[3];
#pragma unroll
              for (int x = 0; x < 3; x++) {
                m2[x] = l2[x * 3] * rp[0] + l2[x * 3 + 1] * rp[1] + l2[x * 3 + 2] * rp[2];   // pa * (l2 rhat)_x
                t0[x] = l0 * rp[x];
                av[x] += t0[x];                                   // 011: l phi_x
                av[3 + x] = fmaf(l1[x], pa, av[3 + x]);           // 101
                av[6 + x] = fmaf(d1, rp[x], av[6 + x]);           // 121: l_x phi_yx -> y
                av[9 + x] += m2[x];                               // 211: l_xy phi_y -> x
              }
#pragma unroll
              for (int x = 0; x < 3; x++) {
#pragma unroll
                for (int y = 0; y < 3; y++) {
                  if (y >= x) ad[x * 3 + y] = fmaf(t0[x], rh[y], ad[x * 3 + y]);      // 022, upper triangle
                  ad[9 + x * 3 + y] = fmaf(l2[x * 3 + y], pa, ad[9 + x * 3 + y]);     // 202
                  ad[18 + x * 3 + y] = fmaf(l1[x], rp[y], ad[18 + x * 3 + y]);        // 112
                  ad[27 + x * 3 + y] = fmaf(m2[x], rh[y], ad[27 + x * 3 + y]);        // 222: l_xy phi_zy -> xz
                }
                // 212: row x of l cross phi
                ad[36 + x * 3 + 0] = fmaf(l2[x * 3 + 1], rp[2], ad[36 + x * 3 + 0]); ad[36 + x * 3 + 0] = fmaf(-l2[x * 3 + 2], rp[1], ad[36 + x * 3 + 0]);
                ad[36 + x * 3 + 1] = fmaf(l2[x * 3 + 2], rp[0], ad[36 + x * 3 + 1]); ad[36 + x * 3 + 1] = fmaf(-l2[x * 3 + 0], rp[2], ad[36 + x * 3 + 1]);
                ad[36 + x * 3 + 2] = fmaf(l2[x * 3 + 0], rp[1], ad[36 + x * 3 + 2]); ad[36 + x * 3 + 2] = fmaf(-l2[x * 3 + 1], rp[0], ad[36 + x * 3 + 2]);
              }
            }
          }
        }
      }
      ad[3] = ad[1]; ad[6] = ad[2]; ad[7] = ad[5];                                       // 022, lower triangle
      av[12] = ad[18 + 1 * 3 + 2] - ad[18 + 2 * 3 + 1];                                  // 111 from 112
      av[13] = ad[18 + 2 * 3 + 0] - ad[18 + 0 * 3 + 2];
      av[14] = ad[18 + 0 * 3 + 1] - ad[18 + 1 * 3 + 0];
      if (cok) {
        if (out_bf16) {
          // the sums feed a tensor-core channel mixing that rounds its operands to BF16 anyway: store them rounded
          // component-major [node][3 | 9][5*chan]: consecutive channels are consecutive addresses, and a (node,
          // component) row is the contiguous K dimension of that channel mixing
          __nv_bfloat16* sv = reinterpret_cast<__nv_bfloat16*>(S_v) + (size_t)v * 3 * 5 * C + c;
          __nv_bfloat16* sd = reinterpret_cast<__nv_bfloat16*>(S_d) + (size_t)v * 9 * 5 * C + c;
#pragma unroll
          for (int k = 0; k < 5; k++) {
#pragma unroll
            for (int x = 0; x < 3; x++) sv[(size_t)x * 5 * C + k * C] = __float2bfloat16_rn(av[k * 3 + x] * scale);
#pragma unroll
            for (int x = 0; x < 9; x++) sd[(size_t)x * 5 * C + k * C] = __float2bfloat16_rn(ad[k * 9 + x] * scale);
          }
        } else {
          float* sv = S_v + (size_t)v * 5 * C * 3;
          float* sd = S_d + (size_t)v * 5 * C * 9;
#pragma unroll
          for (int k = 0; k < 5; k++) {
#pragma unroll
            for (int x = 0; x < 3; x++) sv[((size_t)k * C + c) * 3 + x] = av[k * 3 + x] * scale;
#pragma unroll
            for (int x = 0; x < 9; x++) sd[((size_t)k * C + c) * 9 + x] = ad[k * 9 + x] * scale;
          }
        }
      }
    }
  }
  }
}


// ---- scalar output: per-edge Y maps and mlp_a, then per-node sum -------------------------------------
struct BeeScalarParams {
  BeeEdgeParams g;
  int dim_a;
  const float* Yt;                       // [3*chan][dim_a]: (Y_000 | Y_110 | Y_220) transposed
  const float* W1t; const float* b1;     // mlp_a layers, transposed [in][out]
  const float* W2t; const float* b2;
  const float* W3t; const float* b3;
  const float* Wdt;                      // lin_direct, transposed [dim_a][dim_a]
  float scale;
  float* out_a;                          // [Nt, dim_a]
};

constexpr int BM_LDH = 36;  // row stride of the product tile: 16-byte aligned rows, 4-way instead of 32-way store conflicts

template <int NCOL>
__global__ void __launch_bounds__(MT_THREADS, 1)
bee_scalar_kernel(BeeScalarParams P) {
  extern __shared__ __align__(16) float smem[];
  __shared__ EdgeGeom s_geom[BM_TILE];
  __shared__ int s_dst[BM_TILE];
  __shared__ int s_src[BM_TILE];
  __shared__ float s_jac[72];
  const int C = P.g.chan, A = P.dim_a, tid = threadIdx.x;
  float* hin = smem;                                   // [3C][36]
  float* psi = hin + (size_t)3 * C * BM_LDH;           // [A][32]
  float* bufA = psi + (size_t)A * MT_ROWS;             // [2A][32], later row-major [32][A+1]
  float* bufB = bufA + (size_t)2 * A * MT_ROWS;        // [2A][32]
  float* wstage = bufB + (size_t)2 * A * MT_ROWS;      // 2 x 16 x 2A
  const int ldo = A + 1;
  if (tid < 8) ld_poly8_to_chebyshev(P.g.jacobi + tid * 9, s_jac + tid * 9);   // Chebyshev form of the radial polynomials
  int n_begin, n_end;
  bm_block_range(P.g.row_ptr, 0, P.g.Nt, &n_begin, &n_end);
  if (n_begin >= n_end) return;
  const long long e_begin = P.g.row_ptr[n_begin], e_end = P.g.row_ptr[n_end];
  __syncthreads();

  // per-node sum: thread o < A owns output channel o
  float acc = 0.f;
  int cur = n_begin;
  auto flush_until = [&](int next) {
    if (tid < A)
      for (int v = cur; v < next; v++) P.out_a[(size_t)v * A + tid] = (v == cur ? acc : 0.f) * P.scale;
    acc = 0.f;
    cur = next;
  };

  for (long long e0 = e_begin; e0 < e_end; e0 += BM_TILE) {
    const int cnt = (int)((e_end - e0) < BM_TILE ? (e_end - e0) : BM_TILE);
    if (tid < BM_TILE) {
      int j = 0, sN = -1;
      if (tid < cnt) {
        const long long e = e0 + tid;
        edge_geometry(P.g.rij, e, P.g.r0, s_jac, &s_geom[tid]);
        j = P.g.dst[e];
        int lo = n_begin, hi = n_end;   // largest v with row_ptr[v] <= e
        while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if ((long long)P.g.row_ptr[mid] <= e) lo = mid; else hi = mid; }
        sN = lo;
      }
      s_dst[tid] = j;
      s_src[tid] = sN;
    }
    __syncthreads();
    // scalar products of every (channel, edge): all lanes of a warp read the same neighbour row
    for (int it = tid; it < 2 * C; it += MT_THREADS) {
      const int c = it % C, h = it / C;
      const float wb = P.g.enc_b[c];
      float w8[8];
#pragma unroll
      for (int m = 0; m < 8; m++) w8[m] = P.g.enc_w[c * 8 + m];
      for (int t = h; t < BM_TILE; t += 2) {
        float y0 = 0.f, y1 = 0.f, y2 = 0.f;
        if (t < cnt) {
          const size_t j = (size_t)s_dst[t] * C + c;
          float pa, pv[3], pd[9];
          edge_phi(s_geom[t], w8, wb, &pa, pv, pd);
          y0 = __ldg(P.g.L0 + j) * pa;
#pragma unroll
          for (int k = 0; k < 3; k++) y1 = fmaf(__ldg(P.g.L1 + j * 3 + k), pv[k], y1);
#pragma unroll
          for (int k = 0; k < 9; k++) y2 = fmaf(__ldg(P.g.L2 + j * 9 + k), pd[k], y2);
        }
        hin[(size_t)c * BM_LDH + t] = y0;
        hin[(size_t)(C + c) * BM_LDH + t] = y1;
        hin[(size_t)(2 * C + c) * BM_LDH + t] = y2;
      }
    }
    __syncthreads();
    mt_tile_linear<NCOL, false>(hin, 3 * C, P.Yt, nullptr, A, LD_ACT_NONE, psi, 0, wstage, BM_LDH);
    mt_tile_linear<NCOL, false>(psi, A, P.W1t, P.b1, 2 * A, LD_ACT_LEAKY01, bufA, 0, wstage);
    mt_tile_linear<NCOL, false>(bufA, 2 * A, P.W2t, P.b2, 2 * A, LD_ACT_LEAKY01, bufB, 0, wstage);
    mt_tile_linear<NCOL, true>(bufB, 2 * A, P.W3t, P.b3, A, LD_ACT_NONE, bufA, ldo, wstage);
    // psi + lin_direct(psi) + layers(psi)
    for (int idx = tid; idx < MT_ROWS * A; idx += MT_THREADS) {
      const int r = idx / A, c = idx - r * A;
      float a = psi[(size_t)c * MT_ROWS + r];
      for (int k = 0; k < A; k++) a = fmaf(psi[(size_t)k * MT_ROWS + r], __ldg(P.Wdt + (size_t)k * A + c), a);
      bufA[(size_t)r * ldo + c] += a;
    }
    __syncthreads();
    if (tid < A) {
      for (int t = 0; t < cnt; t++) {
        const int sN = s_src[t];
        if (sN != cur) flush_until(sN);
        acc += bufA[(size_t)t * ldo + tid];
      }
    } else {
      // keep `cur` in step for threads that own no output (uniform control flow is not required, but cheap)
      if (cnt > 0) cur = s_src[cnt - 1];
    }
    __syncthreads();
  }
  flush_until(n_end);
}

}  // namespace

// Per-node sums of the ten rank-1 / rank-2 Bee products of a Messages layer, times `scale`.
// S_v: [Nt, 5*chan, 3] (product order 011,101,121,211,111), S_d: [Nt, 5*chan, 3, 3] (022,202,112,222,212).
// L0/L1/L2 are the node-level left operands: FP32 (feat_bf16 = 0), BF16 (1), or with feat_bf16 = 2
// L0 alone points to the interleaved BF16 form [node][chan][16] = (l0, l1[3], l2[9], 3 unused); enc_w [chan,8] / enc_b [chan] the radial read-in,
// jacobi the 8x9 coefficient matrix of the radial basis. Graph in CSR form sorted by source.
// out_bf16: S_v / S_d are stored as BF16, component-major ([Nt][3][5*chan] and [Nt][9][5*chan]), the input form of
// ld_linear_bf16_tc_in16.
extern "C" int ld_bee_messages_vd_f32(const int* row_ptr, const int* dst, const float* rij, int Nt, int chan, float r0,
                                      const float* L0, const float* L1, const float* L2, const float* enc_w,
                                      const float* enc_b, const float* jacobi, float scale, void* S_v_, void* S_d_,
                                      int feat_bf16, int out_bf16, void* stream) {
  float* S_v = (float*)S_v_;
  float* S_d = (float*)S_d_;
  if (Nt < 0 || chan <= 0 || !(r0 > 0.f)) return LD_ERR_SHAPE;
  if (Nt == 0) return LD_OK;
  int* next_node = nullptr;
  {
    const int rc = ld_work_counter((cudaStream_t)stream, &next_node);
    if (rc != LD_OK) return rc;
  }
  BeeEdgeParams P{row_ptr, dst, rij, Nt, chan, r0, L0, L1, L2, enc_w, enc_b, jacobi, 0, next_node};
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (feat_bf16 == 2 && chan == 128 && out_bf16) bee_vd_kernel<__nv_bfloat16, true, 128><<<sms * 4, 128, 0, (cudaStream_t)stream>>>(P, S_v, S_d, scale, 1);
  else if (feat_bf16 == 2) bee_vd_kernel<__nv_bfloat16, true, 0><<<sms * 4, 128, 0, (cudaStream_t)stream>>>(P, S_v, S_d, scale, out_bf16);
  else if (feat_bf16) bee_vd_kernel<__nv_bfloat16, false, 0><<<sms * 4, 128, 0, (cudaStream_t)stream>>>(P, S_v, S_d, scale, out_bf16);
  else bee_vd_kernel<float, false, 0><<<sms * 4, 128, 0, (cudaStream_t)stream>>>(P, S_v, S_d, scale, out_bf16);
  LD_LAUNCH_CHECK();
  return LD_OK;
}

// Scalar output of a Messages layer: out_a[node] = scale * sum_e (psi_e + mlp_a(psi_e)),
// psi_e = [y_000 | y_110 | y_220] Y^T. Yt: [3*chan][dim_a]; mlp_a = lin_direct + (a -> 2a -> 2a -> a,
// LeakyReLU(0.1)), weights transposed [in][out]. dim_a a multiple of 8, at most 256.
extern "C" int ld_bee_messages_scalar_f32(const int* row_ptr, const int* dst, const float* rij, int Nt, int chan, int dim_a,
                                          float r0, const float* L0, const float* L1, const float* L2, const float* enc_w,
                                          const float* enc_b, const float* jacobi, const float* Yt, const float* W1t,
                                          const float* b1, const float* W2t, const float* b2, const float* W3t,
                                          const float* b3, const float* Wdt, float scale, float* out_a, void* stream) {
  if (Nt < 0 || chan <= 0 || dim_a <= 0 || !(r0 > 0.f)) return LD_ERR_SHAPE;
  if (dim_a % 8 != 0 || dim_a > 256) { ld_set_last_message("bee messages: dim_a must be a multiple of 8, at most 256"); return LD_ERR_UNSUPPORTED; }
  if ((((uintptr_t)Yt | (uintptr_t)W1t | (uintptr_t)W2t | (uintptr_t)W3t) % 16) != 0) return LD_ERR_SHAPE;
  if (Nt == 0) return LD_OK;
  BeeScalarParams P;
  P.g = BeeEdgeParams{row_ptr, dst, rij, Nt, chan, r0, L0, L1, L2, enc_w, enc_b, jacobi, 0};
  P.dim_a = dim_a; P.Yt = Yt; P.W1t = W1t; P.b1 = b1; P.W2t = W2t; P.b2 = b2; P.W3t = W3t; P.b3 = b3; P.Wdt = Wdt;
  P.scale = scale; P.out_a = out_a;
  const size_t floats = (size_t)3 * chan * BM_LDH + (size_t)dim_a * MT_ROWS + (size_t)4 * dim_a * MT_ROWS +
                        (size_t)2 * MT_KC * 2 * dim_a;
  const size_t smem = floats * 4 + 256;
  if (smem > 220 * 1024) { ld_set_last_message("bee messages: shared-memory plan exceeds the limit (chan or dim_a too large)"); return LD_ERR_UNSUPPORTED; }
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (2 * dim_a <= 256) {
    LD_CUDA_TRY(cudaFuncSetAttribute(bee_scalar_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    bee_scalar_kernel<1><<<sms, MT_THREADS, smem, (cudaStream_t)stream>>>(P);
  } else {
    LD_CUDA_TRY(cudaFuncSetAttribute(bee_scalar_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    bee_scalar_kernel<2><<<sms, MT_THREADS, smem, (cudaStream_t)stream>>>(P);
  }
  LD_LAUNCH_CHECK();
  return LD_OK;
}
