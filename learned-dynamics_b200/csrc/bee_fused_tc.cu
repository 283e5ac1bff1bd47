// One edge kernel per l<=2 ("Bee") message layer on the Blackwell tensor cores: Messages.forward of the reference
// (archs/diffuser_atoms15.py:227-253) for chan = 128 product channels and dim_a = 128, with every neighbour row
// gathered exactly once and both the 13 products and their per-node sums formed by the tensor cores.
//
//   pa[e,c]   = lin_enc(radial_encode_8(r_e))[c]                                  (managan/jacobi_radenc.py:27-33)
//   rhat_e    = tens_sigmoid(1, r_e * 7/r0)                                       (managan/tensor_products.py:167-182)
//   the right operands of the Bee products are pa, pa*rhat, pa*rhat rhat^T, so each of the 63 product components
//   of an (edge, channel) is  sum_m (pa[e,c] l[dst_e, c, m]) * G_e[m, o]  with l = (l0, l1[3], l2[9]) the thirteen
//   left values of the neighbour and G_e a 13 x 63 matrix of monomials of rhat_e (degree <= 2, signs of the
//   Levi-Civita symbol) that does not depend on the channel (managan/codegen_tensor_products.py:235-249).
//
// Per edge the sixteen working warps (a warp = 32 channels of every fourth edge) load the neighbour's row
// ([node][2][chan][8] BF16: two 16-byte halves per channel) three edges ahead, and for the current edge compute pa and
// the three scalar products y000, y110, y220 in registers (FP32; the scalar products go as BF16 into the operand tile
// of the per-edge MLP), scale the row by pa and store it into shared memory as a K-major operand L_e [128 channels x
// 16]. The same warps write G_e (102 non-zero BF16 entries at fixed positions, one per thread). One thread then issues one tcgen05
// MMA per edge,
//   S_node[c, 0:64] += L_e * G_e        the 60 rank-1 / rank-2 components ACCUMULATE in tensor memory over the edges
//                                       of a node: the per-node sum of edges_reduce_src costs no instruction at all,
// and the working warps read S_node once per NODE (double-buffered), writing it as BF16 [node][component][5*chan].
// After the 128 edges of a tile: psi = [y000|y110|y220] Y^T, two hidden layers, and the last layer with weights
// [W3 | W_direct + I] as in bee_messages_tc.cu - the last one transposed (weights as the M operand), so that its result
// lies in tensor memory as [channel][edge] and the per-node sum over edges is a sequential sum in one thread per
// channel. All additions happen in an order fixed by the node's edge list alone, so a system's result does not depend
// on the batch (or shard) it is processed in.
//
// Shared memory: MLP operand tile 97 KB | 96 KB ring, used as seven two-edge groups (two rows + two G matrices, 13 KB)
// while the products are formed and as three 32 KB weight slabs while the MLP runs | small operands.
// Tensor memory: [0,128) two node accumulators | [256,512) the MLP accumulators.
// Every wait is bounded; a wait that runs out sets LD_FLAG_TIMEOUT and all roles leave.
#include "common.cuh"
#include "tc05.cuh"
#include "tp_math.h"

namespace {

constexpr int BF_EDGES = 128;
constexpr int BF_C = 128, BF_A = 128;
constexpr int BF_WORK_WARPS = 16;
constexpr int BF_WORK_THREADS = BF_WORK_WARPS * 32;
// 18 warps, at most five per scheduler partition: 96 registers per thread fit (16384 registers per partition)
constexpr int BF_MMA_WARP = 16, BF_WEIGHT_WARP = 17;
constexpr int BF_THREADS = (BF_WORK_WARPS + 2) * 32;                           // 576
constexpr int BF_SYNC_THREADS = (BF_WORK_WARPS + 1) * 32;                      // working warps + MMA warp
constexpr int BF_PANEL = BF_EDGES * 16 + 16;     // byte stride between 8-column panels of the MLP operand tile (padded)
constexpr int BF_NG = 8;                         // ring groups (two edges each)
constexpr int BF_ROW_BYTES = 2 * BF_C * 16;      // 4096: one neighbour row = two K panels of 128 channels
constexpr int BF_GAMMA_ROWS = 64;                // G_e as the N operand: 64 rows (60 used)
constexpr int BF_GAMMA_BYTES = 2 * BF_GAMMA_ROWS * 16;                         // 2560: two K panels
constexpr int BF_GROUP_BYTES = 2 * BF_ROW_BYTES + 2 * BF_GAMMA_BYTES;          // 12288
constexpr int BF_WSTAGES = 3, BF_SLAB_BYTES = 32 * 1024;
constexpr int BF_RING_BYTES = BF_WSTAGES * BF_SLAB_BYTES;                      // 98304
static_assert(BF_NG * BF_GROUP_BYTES <= BF_RING_BYTES, "row groups and weight slabs share the ring");
constexpr int BF_LAYERS = 4;
constexpr int BF_OFF_A = 0;
constexpr int BF_A_BYTES = (3 * BF_C / 8) * BF_PANEL;                          // 99072
constexpr int BF_OFF_RING = BF_OFF_A + BF_A_BYTES;
constexpr int BF_OFF_BIAS = BF_OFF_RING + BF_RING_BYTES;
constexpr int BF_SMEM = BF_OFF_BIAS + 5 * BF_A * 4;
constexpr uint32_t BF_TMEM_COLS = 512, BF_TMEM_MLP = 256;
constexpr int BF_YL = 1;                         // node boundaries are served BF_YL groups of a warp (8 edges) behind its stores
constexpr int BF_GAMMA_ENTRIES = 128;            // 102 used

struct BfLayer {
  const __nv_bfloat16* w;   // packed panels [K/8][N][8]
  int a_panel, ksteps, slab_ksteps, N, act, out_col;
};

struct BfParams {
  const int* row_ptr; const int* dst; const float* rij;
  int Nt;
  float r0, scale;
  const __nv_bfloat16* rows;     // [Nt][2][128][8]
  const float* enc_w; const float* enc_b; const float* jacobi;
  BfLayer layer[BF_LAYERS];
  const float* b1; const float* b2; const float* b3;
  int seg_nodes;
  float* out_a; __nv_bfloat16* S_v; __nv_bfloat16* S_d;
  int* status;
  uint32_t wait_limit;
  int spin;                      // waits on the per-group barriers poll instead of suspending
  long long* prof;               // diagnostics build only
  unsigned short gamma_tab[BF_GAMMA_ENTRIES];   // bits 0-10 (byte offset inside G_e) / 2, 11-14 monomial, 15 sign; 0xffff unused
};

// Diagnostics build (-DLD_PHASE_COUNTERS): cycles per phase of one thread per role (block 0), added into prof[32]:
// working thread 0: 0 geometry, 2 wait free ring group, 3 products + scale + store, 4 barrier after products,
// 5 wait layers, 6 epilogues, 7 scalar sums, 8 end-of-tile barriers, 18 node drains;
// MMA lane: 9 wait rows + G, 10 wait node buffer, 11 wait weights;
// builder 0: 12 wait free group, 13 build; builder 1 lane 0: 15 weight streaming.
struct BfProf {
#ifdef LD_PHASE_COUNTERS
  long long t; long long* prof; bool on;
  __device__ __forceinline__ void start(long long* p, bool enable) { prof = p; on = enable && p != nullptr; t = clock64(); }
  __device__ __forceinline__ void lap(int slot) {   // slot >= 32: restart the clock without recording
    if (on) { const long long n = clock64(); if (slot < 32) atomicAdd((unsigned long long*)&prof[slot], (unsigned long long)(n - t)); t = n; }
  }
#else
  __device__ __forceinline__ void start(long long*, bool) {}
  __device__ __forceinline__ void lap(int) {}
#endif
};

struct BfRange { int n_begin, n_end; long long e_begin, e_end, ntiles; };


__device__ __forceinline__ int bf_work_lb(const int* __restrict__ row_ptr, int lo, int hi, long long target) {
  const long long base = (long long)row_ptr[lo] + lo;
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if ((long long)row_ptr[mid] + mid - base < target) lo = mid + 1; else hi = mid;
  }
  return lo;
}
__device__ __forceinline__ int bf_lb_row(const int* __restrict__ row_ptr, int lo, int hi, long long target) {
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if ((long long)row_ptr[mid] < target) lo = mid + 1; else hi = mid;
  }
  return lo;
}
// this block's node-aligned slice of the segment [seg_lo, seg_hi), balanced over edges + nodes
__device__ __forceinline__ BfRange bf_block_range(const int* __restrict__ row_ptr, int seg_lo, int seg_hi) {
  BfRange r;
  const long long work = ((long long)row_ptr[seg_hi] - row_ptr[seg_lo]) + (seg_hi - seg_lo);
  long long per = (work + gridDim.x - 1) / gridDim.x;
  if (per < BF_EDGES) per = BF_EDGES;
  r.n_begin = blockIdx.x == 0 ? seg_lo : bf_work_lb(row_ptr, seg_lo, seg_hi, per * blockIdx.x);
  r.n_end = blockIdx.x == gridDim.x - 1 ? seg_hi : bf_work_lb(row_ptr, seg_lo, seg_hi, per * (blockIdx.x + 1));
  r.e_begin = r.n_begin < r.n_end ? row_ptr[r.n_begin] : 0;
  r.e_end = r.n_begin < r.n_end ? row_ptr[r.n_end] : 0;
  r.ntiles = (r.e_end - r.e_begin + BF_EDGES - 1) / BF_EDGES;
  return r;
}

__device__ __forceinline__ int bf_sync_or(int flag) {
  int out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "barrier.cta.red.or.pred p, 1, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(out)
      : "r"(flag), "n"(BF_SYNC_THREADS)
      : "memory");
  return out;
}

__device__ __forceinline__ unsigned short bf_bf16(float v) {
  __nv_bfloat16 h = __float2bfloat16_rn(v);
  return *reinterpret_cast<unsigned short*>(&h);
}

// column o of a node accumulator (0..63) -> where it goes. o in [0,15): rank-1 product o/3, component o%3;
// o in [15,60): rank-2 product (o-15)/9, component (o-15)%9; 60..63 unused. Writes the sixteen columns of group G.
template <int G>
__device__ __forceinline__ void bf_store_node(__nv_bfloat16* __restrict__ S_v, __nv_bfloat16* __restrict__ S_d, int node, int c,
                                              const float* acc, float scale) {
#pragma unroll
  for (int k = 0; k < 16; k++) {
    constexpr int base = 16 * G;
    const int o = base + k;
    if (o >= 60) continue;
    const __nv_bfloat16 v = __float2bfloat16_rn(acc[k] * scale);
    if (o < 15) {
      S_v[((size_t)node * 3 + (o % 3)) * (5 * BF_C) + (o / 3) * BF_C + c] = v;
    } else {
      const int di = o - 15;
      S_d[((size_t)node * 9 + (di % 9)) * (5 * BF_C) + (di / 9) * BF_C + c] = v;
    }
  }
}

// End of a node's edge list for one thread (channel c, column group g): write its sixteen sums for `node` (skipped when
// node < 0), then zeros for the nodes without edges from `zero_from` up to `next` (exclusive). One copy of this code,
// called from the few places where a node can end; the sums travel by value so that they stay in registers.
__device__ __noinline__ void bf_flush_node(int g, __nv_bfloat16* S_v, __nv_bfloat16* S_d, int node, int zero_from, int next, int c,
                                           float scale, float a0, float a1, float a2, float a3, float a4, float a5, float a6,
                                           float a7, float a8, float a9, float a10, float a11, float a12, float a13, float a14,
                                           float a15) {
  float acc[16] = {a0, a1, a2, a3, a4, a5, a6, a7, a8, a9, a10, a11, a12, a13, a14, a15};
  for (int v = (node >= 0 ? node : zero_from); v < next; v++) {
    if (v != node) {
#pragma unroll
      for (int i = 0; i < 16; i++) acc[i] = 0.f;
    }
    if (g == 0) bf_store_node<0>(S_v, S_d, v, c, acc, scale);
    else if (g == 1) bf_store_node<1>(S_v, S_d, v, c, acc, scale);
    else if (g == 2) bf_store_node<2>(S_v, S_d, v, c, acc, scale);
    else bf_store_node<3>(S_v, S_d, v, c, acc, scale);
    if (v == node) v = zero_from - 1;   // continue with the nodes that have no edges
  }
}

__global__ void __maxnreg__(96)
bee_fused_tc_kernel(const __grid_constant__ BfParams P) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t bar_full[BF_NG], bar_slot_empty[BF_NG];
  __shared__ __align__(8) uint64_t bar_dfull[2], bar_dempty[2];
  __shared__ __align__(8) uint64_t bar_weights_go;
  __shared__ __align__(8) uint64_t bar_wfull[BF_WSTAGES], bar_wempty[BF_WSTAGES], bar_accum;
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int s_fail;
  // per edge: eight radial functions | 1, rx, ry, rz | rx rx, rx ry, rx rz, ry ry | ry rz, rz rz, 0, 0
  __shared__ __align__(16) float s_geo[BF_EDGES][20];
  __shared__ __align__(16) int s_src[BF_EDGES];
  __shared__ int s_dst[BF_EDGES];
  __shared__ int s_bnd[BF_EDGES];      // edges of the tile at which a new source node starts, ascending
  __shared__ int s_nbnd, s_prev_src;   // their number; source node of the last edge of the previous tile (-1: none)
  __shared__ unsigned s_bmask[BF_EDGES / 32];   // the same as one bit per edge (for the MMA thread)
  __shared__ int s_rowwin[BF_EDGES + 1];
  __shared__ float s_jac[72];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  unsigned char* a_smem = smem + BF_OFF_A;
  unsigned char* ring = smem + BF_OFF_RING;
  float* s_bias = reinterpret_cast<float*>(smem + BF_OFF_BIAS);   // [b1 (2A) | b2 (2A) | b3 (A)]
  const uint32_t wl = P.wait_limit;
  // the per-group barriers (64 groups per tile) complete within a few hundred cycles
  auto hot_wait = [&](uint64_t* bar, uint32_t parity) -> bool {
    return (P.spin & 1) ? tc::mbar_wait_spin(bar, parity, wl << 4) : tc::mbar_wait(bar, parity, wl);
  };
  BfProf pf;

  if (tid < 8) ld_poly8_to_chebyshev(P.jacobi + tid * 9, s_jac + tid * 9);   // Chebyshev form of the radial polynomials
  for (int i = tid; i < 2 * BF_A; i += BF_THREADS) { s_bias[i] = P.b1[i]; s_bias[2 * BF_A + i] = P.b2[i]; }
  for (int i = tid; i < BF_A; i += BF_THREADS) s_bias[4 * BF_A + i] = P.b3[i];
  if (tid == 0) {
    for (int s = 0; s < BF_NG; s++) { tc::mbar_init(&bar_full[s], 4); tc::mbar_init(&bar_slot_empty[s], 1); }   // 4 warps per group
    for (int s = 0; s < 2; s++) { tc::mbar_init(&bar_dfull[s], 1); tc::mbar_init(&bar_dempty[s], BF_WORK_WARPS); }
    tc::mbar_init(&bar_weights_go, 1);
    for (int s = 0; s < BF_WSTAGES; s++) { tc::mbar_init(&bar_wfull[s], 1); tc::mbar_init(&bar_wempty[s], 1); }
    tc::mbar_init(&bar_accum, 1);
    tc::mbar_init_fence();
    // every ring group starts out free: complete the first phase of its "empty" barrier, so that the n-th use of a group
    // always waits for phase n (no special case for the first use)
    for (int s = 0; s < BF_NG; s++) tc::mbar_arrive(&bar_slot_empty[s]);
    s_fail = 0;
  }
  if (warp == 0) { tc::tmem_alloc(&tmem_slot, BF_TMEM_COLS); tc::tmem_relinquish(); }
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  const int seg_nodes = P.seg_nodes > 0 ? P.seg_nodes : P.Nt;
  int fail = 0;

  if (warp == BF_WEIGHT_WARP) {
    // ===== weight slabs of the four layers, once the products of the tile are done with the ring ===================
    if (lane == 0) {
      uint32_t wloads = 0, tiles = 0;
      pf.start(P.prof, blockIdx.x == 0);
      for (int seg_lo = 0; seg_lo < P.Nt && !fail; seg_lo += seg_nodes) {
        const long long ntiles = bf_block_range(P.row_ptr, seg_lo, min(seg_lo + seg_nodes, P.Nt)).ntiles;
        for (long long t = 0; t < ntiles && !fail; t++, tiles++) {
          pf.lap(100);
          // the ring is free for weights once every product MMA of the tile has read its rows
          if (!tc::mbar_wait(&bar_weights_go, tiles & 1, wl)) { fail = 1; break; }
          for (int l = 0; l < BF_LAYERS && !fail; l++) {
            const BfLayer& L = P.layer[l];
            for (int ks = 0; ks < L.ksteps; ks += L.slab_ksteps, wloads++) {
              const uint32_t st = wloads % BF_WSTAGES, use = wloads / BF_WSTAGES;
              const uint32_t bytes = (uint32_t)min(L.slab_ksteps, L.ksteps - ks) * L.N * 32;
              // a slab slot is free when the MMAs that read its previous content are done
              if (use >= 1 && !tc::mbar_wait(&bar_wempty[st], (use - 1) & 1, wl)) { fail = 1; break; }
              if (s_fail) { fail = 1; break; }
              tc::mbar_expect_tx(&bar_wfull[st], bytes);
              tc::bulk_g2s(ring + (size_t)st * BF_SLAB_BYTES, L.w + (size_t)ks * L.N * 16, bytes, &bar_wfull[st]);
            }
          }
          pf.lap(15);
        }
      }
      if (fail) {   // let slabs in flight land (bounded)
        s_fail = 1;
        for (uint32_t i = wloads > BF_WSTAGES ? wloads - BF_WSTAGES : 0; i < wloads; i++)
          tc::mbar_wait(&bar_wfull[i % BF_WSTAGES], (i / BF_WSTAGES) & 1, wl);
      }
    }
  } else if (warp == BF_MMA_WARP) {
    // ===== MMA issue ===========================================================================================
    const bool mma_lane = lane == 0;
    uint32_t wmmas = 0, tiles = 0;
    uint32_t full_ph = 0;       // bit gs: parity of the next phase to wait for on bar_full[gs]
    uint32_t nc = 0;            // nodes (with edges) completed so far: the running node uses accumulator nc & 1
    const uint32_t a_base = tc::smem_u32(a_smem), ring_base = tc::smem_u32(ring);
    const uint64_t row_desc0 = tc::smem_desc(ring_base, BF_C * 16, 128);
    const uint64_t gam_desc0 = tc::smem_desc(ring_base + 2 * BF_ROW_BYTES, BF_GAMMA_ROWS * 16, 128);
    // the byte offset of a ring group (in 16-byte units) only ever changes the low word of a descriptor
    const uint32_t row_lo = (uint32_t)row_desc0, row_hi = (uint32_t)(row_desc0 >> 32);
    const uint32_t gam_lo = (uint32_t)gam_desc0, gam_hi = (uint32_t)(gam_desc0 >> 32);
    const uint32_t idesc_s = tc::idesc_bf16(BF_C, 64);
    pf.start(P.prof, lane == 0 && blockIdx.x == 0);
    for (int seg_lo = 0; seg_lo < P.Nt && !fail; seg_lo += seg_nodes) {
      const BfRange br = bf_block_range(P.row_ptr, seg_lo, min(seg_lo + seg_nodes, P.Nt));
      bool have = false;        // a node is accumulating (none yet in this slice)
      for (long long e0 = br.e_begin; e0 < br.e_end; e0 += BF_EDGES, tiles++) {
        const int cnt = (int)((br.e_end - e0) < BF_EDGES ? (br.e_end - e0) : BF_EDGES);
        const int groups = (cnt + 1) >> 1;
        const bool last_tile = e0 + BF_EDGES >= br.e_end;
        if (bf_sync_or(fail)) { fail = 1; break; }      // [B1] geometry staged (radial functions, monomials, src, dst, boundaries)
        if (mma_lane && !fail) {
          tc::fence_after_sync();
          unsigned bm = 0;
#pragma unroll 1
          for (int grp = 0; grp < groups; grp++) {
            const int gs = grp & (BF_NG - 1);
            if ((grp & 15) == 0) bm = s_bmask[grp >> 4];   // node-boundary flags of the next 32 edges
            pf.lap(100);
            if (!hot_wait(&bar_full[gs], (full_ph >> gs) & 1)) { fail = 1; break; }
            full_ph ^= 1u << gs;
            pf.lap(9);
            tc::fence_after_sync();
            const uint32_t goff = (uint32_t)gs * (BF_GROUP_BYTES >> 4);
#pragma unroll
            for (int u = 0; u < 2; u++) {
              const int e = 2 * grp + u;
              if (e >= cnt) break;
              uint32_t accumulate = 1u;
              if ((bm >> (e & 31)) & 1u) {
                // a new node starts at this edge: hand the accumulator of the finished one to the working warps and
                // take the other one, which must have been read out (it held the node before the previous one)
                if (have) { tc::mma_commit(&bar_dfull[nc & 1]); nc++; }
                have = true;
                if (nc >= 2 && !hot_wait(&bar_dempty[nc & 1], ((nc >> 1) - 1) & 1)) { fail = 1; break; }
                pf.lap(10);
                tc::fence_after_sync();
                accumulate = 0u;
              }
              const uint64_t rd = ((uint64_t)row_hi << 32) | (row_lo + goff + u * (BF_ROW_BYTES >> 4));
              const uint64_t gd = ((uint64_t)gam_hi << 32) | (gam_lo + goff + u * (BF_GAMMA_BYTES >> 4));
              tc::mma_bf16(tmem_base + (nc & 1) * 64, rd, gd, idesc_s, accumulate);
            }
            if (fail) break;
            tc::mma_commit(&bar_slot_empty[gs]);
          }
          if (!fail) {
            if (last_tile && have) { tc::mma_commit(&bar_dfull[nc & 1]); nc++; have = false; }   // last node of the slice
            tc::mma_commit(&bar_weights_go);   // every product MMA of the tile has read its rows: the ring may take weights
          }
        }
        nc = __shfl_sync(0xffffffffu, nc, 0);
        fail = __shfl_sync(0xffffffffu, fail, 0);
        if (bf_sync_or(fail)) { fail = 1; break; }      // [B2] scalar products of the tile are in the operand tile
        for (int l = 0; l < BF_LAYERS; l++) {
          if (mma_lane && !fail) {
            tc::fence_after_sync();
            const int l_ksteps = P.layer[l].ksteps, l_slab = P.layer[l].slab_ksteps, l_N = P.layer[l].N;
            const bool transposed = l == BF_LAYERS - 1;   // last layer: weights are the M operand, the tile the N operand
            const uint32_t idesc = transposed ? tc::idesc_bf16(l_N, BF_EDGES) : tc::idesc_bf16(BF_EDGES, l_N);
            uint64_t ad = tc::smem_desc(a_base + P.layer[l].a_panel * BF_PANEL, BF_PANEL, 128);
            const uint64_t a_step = (uint64_t)((2 * BF_PANEL) >> 4), b_step = (uint64_t)((2 * l_N * 16) >> 4);
            uint32_t accumulate = 0u;
            for (int ks0 = 0; ks0 < l_ksteps; ks0 += l_slab, wmmas++) {
              const uint32_t st = wmmas % BF_WSTAGES, use = wmmas / BF_WSTAGES;
              pf.lap(100);
              if (!tc::mbar_wait(&bar_wfull[st], use & 1, wl)) { fail = 1; break; }
              pf.lap(11);
              tc::fence_after_sync();
              uint64_t bd = tc::smem_desc(ring_base + st * BF_SLAB_BYTES, l_N * 16, 128);
              const int nk = min(l_slab, l_ksteps - ks0);
#pragma unroll 4
              for (int kk = 0; kk < nk; kk++) {
                if (transposed) tc::mma_bf16(tmem_base + BF_TMEM_MLP, bd, ad, idesc, accumulate);
                else tc::mma_bf16(tmem_base + BF_TMEM_MLP, ad, bd, idesc, accumulate);
                accumulate = 1u;
                ad += a_step;
                bd += b_step;
              }
              tc::mma_commit(&bar_wempty[st]);
            }
            if (!fail) {
              tc::mma_commit(&bar_accum);
            }
          }
          fail = __shfl_sync(0xffffffffu, fail, 0);
          if (bf_sync_or(fail)) { fail = 1; break; }    // [B3..B6]
        }
        if (fail) break;
        if (bf_sync_or(fail)) { fail = 1; break; }      // [B7] tile finished
      }
    }
    if (fail) s_fail = 1;
  } else {
    // ===== working warps =========================================================================================
    const int q = warp & 3, j = warp >> 2;              // tensor-memory lane quarter (fixed by the warp id); edges j mod 4
    const int g = j;                                    // column group of the node accumulators this warp reads out
    const int ch = q * 32 + lane;                       // product channel = tensor-memory lane in the product phase
    const int row = q * 32 + lane;                      // edge row = tensor-memory lane in the MLP phase
    const uint32_t tmem_row = tmem_base + ((uint32_t)(q * 32) << 16);
    uint32_t accum_phase = 0, tiles = 0, nc = 0;
    float w8[8];
#pragma unroll
    for (int m = 0; m < 8; m++) w8[m] = P.enc_w[ch * 8 + m];   // lin_enc of this thread's product channel
    const float wb = P.enc_b[ch];
    // this thread's entry of G_e (the four warps of a ring group write all 102 between them)
    const unsigned gtab = P.gamma_tab[q * 32 + lane];
    const int g_mono = 8 + ((gtab >> 11) & 15), g_off = 2 * (gtab & 0x7ffu);
    const bool g_neg = (gtab & 0x8000u) != 0, g_has = gtab != 0xffffu;
    uint32_t empty_ph = 0;      // bit gs: parity of the next phase to wait for on bar_slot_empty[gs]
    pf.start(P.prof, tid == 0 && blockIdx.x == 0);
    for (int seg_lo = 0; seg_lo < P.Nt && !fail; seg_lo += seg_nodes) {
      const BfRange br = bf_block_range(P.row_ptr, seg_lo, min(seg_lo + seg_nodes, P.Nt));
      const int n_begin = br.n_begin, n_end = br.n_end;
      float acc_a = 0.f;
      int cur = -1;               // node whose product sums are accumulating in tensor memory (all working threads agree)
      int zero_from = n_begin;    // first node whose sums have not been written yet
      int cur_a = n_begin;        // node whose scalar sum is running (threads of the warps j == 0)
      int node_lo = n_begin;
      asm volatile("barrier.cta.sync 2, %0;" ::"n"(BF_WORK_THREADS) : "memory");
      if (tid <= BF_EDGES) s_rowwin[tid] = P.row_ptr[min(node_lo + tid, n_end > n_begin ? n_end : n_begin)];
      if (tid == 0) s_prev_src = -1;
      float pre_x = 0.f, pre_y = 0.f, pre_z = 0.f;
      int pre_j = 0;
      if (tid < BF_EDGES && br.e_begin + tid < br.e_end) {
        const long long en = br.e_begin + tid;
        pre_x = P.rij[en * 3]; pre_y = P.rij[en * 3 + 1]; pre_z = P.rij[en * 3 + 2]; pre_j = P.dst[en];
      }
      asm volatile("barrier.cta.sync 2, %0;" ::"n"(BF_WORK_THREADS) : "memory");

      // one node boundary: the node `cur` is complete in its accumulator (the MMA thread has committed it) - read this
      // thread's sixteen columns, release the buffer, write them; then zeros for the nodes without edges before `next`
      auto end_node = [&](int next) {
        float a[16];
#pragma unroll
        for (int i = 0; i < 16; i++) a[i] = 0.f;
        if (cur >= 0) {
          if (!hot_wait(&bar_dfull[nc & 1], (nc >> 1) & 1)) { fail = 1; return; }
          tc::fence_after_sync();
          tc::tmem_ld16(tmem_row + (nc & 1) * 64 + g * 16, a);
          tc::fence_before_sync();
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(&bar_dempty[nc & 1]);
          nc++;
        }
        bf_flush_node(g, P.S_v, P.S_d, cur, zero_from, next, ch, P.scale, a[0], a[1], a[2], a[3], a[4], a[5], a[6], a[7], a[8], a[9],
                      a[10], a[11], a[12], a[13], a[14], a[15]);
      };

      for (long long e0 = br.e_begin; e0 < br.e_end; e0 += BF_EDGES, tiles++) {
        const int cnt = (int)((br.e_end - e0) < BF_EDGES ? (br.e_end - e0) : BF_EDGES);
        const int groups = (cnt + 1) >> 1;
        // ---- 1. edge geometry: radial functions -> operand of the pa product, monomials of rhat, source node ---------
        if (tid < BF_EDGES) {
          const float gx = pre_x, gy = pre_y, gz = pre_z;
          const int gj = pre_j;
          {
            const long long en = e0 + BF_EDGES + tid;   // next tile's edge of this thread
            if (en < br.e_end) { pre_x = P.rij[en * 3]; pre_y = P.rij[en * 3 + 1]; pre_z = P.rij[en * 3 + 2]; pre_j = P.dst[en]; }
          }
          int s = -1;
          float enc[8];
#pragma unroll
          for (int m = 0; m < 8; m++) enc[m] = 0.f;
          float rx = 0.f, ry = 0.f, rz = 0.f;
          if (tid < cnt) {
            const long long e = e0 + tid;
            const float d = sqrtf(gx * gx + gy * gy + gz * gz);
            const float zz = d / P.r0;
            ld_radial_cheb8(zz, fmaxf(1.f - zz, 0.f), s_jac, enc);
            const float sc = 7.f / P.r0;
            const float ux = gx * sc, uy = gy * sc, uz = gz * sc;
            const float inv = rsqrtf(1.f + ux * ux + uy * uy + uz * uz);
            rx = ux * inv; ry = uy * inv; rz = uz * inv;
            if ((long long)s_rowwin[BF_EDGES] > e) {
              int lo = 0, hi = BF_EDGES;
              while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if ((long long)s_rowwin[mid] > e) hi = mid; else lo = mid; }
              s = node_lo + lo;
            } else {
              s = bf_lb_row(P.row_ptr, node_lo + BF_EDGES, n_end, e + 1) - 1;
            }
          }
          s_src[tid] = s;
          s_dst[tid] = tid < cnt ? gj : 0;
          float4* gp = reinterpret_cast<float4*>(&s_geo[tid][0]);
          gp[0] = make_float4(enc[0], enc[1], enc[2], enc[3]);
          gp[1] = make_float4(enc[4], enc[5], enc[6], enc[7]);
          gp[2] = make_float4(1.f, rx, ry, rz);
          gp[3] = make_float4(rx * rx, rx * ry, rx * rz, ry * ry);
          gp[4] = make_float4(ry * rz, rz * rz, 0.f, 0.f);
        }
        // the weight slabs of the previous tile overwrote the G areas of the ring: clear them (32 KB); the entries written
        // later sit at fixed positions among zeros
#pragma unroll
        for (int i = 0; i < (BF_NG * 2 * BF_GAMMA_BYTES / 16) / BF_WORK_THREADS; i++) {
          const int idx = tid + i * BF_WORK_THREADS;
          *reinterpret_cast<uint4*>(ring + (idx >> 8) * BF_GROUP_BYTES + 2 * BF_ROW_BYTES + (idx & 255) * 16) = make_uint4(0u, 0u, 0u, 0u);
        }
        asm volatile("barrier.cta.sync 2, %0;" ::"n"(BF_WORK_THREADS) : "memory");
        if (warp == 0) {
          // boundary list: edges whose source differs from the edge before (the first edge compares with the last edge
          // of the previous tile of this slice), compacted in order by ballots
          int n = 0;
          for (int base = 0; base < cnt; base += 32) {
            const int e = base + lane;
            bool isb = false;
            if (e < cnt) isb = s_src[e] != (e == 0 ? s_prev_src : s_src[e - 1]);
            const unsigned m = __ballot_sync(0xffffffffu, isb);
            if (lane == 0) s_bmask[base >> 5] = m;
            if (isb) s_bnd[n + __popc(m & ((1u << lane) - 1))] = e;
            n += __popc(m);
          }
          __syncwarp();
          if (lane == 0) { s_nbnd = n; s_prev_src = s_src[cnt - 1]; }
        }
        tc::fence_before_sync();
        if (bf_sync_or(fail)) { fail = 1; break; }                                        // [B1]
        pf.lap(0);
        // ---- 2. products ------------------------------------------------------------------------------------------
        // This warp: channels 32q..32q+31 of the ring groups (edge pairs) j, j+4, j+8, ...  Per group: the rows of its
        // next group are requested; for the two edges of this group pa and the three scalar products are formed (FP32),
        // the scalar products go into the MLP's operand tile, the rows scaled by pa go into the ring as MMA operands.
        // Node boundaries (listed by the geometry pass) are served BF_YL groups of this warp behind: all sixteen warps
        // read out their columns of the finished node.
        {
          const __nv_bfloat16* rows_c = P.rows + (size_t)ch * 8;
          uint4 cur_r[4], nxt_r[4];   // two edges x (low, high half) of the group in work and of the next group
          auto request = [&](int grp, uint4* r) {
#pragma unroll
            for (int u = 0; u < 2; u++) {
              const int e = 2 * grp + u;
              r[2 * u] = make_uint4(0u, 0u, 0u, 0u); r[2 * u + 1] = r[2 * u];
              if (e < cnt) {
                const __nv_bfloat16* rp = rows_c + (size_t)s_dst[e] * (2 * BF_C * 8);
                r[2 * u] = __ldg(reinterpret_cast<const uint4*>(rp));
                r[2 * u + 1] = __ldg(reinterpret_cast<const uint4*>(rp + BF_C * 8));
              }
            }
          };
          request(j, cur_r);
          int bi = 0;                                   // next entry of the tile's boundary list
          const int nb = s_nbnd;
#pragma unroll 1
          for (int grp = j; grp < groups + 4 * BF_YL && !fail; grp += 4) {
            if (grp < groups) {
              request(grp + 4, nxt_r);
              const int gs = grp & (BF_NG - 1);
              uint32_t o[2][8];
#pragma unroll
              for (int u = 0; u < 2; u++) {
                const int e = 2 * grp + u;
                if (e < cnt) {
                  const float4* gp = reinterpret_cast<const float4*>(&s_geo[e][0]);
                  const float4 e0v = gp[0], e1v = gp[1], r1 = gp[2], r2 = gp[3], r3 = gp[4];
                  float pa = wb;
                  pa = fmaf(e0v.x, w8[0], pa); pa = fmaf(e0v.y, w8[1], pa); pa = fmaf(e0v.z, w8[2], pa); pa = fmaf(e0v.w, w8[3], pa);
                  pa = fmaf(e1v.x, w8[4], pa); pa = fmaf(e1v.y, w8[5], pa); pa = fmaf(e1v.z, w8[6], pa); pa = fmaf(e1v.w, w8[7], pa);
                  const uint32_t w[8] = {cur_r[2 * u].x, cur_r[2 * u].y, cur_r[2 * u].z, cur_r[2 * u].w,
                                         cur_r[2 * u + 1].x, cur_r[2 * u + 1].y, cur_r[2 * u + 1].z, cur_r[2 * u + 1].w};
                  float l[16];
#pragma unroll
                  for (int i = 0; i < 8; i++) { l[2 * i] = __uint_as_float(w[i] << 16); l[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
                  // y000 = l0 pa, y110 = (l1 . r) pa, y220 = (r^T l2 r) pa with the six distinct products of r
                  const float y1 = l[1] * r1.y + l[2] * r1.z + l[3] * r1.w;
                  const float y2 = l[4] * r2.x + (l[5] + l[7]) * r2.y + (l[6] + l[10]) * r2.z + l[8] * r2.w + (l[9] + l[11]) * r3.x +
                                   l[12] * r3.y;
                  unsigned short* arow = reinterpret_cast<unsigned short*>(a_smem + (size_t)e * 16) + (ch & 7);
                  arow[(ch >> 3) * (BF_PANEL / 2)] = bf_bf16(pa * l[0]);
                  arow[((BF_C + ch) >> 3) * (BF_PANEL / 2)] = bf_bf16(pa * y1);
                  arow[((2 * BF_C + ch) >> 3) * (BF_PANEL / 2)] = bf_bf16(pa * y2);
#pragma unroll
                  for (int i = 0; i < 8; i++) o[u][i] = tc::pack_bf16x2(pa * l[2 * i], pa * l[2 * i + 1]);
                }
              }
              pf.lap(3);
              if (!hot_wait(&bar_slot_empty[gs], (empty_ph >> gs) & 1)) { fail = 1; break; }
              empty_ph ^= 1u << gs;
              pf.lap(2);
#pragma unroll
              for (int u = 0; u < 2; u++) {
                if (2 * grp + u < cnt) {
                  unsigned char* dstp = ring + gs * BF_GROUP_BYTES + u * BF_ROW_BYTES + ch * 16;
                  *reinterpret_cast<uint4*>(dstp) = make_uint4(o[u][0], o[u][1], o[u][2], o[u][3]);
                  *reinterpret_cast<uint4*>(dstp + BF_C * 16) = make_uint4(o[u][4], o[u][5], o[u][6], o[u][7]);
                  if (g_has) {
                    const float gv = s_geo[2 * grp + u][g_mono];
                    *reinterpret_cast<unsigned short*>(ring + gs * BF_GROUP_BYTES + 2 * BF_ROW_BYTES + u * BF_GAMMA_BYTES + g_off) =
                        bf_bf16(g_neg ? -gv : gv);
                  }
                }
              }
              tc::fence_async_smem();
              __syncwarp();
              if (lane == 0) tc::mbar_arrive(&bar_full[gs]);
#pragma unroll
              for (int i = 0; i < 4; i++) cur_r[i] = nxt_r[i];
              pf.lap(3);
            }
            // node boundaries up to the last edge of the group stored BF_YL steps ago
            const int upto = 2 * (grp - 4 * BF_YL) + 1;
            while (bi < nb && s_bnd[bi] <= upto && !fail) {
              const int s = s_src[s_bnd[bi]];
              pf.lap(100); end_node(s); cur = s; zero_from = s + 1; bi++; pf.lap(18);
            }
          }
          // node boundaries among the last edges of the tile
          while (bi < nb && !fail) {
            const int s = s_src[s_bnd[bi]];
            pf.lap(100); end_node(s); cur = s; zero_from = s + 1; bi++; pf.lap(18);
          }
        }
        if (!fail && e0 + BF_EDGES >= br.e_end) {
          // end of this block's slice: its last node, then the nodes without edges up to the end of the slice
          end_node(n_end);
          cur = -1; zero_from = n_end;
        }
        tc::fence_async_smem();
        tc::fence_before_sync();
        if (bf_sync_or(fail)) { fail = 1; break; }                                        // [B2]
        pf.lap(4);
        // ---- 3. four layers ------------------------------------------------------------------------------------
        for (int l = 0; l < BF_LAYERS; l++) {
          {
            int done = 1;
            if (lane == 0) done = tc::mbar_wait(&bar_accum, accum_phase & 1, wl) ? 1 : 0;
            done = __shfl_sync(0xffffffffu, done, 0);
            if (!done) fail = 1;
          }
          accum_phase++;
          tc::fence_after_sync();
          pf.lap(5);
          const int N = P.layer[l].N;
          if (!fail && l < BF_LAYERS - 1) {
            // bias, activation -> BF16 into the operand tile at out_col (this thread: edge `row`, its quarter of the columns)
            const float* bias = l == 0 ? nullptr : s_bias + (l - 1) * 2 * BF_A;
            const int act = P.layer[l].act, oc = P.layer[l].out_col;
            const int cpp = max(N / 4, 32);
            for (int cb = g * cpp; cb < min((g + 1) * cpp, N); cb += 32) {
              float v[32];
              tc::tmem_ld32(tmem_row + BF_TMEM_MLP + cb, v);
#pragma unroll
              for (int g8 = 0; g8 < 4; g8++) {
                float t8[8];
                float b8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                if (bias != nullptr) {
                  const float4 ba = *reinterpret_cast<const float4*>(bias + cb + g8 * 8);
                  const float4 bb = *reinterpret_cast<const float4*>(bias + cb + g8 * 8 + 4);
                  b8[0] = ba.x; b8[1] = ba.y; b8[2] = ba.z; b8[3] = ba.w; b8[4] = bb.x; b8[5] = bb.y; b8[6] = bb.z; b8[7] = bb.w;
                }
#pragma unroll
                for (int jj = 0; jj < 8; jj++) {
                  const float uu = v[g8 * 8 + jj] + b8[jj];
                  t8[jj] = (act == 2) ? fmaxf(uu, 0.1f * uu) : uu;   // LeakyReLU(0.1)
                }
                uint4 qv;
                qv.x = tc::pack_bf16x2(t8[0], t8[1]); qv.y = tc::pack_bf16x2(t8[2], t8[3]);
                qv.z = tc::pack_bf16x2(t8[4], t8[5]); qv.w = tc::pack_bf16x2(t8[6], t8[7]);
                *reinterpret_cast<uint4*>(a_smem + (size_t)(((oc + cb) >> 3) + g8) * BF_PANEL + row * 16) = qv;
              }
            }
            tc::fence_async_smem();
          }
          tc::fence_before_sync();
          if (bf_sync_or(fail)) { fail = 1; break; }                                      // [B3..B6]
          pf.lap(6);
        }
        if (fail) break;
        // ---- 4. per-node sums of the scalar output: tensor memory holds [channel][edge] after the transposed last
        // layer; one thread per channel adds its row in edge order --------------------------------------------------
        tc::fence_after_sync();
        if (j == 0) {
          const float b3 = s_bias[4 * BF_A + ch];
#pragma unroll 1
          for (int cb = 0; cb < cnt; cb += 16) {
            float v[16];
            tc::tmem_ld16(tmem_row + BF_TMEM_MLP + cb, v);
            int sn[16];
#pragma unroll
            for (int i = 0; i < 4; i++) {
              const int4 t = *reinterpret_cast<const int4*>(&s_src[cb + 4 * i]);
              sn[4 * i] = t.x; sn[4 * i + 1] = t.y; sn[4 * i + 2] = t.z; sn[4 * i + 3] = t.w;
            }
            if (cb + 16 <= cnt && sn[0] == cur_a && sn[15] == cur_a) {
              // sixteen edges of the running node (sources are sorted): the same additions in the same order, no tests
#pragma unroll
              for (int i = 0; i < 16; i++) acc_a += v[i] + b3;
            } else {
#pragma unroll
              for (int i = 0; i < 16; i++) {
                if (cb + i < cnt) {
                  if (sn[i] != cur_a) {
                    P.out_a[(size_t)cur_a * BF_A + ch] = acc_a * P.scale;
                    for (int z = cur_a + 1; z < sn[i]; z++) P.out_a[(size_t)z * BF_A + ch] = 0.f;
                    acc_a = 0.f;
                    cur_a = sn[i];
                  }
                  acc_a += v[i] + b3;
                }
              }
            }
          }
        }
        node_lo = s_src[cnt - 1];
        pf.lap(7);
        tc::fence_before_sync();
        if (bf_sync_or(fail)) { fail = 1; break; }                                        // [B7]
        if (tid <= BF_EDGES) s_rowwin[tid] = P.row_ptr[min(node_lo + tid, n_end)];
        // (s_rowwin is read by the geometry of the next tile, after which [B1] orders it against the next refresh)
        asm volatile("barrier.cta.sync 2, %0;" ::"n"(BF_WORK_THREADS) : "memory");
        pf.lap(8);
      }
      if (!fail && n_begin < n_end) {
        if (br.e_begin >= br.e_end) {
          // a slice without any edge: zeros for all its nodes
          bf_flush_node(g, P.S_v, P.S_d, -1, n_begin, n_end, ch, P.scale, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f,
                        0.f, 0.f, 0.f, 0.f);
        }
        if (j == 0) {
          P.out_a[(size_t)cur_a * BF_A + ch] = acc_a * P.scale;
          for (int z = cur_a + 1; z < n_end; z++) P.out_a[(size_t)z * BF_A + ch] = 0.f;
        }
      }
    }
    if (fail) s_fail = 1;
  }
  if (fail && lane == 0 && P.status != nullptr) atomicOr(P.status, LD_FLAG_TIMEOUT);
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem_base, BF_TMEM_COLS);
}

// positions and values of the non-zero entries of G_e: D column o, left component m (0: l0, 1+x: l1[x], 4+3x+y: l2[x][y]),
// monomial of rhat (0: 1, 1..3: r_x, 4..9: r_x r_y for (x,y) = 00,01,02,11,12,22), sign
struct GammaEntry { int o, m, mono, neg; };

int mono2(int x, int y) {
  if (x > y) { int t = x; x = y; y = t; }
  static const int idx[3][3] = {{4, 5, 6}, {5, 7, 8}, {6, 8, 9}};
  return idx[x][y];
}

int build_gamma_entries(GammaEntry* out) {
  int n = 0;
  auto add = [&](int o, int m, int mono, int neg) { out[n++] = GammaEntry{o, m, mono, neg}; };
  add(0, 0, 0, 0);                                                        // y000 = l0
  for (int x = 0; x < 3; x++) add(1, 1 + x, 1 + x, 0);                    // y110 = l1 . r
  for (int x = 0; x < 3; x++) for (int y = 0; y < 3; y++) add(2, 4 + 3 * x + y, mono2(x, y), 0);   // y220 = r^T l2 r
  for (int x = 0; x < 3; x++) {
    add(3 + x, 0, 1 + x, 0);                                              // 011: l0 r_x
    add(6 + x, 1 + x, 0, 0);                                              // 101: l1_x
    for (int y = 0; y < 3; y++) add(9 + x, 1 + y, mono2(y, x), 0);        // 121: (l1 . r) r_x
    for (int y = 0; y < 3; y++) add(12 + x, 4 + 3 * x + y, 1 + y, 0);     // 211: (l2 r)_x
  }
  // 111: l1 x r
  add(15, 2, 3, 0); add(15, 3, 2, 1);
  add(16, 3, 1, 0); add(16, 1, 3, 1);
  add(17, 1, 2, 0); add(17, 2, 1, 1);
  for (int x = 0; x < 3; x++)
    for (int y = 0; y < 3; y++) {
      add(18 + 3 * x + y, 0, mono2(x, y), 0);                             // 022: l0 r_x r_y
      add(27 + 3 * x + y, 4 + 3 * x + y, 0, 0);                           // 202: l2_xy
      add(36 + 3 * x + y, 1 + x, 1 + y, 0);                               // 112: l1_x r_y
      for (int z = 0; z < 3; z++) add(45 + 3 * x + y, 4 + 3 * x + z, mono2(z, y), 0);   // 222: (l2 r)_x r_y
    }
  for (int x = 0; x < 3; x++) {                                           // 212: row x of l2 cross r
    add(54 + 3 * x, 4 + 3 * x + 1, 3, 0); add(54 + 3 * x, 4 + 3 * x + 2, 2, 1);
    add(55 + 3 * x, 4 + 3 * x + 2, 1, 0); add(55 + 3 * x, 4 + 3 * x + 0, 3, 1);
    add(56 + 3 * x, 4 + 3 * x + 0, 2, 0); add(56 + 3 * x, 4 + 3 * x + 1, 1, 1);
  }
  return n;
}

}  // namespace

// The table of G_e as (D column, left component, monomial index, sign) quadruples, for host-side checks of the index
// conventions against the reference's einsum definitions. out: 4 ints per entry, at most 128 entries; returns the count.
extern "C" int ld_bee_gamma_table(int* out) {
  GammaEntry ent[BF_GAMMA_ENTRIES];
  const int n = build_gamma_entries(ent);
  for (int i = 0; i < n; i++) { out[4 * i] = ent[i].o; out[4 * i + 1] = ent[i].m; out[4 * i + 2] = ent[i].mono; out[4 * i + 3] = ent[i].neg; }
  return n;
}

extern "C" int ld_bee_messages_fused_bf16_tc_opt(const int* row_ptr, const int* dst, const float* rij, int Nt, int chan, int dim_a,
                                                 float r0, const void* rows, const float* enc_w, const float* enc_b,
                                                 const float* jacobi, const void* Yp, const void* W1p, const float* b1,
                                                 const void* W2p, const float* b2, const void* W3p, const float* b3, float scale,
                                                 float* out_a, void* S_v, void* S_d, int* status_dev, void* stream, int spin);

// Whole message layer for chan = 128, dim_a = 128 (BF16 tensor-core path, 2e-2 relative):
//   rows    [Nt][2][128][8] BF16: per node and channel (l0, l1[3], l2[0..3] | l2[4..8], 0, 0, 0), written by
//           ld_linear_bf16_tc_out16 / _out16_split; the three unused values must be zero (or any finite number)
//   Yp, W1p, W2p, W3p, biases, enc_w, enc_b, jacobi as in ld_bee_messages_scalar_bf16_tc
//   out_a   [Nt][128] FP32; S_v [Nt][3][640], S_d [Nt][9][640] BF16 (per-node sums of the five rank-1 / rank-2 products,
//           component-major, the input form of ld_linear_bf16_tc_in16), all times `scale`
extern "C" int ld_bee_messages_fused_bf16_tc(const int* row_ptr, const int* dst, const float* rij, int Nt, int chan, int dim_a,
                                             float r0, const void* rows, const float* enc_w, const float* enc_b,
                                             const float* jacobi, const void* Yp, const void* W1p, const float* b1,
                                             const void* W2p, const float* b2, const void* W3p, const float* b3, float scale,
                                             float* out_a, void* S_v, void* S_d, int* status_dev, void* stream) {
  return ld_bee_messages_fused_bf16_tc_opt(row_ptr, dst, rij, Nt, chan, dim_a, r0, rows, enc_w, enc_b, jacobi, Yp, W1p, b1, W2p, b2,
                                           W3p, b3, scale, out_a, S_v, S_d, status_dev, stream, 0);
}

#ifdef LD_PHASE_COUNTERS
long long* ld_internal_phase_counters();
#endif

// `spin`: 1 = the waits on the per-group barriers poll (default), 0 = they suspend with a time hint
extern "C" int ld_bee_messages_fused_bf16_tc_opt(const int* row_ptr, const int* dst, const float* rij, int Nt, int chan, int dim_a,
                                                 float r0, const void* rows, const float* enc_w, const float* enc_b,
                                                 const float* jacobi, const void* Yp, const void* W1p, const float* b1,
                                                 const void* W2p, const float* b2, const void* W3p, const float* b3, float scale,
                                                 float* out_a, void* S_v, void* S_d, int* status_dev, void* stream, int spin) {
  if (Nt < 0 || !(r0 > 0.f)) return LD_ERR_SHAPE;
  if (chan != BF_C || dim_a != BF_A) {
    ld_set_last_message("fused l<=2 message kernel: built for chan = 128 and dim_a = 128 (other widths: the two-kernel path)");
    return LD_ERR_UNSUPPORTED;
  }
  if (b1 == nullptr || b2 == nullptr || b3 == nullptr) return LD_ERR_SHAPE;
  if ((((uintptr_t)Yp | (uintptr_t)W1p | (uintptr_t)W2p | (uintptr_t)W3p | (uintptr_t)rows) % 16) != 0) return LD_ERR_SHAPE;
  if (Nt == 0) return LD_OK;
  BfParams Q;
  Q.row_ptr = row_ptr; Q.dst = dst; Q.rij = rij; Q.Nt = Nt; Q.r0 = r0; Q.scale = scale;
  Q.rows = (const __nv_bfloat16*)rows; Q.enc_w = enc_w; Q.enc_b = enc_b; Q.jacobi = jacobi;
  const int A = BF_A, C = BF_C;
  const int sk1 = BF_SLAB_BYTES / (A * 32), sk2 = BF_SLAB_BYTES / (2 * A * 32);
  Q.layer[0] = BfLayer{(const __nv_bfloat16*)Yp, 0, 3 * C / 16, sk1, A, 0, 2 * A};
  Q.layer[1] = BfLayer{(const __nv_bfloat16*)W1p, 2 * A / 8, A / 16, sk2, 2 * A, 2, 0};
  Q.layer[2] = BfLayer{(const __nv_bfloat16*)W2p, 0, 2 * A / 16, sk2, 2 * A, 2, 0};
  Q.layer[3] = BfLayer{(const __nv_bfloat16*)W3p, 0, 3 * A / 16, sk1, A, 0, -1};
  Q.b1 = b1; Q.b2 = b2; Q.b3 = b3;
  {
    const long long seg = (40LL << 20) / BF_ROW_BYTES;   // about 40 MB of gathered rows per segment: they stay in L2
    Q.seg_nodes = ld_even_segments(Nt, seg);
  }
  Q.out_a = out_a; Q.S_v = (__nv_bfloat16*)S_v; Q.S_d = (__nv_bfloat16*)S_d; Q.status = status_dev;
  Q.wait_limit = tc::TC_WAIT_LIMIT;
  Q.spin = spin;
#ifdef LD_PHASE_COUNTERS
  Q.prof = ld_internal_phase_counters();
#else
  Q.prof = nullptr;
#endif
  {
    GammaEntry ent[BF_GAMMA_ENTRIES];
    const int n = build_gamma_entries(ent);
    for (int i = 0; i < BF_GAMMA_ENTRIES; i++) {
      if (i < n) {
        // operand row = sum index (the three scalar products are formed in registers and have no row)
        const int row = ent[i].o - 3;
        const int off = (ent[i].m / 8) * (BF_GAMMA_ROWS * 16) + row * 16 + (ent[i].m % 8) * 2;
        Q.gamma_tab[i] = ent[i].o < 3 ? (unsigned short)0xffffu
                                      : (unsigned short)((off >> 1) | (ent[i].mono << 11) | (ent[i].neg << 15));
      } else {
        Q.gamma_tab[i] = 0xffffu;
      }
    }
  }
  LD_CUDA_TRY(cudaFuncSetAttribute(bee_fused_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BF_SMEM));
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  bee_fused_tc_kernel<<<sms, BF_THREADS, BF_SMEM, (cudaStream_t)stream>>>(Q);
  LD_LAUNCH_CHECK();
  return LD_OK;
}
