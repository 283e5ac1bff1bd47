// One edge kernel per l<=2 ("Bee") message layer on the Blackwell tensor cores: Messages.forward of the reference
// (archs/diffuser_atoms15.py:227-253) for chan = 128 product channels and dim_a = 128, with every neighbour row
// gathered exactly once and the 13 products formed by the tensor cores instead of the FP32 lanes.
//
//   pa[e,c]   = lin_enc(radial_encode_8(r_e))[c]                                  (managan/jacobi_radenc.py:27-33)
//   rhat_e    = tens_sigmoid(1, r_e * 7/r0)                                       (managan/tensor_products.py:167-182)
//   the right operands of the Bee products are pa, pa*rhat, pa*rhat rhat^T, so each of the 63 product components
//   of an (edge, channel) is  pa[e,c] * sum_m l[dst_e, c, m] * G_e[m, o]  with l = (l0, l1[3], l2[9]) the thirteen
//   left values of the neighbour and G_e a 13 x 63 matrix of monomials of rhat_e (degree <= 2, signs of the
//   Levi-Civita symbol) that does not depend on the channel (managan/codegen_tensor_products.py:235-249).
//
// Per edge ONE tcgen05 MMA  D_e[c, o] = L_e[c, 0:16] * G_e[0:16, 0:64]  (M = 128 channels, N = 64, K = 16, BF16 operands,
// FP32 accumulators in tensor memory):
//   * L_e is the neighbour's row, stored per node as two 16-byte halves per channel, [node][2][chan][8] BF16: a single
//     4 KB bulk copy puts it into shared memory in exactly the K-major operand layout, without passing through
//     registers;
//   * G_e is written by two builder warps (115 non-zero BF16 entries at fixed positions);
//   * pa for the whole tile comes from one more MMA, [chan x 27] x [27 x edges] with lin_enc's weights and the radial
//     functions split into BF16 high and low parts (error 2^-17);
//   * the sixteen working warps read D_e from tensor memory (lane = channel), multiply by pa and add into 60 running
//     sums per channel held in registers (sixteen columns per warp); the three scalar products are rounded to BF16 into
//     the operand tile of the per-edge MLP. Sums are written once per node, in edge order.
// After the 128 edges of a tile: psi = [y000|y110|y220] Y^T, two hidden layers, and the last layer with weights
// [W3 | W_direct + I] as in bee_messages_tc.cu - the last one transposed (weights as the M operand), so that its
// result lies in tensor memory as [channel][edge] and the per-node sum over edges is a plain sequential sum in one
// thread per channel. All additions happen in an order fixed by the node's edge list alone, so a system's result does
// not depend on the batch (or shard) it is processed in.
//
// Shared memory: operand tile 97 KB | 96 KB ring, used as eight two-edge groups (two rows + two G matrices, 12 KB) while
// the products are formed and as three 32 KB weight slabs while the MLP runs | small operands. Tensor memory: columns
// [0, 384) three D groups (two edges each), the first 256 later the MLP accumulators; [384, 512) pa.
// Every wait is bounded; a wait that runs out sets LD_FLAG_TIMEOUT and all roles leave.
#include "common.cuh"
#include "tc05.cuh"
#include "tp_math.h"

namespace {

constexpr int BF_EDGES = 128;
constexpr int BF_C = 128, BF_A = 128;
constexpr int BF_WORK_WARPS = 16;
constexpr int BF_WORK_THREADS = BF_WORK_WARPS * 32;
// 20 warps: five per scheduler partition, the most that fit at 96 registers per thread (16384 registers per partition)
constexpr int BF_MMA_WARP = 16, BF_GATHER_WARP = 17, BF_BUILD_WARP0 = 18, BF_BUILD_WARPS = 2;
constexpr int BF_THREADS = (BF_WORK_WARPS + 2 + BF_BUILD_WARPS) * 32;          // 640
constexpr int BF_SYNC_THREADS = (BF_WORK_WARPS + 1) * 32;                      // working warps + MMA warp
constexpr int BF_PANEL = BF_EDGES * 16 + 16;     // byte stride between 8-column panels of the MLP operand tile (padded)
constexpr int BF_NG = 8;                         // ring groups (two edges each)
constexpr int BF_ROW_BYTES = 2 * BF_C * 16;      // 4096: one neighbour row = two K panels of 128 channels
constexpr int BF_GAMMA_BYTES = 64 * 32;          // 2048: G_e as N = 64 rows x K = 16
constexpr int BF_GROUP_BYTES = 2 * BF_ROW_BYTES + 2 * BF_GAMMA_BYTES;          // 12288
constexpr int BF_RING_BYTES = BF_NG * BF_GROUP_BYTES;                          // 98304
constexpr int BF_WSTAGES = 3, BF_SLAB_BYTES = 32 * 1024;
static_assert(BF_RING_BYTES == BF_WSTAGES * BF_SLAB_BYTES, "the ring is shared by row groups and weight slabs");
constexpr int BF_LAYERS = 4;
constexpr int BF_OFF_A = 0;
constexpr int BF_A_BYTES = (3 * BF_C / 8) * BF_PANEL;                          // 99072
constexpr int BF_OFF_RING = BF_OFF_A + BF_A_BYTES;
constexpr int BF_OFF_W9 = BF_OFF_RING + BF_RING_BYTES;                         // lin_enc operand: 128 rows x 32 (4 panels)
constexpr int BF_OFF_ENC = BF_OFF_W9 + 4 * BF_C * 16;                          // radial operand: 128 edges x 32
constexpr int BF_OFF_BIAS = BF_OFF_ENC + 4 * BF_EDGES * 16;
constexpr int BF_SMEM = BF_OFF_BIAS + 5 * BF_A * 4;
constexpr int BF_ND = 3;                         // D groups in tensor memory (two edges x 64 columns each)
constexpr uint32_t BF_TMEM_COLS = 512, BF_TMEM_PA = BF_ND * 128;
constexpr int BF_GAMMA_ENTRIES = 128;            // 115 used

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
  unsigned short gamma_tab[BF_GAMMA_ENTRIES];   // bits 0-10 byte offset inside G_e, 11-14 monomial, 15 sign; 0xffff unused
};

// Diagnostics build (-DLD_PHASE_COUNTERS): cycles per phase of one thread per role, added into prof[16]:
// working thread 0: 0 geometry, 1 wait pa, 2 wait D, 3 products, 4 barrier after products, 5 wait layers, 6 epilogues,
// 7 scalar sums, 8 end-of-tile barriers; MMA lane: 9 wait rows + G, 10 wait D free, 11 wait weights; builder 0:
// 12 wait free group, 13 build; gather lane 0: 14 wait free group; builder 1 lane 0: 15 weight streaming.
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

// column o of D_e (0..63) -> where its per-node sum goes. o in [3,18): rank-1 product (o-3)/3, component (o-3)%3;
// o in [18,63): rank-2 product (o-18)/9, component (o-18)%9. Writes (or zero-fills) the sixteen columns of group G.
template <int G>
__device__ __forceinline__ void bf_store_node(__nv_bfloat16* __restrict__ S_v, __nv_bfloat16* __restrict__ S_d, int node, int c,
                                              const float* acc, float scale) {
#pragma unroll
  for (int k = 0; k < 16; k++) {
    constexpr int base = 16 * G;
    const int o = base + k;
    if (o < 3 || o == 63) continue;
    const __nv_bfloat16 v = __float2bfloat16_rn(acc[k] * scale);
    if (o < 18) {
      const int vi = o - 3;
      S_v[((size_t)node * 3 + (vi % 3)) * (5 * BF_C) + (vi / 3) * BF_C + c] = v;
    } else {
      const int di = o - 18;
      S_d[((size_t)node * 9 + (di % 9)) * (5 * BF_C) + (di / 9) * BF_C + c] = v;
    }
  }
}

// End of a node's edge list for one thread (channel c, column group g): write its sixteen running sums for `node`, then
// zeros for the nodes without edges up to `next` (exclusive). One copy of this code, called from the few places where
// a node can end; the sums travel by value so that they stay in registers at the call sites.
__device__ __noinline__ void bf_flush_node(int g, __nv_bfloat16* S_v, __nv_bfloat16* S_d, int node, int next, int c, float scale,
                                           float a0, float a1, float a2, float a3, float a4, float a5, float a6, float a7,
                                           float a8, float a9, float a10, float a11, float a12, float a13, float a14, float a15) {
  float acc[16] = {a0, a1, a2, a3, a4, a5, a6, a7, a8, a9, a10, a11, a12, a13, a14, a15};
  for (int v = node; v < next; v++) {
    if (g == 0) bf_store_node<0>(S_v, S_d, v, c, acc, scale);
    else if (g == 1) bf_store_node<1>(S_v, S_d, v, c, acc, scale);
    else if (g == 2) bf_store_node<2>(S_v, S_d, v, c, acc, scale);
    else bf_store_node<3>(S_v, S_d, v, c, acc, scale);
    if (v == node) {
#pragma unroll
      for (int i = 0; i < 16; i++) acc[i] = 0.f;
    }
  }
}
#define BF_FLUSH(node, next)                                                                                              \
  do {                                                                                                                    \
    bf_flush_node(g, P.S_v, P.S_d, (node), (next), ch, P.scale, acc[0], acc[1], acc[2], acc[3], acc[4], acc[5], acc[6],  \
                  acc[7], acc[8], acc[9], acc[10], acc[11], acc[12], acc[13], acc[14], acc[15]);                          \
    _Pragma("unroll") for (int i_ = 0; i_ < 16; i_++) acc[i_] = 0.f;                                                      \
  } while (0)

__global__ void __launch_bounds__(BF_THREADS, 1)
bee_fused_tc_kernel(const __grid_constant__ BfParams P) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t bar_full[BF_NG], bar_slot_empty[BF_NG], bar_dfull[BF_ND], bar_dempty[BF_ND];
  __shared__ __align__(8) uint64_t bar_pa, bar_geom, bar_gather_go, bar_weights_go;
  __shared__ __align__(8) uint64_t bar_wfull[BF_WSTAGES], bar_wempty[BF_WSTAGES], bar_accum;
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int s_fail;
  __shared__ __align__(16) float s_mono[BF_EDGES][12];   // 1, rx, ry, rz, rx rx, rx ry, rx rz, ry ry, ry rz, rz rz
  __shared__ int s_src[BF_EDGES];
  __shared__ int s_rowwin[BF_EDGES + 1];
  __shared__ float s_jac[72];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  unsigned char* a_smem = smem + BF_OFF_A;
  unsigned char* ring = smem + BF_OFF_RING;
  unsigned char* w9_smem = smem + BF_OFF_W9;
  unsigned char* enc_smem = smem + BF_OFF_ENC;
  float* s_bias = reinterpret_cast<float*>(smem + BF_OFF_BIAS);   // [b1 (2A) | b2 (2A) | b3 (A)]
  const uint32_t wl = P.wait_limit;
  // the per-group barriers (64 groups per tile) complete within a few hundred cycles
  auto hot_wait = [&](uint64_t* bar, uint32_t parity) -> bool {
    if (P.spin == 2) return tc::mbar_wait_tight(bar, parity, wl << 6);
    return P.spin ? tc::mbar_wait_spin(bar, parity, wl << 4) : tc::mbar_wait(bar, parity, wl);
  };
  BfProf pf;

  if (tid < 8) ld_poly8_to_chebyshev(P.jacobi + tid * 9, s_jac + tid * 9);   // Chebyshev form of the radial polynomials
  for (int i = tid; i < 2 * BF_A; i += BF_THREADS) { s_bias[i] = P.b1[i]; s_bias[2 * BF_A + i] = P.b2[i]; }
  for (int i = tid; i < BF_A; i += BF_THREADS) s_bias[4 * BF_A + i] = P.b3[i];
  if (tid < BF_C) {
    // lin_enc as the M operand of the pa product: [W_hi (8 weights, bias) | W_hi | W_lo | 0], 32 columns, K-major panels
    float w[9];
#pragma unroll
    for (int m = 0; m < 8; m++) w[m] = P.enc_w[tid * 8 + m];
    w[8] = P.enc_b[tid];
    unsigned short row[32];
#pragma unroll
    for (int m = 0; m < 9; m++) {
      const __nv_bfloat16 hi = __float2bfloat16_rn(w[m]);
      const unsigned short h = *reinterpret_cast<const unsigned short*>(&hi);
      row[m] = h; row[9 + m] = h;
      row[18 + m] = bf_bf16(w[m] - __bfloat162float(hi));
    }
#pragma unroll
    for (int m = 27; m < 32; m++) row[m] = 0;
#pragma unroll
    for (int p = 0; p < 4; p++) {
      uint4 q;
      q.x = row[p * 8] | ((uint32_t)row[p * 8 + 1] << 16); q.y = row[p * 8 + 2] | ((uint32_t)row[p * 8 + 3] << 16);
      q.z = row[p * 8 + 4] | ((uint32_t)row[p * 8 + 5] << 16); q.w = row[p * 8 + 6] | ((uint32_t)row[p * 8 + 7] << 16);
      *reinterpret_cast<uint4*>(w9_smem + p * (BF_C * 16) + tid * 16) = q;
    }
  }
  if (tid == 0) {
    for (int s = 0; s < BF_NG; s++) { tc::mbar_init(&bar_full[s], 2); tc::mbar_init(&bar_slot_empty[s], 1); }
    for (int s = 0; s < BF_ND; s++) { tc::mbar_init(&bar_dfull[s], 1); tc::mbar_init(&bar_dempty[s], BF_WORK_WARPS); }
    tc::mbar_init(&bar_pa, 1); tc::mbar_init(&bar_geom, 1); tc::mbar_init(&bar_gather_go, 1); tc::mbar_init(&bar_weights_go, 1);
    for (int s = 0; s < BF_WSTAGES; s++) { tc::mbar_init(&bar_wfull[s], 1); tc::mbar_init(&bar_wempty[s], 1); }
    tc::mbar_init(&bar_accum, 1);
    tc::mbar_init_fence();
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

  if (warp == BF_GATHER_WARP) {
    // ===== gather: lanes 2k, 2k+1 own ring group k; lane 2k waits for the group to be free and announces the bytes,
    // then each of the two lanes requests one neighbour row (a 4 KB bulk copy straight into operand layout) ==========
    if (lane < 2 * BF_NG) {
      const int k = lane >> 1, u = lane & 1;
      const unsigned pair_mask = 3u << (2 * k);
      long long Gbase = 0;      // groups of all earlier tiles
      uint32_t tiles = 0;
      bool issued = false;
      uint32_t last_use = 0;
      pf.start(P.prof, lane == 0 && blockIdx.x == 0);
      for (int seg_lo = 0; seg_lo < P.Nt && !fail; seg_lo += seg_nodes) {
        const BfRange br = bf_block_range(P.row_ptr, seg_lo, min(seg_lo + seg_nodes, P.Nt));
        for (long long e0 = br.e_begin; e0 < br.e_end && !fail; e0 += BF_EDGES, tiles++) {
          const int cnt = (int)((br.e_end - e0) < BF_EDGES ? (br.e_end - e0) : BF_EDGES);
          const int groups = (cnt + 1) >> 1;
          // the ring holds weight slabs until the last layer of the previous tile has been multiplied
          if (tiles >= 1 && !tc::mbar_wait(&bar_gather_go, (tiles - 1) & 1, wl)) { fail = 1; break; }
          // first group of this tile that lands in ring group k
          int grp = (int)(((long long)k - Gbase) % BF_NG);
          if (grp < 0) grp += BF_NG;
          for (; grp < groups; grp += BF_NG) {
            const long long Gg = Gbase + grp;
            const uint32_t use = (uint32_t)(Gg / BF_NG);
            const int e = min(2 * grp + u, cnt - 1);
            const int j = __ldg(P.dst + e0 + e);
            int ok = 1;
            if (u == 0) {
              pf.lap(100);
              if (use >= 1 && !hot_wait(&bar_slot_empty[k], (use - 1) & 1)) ok = 0;
              pf.lap(14);
              if (ok) tc::mbar_expect_tx(&bar_full[k], 2 * BF_ROW_BYTES);
            }
            ok = __all_sync(pair_mask, ok);
            if (!ok || s_fail) { fail = 1; break; }
            tc::bulk_g2s(ring + k * BF_GROUP_BYTES + u * BF_ROW_BYTES, P.rows + (size_t)j * (2 * BF_C * 8), BF_ROW_BYTES, &bar_full[k]);
            issued = true; last_use = use;
          }
          Gbase += groups;
        }
      }
      if (fail) {
        s_fail = 1;
        if (issued && u == 0) tc::mbar_wait(&bar_full[k], last_use & 1, wl);   // let copies in flight land (bounded)
      }
    }
  } else if (warp >= BF_BUILD_WARP0) {
    // ===== builders: G_e of every edge (B operand, 64 x 16 BF16, K-major panels) =======================================
    // The second builder warp also streams the weight slabs of the four layers: its lane 0 does so after the warp's
    // last G of the tile (the ring belongs to the MLP from then until the last layer has been multiplied).
    const int b = warp - BF_BUILD_WARP0;
    uint32_t wloads = 0;
    unsigned short tab[4];
#pragma unroll
    for (int i = 0; i < 4; i++) tab[i] = P.gamma_tab[lane * 4 + i];
    long long Gbase = 0;
    uint32_t tiles = 0;
    pf.start(P.prof, lane == 0 && blockIdx.x == 0);
    for (int seg_lo = 0; seg_lo < P.Nt && !fail; seg_lo += seg_nodes) {
      const BfRange br = bf_block_range(P.row_ptr, seg_lo, min(seg_lo + seg_nodes, P.Nt));
      for (long long e0 = br.e_begin; e0 < br.e_end && !fail; e0 += BF_EDGES, tiles++) {
        const int cnt = (int)((br.e_end - e0) < BF_EDGES ? (br.e_end - e0) : BF_EDGES);
        const int groups = (cnt + 1) >> 1;
        if (tiles >= 1 && !tc::mbar_wait(&bar_gather_go, (tiles - 1) & 1, wl)) { fail = 1; break; }
        // the weight slabs of the previous tile overwrote the G areas: clear the ones this warp fills in this tile
        // (ring groups of one parity), the entries written below sit at fixed positions among zeros
        {
          const int par = (int)((Gbase + b) & 1);
          for (int gs = par; gs < BF_NG; gs += 2) {
            uint4* gz = reinterpret_cast<uint4*>(ring + gs * BF_GROUP_BYTES + 2 * BF_ROW_BYTES);
            for (int i = lane; i < 2 * BF_GAMMA_BYTES / 16; i += 32) gz[i] = make_uint4(0u, 0u, 0u, 0u);
          }
          __syncwarp();   // the entries written below belong to chunks other lanes have just cleared
        }
        if (!tc::mbar_wait(&bar_geom, tiles & 1, wl)) { fail = 1; break; }    // monomials of this tile are in s_mono
        for (int grp = b; grp < groups; grp += BF_BUILD_WARPS) {
          const long long Gg = Gbase + grp;
          const int gs = (int)(Gg % BF_NG);
          const uint32_t use = (uint32_t)(Gg / BF_NG);
          if (b == 0) pf.lap(100);
          if (use >= 1 && !hot_wait(&bar_slot_empty[gs], (use - 1) & 1)) { fail = 1; break; }
          if (b == 0) pf.lap(12);
          if (s_fail) { fail = 1; break; }
#pragma unroll
          for (int u = 0; u < 2; u++) {
            const int e = min(2 * grp + u, cnt - 1);
            unsigned char* gdst = ring + gs * BF_GROUP_BYTES + 2 * BF_ROW_BYTES + u * BF_GAMMA_BYTES;
#pragma unroll
            for (int i = 0; i < 4; i++) {
              const unsigned t = tab[i];
              if (t != 0xffffu) {
                float v = s_mono[e][(t >> 11) & 15];
                if (t & 0x8000u) v = -v;
                *reinterpret_cast<unsigned short*>(gdst + (t & 0x7ffu)) = bf_bf16(v);
              }
            }
          }
          tc::fence_async_smem();
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(&bar_full[gs]);
          if (b == 0) pf.lap(13);
        }
        Gbase += groups;
        if (b == BF_BUILD_WARPS - 1) {
          pf.lap(100);
          if (lane == 0 && !fail) {
            // the ring is free for weights once every product MMA of the tile has read its rows
            if (!tc::mbar_wait(&bar_weights_go, tiles & 1, wl)) fail = 1;
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
            if (fail) {   // let slabs in flight land (bounded)
              for (uint32_t i = wloads > BF_WSTAGES ? wloads - BF_WSTAGES : 0; i < wloads; i++)
                tc::mbar_wait(&bar_wfull[i % BF_WSTAGES], (i / BF_WSTAGES) & 1, wl);
            }
          }
          pf.lap(15);
          fail = __shfl_sync(0xffffffffu, fail, 0);
        }
      }
    }
    if (fail) s_fail = 1;
  } else if (warp == BF_MMA_WARP) {
    // ===== MMA issue ===========================================================================================
    const bool mma_lane = lane == 0;
    uint32_t wmmas = 0, tiles = 0;
    long long G = 0;
    const uint32_t a_base = tc::smem_u32(a_smem), ring_base = tc::smem_u32(ring);
    const uint64_t row_desc0 = tc::smem_desc(ring_base, BF_C * 16, 128);
    const uint64_t gam_desc0 = tc::smem_desc(ring_base + 2 * BF_ROW_BYTES, 64 * 16, 128);
    const uint32_t idesc_d = tc::idesc_bf16(BF_C, 64), idesc_pa = tc::idesc_bf16(BF_C, BF_EDGES);
    pf.start(P.prof, lane == 0 && blockIdx.x == 0);
    for (int seg_lo = 0; seg_lo < P.Nt && !fail; seg_lo += seg_nodes) {
      const BfRange br = bf_block_range(P.row_ptr, seg_lo, min(seg_lo + seg_nodes, P.Nt));
      for (long long e0 = br.e_begin; e0 < br.e_end; e0 += BF_EDGES, tiles++) {
        const int cnt = (int)((br.e_end - e0) < BF_EDGES ? (br.e_end - e0) : BF_EDGES);
        const int groups = (cnt + 1) >> 1;
        if (bf_sync_or(fail)) { fail = 1; break; }      // [B1] geometry staged (radial operand, monomials)
        if (mma_lane && !fail) {
          tc::fence_after_sync();
          const uint64_t wd = tc::smem_desc(tc::smem_u32(w9_smem), BF_C * 16, 128);
          const uint64_t ed = tc::smem_desc(tc::smem_u32(enc_smem), BF_EDGES * 16, 128);
          tc::mma_bf16(tmem_base + BF_TMEM_PA, wd, ed, idesc_pa, 0u);
          tc::mma_bf16(tmem_base + BF_TMEM_PA, wd + ((2 * BF_C * 16) >> 4), ed + ((2 * BF_EDGES * 16) >> 4), idesc_pa, 1u);
          tc::mma_commit(&bar_pa);
          for (int grp = 0; grp < groups; grp++, G++) {
            const int gs = (int)(G % BF_NG);
            const uint32_t use = (uint32_t)(G / BF_NG), d = (uint32_t)(G % BF_ND), duse = (uint32_t)(G / BF_ND);
            pf.lap(100);
            if (!hot_wait(&bar_full[gs], use & 1)) { fail = 1; break; }
            pf.lap(9);
            if (duse >= 1 && !hot_wait(&bar_dempty[d], (duse - 1) & 1)) { fail = 1; break; }
            pf.lap(10);
            tc::fence_after_sync();
            const uint64_t goff = (uint64_t)((gs * BF_GROUP_BYTES) >> 4);
            tc::mma_bf16(tmem_base + d * 128, row_desc0 + goff, gam_desc0 + goff, idesc_d, 0u);
            tc::mma_bf16(tmem_base + d * 128 + 64, row_desc0 + goff + (BF_ROW_BYTES >> 4), gam_desc0 + goff + (BF_GAMMA_BYTES >> 4),
                         idesc_d, 0u);
            tc::mma_commit(&bar_dfull[d]);
            tc::mma_commit(&bar_slot_empty[gs]);
          }
          if (!fail) tc::mma_commit(&bar_weights_go);   // every product MMA of the tile has read its rows: the ring may take weights
        }
        if (!mma_lane) G += groups;
        fail = __shfl_sync(0xffffffffu, fail, 0);
        G = __shfl_sync(0xffffffffu, G, 0);
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
                if (transposed) tc::mma_bf16(tmem_base, bd, ad, idesc, accumulate);
                else tc::mma_bf16(tmem_base, ad, bd, idesc, accumulate);
                accumulate = 1u;
                ad += a_step;
                bd += b_step;
              }
              tc::mma_commit(&bar_wempty[st]);
            }
            if (!fail) {
              tc::mma_commit(&bar_accum);
              if (l == BF_LAYERS - 1) tc::mma_commit(&bar_gather_go);   // the ring may take rows of the next tile
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
    const int q = warp & 3, g = warp >> 2;              // tensor-memory lane quarter (fixed by the warp id), column group
    const int ch = q * 32 + lane;                       // product channel = tensor-memory lane in the product phase
    const int row = q * 32 + lane;                      // edge row = tensor-memory lane in the MLP phase
    const uint32_t tmem_row = tmem_base + ((uint32_t)(q * 32) << 16);
    uint32_t accum_phase = 0, tiles = 0;
    long long G = 0;
    pf.start(P.prof, tid == 0 && blockIdx.x == 0);
    for (int seg_lo = 0; seg_lo < P.Nt && !fail; seg_lo += seg_nodes) {
      const BfRange br = bf_block_range(P.row_ptr, seg_lo, min(seg_lo + seg_nodes, P.Nt));
      const int n_begin = br.n_begin, n_end = br.n_end;
      float acc[16];
#pragma unroll
      for (int i = 0; i < 16; i++) acc[i] = 0.f;
      float acc_a = 0.f;
      int cur = n_begin;          // node whose product sums are running (all working threads agree)
      int cur_a = n_begin;        // node whose scalar sum is running (threads of column group 0)
      int node_lo = n_begin;
      asm volatile("barrier.cta.sync 2, %0;" ::"n"(BF_WORK_THREADS) : "memory");
      if (tid <= BF_EDGES) s_rowwin[tid] = P.row_ptr[min(node_lo + tid, n_end > n_begin ? n_end : n_begin)];
      float pre_x = 0.f, pre_y = 0.f, pre_z = 0.f;
      if (tid < BF_EDGES && br.e_begin + tid < br.e_end) {
        const long long en = br.e_begin + tid;
        pre_x = P.rij[en * 3]; pre_y = P.rij[en * 3 + 1]; pre_z = P.rij[en * 3 + 2];
      }
      asm volatile("barrier.cta.sync 2, %0;" ::"n"(BF_WORK_THREADS) : "memory");
      for (long long e0 = br.e_begin; e0 < br.e_end; e0 += BF_EDGES, tiles++) {
        const int cnt = (int)((br.e_end - e0) < BF_EDGES ? (br.e_end - e0) : BF_EDGES);
        const int groups = (cnt + 1) >> 1;
        // ---- 1. edge geometry: radial functions -> operand of the pa product, monomials of rhat, source node ---------
        if (tid < BF_EDGES) {
          const float gx = pre_x, gy = pre_y, gz = pre_z;
          {
            const long long en = e0 + BF_EDGES + tid;   // next tile's edge of this thread
            if (en < br.e_end) { pre_x = P.rij[en * 3]; pre_y = P.rij[en * 3 + 1]; pre_z = P.rij[en * 3 + 2]; }
          }
          int s = -1;
          float enc[9];
#pragma unroll
          for (int m = 0; m < 9; m++) enc[m] = 0.f;
          float rx = 0.f, ry = 0.f, rz = 0.f;
          if (tid < cnt) {
            const long long e = e0 + tid;
            const float d = sqrtf(gx * gx + gy * gy + gz * gz);
            const float zz = d / P.r0;
            ld_radial_cheb8(zz, fmaxf(1.f - zz, 0.f), s_jac, enc);
            enc[8] = 1.f;   // multiplies lin_enc's bias
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
          float4* mp = reinterpret_cast<float4*>(&s_mono[tid][0]);
          mp[0] = make_float4(1.f, rx, ry, rz);
          mp[1] = make_float4(rx * rx, rx * ry, rx * rz, ry * ry);
          mp[2] = make_float4(ry * rz, rz * rz, 0.f, 0.f);
          // N operand of the pa product, row = edge: [enc_hi (8 functions, 1) | enc_lo | enc_hi | 0]
          unsigned short rw[32];
#pragma unroll
          for (int m = 0; m < 9; m++) {
            const __nv_bfloat16 hi = __float2bfloat16_rn(enc[m]);
            const unsigned short h = *reinterpret_cast<const unsigned short*>(&hi);
            rw[m] = h; rw[18 + m] = h;
            rw[9 + m] = bf_bf16(enc[m] - __bfloat162float(hi));
          }
#pragma unroll
          for (int m = 27; m < 32; m++) rw[m] = 0;
#pragma unroll
          for (int p = 0; p < 4; p++) {
            uint4 qv;
            qv.x = rw[p * 8] | ((uint32_t)rw[p * 8 + 1] << 16); qv.y = rw[p * 8 + 2] | ((uint32_t)rw[p * 8 + 3] << 16);
            qv.z = rw[p * 8 + 4] | ((uint32_t)rw[p * 8 + 5] << 16); qv.w = rw[p * 8 + 6] | ((uint32_t)rw[p * 8 + 7] << 16);
            *reinterpret_cast<uint4*>(enc_smem + p * (BF_EDGES * 16) + tid * 16) = qv;
          }
        }
        tc::fence_async_smem();
        tc::fence_before_sync();
        if (bf_sync_or(fail)) { fail = 1; break; }                                        // [B1]
        if (tid == 0) tc::mbar_arrive(&bar_geom);       // builders may read the monomials of this tile
        pf.lap(0);
        // ---- 2. products: D_e from tensor memory, times pa, into the running sums / the operand tile -------------
        if (!tc::mbar_wait(&bar_pa, tiles & 1, wl)) fail = 1;
        tc::fence_after_sync();
        pf.lap(1);
#pragma unroll 1
        for (int grp = 0; grp < groups && !fail; grp++) {
          const uint32_t d = (uint32_t)(G % BF_ND), duse = (uint32_t)(G / BF_ND);
          G++;
          pf.lap(3);
          if (!hot_wait(&bar_dfull[d], duse & 1)) { fail = 1; break; }
          pf.lap(2);
          tc::fence_after_sync();
          float v[32], pa[2];
          tc::tmem_ld16x2_2(tmem_row + d * 128 + g * 16, tmem_row + d * 128 + 64 + g * 16, tmem_row + BF_TMEM_PA + 2 * grp, v, pa);
          pf.lap(16);
          tc::fence_before_sync();
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(&bar_dempty[d]);   // this warp has its copy: the group may be overwritten
          pf.lap(17);
          const int e = 2 * grp;
          const bool two = e + 1 < cnt;
          const int s0 = s_src[e], s1 = s_src[two ? e + 1 : e];
          if (s0 != cur) { BF_FLUSH(cur, s0); cur = s0; }
          if (g == 0) {
            // columns 0..2 are the scalar products y000, y110, y220 of this (edge, channel)
            unsigned short* arow = reinterpret_cast<unsigned short*>(a_smem + (size_t)e * 16) + (ch & 7);
            arow[(ch >> 3) * (BF_PANEL / 2)] = bf_bf16(pa[0] * v[0]);
            arow[((BF_C + ch) >> 3) * (BF_PANEL / 2)] = bf_bf16(pa[0] * v[1]);
            arow[((2 * BF_C + ch) >> 3) * (BF_PANEL / 2)] = bf_bf16(pa[0] * v[2]);
            if (two) {
              arow[(ch >> 3) * (BF_PANEL / 2) + 8] = bf_bf16(pa[1] * v[16]);
              arow[((BF_C + ch) >> 3) * (BF_PANEL / 2) + 8] = bf_bf16(pa[1] * v[17]);
              arow[((2 * BF_C + ch) >> 3) * (BF_PANEL / 2) + 8] = bf_bf16(pa[1] * v[18]);
            }
          }
#pragma unroll
          for (int i = 0; i < 16; i++) acc[i] = fmaf(pa[0], v[i], acc[i]);   // (group 0: sums 0..2 are never stored)
          if (two) {
            if (s1 != cur) { BF_FLUSH(cur, s1); cur = s1; }
#pragma unroll
            for (int i = 0; i < 16; i++) acc[i] = fmaf(pa[1], v[16 + i], acc[i]);
          }
        }
        pf.lap(3);
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
              tc::tmem_ld32(tmem_row + cb, v);
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
                for (int j = 0; j < 8; j++) {
                  const float uu = v[g8 * 8 + j] + b8[j];
                  t8[j] = (act == 2) ? fmaxf(uu, 0.1f * uu) : uu;   // LeakyReLU(0.1)
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
        if (g == 0) {
          const float b3 = s_bias[4 * BF_A + ch];
          for (int cb = 0; cb < cnt; cb += 32) {
            float v[32];
            pf.lap(7);
            tc::tmem_ld32(tmem_row + cb, v);
            pf.lap(18);
#pragma unroll
            for (int i = 0; i < 32; i++) {
              const int e = cb + i;
              if (e < cnt) {
                const int s = s_src[e];
                if (s != cur_a) {
                  P.out_a[(size_t)cur_a * BF_A + ch] = acc_a * P.scale;
                  for (int z = cur_a + 1; z < s; z++) P.out_a[(size_t)z * BF_A + ch] = 0.f;
                  acc_a = 0.f;
                  cur_a = s;
                }
                acc_a += v[i] + b3;
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
        // last node of the slice, then nodes without edges up to its end
        BF_FLUSH(cur, n_end);
        if (g == 0) {
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
    Q.seg_nodes = (int)(seg < 1024 ? 1024 : seg);
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
        const int off = (ent[i].m / 8) * (64 * 16) + ent[i].o * 16 + (ent[i].m % 8) * 2;
        Q.gamma_tab[i] = (unsigned short)(off | (ent[i].mono << 11) | (ent[i].neg << 15));
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
