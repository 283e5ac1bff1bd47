// Rank-1 / rank-2 products of the l<=2 ("Bee") message layer, summed per node, on the Blackwell tensor cores:
// the part of Messages.forward of the reference (archs/diffuser_atoms15.py:227-253) that ld_bee_messages_vd_f32
// computes with FP32 FMAs, for chan = 128 product channels and interleaved BF16 neighbour rows.
//
//   pa[e,c]   = lin_enc(radial_encode_8(r_e))[c]                                  (managan/jacobi_radenc.py:27-33)
//   rhat_e    = tens_sigmoid(1, r_e * 7/r0)                                       (managan/tensor_products.py:167-182)
//   the right operands of the Bee products are pa, pa*rhat, pa*rhat rhat^T, so each of the 60 rank-1 / rank-2
//   product components of an (edge, channel) is  sum_m (pa[e,c] l[dst_e, c, m]) * G_e[m, o]  with l = (l0, l1[3], l2[9])
//   the thirteen left values of the neighbour and G_e a 13 x 60 matrix of monomials of rhat_e (degree <= 2, signs of
//   the Levi-Civita symbol) that does not depend on the channel (managan/codegen_tensor_products.py:235-249).
//
// One tcgen05 MMA per edge, S_node[c, 0:64] += L_e * G_e with L_e = [128 channels x 16] the neighbour's row scaled by
// pa and G_e the [16 x 64] monomial matrix: the 60 sums ACCUMULATE in tensor memory over the edges of a node, so the
// per-node sum of edges_reduce_src costs no instruction, and a node's sums are read once per NODE. L_e never touches
// shared memory: the thread that owns a channel scales its 32-byte row in registers (packed BF16 products) and writes
// it with tcgen05.st into the lane of that channel, and the MMA takes its A operand from tensor memory; only G_e
// (2 KB per edge) is a shared-memory operand. Shared-memory bandwidth, which bounds the MMA when both operands and
// their producers' stores go through it, is left to G_e alone.
//
// Roles of a block (one per SM, 64 registers per thread):
//   warps 0..3   stage the geometry of 128 edges at a time (radial functions, monomials of rhat as BF16, source node,
//                node boundaries; two buffers, one tile ahead) and read finished nodes out of tensor memory (four
//                accumulators of 64 columns), writing them as BF16 [node][component][5 * chan];
//   warps 8..27  five sets of four warps (a warp = 32 channels = the tensor-memory lanes it may write); a set takes
//                every fifth group of four edges: loads the neighbours' rows, forms pa, scales the rows and stores
//                them into a ring of eight groups in tensor memory, and writes the 102 non-zero entries of G_e (one
//                per thread) into the ring's shared-memory half;
//   warp 4       one thread issues the MMAs, starts a new accumulator at every node boundary and commits the
//                finished one to the staging warps.
// All additions happen in the order of the node's edge list, so a system's result does not depend on the batch (or
// shard) it is processed in. Every wait is bounded; a wait that runs out sets LD_FLAG_TIMEOUT and all roles leave.
#include <cstdlib>
#include "common.cuh"
#include "tc05.cuh"
#include "tp_math.h"

namespace {

constexpr int VT_C = 128;
constexpr int VT_TILE = 128;                    // edges staged at a time
constexpr int VT_GE = 4;                        // edges per ring group
constexpr int VT_NG = 8;                        // ring groups
constexpr int VT_SETS = 5;                      // sets of four builder warps
constexpr int VT_STAGE_WARPS = 4;
// warps 0..3 stage and read out, warp 4 issues the MMAs, warps 8..27 build (set (w - 8) / 4, channel quarter w % 4: a
// warp can only write the tensor-memory lanes of its own quarter); the other warps are idle
constexpr int VT_MMA_WARP = 4;
constexpr int VT_BUILD_WARP0 = 8;
constexpr int VT_BUILDERS = 4 * VT_SETS;        // 20
constexpr int VT_THREADS = 32 * 32;             // 64 registers per thread
constexpr int VT_STAGE_THREADS = VT_STAGE_WARPS * 32;
constexpr int VT_GAMMA_ROWS = 64;               // G_e as the N operand: 64 rows (60 used)
constexpr int VT_GAMMA_BYTES = 2 * VT_GAMMA_ROWS * 16;                         // 2048: two K panels
constexpr int VT_GROUP_BYTES = VT_GE * VT_GAMMA_BYTES;                         // 8192
constexpr int VT_SMEM = VT_NG * VT_GROUP_BYTES;                                // 65536
constexpr int VT_NACC = 4;                      // node accumulators (64 tensor-memory columns each)
// tensor memory: [0, 256) the node accumulators | [256, 512) the scaled rows L_e of the ring (eight columns per edge)
constexpr uint32_t VT_TMEM_COLS = 512, VT_TMEM_ROWS = 256;
constexpr int VT_GAMMA_ENTRIES = 128;           // 102 used

struct VtParams {
  const int* row_ptr; const int* dst; const float* rij;
  int Nt;
  float r0, scale;
  const __nv_bfloat16* rows;     // [Nt][128][16]: per node and channel (l0, l1[3], l2[9], 3 unused)
  const float* enc_w; const float* enc_b; const float* jacobi;
  int seg_nodes;
  __nv_bfloat16* S_v; __nv_bfloat16* S_d;
  int* status;
  uint32_t wait_limit;
  long long* prof;               // diagnostics build only
  int dbg;                       // diagnostics build only: 1 = issue no MMA, 2 = issue every MMA twice (timing experiments)
  unsigned short gamma_tab[VT_GAMMA_ENTRIES];   // bits 0-10 (byte offset inside G_e) / 2, 11-14 monomial, 15 sign; 0xffff unused
};

struct VtRange { int n_begin, n_end; long long e_begin, e_end, ntiles; };

// Diagnostics build (-DLD_PHASE_COUNTERS): cycles per phase of one thread per role (block 0), added into prof[32]:
// MMA thread: 0 wait staged tile, 1 wait group, 2 wait free accumulator, 3 issue; builder (warp 4, lane 0): 8 wait staged
// tile, 9 wait free ring group, 10 build; staging thread 0: 16 wait free buffer, 17 geometry, 18 wait finished node, 19 write node
struct VtProf {
#ifdef LD_PHASE_COUNTERS
  long long t; long long* prof; bool on;
  __device__ __forceinline__ void start(long long* p, bool enable) { prof = p; on = enable && p != nullptr; t = clock64(); }
  __device__ __forceinline__ void lap(int slot) {
    if (on) { const long long n = clock64(); atomicAdd((unsigned long long*)&prof[slot], (unsigned long long)(n - t)); t = n; }
  }
#else
  __device__ __forceinline__ void start(long long*, bool) {}
  __device__ __forceinline__ void lap(int) {}
#endif
};

__device__ __forceinline__ int vt_work_lb(const int* __restrict__ row_ptr, int lo, int hi, long long target) {
  const long long base = (long long)row_ptr[lo] + lo;
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if ((long long)row_ptr[mid] + mid - base < target) lo = mid + 1; else hi = mid;
  }
  return lo;
}
__device__ __forceinline__ int vt_lb_row(const int* __restrict__ row_ptr, int lo, int hi, long long target) {
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if ((long long)row_ptr[mid] < target) lo = mid + 1; else hi = mid;
  }
  return lo;
}
// this block's node-aligned slice of the segment [seg_lo, seg_hi), balanced over edges + nodes
__device__ __forceinline__ VtRange vt_block_range(const int* __restrict__ row_ptr, int seg_lo, int seg_hi) {
  VtRange r;
  const long long work = ((long long)row_ptr[seg_hi] - row_ptr[seg_lo]) + (seg_hi - seg_lo);
  long long per = (work + gridDim.x - 1) / gridDim.x;
  if (per < VT_TILE) per = VT_TILE;
  r.n_begin = blockIdx.x == 0 ? seg_lo : vt_work_lb(row_ptr, seg_lo, seg_hi, per * blockIdx.x);
  r.n_end = blockIdx.x == gridDim.x - 1 ? seg_hi : vt_work_lb(row_ptr, seg_lo, seg_hi, per * (blockIdx.x + 1));
  r.e_begin = r.n_begin < r.n_end ? row_ptr[r.n_begin] : 0;
  r.e_end = r.n_begin < r.n_end ? row_ptr[r.n_end] : 0;
  r.ntiles = (r.e_end - r.e_begin + VT_TILE - 1) / VT_TILE;
  return r;
}

// barrier of the four staging warps that also ORs a flag over them
__device__ __forceinline__ int vt_stage_sync_or(int flag) {
  int out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "barrier.cta.red.or.pred p, 2, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(out)
      : "r"(flag), "n"(VT_STAGE_THREADS)
      : "memory");
  return out;
}

// sixteen columns [16 G, 16 G + 16) of a node accumulator -> their places. Column o in [0,15): rank-1 product o/3,
// component o%3; o in [15,60): rank-2 product (o-15)/9, component (o-15)%9; 60..63 unused.
template <int G>
__device__ __forceinline__ void vt_store16(__nv_bfloat16* __restrict__ S_v, __nv_bfloat16* __restrict__ S_d, int node, int c,
                                           const float* acc, float scale) {
#pragma unroll
  for (int k = 0; k < 16; k++) {
    constexpr int base = 16 * G;
    const int o = base + k;
    if (o >= 60) continue;
    const __nv_bfloat16 v = __float2bfloat16_rn(acc[k] * scale);
    if (o < 15) {
      S_v[((size_t)node * 3 + (o % 3)) * (5 * VT_C) + (o / 3) * VT_C + c] = v;
    } else {
      const int di = o - 15;
      S_d[((size_t)node * 9 + (di % 9)) * (5 * VT_C) + (di / 9) * VT_C + c] = v;
    }
  }
}

__device__ __noinline__ void vt_store_zero(__nv_bfloat16* __restrict__ S_v, __nv_bfloat16* __restrict__ S_d, int from, int next, int c) {
  const __nv_bfloat16 z = __float2bfloat16_rn(0.f);
  for (int v = from; v < next; v++) {
#pragma unroll
    for (int i = 0; i < 15; i++) S_v[((size_t)v * 3 + (i % 3)) * (5 * VT_C) + (i / 3) * VT_C + c] = z;
#pragma unroll
    for (int i = 0; i < 45; i++) S_d[((size_t)v * 9 + (i % 9)) * (5 * VT_C) + (i / 9) * VT_C + c] = z;
  }
}

__global__ void __launch_bounds__(VT_THREADS, 1)
bee_vd_tc_kernel(const __grid_constant__ VtParams P) {
  extern __shared__ __align__(1024) unsigned char ring[];
  __shared__ __align__(8) uint64_t bar_full[VT_NG], bar_slot_empty[VT_NG];
  __shared__ __align__(8) uint64_t bar_dfull[VT_NACC], bar_dempty[VT_NACC];
  __shared__ __align__(8) uint64_t bar_tfull[2], bar_tempty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int s_fail;
  __shared__ __align__(16) float s_enc[2][VT_TILE][8];            // per edge: the eight radial functions
  // per edge, as BF16: 1, rx, ry, rz, rx rx, rx ry, rx rz, ry ry, ry rz, rz rz, then the same ten negated
  __shared__ __align__(8) unsigned short s_mono[2][VT_TILE][20];
  __shared__ int s_src[2][VT_TILE];
  __shared__ int s_dst[2][VT_TILE];
  __shared__ int s_bnd[2][VT_TILE];      // edges of the tile at which a new source node starts, ascending
  __shared__ int s_nbnd[2];
  __shared__ unsigned s_bmask[2][VT_TILE / 32];   // the same as one bit per edge (for the MMA thread)
  __shared__ int s_prev_src;             // source node of the last edge of the previous tile of the slice (-1: none)
  __shared__ int s_rowwin[VT_TILE + 1];
  __shared__ float s_jac[72];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t wl = P.wait_limit;
  VtProf pf;

  if (tid < 8) ld_poly8_to_chebyshev(P.jacobi + tid * 9, s_jac + tid * 9);   // Chebyshev form of the radial polynomials
  if (tid == 0) {
    for (int s = 0; s < VT_NG; s++) { tc::mbar_init(&bar_full[s], 4); tc::mbar_init(&bar_slot_empty[s], 1); }   // 4 warps per group
    for (int s = 0; s < VT_NACC; s++) { tc::mbar_init(&bar_dfull[s], 1); tc::mbar_init(&bar_dempty[s], VT_STAGE_WARPS); }
    for (int s = 0; s < 2; s++) { tc::mbar_init(&bar_tfull[s], VT_STAGE_WARPS); tc::mbar_init(&bar_tempty[s], VT_BUILDERS + 1); }
    tc::mbar_init_fence();
    // every ring group starts out free: complete the first phase of its "empty" barrier, so that the n-th use of a group
    // always waits for phase n (no special case for the first use)
    for (int s = 0; s < VT_NG; s++) tc::mbar_arrive(&bar_slot_empty[s]);
    s_fail = 0;
  }
  // the entries of G_e sit at fixed positions among zeros: clear the G areas of the ring once
  for (int i = tid; i < VT_SMEM / 16; i += VT_THREADS) *reinterpret_cast<uint4*>(ring + (size_t)i * 16) = make_uint4(0u, 0u, 0u, 0u);
  if (warp == 0) { tc::tmem_alloc(&tmem_slot, VT_TMEM_COLS); tc::tmem_relinquish(); }
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  const int seg_nodes = P.seg_nodes > 0 ? P.seg_nodes : P.Nt;
  int fail = 0;

  if (warp == VT_MMA_WARP) {
    // ===== MMA issue ===========================================================================================
    if (lane == 0) {
      uint32_t gidx = 0, T = 0;   // running group and tile counters (every role counts the same sequence)
      uint32_t nc = 0;            // nodes (with edges) completed so far: the running node uses accumulator nc % VT_NACC
      uint32_t d_addr = tmem_base;
      const uint32_t ring_base = tc::smem_u32(ring);
      const uint64_t gam_desc0 = tc::smem_desc(ring_base, VT_GAMMA_ROWS * 16, 128);
      // the byte offset of an edge's G_e (in 16-byte units) only ever changes the low word of the descriptor
      const uint32_t gam_lo = (uint32_t)gam_desc0, gam_hi = (uint32_t)(gam_desc0 >> 32);
      const uint32_t idesc = tc::idesc_bf16(VT_C, 64);
      pf.start(P.prof, blockIdx.x == 0);
      for (int seg_lo = 0; seg_lo < P.Nt && !fail; seg_lo += seg_nodes) {
        const VtRange br = vt_block_range(P.row_ptr, seg_lo, min(seg_lo + seg_nodes, P.Nt));
        bool have = false;        // a node is accumulating (none yet in this slice)
        for (long long e0 = br.e_begin; e0 < br.e_end && !fail; e0 += VT_TILE, T++) {
          const int cnt = (int)((br.e_end - e0) < VT_TILE ? (br.e_end - e0) : VT_TILE);
          const int groups = (cnt + VT_GE - 1) / VT_GE;
          const int buf = T & 1;
          if (s_fail || !tc::mbar_wait(&bar_tfull[buf], (T >> 1) & 1, wl)) { fail = 1; break; }
          pf.lap(0);
          const unsigned bm0 = s_bmask[buf][0], bm1 = s_bmask[buf][1], bm2 = s_bmask[buf][2], bm3 = s_bmask[buf][3];
#pragma unroll 1
          for (int grp = 0; grp < groups; grp++) {
            const uint32_t g = gidx + grp, slot = g % VT_NG, use = g / VT_NG;
            if (!tc::mbar_wait_tight(&bar_full[slot], use & 1, wl << 4)) { fail = 1; break; }
            pf.lap(1);
            tc::fence_after_sync();
            const unsigned bits = (grp < 8 ? bm0 : grp < 16 ? bm1 : grp < 24 ? bm2 : bm3) >> ((grp & 7) * 4);
            const int nv = cnt - VT_GE * grp;          // edges of this group (at least 1)
            const uint32_t gl = gam_lo + slot * (VT_GROUP_BYTES >> 4);
            const uint32_t al = tmem_base + VT_TMEM_ROWS + slot * (VT_GE * 8);
#pragma unroll
            for (int u = 0; u < VT_GE; u++) {
              if (u >= nv) break;
              uint32_t accumulate = 1u;
              if (bits & (1u << u)) {
                // a new node starts at this edge: hand the accumulator of the finished one to the staging warps and
                // take the next one, which must have been read out (it held the node VT_NACC nodes back)
                if (have) { tc::mma_commit(&bar_dfull[nc % VT_NACC]); nc++; }
                have = true;
                pf.lap(3);
                if (nc >= VT_NACC && !tc::mbar_wait_tight(&bar_dempty[nc % VT_NACC], ((nc / VT_NACC) - 1) & 1, wl << 4)) { fail = 1; break; }
                pf.lap(2);
                tc::fence_after_sync();
                d_addr = tmem_base + (nc % VT_NACC) * 64;
                accumulate = 0u;
              }
              const uint64_t gd = ((uint64_t)gam_hi << 32) | (gl + u * (VT_GAMMA_BYTES >> 4));
#ifdef LD_PHASE_COUNTERS
              if (P.dbg != 1 && P.dbg != 4) tc::mma_bf16_ta(d_addr, al + u * 8, gd, idesc, accumulate);
              if (P.dbg == 2) tc::mma_bf16_ta(d_addr, al + u * 8, gd, idesc, 1u);
#else
              tc::mma_bf16_ta(d_addr, al + u * 8, gd, idesc, accumulate);
#endif
            }
            if (fail) break;
#ifdef LD_PHASE_COUNTERS
            if (P.dbg == 4) tc::mbar_arrive(&bar_slot_empty[slot]); else tc::mma_commit(&bar_slot_empty[slot]);
#else
            tc::mma_commit(&bar_slot_empty[slot]);
#endif
            pf.lap(3);
          }
          if (fail) break;
          if (e0 + VT_TILE >= br.e_end && have) { tc::mma_commit(&bar_dfull[nc % VT_NACC]); nc++; have = false; }   // last node of the slice
          tc::mbar_arrive(&bar_tempty[buf]);
          gidx += groups;
        }
      }
      if (fail) s_fail = 1;
    }
  } else if (warp >= VT_BUILD_WARP0 && warp < VT_BUILD_WARP0 + VT_BUILDERS) {
    // ===== builder warps: rows -> scaled MMA operands in tensor memory, G_e in shared memory ======================
    const int q = warp & 3, set = (warp - VT_BUILD_WARP0) >> 2;
    const int ch = q * 32 + lane;
    const uint32_t tmem_rows = tmem_base + ((uint32_t)(q * 32) << 16) + VT_TMEM_ROWS;
    float w8[8];
#pragma unroll
    for (int m = 0; m < 8; m++) w8[m] = P.enc_w[ch * 8 + m];   // lin_enc of this thread's product channel
    const float wb = P.enc_b[ch];
    // this thread's entry of G_e (the four warps of a set write all 102 between them)
    const unsigned gtab = P.gamma_tab[q * 32 + lane];
    const int g_mono = ((gtab >> 11) & 15) + ((gtab & 0x8000u) ? 10 : 0), g_off = 2 * (gtab & 0x7ffu);
    const bool g_has = gtab != 0xffffu;
    const __nv_bfloat16* rows_c = P.rows + (size_t)ch * 16;
    uint32_t gidx = 0, T = 0;
    pf.start(P.prof, blockIdx.x == 0 && warp == VT_BUILD_WARP0 && lane == 0);
    for (int seg_lo = 0; seg_lo < P.Nt && !fail; seg_lo += seg_nodes) {
      const VtRange br = vt_block_range(P.row_ptr, seg_lo, min(seg_lo + seg_nodes, P.Nt));
      for (long long e0 = br.e_begin; e0 < br.e_end && !fail; e0 += VT_TILE, T++) {
        const int cnt = (int)((br.e_end - e0) < VT_TILE ? (br.e_end - e0) : VT_TILE);
        const int groups = (cnt + VT_GE - 1) / VT_GE;
        const int buf = T & 1;
        pf.lap(10);
        {
          int ok = 1;
          if (lane == 0) ok = (!s_fail && tc::mbar_wait(&bar_tfull[buf], (T >> 1) & 1, wl)) ? 1 : 0;
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) { fail = 1; break; }
        }
        pf.lap(8);
        const int* tdst = s_dst[buf];
        const int last = cnt - 1;
        int grp = (int)((set + VT_SETS - gidx % VT_SETS) % VT_SETS);   // first group of the tile whose running index is this set's
#pragma unroll 1
        for (; grp < groups; grp += VT_SETS) {
          // the four rows of the group are requested together; the other builder warps of the scheduler run meanwhile
          uint32_t raw[VT_GE][8];
#pragma unroll
          for (int u = 0; u < VT_GE; u++) {
            const int e = min(VT_GE * grp + u, last);   // clamped: the load is unconditional
            tc::ldg_raw8(rows_c + (size_t)tdst[e] * (VT_C * 16), raw[u]);
          }
          const uint32_t g = gidx + grp, slot = g % VT_NG, use = g / VT_NG;
          pf.lap(10);
          {
            int ok = 1;
            if (lane == 0) ok = tc::mbar_wait_spin(&bar_slot_empty[slot], use & 1, wl << 4) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) { fail = 1; break; }
          }
          pf.lap(9);
          tc::fence_after_sync();   // the MMAs that read this ring group are complete: its tensor-memory columns may be rewritten
          unsigned char* gbase = ring + (size_t)slot * VT_GROUP_BYTES;
#pragma unroll
          for (int u = 0; u < VT_GE; u++) {
            const int e = VT_GE * grp + u;
            if (e < cnt) {
              const float4* gp = reinterpret_cast<const float4*>(&s_enc[buf][e][0]);
              const float4 e0v = gp[0], e1v = gp[1];
              float pa = wb;
              pa = fmaf(e0v.x, w8[0], pa); pa = fmaf(e0v.y, w8[1], pa); pa = fmaf(e0v.z, w8[2], pa); pa = fmaf(e0v.w, w8[3], pa);
              pa = fmaf(e1v.x, w8[4], pa); pa = fmaf(e1v.y, w8[5], pa); pa = fmaf(e1v.z, w8[6], pa); pa = fmaf(e1v.w, w8[7], pa);
              // the row times pa as packed BF16 products (one rounding of each exact product; pa itself rounded to BF16)
              const __nv_bfloat162 pa2 = __float2bfloat162_rn(pa);
              uint32_t o[8];
#pragma unroll
              for (int i = 0; i < 7; i++) {
                const __nv_bfloat162 v = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&raw[u][i]), pa2);
                o[i] = *reinterpret_cast<const uint32_t*>(&v);
              }
              o[6] &= 0x0000ffffu;   // the three unused values of a row count as zero
              o[7] = 0u;
              tc::tmem_st8(tmem_rows + slot * (VT_GE * 8) + u * 8, o);   // row `ch` of L_e: sixteen BF16 values in K order
              if (g_has)
                *reinterpret_cast<unsigned short*>(gbase + u * VT_GAMMA_BYTES + g_off) = s_mono[buf][e][g_mono];
            }
          }
          pf.lap(11);
          tc::tmem_st_wait();
          pf.lap(12);
          tc::fence_before_sync();
          tc::fence_async_smem();
          pf.lap(13);
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(&bar_full[slot]);
          pf.lap(14);
        }
        if (fail) break;
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&bar_tempty[buf]);
        gidx += groups;
      }
    }
    if (fail) s_fail = 1;
  } else if (warp < VT_STAGE_WARPS) {
    // ===== staging warps: geometry one tile ahead, finished nodes out of tensor memory =============================
    const int q = warp;                               // tensor-memory lane quarter
    const int ch = tid;                               // channel = tensor-memory lane when reading a node out
    const uint32_t tmem_row = tmem_base + ((uint32_t)(q * 32) << 16);
    uint32_t T_stage = 0, T_drain = 0, nc = 0;
    pf.start(P.prof, blockIdx.x == 0 && tid == 0);
    for (int seg_lo = 0; seg_lo < P.Nt && !fail; seg_lo += seg_nodes) {
      const VtRange br = vt_block_range(P.row_ptr, seg_lo, min(seg_lo + seg_nodes, P.Nt));
      const int n_begin = br.n_begin, n_end = br.n_end;
      int cur = -1;               // node whose sums are accumulating in tensor memory
      int zero_from = n_begin;    // first node whose sums have not been written yet
      int node_lo = n_begin;
      float pre_x = 0.f, pre_y = 0.f, pre_z = 0.f;
      int pre_j = 0;
      if (br.e_begin + tid < br.e_end) {
        const long long en = br.e_begin + tid;
        pre_x = P.rij[en * 3]; pre_y = P.rij[en * 3 + 1]; pre_z = P.rij[en * 3 + 2]; pre_j = P.dst[en];
      }
      if (tid == 0) s_prev_src = -1;

      // geometry, source nodes and node boundaries of the tile that starts at edge e0
      auto stage = [&](long long e0) {
        const int cnt = (int)((br.e_end - e0) < VT_TILE ? (br.e_end - e0) : VT_TILE);
        const int buf = T_stage & 1;
        pf.lap(19);
        if (T_stage >= 2) {   // the builders and the MMA thread are done with the tile that used this buffer
          if (lane == 0 && (s_fail || !tc::mbar_wait(&bar_tempty[buf], ((T_stage >> 1) - 1) & 1, wl))) fail = 1;
        }
        pf.lap(16);
        s_rowwin[tid] = P.row_ptr[min(node_lo + tid, n_end)];
        if (tid == 0) s_rowwin[VT_TILE] = P.row_ptr[min(node_lo + VT_TILE, n_end)];
        if (vt_stage_sync_or(fail)) { fail = 1; return; }
        {
          const float gx = pre_x, gy = pre_y, gz = pre_z;
          const int gj = pre_j;
          {
            const long long en = e0 + VT_TILE + tid;   // next tile's edge of this thread
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
            const float inv = 1.0f / sqrtf(1.f + ux * ux + uy * uy + uz * uz);
            rx = ux * inv; ry = uy * inv; rz = uz * inv;
            if ((long long)s_rowwin[VT_TILE] > e) {
              int lo = 0, hi = VT_TILE;
              while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if ((long long)s_rowwin[mid] > e) hi = mid; else lo = mid; }
              s = node_lo + lo;
            } else {
              s = vt_lb_row(P.row_ptr, node_lo + VT_TILE, n_end, e + 1) - 1;
            }
          }
          s_src[buf][tid] = s;
          s_dst[buf][tid] = tid < cnt ? gj : 0;
          float4* gp = reinterpret_cast<float4*>(&s_enc[buf][tid][0]);
          gp[0] = make_float4(enc[0], enc[1], enc[2], enc[3]);
          gp[1] = make_float4(enc[4], enc[5], enc[6], enc[7]);
          const float mono[10] = {1.f, rx, ry, rz, rx * rx, rx * ry, rx * rz, ry * ry, ry * rz, rz * rz};
          uint32_t* mp = reinterpret_cast<uint32_t*>(&s_mono[buf][tid][0]);
#pragma unroll
          for (int i = 0; i < 5; i++) {
            mp[i] = tc::pack_bf16x2(mono[2 * i], mono[2 * i + 1]);
            mp[5 + i] = tc::pack_bf16x2(-mono[2 * i], -mono[2 * i + 1]);
          }
        }
        vt_stage_sync_or(0);
        if (warp == 0) {
          // boundary list: edges whose source differs from the edge before (the first edge compares with the last edge
          // of the previous tile of this slice), compacted in order by ballots
          int n = 0;
          for (int base = 0; base < VT_TILE; base += 32) {
            const int e = base + lane;
            bool isb = false;
            if (e < cnt) isb = s_src[buf][e] != (e == 0 ? s_prev_src : s_src[buf][e - 1]);
            const unsigned m = __ballot_sync(0xffffffffu, isb);
            if (lane == 0) s_bmask[buf][base >> 5] = m;
            if (isb) s_bnd[buf][n + __popc(m & ((1u << lane) - 1))] = e;
            n += __popc(m);
          }
          __syncwarp();
          if (lane == 0) { s_nbnd[buf] = n; s_prev_src = s_src[buf][cnt - 1]; }
        }
        vt_stage_sync_or(0);
        node_lo = s_src[buf][cnt - 1];
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&bar_tfull[buf]);
        T_stage++;
        pf.lap(17);
      };

      // one node boundary: the node `cur` is complete in its accumulator (the MMA thread has committed it) - read this
      // thread's 64 columns, release the accumulator, write them; then zeros for the nodes without edges before `next`
      auto end_node = [&](int next) {
        if (cur >= 0) {
          int ok = 1;
          if (lane == 0) ok = (!s_fail && tc::mbar_wait(&bar_dfull[nc % VT_NACC], (nc / VT_NACC) & 1, wl)) ? 1 : 0;
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) { fail = 1; return; }
          pf.lap(18);
          tc::fence_after_sync();
          const uint32_t t0 = tmem_row + (nc % VT_NACC) * 64;
          float a[16];
          tc::tmem_ld16(t0, a);      vt_store16<0>(P.S_v, P.S_d, cur, ch, a, P.scale);
          tc::tmem_ld16(t0 + 16, a); vt_store16<1>(P.S_v, P.S_d, cur, ch, a, P.scale);
          tc::tmem_ld16(t0 + 32, a); vt_store16<2>(P.S_v, P.S_d, cur, ch, a, P.scale);
          tc::tmem_ld16(t0 + 48, a); vt_store16<3>(P.S_v, P.S_d, cur, ch, a, P.scale);
          tc::fence_before_sync();
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(&bar_dempty[nc % VT_NACC]);
          nc++;
        }
        if (zero_from < next) vt_store_zero(P.S_v, P.S_d, zero_from, next, ch);
        pf.lap(19);
      };

      // The four staging warps meet at block barriers, so they may only leave a loop together: a failure seen by one
      // warp travels through the OR of the next barrier, and every warp acts on that result alone.
      if (br.e_begin < br.e_end) stage(br.e_begin);
      for (long long e0 = br.e_begin; e0 < br.e_end; e0 += VT_TILE, T_drain++) {
        if (vt_stage_sync_or(fail)) { fail = 1; break; }
        if (e0 + VT_TILE < br.e_end) stage(e0 + VT_TILE);
        if (fail) continue;                                  // the same in all four warps (set by a barrier inside stage)
        const int buf = T_drain & 1;
        const int nb = s_nbnd[buf];
        for (int bi = 0; bi < nb && !fail; bi++) {
          const int s = s_src[buf][s_bnd[buf][bi]];
          end_node(s);
          cur = s; zero_from = s + 1;
        }
      }
      // end of this block's slice: its last node, then the nodes without edges up to the end of the slice
      if (!fail) { end_node(n_end); cur = -1; }
      if (vt_stage_sync_or(fail)) fail = 1;
    }
    if (fail) s_fail = 1;
  }
  if (fail && lane == 0 && P.status != nullptr) atomicOr(P.status, LD_FLAG_TIMEOUT);
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem_base, VT_TMEM_COLS);
}

}  // namespace

extern "C" int ld_bee_gamma_table(int* out);
#ifdef LD_PHASE_COUNTERS
long long* ld_internal_phase_counters();
#endif

// Tensor-core variant of ld_bee_messages_vd_f32 for chan = 128:
//   rows    [Nt][128][16] BF16: per node and channel (l0, l1[3], l2[9], 3 unused), the interleaved form written by
//           ld_linear_bf16_tc_out16
//   S_v [Nt][3][640], S_d [Nt][9][640] BF16: per-node sums of the five rank-1 / rank-2 products, component-major
//           (the input form of ld_linear_bf16_tc_in16), times `scale`
extern "C" int ld_bee_messages_vd_bf16_tc(const int* row_ptr, const int* dst, const float* rij, int Nt, int chan, float r0,
                                          const void* rows, const float* enc_w, const float* enc_b, const float* jacobi,
                                          float scale, void* S_v, void* S_d, int* status_dev, void* stream) {
  if (Nt < 0 || !(r0 > 0.f)) return LD_ERR_SHAPE;
  if (chan != VT_C) {
    ld_set_last_message("l<=2 product sums on the tensor cores: built for chan = 128 (other widths: ld_bee_messages_vd_f32)");
    return LD_ERR_UNSUPPORTED;
  }
  if (((uintptr_t)rows % 32) != 0) return LD_ERR_SHAPE;
  if (Nt == 0) return LD_OK;
  VtParams Q;
  Q.row_ptr = row_ptr; Q.dst = dst; Q.rij = rij; Q.Nt = Nt; Q.r0 = r0; Q.scale = scale;
  Q.rows = (const __nv_bfloat16*)rows; Q.enc_w = enc_w; Q.enc_b = enc_b; Q.jacobi = jacobi;
  {
    const long long seg = (40LL << 20) / (VT_C * 32);   // about 40 MB of gathered rows per segment: they stay in L2
    Q.seg_nodes = ld_even_segments(Nt, seg);
  }
  Q.S_v = (__nv_bfloat16*)S_v; Q.S_d = (__nv_bfloat16*)S_d; Q.status = status_dev;
  Q.wait_limit = tc::TC_WAIT_LIMIT;
#ifdef LD_PHASE_COUNTERS
  Q.prof = ld_internal_phase_counters();
  Q.dbg = getenv("LD_VT_DBG") ? atoi(getenv("LD_VT_DBG")) : 0;
#else
  Q.prof = nullptr;
  Q.dbg = 0;
#endif
  {
    // (D column, left component, monomial, sign) of every non-zero entry of G_e; the three scalar products (columns
    // 0..2 of the table) belong to the scalar kernel and have no row here
    int ent[4 * VT_GAMMA_ENTRIES];
    const int n = ld_bee_gamma_table(ent);
    for (int i = 0; i < VT_GAMMA_ENTRIES; i++) {
      Q.gamma_tab[i] = 0xffffu;
      if (i < n && ent[4 * i] >= 3) {
        const int row = ent[4 * i] - 3, m = ent[4 * i + 1], mono = ent[4 * i + 2], neg = ent[4 * i + 3];
        const int off = (m / 8) * (VT_GAMMA_ROWS * 16) + row * 16 + (m % 8) * 2;
        Q.gamma_tab[i] = (unsigned short)((off >> 1) | (mono << 11) | (neg << 15));
      }
    }
  }
  LD_CUDA_TRY(cudaFuncSetAttribute(bee_vd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, VT_SMEM));
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  bee_vd_tc_kernel<<<sms, VT_THREADS, VT_SMEM, (cudaStream_t)stream>>>(Q);
  LD_LAUNCH_CHECK();
  return LD_OK;
}
