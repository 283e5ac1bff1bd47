// PaiNN message step on the Blackwell tensor cores: the same fused computation as
// painn_message.cu (Message.forward, archs/meanflow_painn8.py:77-100, plus the edge gather and
// edges_reduce_src), with the three layers of the per-edge distance MLP running as tcgen05 MMAs:
// BF16 operands, FP32 accumulation in tensor memory. Tolerance of this path: 2e-2 relative.
//
// A block owns a node-aligned, contiguous slice of the CSR and walks it 128 edges at a time.
// Three roles (warp specialised):
//   * 16 working warps (four per 32-lane quarter of tensor memory, each a quarter of the columns): edge geometry,
//     radial features -> BF16 operand tile A in shared memory;
//     between layers they read the accumulators (tcgen05.ld), add bias, apply SiLU and write the
//     next operand tile over A; after the last layer: accumulator x gathered neighbour activation
//     -> vector/scalar messages, staged in shared memory and summed per source node in edge order.
//     Sums of a node that spans tiles stay in registers; every node is written once (no atomics,
//     fixed summation order).
//   * 1 MMA warp (lane 0): per layer, waits for the operand tile and for each 32 KB weight slab,
//     issues the [128 x 4n x 16] MMAs into 128 lanes x 4n columns of TMEM (descriptors built once per
//     layer, one add per K-step), commits stage release and layer completion to mbarriers.
//   * 1 producer warp (lane 0): streams the pre-packed BF16 weight slabs from L2 with bulk
//     asynchronous copies through a ring of stages; weights do not depend on the data, so it runs
//     ahead across layers and tiles as far as the ring allows.
// Edge-sized data never reaches HBM. Every mbarrier wait is bounded (LD_FLAG_TIMEOUT): a failed
// wait is OR-ed into the next block barrier so that all threads leave together.
#include "common.cuh"
#include "tc05.cuh"
#include "tp_math.h"

namespace {

constexpr int MT_EDGES = 128;          // edges per tile = MMA M
constexpr int MT_WORK_WARPS = 16;      // TMEM lane quarter = warp % 4, column part = warp / 4
constexpr int MT_WORK_THREADS = MT_WORK_WARPS * 32;
constexpr int MT_MMA_WARP = MT_WORK_WARPS;
constexpr int MT_PROD_WARP = MT_WORK_WARPS + 1;
constexpr int MT_THREADS_TC = (MT_WORK_WARPS + 2) * 32;
constexpr int MT_SYNC_THREADS = (MT_WORK_WARPS + 1) * 32;  // working warps + MMA warp meet at barrier 1
constexpr int MT_MAX_STAGES = 4;       // weight ring: slabs of K = 32 (as many as fit, at least 2)
constexpr int MT_SLAB_KSTEPS = 2;      // MMA K-steps (K = 16) per slab: larger copies stream faster from L2
constexpr int MT_CG = 64;              // channels per reduction pass
constexpr int MT_MAX_PASS = 2;         // n <= 128
constexpr size_t MT_STAGING_BYTES = (size_t)MT_EDGES * MT_CG * 4 * 4;  // 128 KB

// diagnostics slots (cycles, summed over blocks): 0 geometry, 1 radial features, 2/4/6 waiting for
// layer 1/2/3 accumulators, 3/5 inter-layer epilogues, 7 per-node sums, 8 message staging,
// 9 MMA lane waiting for weights, 10 producer waiting for a free stage
constexpr int MT_PROF_SLOTS = 12;

struct TcMessageParams {
  const int* row_ptr; const int* dst; const float* rij;
  int Nt, n, n_rbf, k0p, radial_kind;
  unsigned stage_off, bias_off;   // byte offsets of the weight ring and the bias copy in dynamic shared memory
  int nstages;                    // slabs in the weight ring
  int seg_nodes;                  // nodes per scheduling segment (all blocks work on one segment at a time: L2 reuse)
  float rmax, pi_over_rmax, eps;
  const __nv_bfloat16* w1; const __nv_bfloat16* w2; const __nv_bfloat16* w3;  // packed panels [K/8][4n][8]
  const float* b1; const float* b2; const float* b3;
  const float* actv; const float* x_v; const float* res_a; const float* res_v;
  const uint32_t* g16;   // optional packed BF16 gather records [Nt][n/8][64] (see ld_painn_pack_gather); replaces actv / x_v
  float* out_a; float* out_v;
  long long* edge_counter;
  int* status;
  long long* prof;   // optional [16] cycle counters (diagnostics)
};

__device__ __forceinline__ int lb_row(const int* __restrict__ row_ptr, int lo, int hi, long long target) {
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if ((long long)row_ptr[mid] < target) lo = mid + 1; else hi = mid;
  }
  return lo;
}

// first node v in [lo, hi] whose preceding work inside the segment, (edges + nodes) in [lo, v), reaches target
__device__ __forceinline__ int work_lower_bound(const int* __restrict__ row_ptr, int lo, int hi, long long target) {
  const long long base = (long long)row_ptr[lo] + lo;
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if ((long long)row_ptr[mid] + mid - base < target) lo = mid + 1; else hi = mid;
  }
  return lo;
}

struct BlockRange { int n_begin, n_end; long long e_begin, e_end, ntiles; };

// node-aligned share of segment [seg_lo, seg_hi) for this block, balanced over edges + nodes
// (nodes without edges still have to be written)
__device__ __forceinline__ BlockRange block_range(const int* __restrict__ row_ptr, int seg_lo, int seg_hi, int tile) {
  BlockRange r;
  const long long work = ((long long)row_ptr[seg_hi] - row_ptr[seg_lo]) + (seg_hi - seg_lo);
  long long per = (work + gridDim.x - 1) / gridDim.x;
  if (per < tile) per = tile;
  r.n_begin = blockIdx.x == 0 ? seg_lo : work_lower_bound(row_ptr, seg_lo, seg_hi, per * blockIdx.x);
  r.n_end = blockIdx.x == gridDim.x - 1 ? seg_hi : work_lower_bound(row_ptr, seg_lo, seg_hi, per * (blockIdx.x + 1));
  r.e_begin = r.n_begin < r.n_end ? row_ptr[r.n_begin] : 0;
  r.e_end = r.n_begin < r.n_end ? row_ptr[r.n_end] : 0;
  r.ntiles = (r.e_end - r.e_begin + tile - 1) / tile;
  return r;
}

// barrier 1: working warps + MMA warp; returns the OR of `flag` over its participants
__device__ __forceinline__ int sync_or(int flag) {
  int out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "barrier.cta.red.or.pred p, 1, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(out)
      : "r"(flag), "n"(MT_SYNC_THREADS)
      : "memory");
  return out;
}
// barrier 2: working warps only
__device__ __forceinline__ void sync_workers() { asm volatile("barrier.cta.sync 2, %0;" ::"n"(MT_WORK_THREADS) : "memory"); }

// NN: the width n as a compile-time constant (0: taken from the parameters)
template <bool PROF, bool G16, int NN>
__global__ void __launch_bounds__(MT_THREADS_TC, 1)
painn_message_tc_kernel(TcMessageParams P) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t bar_full[MT_MAX_STAGES], bar_empty[MT_MAX_STAGES], bar_accum;
  __shared__ uint32_t tmem_slot;
  __shared__ float s_dir[MT_EDGES][3];
  __shared__ float s_dist[MT_EDGES];
  __shared__ int s_dst[MT_EDGES];
  __shared__ int s_src[MT_EDGES];
  __shared__ int s_rowwin[MT_EDGES + 1];  // row_ptr[node_lo .. node_lo+128] of the coming tile
  __shared__ float s_head[2][MT_CG * 4], s_tail[2][MT_CG * 4];   // partial per-node sums of the two row halves

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool mma_lane = warp == MT_MMA_WARP && lane == 0;
  const bool prod_lane = warp == MT_PROD_WARP && lane == 0;
  const int quarter = warp & 3, part = (warp >> 2) & 3;
  const int row = quarter * 32 + lane;  // edge slot / TMEM lane owned in the epilogues
  const int n = NN > 0 ? NN : P.n, N = 4 * n;
  // dynamic shared memory: [ A operand tile, overlaid by the reduction staging | weight ring | biases ]
  unsigned char* a_smem = smem;                                   // 128 x N BF16
  unsigned char* b_smem = smem + P.stage_off;                     // nstages x slab
  float* s_bias = reinterpret_cast<float*>(smem + P.bias_off);    // 3 x N
  float* stage_f = reinterpret_cast<float*>(smem);                // [128][MT_CG*4]
  const uint32_t slab = (uint32_t)N * 32 * MT_SLAB_KSTEPS;        // bytes of a full weight slab
  const uint32_t nst = (uint32_t)P.nstages;

  for (int i = tid; i < N; i += MT_THREADS_TC) {
    s_bias[i] = P.b1[i]; s_bias[N + i] = P.b2[i]; s_bias[2 * N + i] = P.b3[i];
  }
  if (tid == 0) {
    for (int s = 0; s < MT_MAX_STAGES; s++) { tc::mbar_init(&bar_full[s], 1); tc::mbar_init(&bar_empty[s], 1); }
    tc::mbar_init(&bar_accum, 1);
    tc::mbar_init_fence();
  }
  uint32_t ncols = 32;
  while (ncols < (uint32_t)N) ncols <<= 1;
  if (warp == 0) { tc::tmem_alloc(&tmem_slot, ncols); tc::tmem_relinquish(); }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  const uint32_t tmem_row = tmem_base + ((uint32_t)(quarter * 32) << 16);

  const int seg_nodes = P.seg_nodes > 0 ? P.seg_nodes : P.Nt;
  const int k0steps = P.k0p / 16, ksteps = N / 16;
  const int npass = (n + MT_CG - 1) / MT_CG;
  long long pc[PROF ? MT_PROF_SLOTS : 1];
#pragma unroll
  for (int i = 0; i < (PROF ? MT_PROF_SLOTS : 1); i++) pc[i] = 0;
  int fail = 0;

  if (warp == MT_PROD_WARP) {
    // ===== producer: weight slabs through the ring, independent of the data ==============================
    if (prod_lane) {
      uint32_t loads = 0;
      for (int seg_lo = 0; seg_lo < P.Nt && !fail; seg_lo += seg_nodes) {
      const long long ntiles = block_range(P.row_ptr, seg_lo, min(seg_lo + seg_nodes, P.Nt), MT_EDGES).ntiles;
      for (long long t = 0; t < ntiles && !fail; t++) {
        for (int layer = 0; layer < 3 && !fail; layer++) {
          const __nv_bfloat16* wp = layer == 0 ? P.w1 : (layer == 1 ? P.w2 : P.w3);
          const int steps = layer == 0 ? k0steps : ksteps;
          for (int ks = 0; ks < steps; ks += MT_SLAB_KSTEPS, loads++) {
            const uint32_t st = loads % nst, use = loads / nst;
            const uint32_t bytes = (uint32_t)min(MT_SLAB_KSTEPS, steps - ks) * N * 32;
            const long long t0 = PROF ? clock64() : 0;
            if (use >= 1 && !tc::mbar_wait(&bar_empty[st], (use - 1) & 1)) { fail = 1; break; }  // MMAs that read it are done
            if (PROF) pc[10] += clock64() - t0;
            tc::mbar_expect_tx(&bar_full[st], bytes);
            tc::bulk_g2s(b_smem + (size_t)st * slab, wp + (size_t)ks * N * 16, bytes, &bar_full[st]);
          }
        }
      }
      }
      if (fail) {
        // copies already requested still land in this block's shared memory: give them a bounded chance
        for (uint32_t i = loads > nst ? loads - nst : 0; i < loads; i++)
          tc::mbar_wait(&bar_full[i % nst], (i / nst) & 1);
      }
    }
  } else if (warp == MT_MMA_WARP) {
    // ===== MMA issue ========================================================================================
    uint32_t mmas = 0, accum_phase = 0;
    const uint32_t a_base = tc::smem_u32(a_smem);
    for (int seg_lo = 0; seg_lo < P.Nt && !fail; seg_lo += seg_nodes) {
    const long long ntiles = block_range(P.row_ptr, seg_lo, min(seg_lo + seg_nodes, P.Nt), MT_EDGES).ntiles;
    for (long long t = 0; t < ntiles; t++) {
      if (sync_or(fail)) { fail = 1; break; }      // [B1] geometry staged
      if (sync_or(fail)) { fail = 1; break; }      // [B2] first operand tile ready
      for (int layer = 0; layer < 3; layer++) {
        if (mma_lane && !fail) {
          tc::fence_after_sync();
          // everything that is constant over the layer is computed once: the issuing thread runs alone in its warp,
          // so every instruction between two MMAs is exposed latency
          const int steps = layer == 0 ? k0steps : ksteps;
          uint64_t ad = tc::smem_desc(a_base, MT_EDGES * 16, 128);
          const uint64_t a_step = (uint64_t)((2 * MT_EDGES * 16) >> 4), b_step = (uint64_t)((2 * N * 16) >> 4);
          const int n_lo = min(256, N), n_hi = N - n_lo;                       // N = 4n <= 512: one or two instructions per K-step
          const uint32_t idesc_lo = tc::idesc_bf16(MT_EDGES, n_lo), idesc_hi = tc::idesc_bf16(MT_EDGES, n_hi > 0 ? n_hi : 8);
          const uint64_t b_hi = (uint64_t)((256 * 16) >> 4);
          uint32_t accumulate = 0u;
          for (int ks0 = 0; ks0 < steps; ks0 += MT_SLAB_KSTEPS, mmas++) {
            const uint32_t st = mmas % nst, use = mmas / nst;
            const long long t0 = PROF ? clock64() : 0;
            if (!tc::mbar_wait(&bar_full[st], use & 1)) { fail = 1; break; }
            if (PROF) pc[9] += clock64() - t0;
            tc::fence_after_sync();
            uint64_t bd = tc::smem_desc(tc::smem_u32(b_smem + (size_t)st * slab), N * 16, 128);
            const int nk = min(MT_SLAB_KSTEPS, steps - ks0);
            for (int kk = 0; kk < nk; kk++) {
              tc::mma_bf16(tmem_base, ad, bd, idesc_lo, accumulate);
              if (n_hi > 0) tc::mma_bf16(tmem_base + 256, ad, bd + b_hi, idesc_hi, accumulate);
              accumulate = 1u;
              ad += a_step;   // the address field of a descriptor counts 16-byte units: next K-step = two panels on
              bd += b_step;
            }
            tc::mma_commit(&bar_empty[st]);
          }
          if (!fail) tc::mma_commit(&bar_accum);
          // the issuing lane polls for the completion itself and passes it on through the block barrier below: a
          // hardware barrier wakes the sixteen working warps faster than sixteen suspended mbarrier waits
          if (!fail && !tc::mbar_wait_tight(&bar_accum, accum_phase & 1)) fail = 1;
          tc::fence_before_sync();
        }
        accum_phase++;
        fail = __shfl_sync(0xffffffffu, fail, 0);
        if (sync_or(fail)) { fail = 1; break; }    // [A0..A2] accumulators of this layer complete
        if (sync_or(fail)) { fail = 1; break; }    // [B3..B5] accumulators consumed / next operand tile ready
      }
      if (fail) break;
      if (sync_or(fail)) { fail = 1; break; }      // [B6] tile finished: TMEM and A free again
    }
    }
  } else {
    // ===== working warps =========================================================================================
    // reduction role: column `tid` of the staging tile = (channel tid/4 of the pass, component tid%4)
    const int red_c = (tid >> 2) & (MT_CG - 1), red_k = tid & 3;
    long long tprev = PROF ? clock64() : 0;
    auto lap = [&](int i) {
      if (PROF) { const long long t = clock64(); pc[i] += t - tprev; tprev = t; }
    };
    const bool reducer = tid < MT_CG * 4;  // the staging tile has MT_CG * 4 columns, one per reducing thread

    auto flush_until = [&](int pass, int from, int next, float value) {
      // write node `from` (value), zero-fill (from, next) for this pass's channel
      const int c = pass * MT_CG + red_c;
      if (c >= n || !reducer) return;
      for (int v = from; v < next; v++) {
        float val = (v == from) ? value : 0.f;
        if (red_k < 3) {
          const size_t off = ((size_t)v * n + c) * 3 + red_k;
          if (P.res_v != nullptr) val += P.res_v[off];
          P.out_v[off] = val;
        } else {
          const size_t off = (size_t)v * n + c;
          if (P.res_a != nullptr) val += P.res_a[off];
          P.out_a[off] = val;
        }
      }
    };

    long long edges_done = 0;
    for (int seg_lo = 0; seg_lo < P.Nt && !fail; seg_lo += seg_nodes) {
    const BlockRange br = block_range(P.row_ptr, seg_lo, min(seg_lo + seg_nodes, P.Nt), MT_EDGES);
    const int n_begin = br.n_begin, n_end = br.n_end;
    const long long e_begin = br.e_begin, e_end = br.e_end;
    float acc[MT_MAX_PASS] = {0.f, 0.f};
    int cur = n_begin;
    int node_lo = n_begin;  // source node of the next tile's first edge (or an earlier node)
    sync_workers();         // the previous segment's last readers of s_rowwin are done
    if (tid <= MT_EDGES) s_rowwin[tid] = P.row_ptr[min(node_lo + tid, n_end > n_begin ? n_end : n_begin)];
    sync_workers();
    for (long long e0 = e_begin; e0 < e_end; e0 += MT_EDGES) {
      const int cnt = (int)((e_end - e0) < MT_EDGES ? (e_end - e0) : MT_EDGES);
      // ---- 1. edge geometry ------------------------------------------------------------------------
      if (tid < MT_EDGES) {
        float dx = 0.f, dy = 0.f, dz = 0.f;
        int j = 0, s = -1;
        if (tid < cnt) {
          const long long e = e0 + tid;
          dx = P.rij[e * 3]; dy = P.rij[e * 3 + 1]; dz = P.rij[e * 3 + 2];
          j = P.dst[e];
          // source node: largest v with row_ptr[v] <= e, searched in the staged window first
          if ((long long)s_rowwin[MT_EDGES] > e) {
            int lo = 0, hi = MT_EDGES;  // win[lo] <= e < win[hi]
            while (hi - lo > 1) {
              const int mid = (lo + hi) >> 1;
              if ((long long)s_rowwin[mid] > e) hi = mid; else lo = mid;
            }
            s = node_lo + lo;
          } else {
            s = lb_row(P.row_ptr, node_lo + MT_EDGES, n_end, e + 1) - 1;
          }
        }
        const float r2 = dx * dx + dy * dy + dz * dz;
        const float inv = rsqrtf(P.eps + r2);
        s_dir[tid][0] = dx * inv; s_dir[tid][1] = dy * inv; s_dir[tid][2] = dz * inv;
        s_dist[tid] = sqrtf(r2);
        s_dst[tid] = j;
        s_src[tid] = s;
      }
      if (sync_or(fail)) { fail = 1; break; }                                            // [B1]
      lap(0);
      // ---- 2. radial features -> operand tile ---------------------------------------------------------------
      {
        const int e = tid & (MT_EDGES - 1);
        const float d = s_dist[e];
        // Gaussian basis: envelope once per edge, fast exponentials (the features are rounded to BF16)
        const float width = P.n_rbf > 1 ? P.rmax / (float)(P.n_rbf - 1) : P.rmax;
        const float inv_w = 1.0f / width;
        const float env = d < P.rmax ? 0.5f * (__cosf(P.pi_over_rmax * d) + 1.0f) : 0.f;
        for (int p = tid >> 7; p < P.k0p / 8; p += MT_WORK_THREADS / MT_EDGES) {
          float v[8];
#pragma unroll
          for (int j = 0; j < 8; j++) {
            const int k = p * 8 + j;
            float f = 0.f;
            if (e < cnt && k < P.n_rbf) {
              if (P.radial_kind == 1) {
                const float u = (d - (float)k * width) * inv_w;
                f = __expf(-0.5f * u * u) * env;
              } else {
                f = radial_feature(P.radial_kind, k, P.n_rbf, d, P.rmax, P.pi_over_rmax);
              }
            }
            v[j] = f;
          }
          uint4 q;
          q.x = tc::pack_bf16x2(v[0], v[1]); q.y = tc::pack_bf16x2(v[2], v[3]);
          q.z = tc::pack_bf16x2(v[4], v[5]); q.w = tc::pack_bf16x2(v[6], v[7]);
          *reinterpret_cast<uint4*>(a_smem + (size_t)p * (MT_EDGES * 16) + e * 16) = q;
        }
        tc::fence_async_smem();
      }
      tc::fence_before_sync();
      if (sync_or(fail)) { fail = 1; break; }                                            // [B2]
      lap(1);

      // ---- 3. three layers -------------------------------------------------------------------------------------
      for (int layer = 0; layer < 3; layer++) {
        if (sync_or(fail)) { fail = 1; break; }                                          // [A0..A2] this layer's accumulators are complete
        tc::fence_after_sync();
        lap(2 + 2 * layer);
        if (!fail && layer < 2) {
          // bias + SiLU -> next operand tile (this thread: row `row`, columns of its part)
          const float* bias = s_bias + layer * N;
          const int cpp = ((N / 4 + 31) / 32) * 32;  // columns per part (N is a multiple of 32)
          for (int cb = part * cpp; cb < min((part + 1) * cpp, N); cb += 32) {
            float v[32];
            tc::tmem_ld32(tmem_row + cb, v);
#pragma unroll
            for (int g8 = 0; g8 < 4; g8++) {
              float t[8];
              const float4 ba = *reinterpret_cast<const float4*>(bias + cb + g8 * 8);       // eight biases, two 16-byte loads
              const float4 bb = *reinterpret_cast<const float4*>(bias + cb + g8 * 8 + 4);
              const float b8[8] = {ba.x, ba.y, ba.z, ba.w, bb.x, bb.y, bb.z, bb.w};
#pragma unroll
              for (int j = 0; j < 8; j++) t[j] = tc::silu_fast(v[g8 * 8 + j] + b8[j]);
              uint4 q;
              q.x = tc::pack_bf16x2(t[0], t[1]); q.y = tc::pack_bf16x2(t[2], t[3]);
              q.z = tc::pack_bf16x2(t[4], t[5]); q.w = tc::pack_bf16x2(t[6], t[7]);
              *reinterpret_cast<uint4*>(a_smem + (size_t)((cb >> 3) + g8) * (MT_EDGES * 16) + row * 16) = q;
            }
          }
          tc::fence_async_smem();
          tc::fence_before_sync();
        }
        if (sync_or(fail)) { fail = 1; break; }                                          // [B3], [B4], [B5]
        if (layer < 2) lap(3 + 2 * layer);
      }
      if (fail) break;

      // ---- 4. messages and per-node sums -----------------------------------------------------------------------
      const float* b3 = s_bias + 2 * N;
      const int j_node = s_dst[row];
      const float* Aj = P.actv + (size_t)j_node * N;
      const float* Xj = P.x_v + (size_t)j_node * n * 3;
      const float dir0 = s_dir[row][0], dir1 = s_dir[row][1], dir2 = s_dir[row][2];
      const int tile_cur = cur;
      node_lo = s_src[cnt - 1];
      // stage the row_ptr window of the next tile (read after the barrier that ends this tile)
      if (tid <= MT_EDGES) s_rowwin[tid] = P.row_ptr[min(node_lo + tid, n_end)];
      for (int pass = 0; pass < npass; pass++) {
        // this thread: edge `row`, channels [pass*CG + part*CG/4, +CG/4) in groups of 8
        for (int g8 = 0; g8 < MT_CG / 32; g8++) {
          const int c0 = pass * MT_CG + part * (MT_CG / 4) + g8 * 8;
          if (c0 < n) {  // n is a multiple of 8: a group is entirely valid or entirely not
            // 32-byte loads: every fetched sector is requested exactly once
            float a[32];
            float xv[24];
            if (G16) {
              // one 128-byte BF16 record per (neighbour, 8 channels): actv planes 0..3 (8 values each), x_v (24), 8 unused
              uint32_t raw[32];
              const uint32_t* rec = P.g16 + ((size_t)j_node * (n >> 3) + (c0 >> 3)) * 32;
#pragma unroll
              for (int q = 0; q < 4; q++) tc::ldg_raw8(rec + 8 * q, raw + 8 * q);
#pragma unroll
              for (int i = 0; i < 32; i++) a[i] = tc::bf16_at(raw, i);
#pragma unroll
              for (int i = 0; i < 24; i++) xv[i] = tc::bf16_at(raw + 16, i);
            } else {
#pragma unroll
              for (int k = 0; k < 4; k++) tc::ldg_v8(Aj + k * n + c0, a + 8 * k);
#pragma unroll
              for (int q8 = 0; q8 < 3; q8++) tc::ldg_v8(Xj + (size_t)c0 * 3 + 8 * q8, xv + 8 * q8);
            }
            // p_k = (D_k + b3_k) * actv_k in place, one 8-column read of tensor memory per k (keeps registers low)
#pragma unroll
            for (int k = 0; k < 4; k++) {
              float d8[8];
              tc::tmem_ld8(tmem_row + c0 + k * n, d8);
              const float4 ba = *reinterpret_cast<const float4*>(b3 + k * n + c0);
              const float4 bb = *reinterpret_cast<const float4*>(b3 + k * n + c0 + 4);
              const float b8[8] = {ba.x, ba.y, ba.z, ba.w, bb.x, bb.y, bb.z, bb.w};
#pragma unroll
              for (int j = 0; j < 8; j++) a[k * 8 + j] *= d8[j] + b8[j];
            }
#pragma unroll
            for (int j = 0; j < 8; j++) {
              const int c = c0 + j;
              const float p0 = a[j], p1 = a[8 + j], p2 = a[16 + j], p3 = a[24 + j];
              const float x0 = xv[3 * j], x1 = xv[3 * j + 1], x2 = xv[3 * j + 2];
              float4 m;
              m.x = x0 * p0 + (x1 * dir2 - x2 * dir1) * p1 + dir0 * p2;
              m.y = x1 * p0 + (x2 * dir0 - x0 * dir2) * p1 + dir1 * p2;
              m.z = x2 * p0 + (x0 * dir1 - x1 * dir0) * p1 + dir2 * p2;
              m.w = p3;
              if (row >= cnt) m = make_float4(0.f, 0.f, 0.f, 0.f);
              // staging row `row`, 16-byte slot (channel within pass) xor-swizzled by row within groups of 8
              const int slot = (c - pass * MT_CG);
              const int sw = (slot & ~7) | ((slot ^ row) & 7);
              *reinterpret_cast<float4*>(stage_f + (size_t)row * (MT_CG * 4) + sw * 4) = m;
            }
          }
        }
        sync_workers();
        lap(8);
        // Sum per source node in edge order, in two steps. (a) Thread (column, row half) adds up its 64 rows: the sum
        // for the half's first node goes to s_head, for its last node (when different) to s_tail, nodes strictly
        // inside the half are complete and written at once. (b) One thread per column joins the two halves with the
        // sum carried over from earlier tiles. Column = (channel, component); every addition is in a fixed order.
        {
          const int col = tid & (MT_CG * 4 - 1), rh = tid / (MT_CG * 4);   // 256 columns x 2 row halves
          const int r_lo = rh * (MT_EDGES / 2), r_hi = min(r_lo + MT_EDGES / 2, cnt);
          const int c_chan = pass * MT_CG + ((col >> 2) & (MT_CG - 1)), c_k = col & 3;
          if (rh < 2 && r_lo < cnt && c_chan < n) {
            const int slot = (col >> 2) & (MT_CG - 1);
            auto write_node = [&](int v, float val) {
              if (c_k < 3) {
                const size_t off = ((size_t)v * n + c_chan) * 3 + c_k;
                P.out_v[off] = P.res_v != nullptr ? val + P.res_v[off] : val;
              } else {
                const size_t off = (size_t)v * n + c_chan;
                P.out_a[off] = P.res_a != nullptr ? val + P.res_a[off] : val;
              }
            };
            int c_node = s_src[r_lo];
            float sum = 0.f, head = 0.f;
            bool first = true;
            // row e keeps this column at slot (slot & ~7) | ((slot ^ e) & 7); eb is a multiple of 8, so within a group
            // of eight rows the offsets are loop-invariant
            const float* sp = stage_f + (size_t)r_lo * (MT_CG * 4) + (slot & ~7) * 4 + c_k;
            const int sx = slot & 7;
            for (int eb = r_lo; eb < r_hi; eb += 8, sp += 8 * (MT_CG * 4)) {
              float v[8];
#pragma unroll
              for (int i = 0; i < 8; i++) v[i] = sp[i * (MT_CG * 4) + ((sx ^ i) << 2)];   // rows beyond cnt hold zeros
              const int last = min(eb + 7, r_hi - 1);
              if (s_src[eb] == c_node && s_src[last] == c_node) {
                sum += ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
              } else {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                  if (eb + i < r_hi) {
                    const int s = s_src[eb + i];
                    if (s != c_node) {
                      if (first) { head = sum; first = false; }
                      else write_node(c_node, sum);
                      for (int z = c_node + 1; z < s; z++) write_node(z, 0.f);   // nodes without edges
                      sum = 0.f;
                      c_node = s;
                    }
                    sum += v[i];
                  }
                }
              }
            }
            s_head[rh][col] = first ? sum : head;
            s_tail[rh][col] = first ? 0.f : sum;
          }
        }
        sync_workers();
        lap(11);
        if (reducer) {
          int c_node = tile_cur;
          float a_sum = acc[pass];
          const bool live = pass * MT_CG + red_c < n;
          for (int q = 0; q < 2 && q * (MT_EDGES / 2) < cnt; q++) {
            const int f = s_src[q * (MT_EDGES / 2)], l = s_src[min(q * (MT_EDGES / 2) + MT_EDGES / 2 - 1, cnt - 1)];
            if (f != c_node) { flush_until(pass, c_node, f, a_sum); a_sum = 0.f; c_node = f; }
            if (live) a_sum += s_head[q][tid];
            if (l != f) {
              flush_until(pass, f, f + 1, a_sum);   // node f alone: the gaps after it were filled by the half's thread
              a_sum = live ? s_tail[q][tid] : 0.f;
              c_node = l;
            }
          }
          acc[pass] = a_sum;
          if (pass == npass - 1) cur = c_node;
        }
        if (pass + 1 < npass) sync_workers();  // staging is rewritten by the next pass
        lap(7);
      }
      tc::fence_before_sync();
      if (sync_or(fail)) { fail = 1; break; }                                            // [B6]
    }
    if (!fail && n_begin < n_end) {
      for (int pass = 0; pass < npass; pass++) flush_until(pass, cur, n_end, acc[pass]);
      edges_done += e_end - e_begin;
    }
    }
    if (!fail && P.edge_counter != nullptr && tid == 0 && edges_done > 0)
      atomicAdd((unsigned long long*)P.edge_counter, (unsigned long long)edges_done);
  }
  if (PROF && P.prof != nullptr && (tid == 0 || mma_lane || prod_lane)) {
    for (int i = 0; i < MT_PROF_SLOTS; i++)
      if (pc[i]) atomicAdd((unsigned long long*)&P.prof[i], (unsigned long long)pc[i]);
  }
  if (fail && lane == 0 && P.status != nullptr) atomicOr(P.status, LD_FLAG_TIMEOUT);
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem_base, ncols);
}

// actv [Nt][4n] and x_v [Nt][n][3] (FP32) -> BF16 records [Nt][n/8][64]: for 8 consecutive channels c0..c0+7 the four
// actv planes (8 values each, plane k = columns k*n + c), the 24 vector components, 8 unused values. 128 bytes, so a
// fused-message thread fetches everything it needs of a neighbour with four 32-byte loads.
__global__ void painn_pack_gather_kernel(const float* __restrict__ actv, const float* __restrict__ x_v, long long groups,
                                         int n, uint4* __restrict__ out) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= groups) return;
  const int gpn = n >> 3;
  const long long node = idx / gpn;
  const int c0 = (int)(idx % gpn) * 8;
  float v[64];
#pragma unroll
  for (int k = 0; k < 4; k++) tc::ldg_v8(actv + node * 4 * n + k * n + c0, v + 8 * k);
#pragma unroll
  for (int q = 0; q < 3; q++) tc::ldg_v8(x_v + (node * n + c0) * 3 + 8 * q, v + 32 + 8 * q);
#pragma unroll
  for (int i = 56; i < 64; i++) v[i] = 0.f;
#pragma unroll
  for (int q = 0; q < 8; q++) {
    uint4 w;
    w.x = tc::pack_bf16x2(v[8 * q], v[8 * q + 1]); w.y = tc::pack_bf16x2(v[8 * q + 2], v[8 * q + 3]);
    w.z = tc::pack_bf16x2(v[8 * q + 4], v[8 * q + 5]); w.w = tc::pack_bf16x2(v[8 * q + 6], v[8 * q + 7]);
    out[idx * 8 + q] = w;
  }
}

#ifdef LD_PHASE_COUNTERS
long long* g_prof_buffer = nullptr;
#endif

}  // namespace

#ifdef LD_PHASE_COUNTERS
// Diagnostics build only (-DLD_PHASE_COUNTERS; not part of the library's interface): device buffer of 16 int64 that
// later launches of the fused tensor-core kernels add per-phase cycle counts to; NULL switches it off. Process-wide
// and not thread safe, which is why the regular build has neither this switch nor the counting kernel instances.
extern "C" int ld_debug_set_phase_counters(long long* device_buffer16) { g_prof_buffer = device_buffer16; return LD_OK; }
long long* ld_internal_phase_counters() { return g_prof_buffer; }
#endif

extern "C" int ld_painn_pack_gather(const float* actv, const float* x_v, int Nt, int n, void* out_bf16, void* stream) {
  if (Nt < 0 || n <= 0 || n % 8 != 0) return LD_ERR_SHAPE;
  if ((((uintptr_t)actv | (uintptr_t)x_v | (uintptr_t)out_bf16) % 32) != 0) return LD_ERR_SHAPE;
  const long long groups = (long long)Nt * (n / 8);
  if (groups == 0) return LD_OK;
  painn_pack_gather_kernel<<<(unsigned)((groups + 127) / 128), 128, 0, (cudaStream_t)stream>>>(actv, x_v, groups, n, (uint4*)out_bf16);
  LD_LAUNCH_CHECK();
  return LD_OK;
}

// Tensor-core variant of ld_painn_message_f32 (same graph / feature arguments). w1p/w2p/w3p are the
// distance-MLP weights packed by ld_pack_weights_bf16 ([4n][n_rbf], [4n][4n], [4n][4n]); biases FP32.
// n a multiple of 8, n <= 128. status_dev receives LD_FLAG_TIMEOUT if a bounded wait ran out.
// gather16 (optional): the node features as BF16 records written by ld_painn_pack_gather; the kernel then reads
// 2 KB per neighbour (n = 128) instead of 3.5 KB and actv / x_v are not touched.
extern "C" int ld_painn_message_bf16_tc(const int* row_ptr, const int* dst, const float* rij, int Nt, int n, int n_rbf,
                                        int radial_kind, float rmax, float eps, const void* w1p, const float* b1,
                                        const void* w2p, const float* b2, const void* w3p, const float* b3,
                                        const float* actv, const float* x_v, const void* gather16, const float* res_a,
                                        const float* res_v, float* out_a, float* out_v, long long* edge_counter,
                                        int* status_dev, void* stream) {
  if (Nt < 0 || n <= 0 || n_rbf <= 0) return LD_ERR_SHAPE;
  if (n % 8 != 0 || n > 128) { ld_set_last_message("painn message (tensor-core path): n must be a multiple of 8, at most 128"); return LD_ERR_UNSUPPORTED; }
  if (b1 == nullptr || b2 == nullptr || b3 == nullptr) { ld_set_last_message("painn message: biases are required"); return LD_ERR_SHAPE; }
  if (gather16 == nullptr && (actv == nullptr || x_v == nullptr)) {
    ld_set_last_message("painn message (tensor-core path): pass either actv and x_v or the packed gather records");
    return LD_ERR_SHAPE;
  }
  if ((((uintptr_t)w1p | (uintptr_t)w2p | (uintptr_t)w3p) % 16) != 0 ||
      (((uintptr_t)actv | (uintptr_t)x_v | (uintptr_t)gather16) % 32) != 0) {
    ld_set_last_message("painn message (tensor-core path): packed weights must be 16-byte, node features 32-byte aligned");
    return LD_ERR_SHAPE;
  }
  if (Nt == 0) return LD_OK;
  TcMessageParams P;
  P.row_ptr = row_ptr; P.dst = dst; P.rij = rij; P.Nt = Nt; P.n = n; P.n_rbf = n_rbf; P.k0p = (n_rbf + 15) / 16 * 16;
  P.radial_kind = radial_kind; P.rmax = rmax; P.pi_over_rmax = (float)(3.14159265358979323846 / (double)rmax); P.eps = eps;
  P.w1 = (const __nv_bfloat16*)w1p; P.w2 = (const __nv_bfloat16*)w2p; P.w3 = (const __nv_bfloat16*)w3p;
  P.b1 = b1; P.b2 = b2; P.b3 = b3; P.actv = actv; P.x_v = x_v; P.g16 = (const uint32_t*)gather16; P.res_a = res_a; P.res_v = res_v;
  P.out_a = out_a; P.out_v = out_v; P.edge_counter = edge_counter; P.status = status_dev;
#ifdef LD_PHASE_COUNTERS
  P.prof = g_prof_buffer;
#else
  P.prof = nullptr;
#endif
  const int N = 4 * n;
  if (P.k0p > N) { ld_set_last_message("painn message (tensor-core path): n_rbf above 4n is not supported"); return LD_ERR_UNSUPPORTED; }
  // the staging tile overlays only the operand tile, never the weight ring (the producer runs ahead)
  const size_t a_bytes = (size_t)MT_EDGES * N * 2;
  const size_t front = a_bytes > MT_STAGING_BYTES ? a_bytes : MT_STAGING_BYTES;
  const size_t slab = (size_t)N * 32 * MT_SLAB_KSTEPS;
  const size_t fixed = front + (size_t)3 * N * 4 + 1024 + 6 * 1024;  // + static shared memory of the kernel
  int nstages = (int)((227 * 1024 - fixed) / slab);
  if (nstages > MT_MAX_STAGES) nstages = MT_MAX_STAGES;
  if (nstages < 2) return LD_ERR_UNSUPPORTED;
  const size_t ring = (size_t)nstages * slab;
  P.nstages = nstages;
  // all blocks walk the node range segment by segment so that the gathered rows of a segment
  // (28n bytes per node) stay resident in L2 while its edges are processed
  {
    const long long seg = (40LL << 20) / (28LL * n);
    P.seg_nodes = ld_even_segments(Nt, seg);
  }
  P.stage_off = (unsigned)front;
  P.bias_off = (unsigned)(front + ring);
  const size_t smem = front + ring + (size_t)3 * N * 4 + 1024;
#ifdef LD_PHASE_COUNTERS
  auto kern = gather16 != nullptr ? (P.prof != nullptr ? painn_message_tc_kernel<true, true, 0> : (n == 128 ? painn_message_tc_kernel<false, true, 128> : painn_message_tc_kernel<false, true, 0>))
                                  : (P.prof != nullptr ? painn_message_tc_kernel<true, false, 0> : painn_message_tc_kernel<false, false, 0>);
#else
  auto kern = gather16 != nullptr ? (n == 128 ? painn_message_tc_kernel<false, true, 128> : painn_message_tc_kernel<false, true, 0>)
                                  : painn_message_tc_kernel<false, false, 0>;
#endif
  LD_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  kern<<<sms, MT_THREADS_TC, smem, (cudaStream_t)stream>>>(P);
  LD_LAUNCH_CHECK();
  return LD_OK;
}
