// Scalar channel of the l<=2 ("Bee") message layer on the Blackwell tensor cores: the per-edge
// work of Messages.forward (archs/diffuser_atoms15.py:227-253) that cannot be hoisted to nodes,
//   psi_e = [y_000 | y_110 | y_220] Y^T ;  out_e = psi_e + lin_direct(psi_e) + layers(psi_e)
//   B_a[i] = scale * sum_{e: src_e = i} out_e
// as four tcgen05 GEMMs per 128-edge tile (BF16 operands, FP32 accumulation in tensor memory;
// 2e-2 relative). Same block structure as the fused PaiNN kernel (painn_message_tc.cu): 16 working
// warps build the operand tile and run the epilogues, one warp issues MMAs, one warp streams
// weight slabs from L2 with bulk copies; node-aligned CSR slices, one write per node, no atomics.
//
// Operand tile A (K-major panels, 128 rows): columns [0, 3*chan) hold the products for the Y
// map; afterwards columns [0, 2a) hold the hidden activations and [2a, 3a) keep psi, so that the
// last layer is ONE GEMM over K = 3a with weights [W3 | W_direct + I]: the residual and the direct
// term ride on the tensor cores.
#include "common.cuh"
#include "tc05.cuh"
#include "tp_math.h"

#ifdef LD_PHASE_COUNTERS
long long* ld_internal_phase_counters();  // diagnostics build only: buffer set by ld_debug_set_phase_counters
#endif

namespace {

constexpr int BT_EDGES = 128;
constexpr int BT_WORK_WARPS = 16;     // four warps per 32-lane quarter of tensor memory; each takes a quarter of the columns
constexpr int BT_WORK_THREADS = BT_WORK_WARPS * 32;
constexpr int BT_MMA_WARP = BT_WORK_WARPS;
constexpr int BT_PROD_WARP = BT_WORK_WARPS + 1;
constexpr int BT_THREADS = (BT_WORK_WARPS + 2) * 32;
constexpr int BT_SYNC_THREADS = (BT_WORK_WARPS + 1) * 32;
// weight ring: two slabs of 48 KB. Every slab costs the issuing thread and the producer a few hundred cycles whatever its
// size, so few large slabs beat many small ones at the same 96 KB in flight: per 21.5M-edge launch 23.0 ms with 2 x 48 KB,
// 23.5 with 3 x 32, 24.9 with 4 x 24, 26.4 with 6 x 16, 32.3 with 12 x 8
constexpr int BT_STAGES = 2;
constexpr int BT_SLAB_BYTES = 48 * 1024;
constexpr int BT_LAYERS = 4;
constexpr uint32_t BT_WRES_COL = 384;   // tensor-memory columns [384, 512): resident weights of the transposed last layer
// Byte stride between the 8-column panels of the operand tile: 128 rows x 16 bytes plus one 16-byte pad, so that the
// panels a warp of the product phase writes to (32 channels = 4 panels, same row) fall into different banks
constexpr int BT_PANEL = BT_EDGES * 16 + 16;

struct BtLayer {
  const __nv_bfloat16* w;   // packed panels [K/8][N][8]
  const float* bias;        // may be null
  int a_panel;              // first 8-column panel of A this layer reads
  int ksteps;               // K / 16
  int slab_ksteps;          // K-steps per weight slab: BT_SLAB_BYTES / (N * 32 B)
  int N;                    // output width (multiple of 64, <= 256)
  int act;                  // 0 none, 2 LeakyReLU(0.1)
  int out_col;              // A column where the epilogue writes its BF16 result (-1: last layer)
  int ks_resident;          // leading K-steps whose weights stay in tensor memory for the whole kernel (transposed last layer)
};

struct BtParams {
  const int* row_ptr; const int* dst; const float* rij;
  int Nt, chan, dim_a;
  float r0, scale;
  const float* L0; const float* L1; const float* L2;
  const float* enc_w; const float* enc_b; const float* jacobi;
  BtLayer layer[BT_LAYERS];
  unsigned stage_off, bias_off, slab_bytes;
  int seg_nodes;
  int feat_bf16;            // 0: L0/L1/L2 FP32; 1: BF16; 2: L0 = interleaved BF16 [node][chan][16]
  float* out_a;
  int* status;
  long long* prof;          // optional cycle counters, 3 x 12: 0 geometry, 11 products, 1 barrier after them, 2/4/6/8 waiting for layers, 3/5/7 epilogues, 9 staging, 10 sums
};

struct __align__(16) BtGeom { float enc[8]; float rhat[3]; float pad; };   // 48 bytes: three 16-byte shared-memory loads

__device__ __forceinline__ int bt_lb_row(const int* __restrict__ row_ptr, int lo, int hi, long long target) {
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if ((long long)row_ptr[mid] < target) lo = mid + 1; else hi = mid;
  }
  return lo;
}

__device__ __forceinline__ int bt_work_lb(const int* __restrict__ row_ptr, int lo, int hi, long long target) {
  const long long base = (long long)row_ptr[lo] + lo;
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if ((long long)row_ptr[mid] + mid - base < target) lo = mid + 1; else hi = mid;
  }
  return lo;
}

struct BtRange { int n_begin, n_end; long long e_begin, e_end, ntiles; };

__device__ __forceinline__ BtRange bt_block_range(const int* __restrict__ row_ptr, int seg_lo, int seg_hi) {
  BtRange r;
  const long long work = ((long long)row_ptr[seg_hi] - row_ptr[seg_lo]) + (seg_hi - seg_lo);
  long long per = (work + gridDim.x - 1) / gridDim.x;
  if (per < BT_EDGES) per = BT_EDGES;
  r.n_begin = blockIdx.x == 0 ? seg_lo : bt_work_lb(row_ptr, seg_lo, seg_hi, per * blockIdx.x);
  r.n_end = blockIdx.x == gridDim.x - 1 ? seg_hi : bt_work_lb(row_ptr, seg_lo, seg_hi, per * (blockIdx.x + 1));
  r.e_begin = r.n_begin < r.n_end ? row_ptr[r.n_begin] : 0;
  r.e_end = r.n_begin < r.n_end ? row_ptr[r.n_end] : 0;
  r.ntiles = (r.e_end - r.e_begin + BT_EDGES - 1) / BT_EDGES;
  return r;
}

__device__ __forceinline__ int bt_sync_or(int flag) {
  int out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "barrier.cta.red.or.pred p, 1, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(out)
      : "r"(flag), "n"(BT_SYNC_THREADS)
      : "memory");
  return out;
}
__device__ __forceinline__ void bt_sync_workers() { asm volatile("barrier.cta.sync 2, %0;" ::"n"(BT_WORK_THREADS) : "memory"); }

__device__ __forceinline__ void bt_geometry(float x, float y, float z, float r0, const float* jac, BtGeom* g) {
  const float d = sqrtf(x * x + y * y + z * z);
  const float zz = d / r0;
  const float env = fmaxf(1.f - zz, 0.f);
  ld_radial_cheb8(zz, env, jac, g->enc);
  const float s = 7.f / r0;
  const float ux = x * s, uy = y * s, uz = z * s;
  const float inv = rsqrtf(1.f + ux * ux + uy * uy + uz * uz);
  g->rhat[0] = ux * inv; g->rhat[1] = uy * inv; g->rhat[2] = uz * inv;
  g->pad = 1.f;   // weight of the edge; the unused slots of a ragged last tile carry 0
}

__device__ __forceinline__ unsigned short bt_bf16(float v) {
  __nv_bfloat16 h = __float2bfloat16_rn(v);
  return *reinterpret_cast<unsigned short*>(&h);
}

// FAST: the instance for chan = dim_a = 128 with interleaved BF16 rows (widths and row format are compile-time constants)
template <bool PROF, bool FAST>
__global__ void __launch_bounds__(BT_THREADS, 1)
bee_scalar_tc_kernel(BtParams P) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t bar_full[BT_STAGES], bar_empty[BT_STAGES], bar_accum;
  __shared__ uint32_t tmem_slot;
  __shared__ BtGeom s_geom[2][BT_EDGES];          // two tiles: the overlapped schedule fills one while the other is read
  __shared__ int s_dst[2][BT_EDGES];
  __shared__ __align__(16) int s_src[2][BT_EDGES];
  __shared__ int s_rowwin[BT_EDGES + 1];
  __shared__ float s_jac[72];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool mma_lane = warp == BT_MMA_WARP && lane == 0;
  const bool prod_lane = warp == BT_PROD_WARP && lane == 0;
  const int quarter = warp & 3, part = (warp >> 2) & 3;  // TMEM lane quarter (fixed by the warp id), column part
  const int row = quarter * 32 + lane;
  const int C = FAST ? 128 : P.chan, A = FAST ? 128 : P.dim_a;
  const int feat = FAST ? 2 : P.feat_bf16;
  unsigned char* a_smem = smem;                                   // 128 x max(3C, 3A) BF16, overlaid by the staging tile
  unsigned char* b_smem = smem + P.stage_off;                     // BT_STAGES x slab
  float* s_bias = reinterpret_cast<float*>(smem + P.bias_off);    // biases of layers 1..3: [2A | 2A | A]
  float* stage_f = reinterpret_cast<float*>(smem);                // [128][A] FP32
  const uint32_t slab = P.slab_bytes;

  if (tid < 8) ld_poly8_to_chebyshev(P.jacobi + tid * 9, s_jac + tid * 9);   // Chebyshev form of the radial polynomials
  for (int i = tid; i < 2 * A; i += BT_THREADS) { s_bias[i] = P.layer[1].bias[i]; s_bias[2 * A + i] = P.layer[2].bias[i]; }
  for (int i = tid; i < A; i += BT_THREADS) s_bias[4 * A + i] = P.layer[3].bias[i];
  if (tid == 0) {
    for (int s = 0; s < BT_STAGES; s++) { tc::mbar_init(&bar_full[s], 1); tc::mbar_init(&bar_empty[s], 1); }
    tc::mbar_init(&bar_accum, 1);
    tc::mbar_init_fence();
  }
  uint32_t ncols = 32;
  while (ncols < (uint32_t)(A == 128 ? 512 : 2 * A)) ncols <<= 1;   // dim_a = 128 keeps the last layer's result in columns [256, 384)
  if (warp == 0) { tc::tmem_alloc(&tmem_slot, ncols); tc::tmem_relinquish(); }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  const uint32_t tmem_row = tmem_base + ((uint32_t)(quarter * 32) << 16);
  const int seg_nodes = P.seg_nodes > 0 ? P.seg_nodes : P.Nt;
  int fail = 0;
  if (P.layer[BT_LAYERS - 1].ks_resident > 0 && tid < 128) {
    // Weights of the last layer that multiply the second hidden layer (K = 2a of its 3a), once per kernel into tensor
    // memory: lane = output channel, eight columns per K-step (sixteen BF16 values, two per column). The last layer is
    // issued with the weights as the M operand, so these K-steps take their A operand from here and only the K = a
    // of the direct term streams through the ring: 329 KB instead of 393 KB of weights per tile, one slab fewer to wait for.
    const BtLayer& L = P.layer[BT_LAYERS - 1];
    const uint4* wp = reinterpret_cast<const uint4*>(L.w);
    for (int ks = 0; ks < L.ks_resident; ks++) {
      const uint4 c0 = __ldg(wp + (size_t)(2 * ks) * L.N + tid), c1 = __ldg(wp + (size_t)(2 * ks + 1) * L.N + tid);
      const uint32_t r[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
      tc::tmem_st8(tmem_row + BT_WRES_COL + (uint32_t)ks * 8u, r);
    }
    tc::tmem_st_wait();
    tc::fence_before_sync();
  }
  __syncthreads();
  tc::fence_after_sync();

  if (warp == BT_PROD_WARP) {
    // ===== producer: weight slabs through the ring =========================================================
    if (prod_lane) {
      uint32_t loads = 0;
      for (int seg_lo = 0; seg_lo < P.Nt && !fail; seg_lo += seg_nodes) {
        const long long ntiles = bt_block_range(P.row_ptr, seg_lo, min(seg_lo + seg_nodes, P.Nt)).ntiles;
        for (long long t = 0; t < ntiles && !fail; t++) {
          for (int l = 0; l < BT_LAYERS && !fail; l++) {
            const BtLayer& L = P.layer[l];
            for (int ks = L.ks_resident; ks < L.ksteps; ks += L.slab_ksteps, loads++) {
              const uint32_t st = loads % BT_STAGES, use = loads / BT_STAGES;
              const uint32_t bytes = (uint32_t)min(L.slab_ksteps, L.ksteps - ks) * L.N * 32;
              if (use >= 1 && !tc::mbar_wait(&bar_empty[st], (use - 1) & 1)) { fail = 1; break; }
              tc::mbar_expect_tx(&bar_full[st], bytes);
              tc::bulk_g2s(b_smem + (size_t)st * slab, L.w + (size_t)ks * L.N * 16, bytes, &bar_full[st]);
            }
          }
        }
      }
      if (fail) {
        for (uint32_t i = loads > BT_STAGES ? loads - BT_STAGES : 0; i < loads; i++)
          tc::mbar_wait(&bar_full[i % BT_STAGES], (i / BT_STAGES) & 1);
      }
    }
  } else if (warp == BT_MMA_WARP) {
    // ===== MMA issue =========================================================================================
    uint32_t mmas = 0, accum_phase = 0;
    const uint32_t a_base = tc::smem_u32(a_smem);
    const bool OV = FAST || A == 128;   // overlapped schedule of the working warps: barriers B1, B6 and B7 fall away
    for (int seg_lo = 0; seg_lo < P.Nt && !fail; seg_lo += seg_nodes) {
      const long long ntiles = bt_block_range(P.row_ptr, seg_lo, min(seg_lo + seg_nodes, P.Nt)).ntiles;
      bool stop = false;   // a barrier reported a failure: every warp leaves at that barrier
      for (long long t = 0; t < ntiles; t++) {
        if (!OV && bt_sync_or(fail)) { fail = 1; stop = true; break; }      // [B1] geometry staged
        if (bt_sync_or(fail)) { fail = 1; stop = true; break; }             // [B2] product tile ready
        for (int l = 0; l < BT_LAYERS; l++) {
          if (mma_lane && !fail) {
            tc::fence_after_sync();
            // everything that is constant over the layer is computed once: the issuing thread runs alone in its warp,
            // so every instruction between two MMAs is exposed latency
            const int l_ksteps = P.layer[l].ksteps, l_slab = P.layer[l].slab_ksteps, l_N = P.layer[l].N;
            // dim_a = 128: the last layer is issued transposed (weights as the M operand, the tile as the N operand), so its
            // result lies in tensor memory as [channel][edge] and the per-node sum is a walk along columns in one thread.
            // It goes to columns [256, 384), which stay untouched while the next tile's first layers run.
            const bool transposed = l == BT_LAYERS - 1 && OV;
            const uint32_t d_tmem = tmem_base + (transposed ? 256u : 0u);
            const uint32_t idesc = transposed ? tc::idesc_bf16(l_N, BT_EDGES) : tc::idesc_bf16(BT_EDGES, l_N);
            uint64_t ad = tc::smem_desc(a_base + P.layer[l].a_panel * BT_PANEL, BT_PANEL, 128);
            const uint64_t a_step = (uint64_t)((2 * BT_PANEL) >> 4), b_step = (uint64_t)((2 * l_N * 16) >> 4);
            uint32_t accumulate = 0u;
            const int l_res = P.layer[l].ks_resident;
            // the part of the last layer's weights that lives in tensor memory (columns [384, 512), A operand of the
            // transposed product) needs no slab: its MMAs go first, while the one streamed slab is on its way
            for (int kk = 0; kk < l_res; kk++) {
              tc::mma_bf16_ta(d_tmem, tmem_base + BT_WRES_COL + (uint32_t)kk * 8u, ad, idesc, accumulate);
              accumulate = 1u;
              ad += a_step;
            }
            for (int ks0 = l_res; ks0 < l_ksteps; ks0 += l_slab, mmas++) {
              const uint32_t st = mmas % BT_STAGES, use = mmas / BT_STAGES;
              if (!tc::mbar_wait(&bar_full[st], use & 1)) { fail = 1; break; }
              tc::fence_after_sync();
              uint64_t bd = tc::smem_desc(tc::smem_u32(b_smem + (size_t)st * slab), l_N * 16, 128);
              const int nk = min(l_slab, l_ksteps - ks0);
#pragma unroll 4
              for (int kk = 0; kk < nk; kk++) {
                if (transposed) tc::mma_bf16(d_tmem, bd, ad, idesc, accumulate);
                else tc::mma_bf16(d_tmem, ad, bd, idesc, accumulate);
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
          if (bt_sync_or(fail)) { fail = 1; stop = true; break; }    // [A0..A3] accumulators of layer l complete
          if (OV && l == BT_LAYERS - 1) break;          // the next barrier is B2 of the following tile (or the segment's end)
          if (bt_sync_or(fail)) { fail = 1; stop = true; break; }    // [B3..B6] accumulators consumed / next operand ready
        }
        if (stop) break;
        if (!OV && bt_sync_or(fail)) { fail = 1; stop = true; break; }      // [B7] tile finished
      }
      if (!stop && bt_sync_or(fail)) fail = 1;                              // [B8] segment finished
    }
  } else {
    // ===== working warps =========================================================================================
    // dim_a = 128 runs the overlapped schedule: the geometry of the next tile is computed by warps 4..7 while the
    // first GEMM of this tile runs, and the per-node sums of a tile (warps 0..3, reading tensor-memory columns
    // [256, 384)) run while the other warps already form the products of the next tile.
    const bool OV = FAST || A == 128;
    long long pc[PROF ? 12 : 1];
#pragma unroll
    for (int i = 0; i < (PROF ? 12 : 1); i++) pc[i] = 0;
    long long tprev = PROF ? clock64() : 0;
    unsigned long long t_block0 = 0, tiles_done = 0;
    if (PROF) asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t_block0));
    auto lap = [&](int i) {
      if (PROF) { const long long t = clock64(); pc[i] += t - tprev; tprev = t; }
    };
    auto flush_until = [&](int from, int next, float value) {
      if (tid < A)
        for (int v = from; v < next; v++) P.out_a[(size_t)v * A + tid] = (v == from ? value : 0.f) * P.scale;
    };
    // product role: channel c; the lanes of a warp share the edge, so loads stay coalesced. The edges of a tile are
    // taken in batches of UNR: edge(b, u) = pb_base + b * pb_step + u * pu_step for b in [pb_lo, pb_hi)
    constexpr int UNR = 4;  // neighbour rows in flight per thread (the loop is bound by L2 latency otherwise)
    const int pc_c = tid % C, pc_h = tid / C, pc_stride = BT_WORK_THREADS / C;
    int pb_base = pc_h, pb_step = pc_stride * UNR, pu_step = pc_stride, pb_lo = 0,
        pb_hi = pc_h < pc_stride ? (BT_EDGES - pc_h + pc_stride * UNR - 1) / (pc_stride * UNR) : 0;
    if (OV && C == 128) {
      // the warps that add up the previous tile first (pc_h = 0) take 5 of the 32 batches, the others 9 each
      pb_base = 0; pb_step = UNR; pu_step = 1;
      pb_lo = pc_h == 0 ? 0 : 5 + 9 * (pc_h - 1);
      pb_hi = 5 + 9 * pc_h;
    }
    // this thread's three columns of the operand tile (element offsets within a row's panels)
    const int a_off0 = (pc_c >> 3) * (BT_PANEL / 2) + (pc_c & 7), a_off1 = ((C + pc_c) >> 3) * (BT_PANEL / 2) + (pc_c & 7),
              a_off2 = ((2 * C + pc_c) >> 3) * (BT_PANEL / 2) + (pc_c & 7);
    float w8[8], wb = 0.f;
    if (pc_h < pc_stride) {
#pragma unroll
      for (int m = 0; m < 8; m++) w8[m] = P.enc_w[pc_c * 8 + m];
      wb = P.enc_b[pc_c];
    }
    const int gt = OV ? tid - BT_EDGES : tid;   // geometry role: thread gt in [0, 128) owns edge gt of a tile
    const uint32_t sum_col = OV ? 256u : 0u;
    for (int seg_lo = 0; seg_lo < P.Nt && !fail; seg_lo += seg_nodes) {
      const BtRange br = bt_block_range(P.row_ptr, seg_lo, min(seg_lo + seg_nodes, P.Nt));
      const int n_begin = br.n_begin, n_end = br.n_end;
      if (PROF) tiles_done += (unsigned long long)br.ntiles;
      float acc = 0.f;
      int cur = n_begin, node_lo = n_begin;
      float pre_x = 0.f, pre_y = 0.f, pre_z = 0.f;
      int pre_j = 0;
      // edge geometry of the tile that starts at edge e0 into buffer b (the displacement and neighbour index were
      // fetched one tile ahead); nlo: a node at or before the tile's first source node, s_rowwin starts there
      auto geometry = [&](long long e0, int cnt, int b, int nlo) {
        int j = 0, s = -1;
        const float gx = pre_x, gy = pre_y, gz = pre_z;
        const int gj = pre_j;
        {
          const long long en = e0 + BT_EDGES + gt;   // next tile's edge for this thread
          if (en < br.e_end) { pre_x = P.rij[en * 3]; pre_y = P.rij[en * 3 + 1]; pre_z = P.rij[en * 3 + 2]; pre_j = P.dst[en]; }
        }
        if (gt < cnt) {
          const long long e = e0 + gt;
          bt_geometry(gx, gy, gz, P.r0, s_jac, &s_geom[b][gt]);
          j = gj;
          if ((long long)s_rowwin[BT_EDGES] > e) {
            int lo = 0, hi = BT_EDGES;
            while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if ((long long)s_rowwin[mid] > e) hi = mid; else lo = mid; }
            s = nlo + lo;
          } else {
            s = bt_lb_row(P.row_ptr, nlo + BT_EDGES, n_end, e + 1) - 1;
          }
        } else {
          // a slot past the end of the block's edges: weight 0 and neighbour 0, so that the product phase needs no bounds check
          float4* gp = reinterpret_cast<float4*>(&s_geom[b][gt]);
          gp[0] = gp[1] = gp[2] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        s_dst[b][gt] = j;
        s_src[b][gt] = s;
      };
      // transposed last layer: thread tid < 128 owns channel tid (its tensor-memory lane) and adds the tile's edges
      // (columns) in order, carrying the sum of the node that continues from the previous tile. The order of the
      // additions depends on the node's edge list alone, so a system's result does not depend on its batch.
      auto sums_transposed = [&](int b, int cnt) {
        const float b3 = s_bias[4 * A + tid];
        int c_node = cur;
        float a_sum = acc;
        // sixteen edges (columns cb .. cb + 15) of this thread's channel
        auto add16 = [&](const uint32_t* r, int cb) {
          if (cb + 16 <= cnt && s_src[b][cb] == c_node && s_src[b][cb + 15] == c_node) {
#pragma unroll
            for (int i = 0; i < 16; i++) a_sum += __uint_as_float(r[i]) + b3;   // sixteen edges of the running node (sources are sorted)
          } else {
#pragma unroll
            for (int i4 = 0; i4 < 4; i4++) {
              const int4 t = *reinterpret_cast<const int4*>(&s_src[b][cb + 4 * i4]);
              const int sn[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
              for (int k = 0; k < 4; k++) {
                const int i = 4 * i4 + k;
                if (cb + i < cnt) {
                  if (sn[k] != c_node) { flush_until(c_node, sn[k], a_sum); a_sum = 0.f; c_node = sn[k]; }
                  a_sum += __uint_as_float(r[i]) + b3;
                }
              }
            }
          }
        };
        uint32_t ra[16];
        const uint32_t t0 = tmem_row + sum_col;
#pragma unroll 1
        for (int cb = 0; cb < cnt; cb += 16) {
          tc::tmem_ld16_issue(t0 + cb, ra);
          tc::tmem_ld16_wait(ra);
          add16(ra, cb);
        }
        acc = a_sum;
        cur = c_node;
      };
      bt_sync_workers();
      if (gt >= 0 && gt <= BT_EDGES) s_rowwin[gt] = P.row_ptr[min(node_lo + gt, n_end > n_begin ? n_end : n_begin)];
      if (gt >= 0 && gt < BT_EDGES && br.e_begin + gt < br.e_end) {
        const long long en = br.e_begin + gt;
        pre_x = P.rij[en * 3]; pre_y = P.rij[en * 3 + 1]; pre_z = P.rij[en * 3 + 2]; pre_j = P.dst[en];
      }
      bt_sync_workers();
      if (OV) {
        if (gt >= 0 && gt < BT_EDGES && br.e_begin < br.e_end)
          geometry(br.e_begin, (int)min((long long)BT_EDGES, br.e_end - br.e_begin), 0, node_lo);
        bt_sync_workers();
      }
      int prev_cnt = 0, tile_no = 0, win = 0;
      bool stop = false;   // a barrier reported a failure: every warp leaves at that barrier
      for (long long e0 = br.e_begin; e0 < br.e_end; e0 += BT_EDGES, tile_no++) {
        const int cnt = (int)((br.e_end - e0) < BT_EDGES ? (br.e_end - e0) : BT_EDGES);
        const int gb = OV ? (tile_no & 1) : 0;   // buffer of this tile's geometry
        if (!OV) {
          // ---- 1. edge geometry ---------------------------------------------------------------------------------
          if (tid < BT_EDGES) geometry(e0, cnt, 0, node_lo);
          if (bt_sync_or(fail)) { fail = 1; stop = true; break; }                         // [B1]
          lap(0);
        } else {
          // ---- 1. per-node sums of the previous tile; source-node window of the next tile ----------------------
          if (tid < A && tile_no > 0 && !fail) { sums_transposed(gb ^ 1, prev_cnt); tc::fence_before_sync(); }
          node_lo = s_src[gb][cnt - 1];
          if (gt >= 0 && gt <= BT_EDGES) win = P.row_ptr[min(node_lo + gt, n_end)];   // stored after the products
          lap(10);
        }
        // ---- 2. scalar products -> operand tile (columns c, C+c, 2C+c of row t) ------------------------------
        if (pb_lo < pb_hi) {
          const __nv_bfloat16* Lp = reinterpret_cast<const __nv_bfloat16*>(P.L0);
          const int* tdst = s_dst[gb];
#pragma unroll 1
          for (int pb = pb_lo; pb < pb_hi; pb++) {
            // the batch's rows are requested together and waited for together: the loads of a warp share a scoreboard,
            // so a rotating prefetch (reload a slot as soon as it is unpacked) would wait for the newest load every time
            uint32_t raw[UNR][8];
            if (feat == 2) {
#pragma unroll
              for (int u = 0; u < UNR; u++) {
                const int tu = pb_base + pb * pb_step + u * pu_step;       // slots past the edges name neighbour 0
                const int t = FAST ? tu : min(tu, BT_EDGES - 1);
                tc::ldg_raw8(Lp + ((size_t)tdst[t] * C + pc_c) * 16, raw[u]);
              }
            }
#pragma unroll
            for (int u = 0; u < UNR; u++) {
              const int t = pb_base + pb * pb_step + u * pu_step;
              if (!FAST && t >= BT_EDGES) break;
              float l0 = 0.f, l1[3] = {0.f, 0.f, 0.f}, l2[9] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
              if (feat == 2) {
                l0 = tc::bf16_at(raw[u], 0);
#pragma unroll
                for (int k = 0; k < 3; k++) l1[k] = tc::bf16_at(raw[u], 1 + k);
#pragma unroll
                for (int k = 0; k < 9; k++) l2[k] = tc::bf16_at(raw[u], 4 + k);
              }
              float y0 = 0.f, y1 = 0.f, y2 = 0.f;
              {
                const float4* gp = reinterpret_cast<const float4*>(&s_geom[gb][t]);
                const float4 e0 = gp[0], e1 = gp[1], rr = gp[2];
                float pa = wb;
                pa = fmaf(e0.x, w8[0], pa); pa = fmaf(e0.y, w8[1], pa); pa = fmaf(e0.z, w8[2], pa); pa = fmaf(e0.w, w8[3], pa);
                pa = fmaf(e1.x, w8[4], pa); pa = fmaf(e1.y, w8[5], pa); pa = fmaf(e1.z, w8[6], pa); pa = fmaf(e1.w, w8[7], pa);
                pa *= rr.w;   // 1 for an edge, 0 for a slot past the block's edges: the three products carry pa as a factor
                const float rh[3] = {rr.x, rr.y, rr.z};
                if (feat != 2) {
                  const size_t j = (size_t)tdst[t] * C + pc_c;
                  if (feat) {
                    const __nv_bfloat16* F0 = reinterpret_cast<const __nv_bfloat16*>(P.L0);
                    const __nv_bfloat16* F1 = reinterpret_cast<const __nv_bfloat16*>(P.L1);
                    const __nv_bfloat16* F2 = reinterpret_cast<const __nv_bfloat16*>(P.L2);
                    l0 = __bfloat162float(F0[j]);
#pragma unroll
                    for (int k = 0; k < 3; k++) l1[k] = __bfloat162float(F1[j * 3 + k]);
#pragma unroll
                    for (int k = 0; k < 9; k++) l2[k] = __bfloat162float(F2[j * 9 + k]);
                  } else {
                    l0 = __ldg(P.L0 + j);
#pragma unroll
                    for (int k = 0; k < 3; k++) l1[k] = __ldg(P.L1 + j * 3 + k);
#pragma unroll
                    for (int k = 0; k < 9; k++) l2[k] = __ldg(P.L2 + j * 9 + k);
                  }
                }
                // every rounding is spelled out, so that all instances of the kernel (and any later build) give the same bits
                y0 = l0 * pa;
                y1 = fmaf(l1[2], rh[2], fmaf(l1[1], rh[1], l1[0] * rh[0])) * pa;
                // r^T l2 r, row by row
                const float m0 = fmaf(l2[2], rh[2], fmaf(l2[1], rh[1], l2[0] * rh[0]));
                const float m1 = fmaf(l2[5], rh[2], fmaf(l2[4], rh[1], l2[3] * rh[0]));
                const float m2 = fmaf(l2[8], rh[2], fmaf(l2[7], rh[1], l2[6] * rh[0]));
                y2 = fmaf(m2, rh[2], fmaf(m1, rh[1], m0 * rh[0])) * pa;
              }
              unsigned short* arow = reinterpret_cast<unsigned short*>(a_smem + (size_t)t * 16);
              arow[a_off0] = bt_bf16(y0);
              arow[a_off1] = bt_bf16(y1);
              arow[a_off2] = bt_bf16(y2);
            }
          }
        }
        if (OV && gt >= 0 && gt <= BT_EDGES) s_rowwin[gt] = win;
        tc::fence_async_smem();
        tc::fence_before_sync();
        lap(11);
        if (bt_sync_or(fail)) { fail = 1; stop = true; break; }                           // [B2]
        lap(1);
        // overlapped schedule: the geometry of the next tile, while the first GEMM of this one runs
        if (OV && gt >= 0 && gt < BT_EDGES && e0 + BT_EDGES < br.e_end) {
          const long long en0 = e0 + BT_EDGES;
          geometry(en0, (int)min((long long)BT_EDGES, br.e_end - en0), gb ^ 1, node_lo);
          lap(0);
        }
        // ---- 3. four layers ------------------------------------------------------------------------------------
        for (int l = 0; l < BT_LAYERS; l++) {
          if (bt_sync_or(fail)) { fail = 1; stop = true; break; }                         // [A0..A3] layer l complete
          tc::fence_after_sync();
          lap(2 + 2 * l);
          const int N = P.layer[l].N;
          if (!fail && l < BT_LAYERS - 1) {
            // bias, activation -> BF16 into the operand tile at out_col (this thread: row `row`, its quarter of the columns)
            const float* bias = l == 0 ? nullptr : s_bias + (l - 1) * 2 * A;
            const int act = P.layer[l].act, oc = P.layer[l].out_col;
            const int cpp = max(N / 4, 32);  // columns per part
            // eight columns from `cb` on: bias, activation, BF16, one 16-byte store into the operand tile
            auto put8 = [&](const float* v8, int cb) {
              float t8[8];
              float b8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
              if (bias != nullptr) {   // two 16-byte shared-memory loads for eight biases
                const float4 ba = *reinterpret_cast<const float4*>(bias + cb);
                const float4 bb = *reinterpret_cast<const float4*>(bias + cb + 4);
                b8[0] = ba.x; b8[1] = ba.y; b8[2] = ba.z; b8[3] = ba.w; b8[4] = bb.x; b8[5] = bb.y; b8[6] = bb.z; b8[7] = bb.w;
              }
#pragma unroll
              for (int j = 0; j < 8; j++) {
                const float u = v8[j] + b8[j];
                t8[j] = (act == 2) ? fmaxf(u, 0.1f * u) : u;   // LeakyReLU(0.1) = max(u, 0.1 u)
              }
              uint4 q;
              q.x = tc::pack_bf16x2(t8[0], t8[1]); q.y = tc::pack_bf16x2(t8[2], t8[3]);
              q.z = tc::pack_bf16x2(t8[4], t8[5]); q.w = tc::pack_bf16x2(t8[6], t8[7]);
              *reinterpret_cast<uint4*>(a_smem + (size_t)((oc + cb) >> 3) * BT_PANEL + row * 16) = q;
            };
            if (FAST) {
              // sixteen columns at a time through two register blocks: the next block is on its way from tensor memory
              // while this one is converted and stored
              auto put16 = [&](const uint32_t* r, int cb) {
                float v[16];
#pragma unroll
                for (int i = 0; i < 16; i++) v[i] = __uint_as_float(r[i]);
                put8(v, cb);
                put8(v + 8, cb + 8);
              };
              uint32_t ra[16], rb[16];
              const int c_lo = part * cpp, c_hi = min((part + 1) * cpp, N);
              tc::tmem_ld16_issue(tmem_row + c_lo, ra);
              tc::tmem_ld16_wait(ra);
#pragma unroll 1
              for (int cb = c_lo; cb < c_hi; cb += 32) {
                const bool more2 = cb + 32 < c_hi;
                tc::tmem_ld16_issue(tmem_row + cb + 16, rb);
                put16(ra, cb);
                tc::tmem_ld16_wait(rb);
                if (more2) tc::tmem_ld16_issue(tmem_row + cb + 32, ra);
                put16(rb, cb + 16);
                if (more2) tc::tmem_ld16_wait(ra);
              }
            } else {
              for (int cb = part * cpp; cb < min((part + 1) * cpp, N); cb += 32) {
                float v[32];
                tc::tmem_ld32(tmem_row + cb, v);
#pragma unroll
                for (int g8 = 0; g8 < 4; g8++) put8(v + g8 * 8, cb + g8 * 8);
              }
            }
            tc::fence_async_smem();
            tc::fence_before_sync();
          }
          if (OV && l == BT_LAYERS - 1) break;   // the sums of this tile follow at the top of the next one
          if (bt_sync_or(fail)) { fail = 1; stop = true; break; }                         // [B3..B6]
          if (l < BT_LAYERS - 1) lap(3 + 2 * l);
        }
        if (stop) break;
        prev_cnt = cnt;
        if (OV) continue;
        // ---- 4. last layer's accumulators -> per-node sums (dim_a = 64) -----------------------------------------
        const int tile_cur = cur;
        node_lo = s_src[0][cnt - 1];
        if (tid <= BT_EDGES) s_rowwin[tid] = P.row_ptr[min(node_lo + tid, n_end)];
        {
          const float* bias = s_bias + 4 * A;
          const int cpp = max(A / 4, 32);
          for (int cb = part * cpp; cb < min((part + 1) * cpp, A); cb += 32) {
            float v[32];
            tc::tmem_ld32(tmem_row + cb, v);
#pragma unroll
            for (int g4 = 0; g4 < 8; g4++) {
              float4 m = make_float4(v[g4 * 4] + bias[cb + g4 * 4], v[g4 * 4 + 1] + bias[cb + g4 * 4 + 1],
                                     v[g4 * 4 + 2] + bias[cb + g4 * 4 + 2], v[g4 * 4 + 3] + bias[cb + g4 * 4 + 3]);
              if (row >= cnt) m = make_float4(0.f, 0.f, 0.f, 0.f);
              // 16-byte slot = 4 consecutive channels, xor-swizzled by row within groups of 8 slots
              const int slot = (cb >> 2) + g4;
              const int sw = (slot & ~7) | ((slot ^ row) & 7);
              *reinterpret_cast<float4*>(stage_f + (size_t)row * A + sw * 4) = m;
            }
          }
        }
        tc::fence_before_sync();
        bt_sync_workers();
        lap(9);
        // Per-node sums: one thread per output column adds the rows of the tile in edge order, carrying the sum of the
        // node that continues from the previous tile. The order of the additions depends on the node's edge list
        // alone, not on where the tiles of this block happen to start, so the result for a system is bit-identical
        // whatever batch (or shard of a batch) it is processed in.
        if (tid < A) {
          const int col = tid, slot = col >> 2, sub = col & 3;
          int c_node = tile_cur;
          float a_sum = acc;
          const float* sp = stage_f + (slot & ~7) * 4 + sub;
          const int sx = slot & 7;
          for (int e = 0; e < cnt; e++) {
            const int s = s_src[0][e];
            if (s != c_node) { flush_until(c_node, s, a_sum); a_sum = 0.f; c_node = s; }
            a_sum += sp[(size_t)e * A + ((sx ^ (e & 7)) << 2)];
          }
          acc = a_sum;
          cur = c_node;
        }
        if (bt_sync_or(fail)) { fail = 1; stop = true; break; }                           // [B7]
        lap(10);
      }
      if (OV && !fail && tid < A && tile_no > 0) { sums_transposed((tile_no - 1) & 1, prev_cnt); tc::fence_before_sync(); lap(9); }
      if (!stop && bt_sync_or(fail)) fail = 1;                                            // [B8] segment finished
      if (!fail && n_begin < n_end) flush_until(cur, n_end, acc);
    }
    // one thread of each role: tid 0 (adds up the previous tile), 128 (geometry of the next tile), 256 (neither)
    if (PROF && P.prof != nullptr && (tid == 0 || tid == 128 || tid == 256))
      for (int i = 0; i < 12; i++) atomicAdd((unsigned long long*)&P.prof[(tid >> 7) * 12 + i], (unsigned long long)pc[i]);
    if (PROF && P.prof != nullptr && tid == 0 && blockIdx.x < 256) {
      // per block: start and end on the global timer (ns), tiles processed, the SM it ran on
      unsigned long long t1; unsigned smid;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
      asm volatile("mov.u32 %0, %smid;" : "=r"(smid));
      P.prof[64 + blockIdx.x] = (long long)t_block0;
      P.prof[64 + 256 + blockIdx.x] = (long long)t1;
      P.prof[64 + 512 + blockIdx.x] = (long long)tiles_done;
      P.prof[64 + 768 + blockIdx.x] = (long long)smid;
    }
  }
  if (fail && lane == 0 && P.status != nullptr) atomicOr(P.status, LD_FLAG_TIMEOUT);
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem_base, ncols);
}

}  // namespace

// Tensor-core variant of ld_bee_messages_scalar_f32. Packed BF16 weights (ld_pack_weights_bf16):
// Yp = [dim_a][3*chan] (Y_000 | Y_110 | Y_220), W1p = [2a][a], W2p = [2a][2a],
// W3p = [a][3a] = (W3 | W_direct + identity). Biases FP32. chan a multiple of 32 (<= 256), dim_a 64 or 128.
extern "C" int ld_bee_messages_scalar_bf16_tc(const int* row_ptr, const int* dst, const float* rij, int Nt, int chan,
                                              int dim_a, float r0, const float* L0, const float* L1, const float* L2,
                                              const float* enc_w, const float* enc_b, const float* jacobi, const void* Yp,
                                              const void* W1p, const float* b1, const void* W2p, const float* b2,
                                              const void* W3p, const float* b3, float scale, float* out_a, int feat_bf16,
                                              int* status_dev, void* stream) {
  if (Nt < 0 || chan <= 0 || dim_a <= 0 || !(r0 > 0.f)) return LD_ERR_SHAPE;
  if (chan % 32 != 0 || chan > 256 || (dim_a != 64 && dim_a != 128)) {
    ld_set_last_message("bee messages (tensor-core path): chan must be a multiple of 32 up to 256, dim_a 64 or 128");
    return LD_ERR_UNSUPPORTED;
  }
  if (b1 == nullptr || b2 == nullptr || b3 == nullptr) return LD_ERR_SHAPE;
  if ((((uintptr_t)Yp | (uintptr_t)W1p | (uintptr_t)W2p | (uintptr_t)W3p) % 16) != 0) return LD_ERR_SHAPE;
  if (Nt == 0) return LD_OK;
  const int A = dim_a, C = chan;
  BtParams P;
  P.row_ptr = row_ptr; P.dst = dst; P.rij = rij; P.Nt = Nt; P.chan = C; P.dim_a = A; P.r0 = r0; P.scale = scale;
  P.L0 = L0; P.L1 = L1; P.L2 = L2; P.enc_w = enc_w; P.enc_b = enc_b; P.jacobi = jacobi;
  const int sk1 = BT_SLAB_BYTES / (A * 32), sk2 = BT_SLAB_BYTES / (2 * A * 32);
  P.layer[0] = BtLayer{(const __nv_bfloat16*)Yp, nullptr, 0, 3 * C / 16, sk1, A, 0, 2 * A, 0};
  P.layer[1] = BtLayer{(const __nv_bfloat16*)W1p, b1, 2 * A / 8, A / 16, sk2, 2 * A, 2, 0, 0};
  P.layer[2] = BtLayer{(const __nv_bfloat16*)W2p, b2, 0, 2 * A / 16, sk2, 2 * A, 2, 0, 0};
  P.layer[3] = BtLayer{(const __nv_bfloat16*)W3p, b3, 0, 3 * A / 16, sk1, A, 0, -1, A == 128 ? 2 * A / 16 : 0};
  const int cols = 3 * (C > A ? C : A);
  const size_t a_bytes = (size_t)(cols / 8) * BT_PANEL;
  const size_t staging = (size_t)BT_EDGES * A * 4;
  const size_t front = a_bytes > staging ? a_bytes : staging;
  P.slab_bytes = (unsigned)BT_SLAB_BYTES;
  P.stage_off = (unsigned)front;
  P.bias_off = (unsigned)(front + (size_t)BT_STAGES * P.slab_bytes);
  const size_t smem = P.bias_off + (size_t)5 * A * 4 + 256;
  if (smem > 215 * 1024) { ld_set_last_message("bee messages (tensor-core path): shared-memory plan exceeds the limit"); return LD_ERR_UNSUPPORTED; }
  {
    // The blocks walk the node range in segments so that the rows a segment gathers stay in L2 (126 MB): 80 MB of rows
    // per segment. Every segment costs each block a ragged last tile and a pipeline refill, and fewer segments average
    // the blocks' shares better; measured on 256-bead polymers, 1024 systems: 23.34 ms with 40 MB segments, 23.26 with
    // 80, 23.2 with one; 128 systems: 3.12, 3.07, 3.00. Systems whose nodes have neighbours all over a large periodic
    // box need the segments: the PaiNN kernel on 8192-node boxes loses 0.3 % at 80 MB and 5 to 8 % at 160 MB or more.
    const long long row_bytes = (feat_bf16 == 2 ? 32LL : feat_bf16 ? 26LL : 52LL) * C;   // 13*chan values gathered per neighbour
    // (a range whose rows come to little more than L2 is walked as one segment: 134 MB of rows, 128 polymers, 3.00 ms
    // against 3.07 ms in two segments)
    const long long seg = (long long)Nt * row_bytes <= (160LL << 20) ? (long long)Nt : (80LL << 20) / row_bytes;
    P.seg_nodes = ld_even_segments(Nt, seg);
  }
  P.out_a = out_a; P.status = status_dev; P.feat_bf16 = feat_bf16;
#ifdef LD_PHASE_COUNTERS
  P.prof = ld_internal_phase_counters();
  const bool fast = C == 128 && A == 128 && feat_bf16 == 2;
  auto kern = P.prof != nullptr ? (fast ? bee_scalar_tc_kernel<true, true> : bee_scalar_tc_kernel<true, false>)
                                : (fast ? bee_scalar_tc_kernel<false, true> : bee_scalar_tc_kernel<false, false>);
#else
  P.prof = nullptr;
  auto kern = (C == 128 && A == 128 && feat_bf16 == 2) ? bee_scalar_tc_kernel<false, true> : bee_scalar_tc_kernel<false, false>;
#endif
  LD_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  kern<<<sms, BT_THREADS, smem, (cudaStream_t)stream>>>(P);
  LD_LAUNCH_CHECK();
  return LD_OK;
}
