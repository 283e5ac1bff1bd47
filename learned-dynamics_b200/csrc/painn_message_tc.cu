// PaiNN message step on the Blackwell tensor cores: the same fused computation as
// painn_message.cu (Message.forward, archs/meanflow_painn8.py:77-100, plus the edge gather and
// edges_reduce_src), with the three layers of the per-edge distance MLP running as tcgen05 MMAs:
// BF16 operands, FP32 accumulation in tensor memory. Tolerance of this path: 2e-2 relative.
//
// A block owns a node-aligned, contiguous slice of the CSR and walks it 128 edges at a time:
//   1. radial features of the 128 edges -> BF16 operand tile A in shared memory
//   2. three layers: weights stream from L2 as pre-packed BF16 panels (bulk asynchronous copies,
//      4 stages of K=16), one thread issues [128 x 4n x 16] MMAs into 128 lanes x 4n columns of TMEM;
//      between layers all threads read the accumulators (tcgen05.ld), add bias, apply SiLU and
//      write the next operand tile back over A
//   3. last layer: accumulator x gathered neighbour activation -> vector/scalar messages, staged
//      in shared memory, then summed per source node in edge order; sums for the node that spans
//      tiles stay in registers, every node is written once (no atomics, fixed summation order)
// Edge-sized data never reaches HBM. Every mbarrier wait is bounded (LD_FLAG_TIMEOUT).
#include "common.cuh"
#include "tc05.cuh"
#include "tp_math.h"

namespace {

constexpr int MT_EDGES = 128;          // edges per tile = MMA M
constexpr int MT_WORK_WARPS = 8;       // working warps: TMEM lane quarter = warp % 4, column half = warp / 4
constexpr int MT_THREADS_TC = (MT_WORK_WARPS + 1) * 32;  // + one warp whose lane 0 streams weights and issues MMAs
constexpr int MT_STAGES = 4;           // weight stages of K = 16
constexpr int MT_CG = 64;              // channels per reduction pass
constexpr int MT_MAX_PASS = 2;         // n <= 128

struct TcMessageParams {
  const int* row_ptr; const int* dst; const float* rij;
  int Nt, n, n_rbf, k0p, radial_kind;
  unsigned bias_off;   // byte offset of the bias copy in dynamic shared memory
  float rmax, pi_over_rmax, eps;
  const __nv_bfloat16* w1; const __nv_bfloat16* w2; const __nv_bfloat16* w3;  // packed panels [K/8][4n][8]
  const float* b1; const float* b2; const float* b3;
  const float* actv; const float* x_v; const float* res_a; const float* res_v;
  float* out_a; float* out_v;
  long long* edge_counter;
  int* status;
};

__device__ __forceinline__ int lb_row(const int* __restrict__ row_ptr, int lo, int hi, long long target) {
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if ((long long)row_ptr[mid] < target) lo = mid + 1; else hi = mid;
  }
  return lo;
}


// first node v in [0, Nt] with row_ptr[v] + v >= target (work = edges + nodes before v)
__device__ __forceinline__ int work_lower_bound(const int* __restrict__ row_ptr, int Nt, long long target) {
  int lo = 0, hi = Nt;
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if ((long long)row_ptr[mid] + mid < target) lo = mid + 1; else hi = mid;
  }
  return lo;
}

struct Pipe {
  uint32_t loads;   // weight slabs requested so far (block lifetime)
  uint32_t mmas;    // weight slabs consumed so far
  int requested;    // slabs of the current layer requested so far
};

struct IssueCtx {
  unsigned char* b_smem; uint64_t* bar_full; uint64_t* bar_empty; uint64_t* bar_accum;
  uint32_t a_base, tmem_base; int N;
};

// request the K=16 weight slab `ks` of a layer into the next free stage (one thread)
__device__ __forceinline__ bool request_slab(const IssueCtx& c, Pipe& pipe, const __nv_bfloat16* __restrict__ wp, int ks) {
  const uint32_t slab = (uint32_t)c.N * 32;  // 2 panels x N rows x 16 B
  const uint32_t st = pipe.loads % MT_STAGES, use = pipe.loads / MT_STAGES;
  if (use >= 1 && !tc::mbar_wait(&c.bar_empty[st], (use - 1) & 1)) return false;  // MMAs that read the stage are done
  tc::mbar_expect_tx(&c.bar_full[st], slab);
  tc::bulk_g2s(c.b_smem + (size_t)st * slab, wp + (size_t)ks * c.N * 16, slab, &c.bar_full[st]);
  pipe.loads++;
  return true;
}

__device__ __forceinline__ bool prefetch_layer(const IssueCtx& c, Pipe& pipe, const __nv_bfloat16* __restrict__ wp, int ksteps) {
  for (pipe.requested = 0; pipe.requested < ksteps && pipe.requested < MT_STAGES - 1; pipe.requested++)
    if (!request_slab(c, pipe, wp, pipe.requested)) return false;
  return true;
}

// issue the MMAs of one layer (operand tile A is ready), keep the weight pipeline full, signal bar_accum
__device__ __forceinline__ bool run_layer(const IssueCtx& c, Pipe& pipe, const __nv_bfloat16* __restrict__ wp, int ksteps) {
  const uint32_t slab = (uint32_t)c.N * 32;
  for (int ks = 0; ks < ksteps; ks++) {
    const uint32_t st = pipe.mmas % MT_STAGES, use = pipe.mmas / MT_STAGES;
    if (!tc::mbar_wait(&c.bar_full[st], use & 1)) return false;
    tc::fence_after_sync();
    const uint64_t ad = tc::smem_desc(c.a_base + ks * 2 * (MT_EDGES * 16), MT_EDGES * 16, 128);
    const uint32_t b_base = tc::smem_u32(c.b_smem + (size_t)st * slab);
    for (int n0 = 0; n0 < c.N; n0 += 256) {
      const int n1 = min(256, c.N - n0);
      const uint64_t bd = tc::smem_desc(b_base + n0 * 16, c.N * 16, 128);
      tc::mma_bf16(c.tmem_base + n0, ad, bd, tc::idesc_bf16(MT_EDGES, n1), ks > 0 ? 1u : 0u);
    }
    tc::mma_commit(&c.bar_empty[st]);
    pipe.mmas++;
    if (pipe.requested < ksteps) {
      if (!request_slab(c, pipe, wp, pipe.requested)) return false;
      pipe.requested++;
    }
  }
  tc::mma_commit(c.bar_accum);
  return true;
}

// Warps 0..7: geometry, operand tiles, epilogues, reduction (thread = one edge row / one output
// column). Warp 8: lane 0 streams weights and issues MMAs; it never spins in the same warp as
// working threads. All 288 threads meet at the same sequence of block barriers; a failed bounded
// wait is OR-ed in at the next barrier so that everybody leaves together.
__global__ void __launch_bounds__(MT_THREADS_TC, 1)
painn_message_tc_kernel(TcMessageParams P) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t bar_full[MT_STAGES], bar_empty[MT_STAGES], bar_accum;
  __shared__ uint32_t tmem_slot;
  __shared__ float s_dir[MT_EDGES][3];
  __shared__ float s_dist[MT_EDGES];
  __shared__ int s_dst[MT_EDGES];
  __shared__ int s_src[MT_EDGES];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool issuer_warp = warp == MT_WORK_WARPS;
  const bool issuer = issuer_warp && lane == 0;
  const int quarter = warp & 3, half = (warp >> 2) & 1;
  const int row = quarter * 32 + lane;  // edge slot / TMEM lane owned in the epilogues
  const int n = P.n, N = 4 * n;
  // shared-memory carve-up: A operand tile | weight stages ; reduction staging overlays both ; biases after
  unsigned char* a_smem = smem;                                   // 128 x N BF16
  unsigned char* b_smem = a_smem + (size_t)MT_EDGES * N * 2;      // MT_STAGES x N*32
  float* s_bias = reinterpret_cast<float*>(smem + P.bias_off);    // 3 x N
  float* stage_f = reinterpret_cast<float*>(smem);                // [128][MT_CG*4]

  for (int i = tid; i < N; i += MT_THREADS_TC) {
    s_bias[i] = P.b1[i]; s_bias[N + i] = P.b2[i]; s_bias[2 * N + i] = P.b3[i];
  }
  if (tid == 0) {
    for (int s = 0; s < MT_STAGES; s++) { tc::mbar_init(&bar_full[s], 1); tc::mbar_init(&bar_empty[s], 1); }
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
  IssueCtx ctx{b_smem, bar_full, bar_empty, &bar_accum, tc::smem_u32(a_smem), tmem_base, N};

  // node-aligned share, balanced over edges + nodes: nodes without edges still have to be written
  const long long E = P.row_ptr[P.Nt];
  long long per = (E + P.Nt + gridDim.x - 1) / gridDim.x;
  if (per < MT_EDGES) per = MT_EDGES;
  const int n_begin = blockIdx.x == 0 ? 0 : work_lower_bound(P.row_ptr, P.Nt, per * blockIdx.x);
  const int n_end = blockIdx.x == gridDim.x - 1 ? P.Nt : work_lower_bound(P.row_ptr, P.Nt, per * (blockIdx.x + 1));
  const long long e_begin = n_begin < n_end ? P.row_ptr[n_begin] : 0;
  const long long e_end = n_begin < n_end ? P.row_ptr[n_end] : 0;

  // reduction role: column `tid` of the staging tile = (channel tid/4 of the pass, component tid%4)
  const int red_c = (tid >> 2) & (MT_CG - 1), red_k = tid & 3;
  const int npass = (n + MT_CG - 1) / MT_CG;
  const int k0steps = P.k0p / 16, ksteps = N / 16;
  float acc[MT_MAX_PASS] = {0.f, 0.f};
  int cur = n_begin;
  Pipe pipe{0, 0, 0};
  uint32_t accum_phase = 0;
  int fail = 0;

  auto flush_until = [&](int pass, int from, int next, float value) {
    // write node `from` (value), zero-fill (from, next) for this pass's channel
    const int c = pass * MT_CG + red_c;
    if (c >= n) return;
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
        s = lb_row(P.row_ptr, n_begin, n_end, e + 1) - 1;
      }
      const float r2 = dx * dx + dy * dy + dz * dz;
      const float inv = 1.0f / sqrtf(P.eps + r2);
      s_dir[tid][0] = dx * inv; s_dir[tid][1] = dy * inv; s_dir[tid][2] = dz * inv;
      s_dist[tid] = sqrtf(r2);
      s_dst[tid] = j;
      s_src[tid] = s;
    }
    if (__syncthreads_or(fail)) { fail = 1; break; }                                   // [S1]
    // ---- 2. radial features -> operand tile ; issuer prefetches the first layer's weights --------------
    if (issuer) {
      if (!prefetch_layer(ctx, pipe, P.w1, k0steps)) fail = 1;
    } else if (!issuer_warp) {
      const int e = tid & (MT_EDGES - 1);
      const float d = s_dist[e];
      for (int p = tid >> 7; p < P.k0p / 8; p += MT_WORK_WARPS * 32 / MT_EDGES) {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
          const int k = p * 8 + j;
          v[j] = (e < cnt && k < P.n_rbf) ? radial_feature(P.radial_kind, k, P.n_rbf, d, P.rmax, P.pi_over_rmax) : 0.f;
        }
        uint4 q;
        q.x = tc::pack_bf16x2(v[0], v[1]); q.y = tc::pack_bf16x2(v[2], v[3]);
        q.z = tc::pack_bf16x2(v[4], v[5]); q.w = tc::pack_bf16x2(v[6], v[7]);
        *reinterpret_cast<uint4*>(a_smem + (size_t)p * (MT_EDGES * 16) + e * 16) = q;
      }
      tc::fence_async_smem();
    }
    tc::fence_before_sync();
    if (__syncthreads_or(fail)) { fail = 1; break; }                                   // [S2]

    // ---- 3. three layers ---------------------------------------------------------------------------------
    for (int layer = 0; layer < 3; layer++) {
      if (issuer) {
        tc::fence_after_sync();
        const __nv_bfloat16* wp = layer == 0 ? P.w1 : (layer == 1 ? P.w2 : P.w3);
        if (!run_layer(ctx, pipe, wp, layer == 0 ? k0steps : ksteps)) fail = 1;
        if (!fail && layer < 2 && !prefetch_layer(ctx, pipe, layer == 0 ? P.w2 : P.w3, ksteps)) fail = 1;
      } else if (!issuer_warp) {
        if (!tc::mbar_wait(&bar_accum, accum_phase & 1)) fail = 1;
        tc::fence_after_sync();
        if (!fail && layer < 2) {
          // bias + SiLU -> next operand tile (this thread: row `row`, columns of its half)
          const float* bias = s_bias + layer * N;
          for (int cb = half * (N / 2); cb < (half + 1) * (N / 2); cb += 32) {
            float v[32];
            tc::tmem_ld32(tmem_row + cb, v);
#pragma unroll
            for (int g8 = 0; g8 < 4; g8++) {
              float t[8];
#pragma unroll
              for (int j = 0; j < 8; j++) t[j] = silu_f(v[g8 * 8 + j] + bias[cb + g8 * 8 + j]);
              uint4 q;
              q.x = tc::pack_bf16x2(t[0], t[1]); q.y = tc::pack_bf16x2(t[2], t[3]);
              q.z = tc::pack_bf16x2(t[4], t[5]); q.w = tc::pack_bf16x2(t[6], t[7]);
              *reinterpret_cast<uint4*>(a_smem + (size_t)((cb >> 3) + g8) * (MT_EDGES * 16) + row * 16) = q;
            }
          }
          tc::fence_async_smem();
        }
      }
      accum_phase++;
      tc::fence_before_sync();
      if (__syncthreads_or(fail)) { fail = 1; break; }                                 // [S3], [S4], [S5]
    }
    if (fail) break;  // uniform: the flag was OR-ed across the block at the barrier above

    // ---- 4. messages and per-node sums (working warps; the issuer warp only keeps the barriers) ------------
    const float* b3 = s_bias + 2 * N;
    const int j_node = issuer_warp ? 0 : s_dst[row];
    const float* Aj = P.actv + (size_t)j_node * N;
    const float* Xj = P.x_v + (size_t)j_node * n * 3;
    const float dir0 = s_dir[row][0], dir1 = s_dir[row][1], dir2 = s_dir[row][2];
    const int tile_cur = cur;
    for (int pass = 0; pass < npass; pass++) {
      if (!issuer_warp) {
        // this thread: edge `row`, channels [pass*CG + half*CG/2, +CG/2) in groups of 8
        for (int g8 = 0; g8 < MT_CG / 16; g8++) {
          const int c0 = pass * MT_CG + half * (MT_CG / 2) + g8 * 8;
          if (c0 < n) {  // n is a multiple of 8: a group is entirely valid or entirely not
            float d[32];
            tc::tmem_ld8x4(tmem_row + c0, (uint32_t)n, d);  // D[.., c0 + k*n + j] at d[k*8 + j]
            float a[32];
#pragma unroll
            for (int k = 0; k < 4; k++) {
              const float4 u0 = __ldg(reinterpret_cast<const float4*>(Aj + k * n + c0));
              const float4 u1 = __ldg(reinterpret_cast<const float4*>(Aj + k * n + c0 + 4));
              a[k * 8 + 0] = u0.x; a[k * 8 + 1] = u0.y; a[k * 8 + 2] = u0.z; a[k * 8 + 3] = u0.w;
              a[k * 8 + 4] = u1.x; a[k * 8 + 5] = u1.y; a[k * 8 + 6] = u1.z; a[k * 8 + 7] = u1.w;
            }
            float xv[24];
#pragma unroll
            for (int q4 = 0; q4 < 6; q4++) {
              const float4 u = __ldg(reinterpret_cast<const float4*>(Xj + (size_t)c0 * 3) + q4);
              xv[q4 * 4 + 0] = u.x; xv[q4 * 4 + 1] = u.y; xv[q4 * 4 + 2] = u.z; xv[q4 * 4 + 3] = u.w;
            }
#pragma unroll
            for (int j = 0; j < 8; j++) {
              const int c = c0 + j;
              const float p0 = (d[j] + b3[c]) * a[j];
              const float p1 = (d[8 + j] + b3[n + c]) * a[8 + j];
              const float p2 = (d[16 + j] + b3[2 * n + c]) * a[16 + j];
              const float p3 = (d[24 + j] + b3[3 * n + c]) * a[24 + j];
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
      }
      __syncthreads();
      // sum per source node, in edge order; thread = one (channel, component) column
      if (!issuer_warp) {
        int c_node = tile_cur;
        float a_sum = acc[pass];
        const int slot = red_c;
        for (int e = 0; e < cnt; e++) {
          const int s = s_src[e];
          if (s != c_node) {
            flush_until(pass, c_node, s, a_sum);
            a_sum = 0.f;
            c_node = s;
          }
          const int sw = (slot & ~7) | ((slot ^ e) & 7);
          a_sum += stage_f[(size_t)e * (MT_CG * 4) + sw * 4 + red_k];
        }
        acc[pass] = a_sum;
        if (pass == npass - 1) cur = c_node;
      }
      tc::fence_before_sync();
      __syncthreads();  // staging (and TMEM after the last pass) is rewritten by the next pass / tile
    }
  }
  if (!fail && !issuer_warp && n_begin < n_end) {
    for (int pass = 0; pass < npass; pass++) flush_until(pass, cur, n_end, acc[pass]);
    if (P.edge_counter != nullptr && tid == 0) atomicAdd((unsigned long long*)P.edge_counter, (unsigned long long)(e_end - e_begin));
  }
  if (fail && tid == 0 && P.status != nullptr) atomicOr(P.status, LD_FLAG_TIMEOUT);
  if (fail && issuer) {
    // give copies still in flight a bounded chance to land before the block's shared memory is released
    for (uint32_t i = pipe.mmas; i < pipe.loads; i++) tc::mbar_wait(&bar_full[i % MT_STAGES], (i / MT_STAGES) & 1);
  }
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem_base, ncols);
}

}  // namespace

// Tensor-core variant of ld_painn_message_f32 (same graph / feature arguments). w1p/w2p/w3p are the
// distance-MLP weights packed by ld_pack_weights_bf16 ([4n][n_rbf], [4n][4n], [4n][4n]); biases FP32.
// n a multiple of 8, n <= 128. status_dev receives LD_FLAG_TIMEOUT if a bounded wait ran out.
extern "C" int ld_painn_message_bf16_tc(const int* row_ptr, const int* dst, const float* rij, int Nt, int n, int n_rbf,
                                        int radial_kind, float rmax, float eps, const void* w1p, const float* b1,
                                        const void* w2p, const float* b2, const void* w3p, const float* b3,
                                        const float* actv, const float* x_v, const float* res_a, const float* res_v,
                                        float* out_a, float* out_v, long long* edge_counter, int* status_dev, void* stream) {
  if (Nt < 0 || n <= 0 || n_rbf <= 0) return LD_ERR_SHAPE;
  if (n % 8 != 0 || n > 128) { ld_set_last_message("painn message (tensor-core path): n must be a multiple of 8, at most 128"); return LD_ERR_UNSUPPORTED; }
  if (b1 == nullptr || b2 == nullptr || b3 == nullptr) { ld_set_last_message("painn message: biases are required"); return LD_ERR_SHAPE; }
  if ((((uintptr_t)w1p | (uintptr_t)w2p | (uintptr_t)w3p | (uintptr_t)actv | (uintptr_t)x_v) % 16) != 0) {
    ld_set_last_message("painn message (tensor-core path): weights and node features must be 16-byte aligned");
    return LD_ERR_SHAPE;
  }
  if (Nt == 0) return LD_OK;
  TcMessageParams P;
  P.row_ptr = row_ptr; P.dst = dst; P.rij = rij; P.Nt = Nt; P.n = n; P.n_rbf = n_rbf; P.k0p = (n_rbf + 15) / 16 * 16;
  P.radial_kind = radial_kind; P.rmax = rmax; P.pi_over_rmax = (float)(3.14159265358979323846 / (double)rmax); P.eps = eps;
  P.w1 = (const __nv_bfloat16*)w1p; P.w2 = (const __nv_bfloat16*)w2p; P.w3 = (const __nv_bfloat16*)w3p;
  P.b1 = b1; P.b2 = b2; P.b3 = b3; P.actv = actv; P.x_v = x_v; P.res_a = res_a; P.res_v = res_v;
  P.out_a = out_a; P.out_v = out_v; P.edge_counter = edge_counter; P.status = status_dev;
  const int N = 4 * n;
  if (P.k0p > N) { ld_set_last_message("painn message (tensor-core path): n_rbf above 4n is not supported"); return LD_ERR_UNSUPPORTED; }
  size_t a_bytes = (size_t)MT_EDGES * N * 2, b_bytes = (size_t)MT_STAGES * N * 32;
  size_t staging = (size_t)MT_EDGES * MT_CG * 4 * 4;  // 128 KB, overlays A and the weight stages
  size_t front = a_bytes + b_bytes > staging ? a_bytes + b_bytes : staging;
  P.bias_off = (unsigned)front;
  const size_t smem = front + (size_t)3 * N * 4 + 1024;
  if (smem > 227 * 1024) return LD_ERR_UNSUPPORTED;
  LD_CUDA_TRY(cudaFuncSetAttribute(painn_message_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  painn_message_tc_kernel<<<sms, MT_THREADS_TC, smem, (cudaStream_t)stream>>>(P);
  LD_LAUNCH_CHECK();
  return LD_OK;
}
