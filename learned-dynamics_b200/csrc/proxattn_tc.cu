// Dense proximity attention, forward pass on the tensor cores in TF32 (tcgen05, accumulators in TMEM):
//   out[z,m,:] = sum_n w(m,n) * (q_m . k_n) * v_n,   w(m,n) = r0sq / (r0sq + dist2(x_m, y_n))
// Same operator as ld_proxattn_fwd (FP32 FMA); this is the precision the reference's Triton kernel computes
// in (its tl.dot calls on FP32 inputs run as TF32; managan/triton_kernels/proxattn.py:30-83).
//
// A block owns 128 queries (one TMEM lane each) and walks the keys in steps of TN = 64; up to dim 64 two blocks
// share an SM (shared memory about 100 KB, 128 TMEM columns each), so that one block's staging and weights
// overlap the other's MMAs:
//   1. K, V and the key positions of the step are staged in shared memory (K by asynchronous copies and V through registers, both
//      issued during the weights of the step before) as K-major, no-swizzle operand
//      panels of 32-bit elements: element (row, k) at (k / 4) * LBO + row * 16 + (k % 4) * 4 bytes. For V the
//      "row" is the feature and k the key, so the staging transposes 4 keys per 16-byte store.
//   2. one thread issues S = Q K^T (dim / 8 MMAs of 128 x TN x 8) into TMEM columns [0, TN)
//   3. all 256 threads (thread = query row x column half) read their part of S, multiply by the pair
//      weights and store P = w o S as the A-operand panel of the second product
//   4. one thread issues O += P V (TN / 8 MMAs of 128 x dim x 8) into TMEM columns [TN, TN + dim)
// Rows past N are zero-filled, so they contribute nothing; only the final store is masked. Every wait on an
// mbarrier is bounded; on a timeout the block sets LD_FLAG_TIMEOUT in the status word, frees its TMEM and returns.
#include <cuda_runtime.h>
#include "common.cuh"
#include "tc05.cuh"

namespace {

constexpr int QT = 128;          // queries per block
constexpr int PTC_THREADS = 256;
constexpr int PANEL_PAD = 16;    // bytes added to every K-group stride (spreads staging stores over banks)

struct PtcArgs {
  const float *Q, *K, *V, *X, *Y, *r0sq;
  float* out;
  int* status;
  int heads, N;
  float lx, ly, lz;
};

__host__ __device__ constexpr uint32_t idesc_tf32(uint32_t M, uint32_t N) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((N >> 3) << 17) | ((M >> 4) << 24);
}

__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// round to nearest TF32 (the MMA itself would drop the low mantissa bits)
__device__ __forceinline__ float to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

template <int D>
struct Ptc {
  static constexpr int TN = 64;                               // keys per step
  static constexpr int TMEM_COLS = (D <= 64) ? 128 : 256;     // S in columns [0, 64), O in [64, 64 + D)
  static constexpr int MIN_BLOCKS = (D <= 64) ? 2 : 1;        // two blocks per SM overlap each other's phases
  static constexpr int LBO_Q = QT * 16 + PANEL_PAD;         // bytes between K-groups of the Q panel (rows = queries)
  static constexpr int LBO_K = TN * 16 + PANEL_PAD;         // K panel (rows = keys)
  static constexpr int LBO_V = D * 16 + PANEL_PAD;          // V panel (rows = features, K-groups = 4 keys)
  static constexpr int LBO_P = QT * 16 + PANEL_PAD;         // P panel (rows = queries, K-groups = 4 keys)
  static constexpr int Q_BYTES = (D / 4) * LBO_Q;
  static constexpr int K_BYTES = (D / 4) * LBO_K;
  static constexpr int V_BYTES = (TN / 4) * LBO_V;
  static constexpr int P_BYTES = (TN / 4) * LBO_P;
  static constexpr int Y_BYTES = TN * 6 * 4;
  static constexpr int SMEM = Q_BYTES + K_BYTES + V_BYTES + P_BYTES + Y_BYTES + 64;
};

// rows [row0, row0 + ROWS) of g [N][D] -> panel with K-groups along the feature dimension
template <int D, int ROWS>
__device__ __forceinline__ void ptc_stage_rows(uint8_t* __restrict__ panel, int lbo, const float* __restrict__ g, int row0, int N) {
  constexpr int G = D / 4;
  for (int idx = threadIdx.x; idx < ROWS * G; idx += PTC_THREADS) {
    const int r = idx / G, k4 = idx % G;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (row0 + r < N) v = __ldg(reinterpret_cast<const float4*>(g + (size_t)(row0 + r) * D) + k4);
    *reinterpret_cast<float4*>(panel + (size_t)k4 * lbo + r * 16) = make_float4(to_tf32(v.x), to_tf32(v.y), to_tf32(v.z), to_tf32(v.w));
  }
}

// the same panel filled by 16-byte asynchronous copies (rows past N are zero-filled by a zero source size); the
// MMA then drops the low mantissa bits of these operands instead of rounding them
template <int D, int ROWS>
__device__ __forceinline__ void ptc_stage_rows_async(uint32_t panel_addr, int lbo, const float* __restrict__ g, int row0, int N) {
  constexpr int G = D / 4;
  for (int idx = threadIdx.x; idx < ROWS * G; idx += PTC_THREADS) {
    const int r = idx / G, k4 = idx % G;
    const bool in = row0 + r < N;
    const float* src = g + (size_t)(in ? row0 + r : 0) * D + 4 * k4;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(panel_addr + (uint32_t)(k4 * lbo + r * 16)), "l"(src),
                 "r"(in ? 16 : 0)
                 : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
}

// rows [row0, row0 + TN) of V [N][D] -> panel whose rows are features and whose K-groups are 4 consecutive keys.
// In two halves, so that the loads of the next step can be in flight while this step's weights are computed:
// ptc_load_v reads 4 keys x one feature per thread and iteration into registers, ptc_store_v rounds and stores them.
template <int D, int TN>
__device__ __forceinline__ void ptc_load_v(float (&e)[D / 16][4], const float* __restrict__ g, int row0, int N) {
#pragma unroll
  for (int it = 0; it < D / 16; it++) {
    const int idx = threadIdx.x + it * PTC_THREADS, d = idx % D, n4 = idx / D;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int n = row0 + 4 * n4 + j;
      e[it][j] = (n < N) ? __ldg(g + (size_t)n * D + d) : 0.f;
    }
  }
}
template <int D, int TN>
__device__ __forceinline__ void ptc_store_v(uint8_t* __restrict__ panel, int lbo, const float (&e)[D / 16][4]) {
#pragma unroll
  for (int it = 0; it < D / 16; it++) {
    const int idx = threadIdx.x + it * PTC_THREADS, d = idx % D, n4 = idx / D;
    *reinterpret_cast<float4*>(panel + (size_t)n4 * lbo + d * 16) =
        make_float4(to_tf32(e[it][0]), to_tf32(e[it][1]), to_tf32(e[it][2]), to_tf32(e[it][3]));
  }
}

// positions of a tile: open space (x, y, z); periodic (cos, sin) of 2 pi x_a / L_a per axis
template <bool PER>
__device__ __forceinline__ void ptc_point(const float* __restrict__ g, int row, int N, const PtcArgs& p, float* o) {
  const float L[3] = {p.lx, p.ly, p.lz};
#pragma unroll
  for (int a = 0; a < 3; a++) {
    const float v = (row < N) ? __ldg(g + (size_t)row * 3 + a) : 0.f;
    if (PER) {
      float sn, cs;
      sincosf(6.283185307179586f * v / L[a], &sn, &cs);
      o[2 * a] = cs; o[2 * a + 1] = sn;
    } else {
      o[a] = v;
    }
  }
}

template <bool PER>
__device__ __forceinline__ float ptc_weight(const float* x, const float* y, float r0sq, const float* kc) {
  float dd = 0.f;
#pragma unroll
  for (int a = 0; a < 3; a++) {
    if (PER) {
      const float cs = fmaf(x[2 * a], y[2 * a], x[2 * a + 1] * y[2 * a + 1]);
      dd = fmaf(1.f - cs, kc[a], dd);
    } else {
      const float R = x[a] - y[a];
      dd = fmaf(R, R, dd);
    }
  }
  return __fdividef(r0sq, r0sq + dd);
}

template <int D, bool PER>
__global__ void __launch_bounds__(PTC_THREADS, Ptc<D>::MIN_BLOCKS) proxattn_fwd_tc_kernel(PtcArgs p) {
  using C = Ptc<D>;
  constexpr int TN = C::TN, TNH = TN / 2, PS = PER ? 6 : 3;
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + C::Q_BYTES;
  uint8_t* sV = sK + C::K_BYTES;
  uint8_t* sP = sV + C::V_BYTES;
  float* sY = reinterpret_cast<float*>(sP + C::P_BYTES);
  uint64_t* bar_s = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(sY) + C::Y_BYTES);
  uint64_t* bar_o = bar_s + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_o + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row = 32 * (warp & 3) + lane, half = warp >> 2;   // TMEM lane of this thread, and its half of the columns
  const int z = blockIdx.y, m0 = blockIdx.x * QT, N = p.N;
  const size_t zf = (size_t)z * N * D, zp = (size_t)z * N * 3;
  const float r0sq = __ldg(p.r0sq + z % p.heads);
  const float kc[3] = {p.lx * p.lx * 0.05066059182116889f, p.ly * p.ly * 0.05066059182116889f, p.lz * p.lz * 0.05066059182116889f};

  if (tid == 0) {
    tc::mbar_init(bar_s, 1);
    tc::mbar_init(bar_o, 1);
    tc::mbar_init_fence();
  }
  if (warp == 0) { tc::tmem_alloc(tmem_slot, C::TMEM_COLS); tc::tmem_relinquish(); }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + TN;
  const uint32_t lane_bits = (uint32_t)(32 * (warp & 3)) << 16;

  ptc_stage_rows<D, QT>(sQ, C::LBO_Q, p.Q + zf, m0, N);
  ptc_stage_rows<D, TN>(sK, C::LBO_K, p.K + zf, 0, N);
  float vreg[D / 16][4];
  ptc_load_v<D, TN>(vreg, p.V + zf, 0, N);
  float xq[PS];
  ptc_point<PER>(p.X + zp, m0 + row, N, p, xq);
  tc::fence_async_smem();
  __syncthreads();

  const uint32_t q_addr = tc::smem_u32(sQ), k_addr = tc::smem_u32(sK), v_addr = tc::smem_u32(sV), p_addr = tc::smem_u32(sP);
  const int ntiles = (N + TN - 1) / TN;
  bool ok = true;
  for (int t = 0; t < ntiles && ok; t++) {
    const int n0 = t * TN;
    if (tid == 0) {   // K of this step is in shared memory (prologue, or the asynchronous copies of the previous step)
      tc::fence_after_sync();
#pragma unroll
      for (int ks = 0; ks < D / 8; ks++) {
        const uint64_t ad = tc::smem_desc(q_addr + ks * 2 * C::LBO_Q, C::LBO_Q, 128);
        const uint64_t bd = tc::smem_desc(k_addr + ks * 2 * C::LBO_K, C::LBO_K, 128);
        mma_tf32(tmem_s, ad, bd, idesc_tf32(QT, TN), ks > 0 ? 1u : 0u);
      }
      tc::mma_commit(bar_s);
    }
    if (t > 0) {   // the second product of the previous step still reads sP and sV
      const bool w = tc::mbar_wait(bar_o, (t - 1) & 1);
      ok = __syncthreads_and(w);
      if (!ok) break;
    }
    ptc_store_v<D, TN>(sV, C::LBO_V, vreg);   // loaded during the weights of the previous step
    if (tid < TN) ptc_point<PER>(p.Y + zp, n0 + tid, N, p, sY + tid * PS);
    {
      const bool w = tc::mbar_wait(bar_s, t & 1);
      ok = __syncthreads_and(w);   // also orders the position stores before the weights below
      if (!ok) break;
    }
    if (t + 1 < ntiles) {   // sK is free; both land during the weights
      ptc_stage_rows_async<D, TN>(k_addr, C::LBO_K, p.K + zf, n0 + TN, N);
      ptc_load_v<D, TN>(vreg, p.V + zf, n0 + TN, N);
    }
    tc::fence_after_sync();
#pragma unroll
    for (int c0 = 0; c0 < TNH; c0 += 32) {
      float s[32];
      tc::tmem_ld32(tmem_s + lane_bits + half * TNH + c0, s);
#pragma unroll
      for (int c = 0; c < 32; c += 4) {
        const int n = half * TNH + c0 + c;
        float4 o;
        o.x = to_tf32(s[c + 0] * ptc_weight<PER>(xq, sY + (n + 0) * PS, r0sq, kc));
        o.y = to_tf32(s[c + 1] * ptc_weight<PER>(xq, sY + (n + 1) * PS, r0sq, kc));
        o.z = to_tf32(s[c + 2] * ptc_weight<PER>(xq, sY + (n + 2) * PS, r0sq, kc));
        o.w = to_tf32(s[c + 3] * ptc_weight<PER>(xq, sY + (n + 3) * PS, r0sq, kc));
        *reinterpret_cast<float4*>(sP + (size_t)(n >> 2) * C::LBO_P + row * 16) = o;
      }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    tc::fence_async_smem();
    tc::fence_before_sync();
    __syncthreads();
    if (tid == 0) {
      tc::fence_after_sync();
#pragma unroll
      for (int ks = 0; ks < TN / 8; ks++) {
        const uint64_t ad = tc::smem_desc(p_addr + ks * 2 * C::LBO_P, C::LBO_P, 128);
        const uint64_t bd = tc::smem_desc(v_addr + ks * 2 * C::LBO_V, C::LBO_V, 128);
        mma_tf32(tmem_o, ad, bd, idesc_tf32(QT, D), (t > 0 || ks > 0) ? 1u : 0u);
      }
      tc::mma_commit(bar_o);
    }
  }
  if (ok && ntiles > 0) {
    const bool w = tc::mbar_wait(bar_o, (ntiles - 1) & 1);
    ok = __syncthreads_and(w);
  }
  if (ok) {
    tc::fence_after_sync();
    const int m = m0 + row;
#pragma unroll
    for (int c0 = 0; c0 < D / 2; c0 += 8) {
      float o[8];
      tc::tmem_ld8(tmem_o + lane_bits + half * (D / 2) + c0, o);
      if (m < N) {
        float4* dst = reinterpret_cast<float4*>(p.out + zf + (size_t)m * D + half * (D / 2) + c0);
        dst[0] = make_float4(o[0], o[1], o[2], o[3]);
        dst[1] = make_float4(o[4], o[5], o[6], o[7]);
      }
    }
  } else if (tid == 0 && p.status != nullptr) {
    atomicOr(p.status, LD_FLAG_TIMEOUT);
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem_base, C::TMEM_COLS);
}

template <int D, bool PER>
int ptc_launch(const PtcArgs& a, int Z, cudaStream_t st) {
  constexpr int sm = Ptc<D>::SMEM;
  static_assert(sm <= 227 * 1024, "shared memory of the proximity attention tile");
  LD_CUDA_TRY(cudaFuncSetAttribute(proxattn_fwd_tc_kernel<D, PER>, cudaFuncAttributeMaxDynamicSharedMemorySize, sm));
  proxattn_fwd_tc_kernel<D, PER><<<dim3((a.N + QT - 1) / QT, Z), PTC_THREADS, sm, st>>>(a);
  LD_LAUNCH_CHECK();
  return LD_OK;
}

template <bool PER>
int ptc_dispatch(const PtcArgs& a, int Z, int dim, cudaStream_t st) {
  switch (dim) {
    case 16: return ptc_launch<16, PER>(a, Z, st);
    case 32: return ptc_launch<32, PER>(a, Z, st);
    case 64: return ptc_launch<64, PER>(a, Z, st);
    case 128: return ptc_launch<128, PER>(a, Z, st);
  }
  ld_set_last_message("proximity attention: dim must be 16, 32, 64 or 128");
  return LD_ERR_UNSUPPORTED;
}

}  // namespace

extern "C" int ld_proxattn_fwd_tf32_tc(const float* Q, const float* K, const float* V, const float* X, const float* Y,
                                       const float* r0sq, int heads, int Z, int N, int dim, int periodic, float box_x, float box_y,
                                       float box_z, float* out, int* status_dev, void* stream) {
  if (heads <= 0 || Z < 0 || N < 0 || Z % heads != 0 || Z > 65535) return LD_ERR_SHAPE;
  if (periodic && !(box_x > 0.f && box_y > 0.f && box_z > 0.f)) return LD_ERR_SHAPE;
  if (Z == 0 || N == 0) return LD_OK;
  PtcArgs a{};
  a.Q = Q; a.K = K; a.V = V; a.X = X; a.Y = Y; a.r0sq = r0sq; a.out = out; a.status = status_dev; a.heads = heads; a.N = N;
  a.lx = box_x; a.ly = box_y; a.lz = box_z;
  return periodic ? ptc_dispatch<true>(a, Z, dim, (cudaStream_t)stream) : ptc_dispatch<false>(a, Z, dim, (cudaStream_t)stream);
}
