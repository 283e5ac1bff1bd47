// The three channel mixings L0, L1, L2 of an l<=2 message layer (Messages.forward of the reference,
// archs/diffuser_atoms15.py:244-246: TensLinear of ranks 0, 1, 2 to `chan` = 128 channels) in ONE launch that writes the
// neighbour rows the edge kernels gather, [node][chan][16] BF16 = (l0, l1[3], l2[9], three zeros), as whole rows.
//
// As three launches of the general tensor-core linear the rows are written 2, 6 and 18 bytes at a time at a 32-byte
// stride: every launch moves the whole buffer through L2 and DRAM as partially written sectors, which costs more
// than the arithmetic and the inputs together. Here a block owns 128 nodes: each thread reads its node's three
// feature rows with 16-byte loads (they are contiguous per node: [K][3^l] floats), rounds them to BF16 and stores
// them component by component as K-major operand tiles (eight channels of one component are one 16-byte piece: the
// transposition happens in registers); for every 32 nodes thirteen small GEMMs follow, one per Cartesian component,
// issued TRANSPOSED (weights as the M operand, 32 nodes as the N operand), so that a tensor-memory lane is an output
// channel and a column a node: 13 accumulators of 32 columns. Thread c then holds all thirteen values of (node, c),
// packs them into the 32-byte row, and the warp's 32 rows of a node (1 KB of consecutive addresses) leave as two
// fully coalesced stores after a transposition through a per-warp staging buffer: every sector is written once, whole.
// Every wait is bounded; a wait that runs out sets LD_FLAG_TIMEOUT and the block leaves.
#include "common.cuh"
#include "tc05.cuh"

namespace {

constexpr int LR_NODES = 128;     // nodes per tile
constexpr int LR_SUB = 32;        // nodes per group of GEMMs (N of the MMAs)
constexpr int LR_C = 128;         // output channels (M of the MMAs)
constexpr int LR_THREADS = 128;
constexpr int LR_PANEL = LR_NODES * 16;   // bytes of one 8-wide K panel of a 128-row operand

struct LeftRowsParams {
  const float* xa; const float* xv; const float* xd;   // [Nt][da], [Nt][dv][3], [Nt][dd][9]
  long long Nt;
  int da, dv, dd;
  const __nv_bfloat16* w0; const __nv_bfloat16* w1; const __nv_bfloat16* w2;   // packed panels [K/8][128][8]
  __nv_bfloat16* rows;       // [Nt][128][16]
  int* status;
  uint32_t wait_limit;
};

__device__ __forceinline__ uint4 lr_pack8(const float* v) {
  uint4 q;
  q.x = tc::pack_bf16x2(v[0], v[1]); q.y = tc::pack_bf16x2(v[2], v[3]);
  q.z = tc::pack_bf16x2(v[4], v[5]); q.w = tc::pack_bf16x2(v[6], v[7]);
  return q;
}

// eight channels x S components of one node (8 * S consecutive floats) -> S pieces of eight BF16 values, one per
// component, each stored as this node's 16 bytes of panel `g` of that component's operand tile
template <int S>
__device__ __forceinline__ void lr_stage_group(const float* __restrict__ src, bool ok, unsigned char* tile0, int comp_bytes, int g,
                                               int row) {
  float v[8 * S];
#pragma unroll
  for (int i = 0; i < 2 * S; i++) {
    const float4 q = ok ? __ldg(reinterpret_cast<const float4*>(src) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    v[4 * i] = q.x; v[4 * i + 1] = q.y; v[4 * i + 2] = q.z; v[4 * i + 3] = q.w;
  }
#pragma unroll
  for (int s = 0; s < S; s++) {
    float c8[8];
#pragma unroll
    for (int i = 0; i < 8; i++) c8[i] = v[i * S + s];
    *reinterpret_cast<uint4*>(tile0 + (size_t)s * comp_bytes + (size_t)g * LR_PANEL + row * 16) = lr_pack8(c8);
  }
}

__global__ void __launch_bounds__(LR_THREADS, 1)
bee_left_rows_kernel(const __grid_constant__ LeftRowsParams P) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t bar_w, bar_acc;
  __shared__ uint32_t tmem_slot;
  __shared__ __align__(16) unsigned char s_stage[LR_THREADS / 32][1024];   // per warp: 32 rows of 32 bytes on their way out

  const int tid = threadIdx.x, warp = tid >> 5;
  const int da = P.da, dv = P.dv, dd = P.dd;
  // operand tiles of the thirteen components, then the three weight matrices
  const int a_bytes = (da / 8) * LR_PANEL, v_bytes = (dv / 8) * LR_PANEL, d_bytes = (dd / 8) * LR_PANEL;
  unsigned char* t_a = smem;
  unsigned char* t_v = t_a + a_bytes;
  unsigned char* t_d = t_v + 3 * v_bytes;
  unsigned char* w_a = t_d + 9 * d_bytes;
  unsigned char* w_v = w_a + (da / 8) * (LR_C * 16);
  unsigned char* w_d = w_v + (dv / 8) * (LR_C * 16);
  const uint32_t wl = P.wait_limit;

  if (tid == 0) {
    tc::mbar_init(&bar_w, 1);
    tc::mbar_init(&bar_acc, 1);
    tc::mbar_init_fence();
  }
  if (warp == 0) { tc::tmem_alloc(&tmem_slot, 512); tc::tmem_relinquish(); }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  if (tid == 0) {
    const uint32_t b0 = (uint32_t)(da / 8) * LR_C * 16, b1 = (uint32_t)(dv / 8) * LR_C * 16, b2 = (uint32_t)(dd / 8) * LR_C * 16;
    tc::mbar_expect_tx(&bar_w, b0 + b1 + b2);
    tc::bulk_g2s(w_a, P.w0, b0, &bar_w);
    tc::bulk_g2s(w_v, P.w1, b1, &bar_w);
    tc::bulk_g2s(w_d, P.w2, b2, &bar_w);
  }
  const long long ntiles = (P.Nt + LR_NODES - 1) / LR_NODES;
  const uint32_t idesc = tc::idesc_bf16(LR_C, LR_SUB);
  uint32_t acc_phase = 0;
  bool ok = true, have_w = false;

  for (long long tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
    // ---- 1. this thread's node: three feature rows -> BF16 operand tiles, component-major ---------------------------
    const long long node = tile * LR_NODES + tid;
    const bool node_ok = node < P.Nt;
    const long long nc = node_ok ? node : 0;
    {
      const float* xa = P.xa + nc * da;
      for (int g = 0; g < da / 8; g++) lr_stage_group<1>(xa + g * 8, node_ok, t_a, a_bytes, g, tid);
      const float* xv = P.xv + nc * dv * 3;
      for (int g = 0; g < dv / 8; g++) lr_stage_group<3>(xv + g * 24, node_ok, t_v, v_bytes, g, tid);
      const float* xd = P.xd + nc * dd * 9;
      for (int g = 0; g < dd / 8; g++) lr_stage_group<9>(xd + g * 72, node_ok, t_d, d_bytes, g, tid);
    }
    tc::fence_async_smem();
    tc::fence_before_sync();
    __syncthreads();
    // ---- 2. per 32 nodes: thirteen GEMMs into 13 x 32 tensor-memory columns, then whole 32-byte rows ---------------
    const int nvalid = (int)min((long long)LR_NODES, P.Nt - tile * LR_NODES);
    for (int sub = 0; sub < LR_NODES / LR_SUB && ok; sub++) {
      if (sub * LR_SUB >= nvalid) break;
      if (tid == 0) {
        if (!have_w) { have_w = tc::mbar_wait(&bar_w, 0, wl); }
        if (have_w) {
          tc::fence_after_sync();
#pragma unroll 1
          for (int m = 0; m < 13; m++) {                      // slot of the row: 0 = l0, 1..3 = l1, 4..12 = l2
            const unsigned char* a_tile = m == 0 ? t_a : (m < 4 ? t_v + (size_t)(m - 1) * v_bytes : t_d + (size_t)(m - 4) * d_bytes);
            const unsigned char* w_tile = m == 0 ? w_a : (m < 4 ? w_v : w_d);
            const int K = m == 0 ? da : (m < 4 ? dv : dd);
            uint64_t wd = tc::smem_desc(tc::smem_u32(w_tile), LR_C * 16, 128);
            uint64_t xd = tc::smem_desc(tc::smem_u32(a_tile) + sub * LR_SUB * 16, LR_PANEL, 128);
            for (int ks = 0; ks < K / 16; ks++) {
              tc::mma_bf16(tmem_base + m * LR_SUB, wd, xd, idesc, ks > 0 ? 1u : 0u);
              wd += (uint64_t)((2 * LR_C * 16) >> 4);         // the address field of a descriptor counts 16-byte units
              xd += (uint64_t)((2 * LR_PANEL) >> 4);
            }
          }
          tc::mma_commit(&bar_acc);
        }
      }
      ok = tc::mbar_wait(&bar_acc, acc_phase & 1, wl);
      acc_phase++;
      ok = __syncthreads_and(ok);
      if (!ok) break;
      tc::fence_after_sync();
      // thread = channel (its tensor-memory lane); columns = nodes. Eight nodes at a time: the thirteen values of
      // (node, channel) become one 32-byte row; a warp's 32 rows of a node are 1 KB of consecutive addresses, written
      // as two fully coalesced 512-byte stores after a transposition through the warp's staging buffer.
      const uint32_t t_lane = tmem_base + ((uint32_t)(warp * 32) << 16);
      const int lane = tid & 31;
      unsigned char* stage = s_stage[warp];
#pragma unroll 1
      for (int q = 0; q < LR_SUB / 8; q++) {
        const int n0 = sub * LR_SUB + q * 8;
        if (n0 >= nvalid) break;
        float v[13][8];
#pragma unroll
        for (int m = 0; m < 13; m++) tc::tmem_ld8_issue(t_lane + m * LR_SUB + q * 8, v[m]);
        tc::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 8; i++) {
          if (n0 + i >= nvalid) break;
          uint4 lo, hi;
          lo.x = tc::pack_bf16x2(v[0][i], v[1][i]);   lo.y = tc::pack_bf16x2(v[2][i], v[3][i]);
          lo.z = tc::pack_bf16x2(v[4][i], v[5][i]);   lo.w = tc::pack_bf16x2(v[6][i], v[7][i]);
          hi.x = tc::pack_bf16x2(v[8][i], v[9][i]);   hi.y = tc::pack_bf16x2(v[10][i], v[11][i]);
          hi.z = tc::pack_bf16x2(v[12][i], 0.f);      hi.w = 0u;                       // the three unused values of a row
          *reinterpret_cast<uint4*>(stage + lane * 32) = lo;
          *reinterpret_cast<uint4*>(stage + lane * 32 + 16) = hi;
          __syncwarp();
          const uint4 p0 = *reinterpret_cast<const uint4*>(stage + lane * 16);
          const uint4 p1 = *reinterpret_cast<const uint4*>(stage + 512 + lane * 16);
          unsigned char* out = reinterpret_cast<unsigned char*>(P.rows) + ((size_t)(tile * LR_NODES + n0 + i) * LR_C + warp * 32) * 32;
          *reinterpret_cast<uint4*>(out + lane * 16) = p0;
          *reinterpret_cast<uint4*>(out + 512 + lane * 16) = p1;
          __syncwarp();
        }
      }
      tc::fence_before_sync();
      __syncthreads();   // the accumulators are free for the next 32 nodes (after the last: the tiles for the next nodes)
    }
  }
  if (!ok && tid == 0 && P.status != nullptr) atomicOr(P.status, LD_FLAG_TIMEOUT);
  // the weight copies were waited for before the first MMA; a block without tiles waits for them here (bounded)
  if (tid == 0 && !have_w) tc::mbar_wait(&bar_w, 0, wl);
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem_base, 512);
}

}  // namespace

// rows [Nt][128][16] BF16 = (L0 x_a, L1 x_v [3], L2 x_d [9], 0, 0, 0) per (node, channel).
// x_a [Nt][da], x_v [Nt][dv][3], x_d [Nt][dd][3][3] FP32 contiguous; W0p, W1p, W2p from ld_pack_weights_bf16 for the
// [128][da], [128][dv], [128][dd] weight matrices. da, dv, dd multiples of 16 with da + 3 dv + 9 dd <= 640; chan = 128.
// BF16 operands, FP32 accumulation: the same values as three ld_linear_bf16_tc_out16 launches into the same buffer.
extern "C" int ld_bee_left_rows_bf16_tc(const float* x_a, const float* x_v, const float* x_d, long long Nt, int da, int dv, int dd,
                                        int chan, const void* W0p, const void* W1p, const void* W2p, void* rows, int* status_dev,
                                        void* stream) {
  if (Nt < 0 || da <= 0 || dv <= 0 || dd <= 0) return LD_ERR_SHAPE;
  if (chan != LR_C || da % 16 || dv % 16 || dd % 16 || da + 3 * dv + 9 * dd > 640) {
    ld_set_last_message("left rows of the l<=2 layer in one launch: chan = 128, widths multiples of 16, da + 3 dv + 9 dd <= 640");
    return LD_ERR_UNSUPPORTED;
  }
  if ((((uintptr_t)x_a | (uintptr_t)x_v | (uintptr_t)x_d | (uintptr_t)W0p | (uintptr_t)W1p | (uintptr_t)W2p | (uintptr_t)rows) % 16) != 0)
    return LD_ERR_SHAPE;
  if (Nt == 0) return LD_OK;
  LeftRowsParams P;
  P.xa = x_a; P.xv = x_v; P.xd = x_d; P.Nt = Nt; P.da = da; P.dv = dv; P.dd = dd;
  P.w0 = (const __nv_bfloat16*)W0p; P.w1 = (const __nv_bfloat16*)W1p; P.w2 = (const __nv_bfloat16*)W2p;
  P.rows = (__nv_bfloat16*)rows; P.status = status_dev; P.wait_limit = tc::TC_WAIT_LIMIT;
  const size_t smem = (size_t)(da / 8 + 3 * (dv / 8) + 9 * (dd / 8)) * LR_PANEL + (size_t)(da / 8 + dv / 8 + dd / 8) * (LR_C * 16) + 1024;
  LD_CUDA_TRY(cudaFuncSetAttribute(bee_left_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long ntiles = (Nt + LR_NODES - 1) / LR_NODES;
  bee_left_rows_kernel<<<(int)(ntiles < sms ? ntiles : sms), LR_THREADS, smem, (cudaStream_t)stream>>>(P);
  LD_LAUNCH_CHECK();
  return LD_OK;
}
