// Front half of the node-local l<=2 products (SelfTensProds.forward of the reference, archs/diffuser_atoms15.py:59-95)
// in one launch: the six channel mixings L0, L1, L2, R0, R1, R2 (TensLinear of ranks 0, 1, 2 to `chan` = 128 channels,
// left and right weights stacked) and the thirteen Bee products of their results
// (managan/codegen_tensor_products.py:64-75), written in the form the Y maps read:
//   P_a [Nt][3*chan] FP32 = (000 | 110 | 220), P_v [Nt][3][5*chan] BF16 = (011 | 101 | 121 | 211 | 111),
//   P_d [Nt][9][5*chan] BF16 = (022 | 202 | 112 | 222 | 212), component-major.
// As separate launches the stacked mixings write 13 KB of FP32 per node (with element strides of 3 and 9 floats) that
// the product kernel reads back at once; here they never leave the SM. A block owns 64 nodes: its threads read the
// nodes' feature rows with 16-byte loads, round to BF16 and store them component by component as K-major operand
// tiles (the transposition happens in registers); for every 16 nodes, 26 small GEMMs are issued TRANSPOSED (the left
// or right weights of a rank as the M operand, 16 nodes of one Cartesian component as the N operand): 26
// accumulators of 16 tensor-memory columns, a lane = a channel. Thread c then holds all thirteen left and right
// values of (node, c) for four nodes at a time, forms the products in FP32 (ld_hotpath's bee_fwd_point) and stores
// them; consecutive lanes are consecutive addresses of every output row.
// Every wait is bounded; a wait that runs out sets LD_FLAG_TIMEOUT and the block leaves.
#include "common.cuh"
#include "tc05.cuh"
#include "tp_math.h"

namespace {

constexpr int SF_NODES = 64;      // nodes per tile
constexpr int SF_SUB = 16;        // nodes per group of GEMMs (N of the MMAs)
constexpr int SF_C = 128;         // channels (M of the MMAs)
constexpr int SF_THREADS = 128;
constexpr int SF_PANEL = SF_NODES * 16;        // bytes of one 8-wide K panel of a 64-row operand tile
constexpr int SF_WPANEL = 2 * SF_C * 16;       // bytes of one K panel of the stacked weights (256 rows)

struct SelfFrontParams {
  const float* xa; const float* xv; const float* xd;   // [Nt][da], [Nt][dv][3], [Nt][dd][9]
  long long Nt;
  int da, dv, dd;
  const __nv_bfloat16* w0; const __nv_bfloat16* w1; const __nv_bfloat16* w2;   // packed panels [K/8][256][8] (left | right)
  float* P_a; __nv_bfloat16* P_v; __nv_bfloat16* P_d;
  int* status;
  uint32_t wait_limit;
};

__device__ __forceinline__ uint4 sf_pack8(const float* v) {
  uint4 q;
  q.x = tc::pack_bf16x2(v[0], v[1]); q.y = tc::pack_bf16x2(v[2], v[3]);
  q.z = tc::pack_bf16x2(v[4], v[5]); q.w = tc::pack_bf16x2(v[6], v[7]);
  return q;
}

// eight channels x S components of one node (8 * S consecutive floats) -> S pieces of eight BF16 values, one per
// component, each stored as this node's 16 bytes of panel `g` of that component's operand tile
template <int S>
__device__ __forceinline__ void sf_stage_group(const float* __restrict__ src, bool ok, unsigned char* tile0, int comp_bytes, int g,
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
    *reinterpret_cast<uint4*>(tile0 + (size_t)s * comp_bytes + (size_t)g * SF_PANEL + row * 16) = sf_pack8(c8);
  }
}

__global__ void __launch_bounds__(SF_THREADS, 1)
bee_self_front_kernel(const __grid_constant__ SelfFrontParams P) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t bar_w, bar_acc;
  __shared__ uint32_t tmem_slot;

  const int tid = threadIdx.x, warp = tid >> 5;
  const int da = P.da, dv = P.dv, dd = P.dd;
  // operand tiles of the thirteen components, then the three stacked weight matrices
  const int a_bytes = (da / 8) * SF_PANEL, v_bytes = (dv / 8) * SF_PANEL, d_bytes = (dd / 8) * SF_PANEL;
  unsigned char* t_a = smem;
  unsigned char* t_v = t_a + a_bytes;
  unsigned char* t_d = t_v + 3 * v_bytes;
  unsigned char* w_a = t_d + 9 * d_bytes;
  unsigned char* w_v = w_a + (da / 8) * SF_WPANEL;
  unsigned char* w_d = w_v + (dv / 8) * SF_WPANEL;
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
    const uint32_t b0 = (uint32_t)(da / 8) * SF_WPANEL, b1 = (uint32_t)(dv / 8) * SF_WPANEL, b2 = (uint32_t)(dd / 8) * SF_WPANEL;
    tc::mbar_expect_tx(&bar_w, b0 + b1 + b2);
    tc::bulk_g2s(w_a, P.w0, b0, &bar_w);
    tc::bulk_g2s(w_v, P.w1, b1, &bar_w);
    tc::bulk_g2s(w_d, P.w2, b2, &bar_w);
  }
  const long long ntiles = (P.Nt + SF_NODES - 1) / SF_NODES;
  const uint32_t idesc = tc::idesc_bf16(SF_C, SF_SUB);
  uint32_t acc_phase = 0;
  bool ok = true, have_w = false;
  const int c = tid;                                       // this thread's channel when it forms products
  const uint32_t t_lane = tmem_base + ((uint32_t)(warp * 32) << 16);

  for (long long tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
    // ---- 1. two threads per node: feature rows -> BF16 operand tiles, component-major (the halves take alternate groups)
    {
      const int row = tid & (SF_NODES - 1), half = tid >> 6;
      const long long node = tile * SF_NODES + row;
      const bool node_ok = node < P.Nt;
      const long long nc = node_ok ? node : 0;
      const float* xa = P.xa + nc * da;
      for (int g = half; g < da / 8; g += 2) sf_stage_group<1>(xa + g * 8, node_ok, t_a, a_bytes, g, row);
      const float* xv = P.xv + nc * dv * 3;
      for (int g = half; g < dv / 8; g += 2) sf_stage_group<3>(xv + g * 24, node_ok, t_v, v_bytes, g, row);
      const float* xd = P.xd + nc * dd * 9;
      for (int g = half; g < dd / 8; g += 2) sf_stage_group<9>(xd + g * 72, node_ok, t_d, d_bytes, g, row);
    }
    tc::fence_async_smem();
    tc::fence_before_sync();
    __syncthreads();
    const int nvalid = (int)min((long long)SF_NODES, P.Nt - tile * SF_NODES);
    // ---- 2. per 16 nodes: 26 GEMMs (left and right of the thirteen components), then the products ----------------------
    for (int sub = 0; sub < SF_NODES / SF_SUB && ok; sub++) {
      if (sub * SF_SUB >= nvalid) break;
      if (tid == 0) {
        if (!have_w) { have_w = tc::mbar_wait(&bar_w, 0, wl); }
        if (have_w) {
          tc::fence_after_sync();
#pragma unroll 1
          for (int m = 0; m < 13; m++) {                        // slot: 0 = rank 0, 1..3 = rank 1, 4..12 = rank 2
            const unsigned char* a_tile = m == 0 ? t_a : (m < 4 ? t_v + (size_t)(m - 1) * v_bytes : t_d + (size_t)(m - 4) * d_bytes);
            const unsigned char* w_tile = m == 0 ? w_a : (m < 4 ? w_v : w_d);
            const int K = m == 0 ? da : (m < 4 ? dv : dd);
            uint64_t wd = tc::smem_desc(tc::smem_u32(w_tile), SF_WPANEL, 128);
            uint64_t xd = tc::smem_desc(tc::smem_u32(a_tile) + sub * SF_SUB * 16, SF_PANEL, 128);
            for (int ks = 0; ks < K / 16; ks++) {
              tc::mma_bf16(tmem_base + (2 * m) * SF_SUB, wd, xd, idesc, ks > 0 ? 1u : 0u);                              // left
              tc::mma_bf16(tmem_base + (2 * m + 1) * SF_SUB, wd + (uint64_t)((SF_C * 16) >> 4), xd, idesc, ks > 0 ? 1u : 0u);   // right
              wd += (uint64_t)((2 * SF_WPANEL) >> 4);           // the address field of a descriptor counts 16-byte units
              xd += (uint64_t)((2 * SF_PANEL) >> 4);
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
      // thread = channel (its tensor-memory lane); four nodes (columns) at a time
#pragma unroll 1
      for (int q = 0; q < SF_SUB / 4; q++) {
        const int n0 = sub * SF_SUB + q * 4;
        if (n0 >= nvalid) break;
        float v[26][4];
#pragma unroll
        for (int a = 0; a < 26; a++) tc::tmem_ld4(t_lane + a * SF_SUB + q * 4, v[a]);
#pragma unroll
        for (int i = 0; i < 4; i++) {
          if (n0 + i >= nvalid) break;
          float l1[3], r1[3], l2[9], r2[9];
#pragma unroll
          for (int x = 0; x < 3; x++) { l1[x] = v[2 + 2 * x][i]; r1[x] = v[3 + 2 * x][i]; }
#pragma unroll
          for (int x = 0; x < 9; x++) { l2[x] = v[8 + 2 * x][i]; r2[x] = v[9 + 2 * x][i]; }
          BeeOut o;
          bee_fwd_point(v[0][i], l1, l2, v[1][i], r1, r2, &o);
          const size_t node = (size_t)tile * SF_NODES + n0 + i;
          float* pa = P.P_a + node * 3 * SF_C + c;
          pa[0] = o.y000; pa[SF_C] = o.y110; pa[2 * SF_C] = o.y220;
          __nv_bfloat16* pv = P.P_v + node * 3 * 5 * SF_C + c;
          __nv_bfloat16* pd = P.P_d + node * 9 * 5 * SF_C + c;
          const float* vs[5] = {o.y011, o.y101, o.y121, o.y211, o.y111};
          const float* ds[5] = {o.y022, o.y202, o.y112, o.y222, o.y212};
#pragma unroll
          for (int k = 0; k < 5; k++) {
#pragma unroll
            for (int x = 0; x < 3; x++) pv[(size_t)x * 5 * SF_C + k * SF_C] = __float2bfloat16_rn(vs[k][x]);
#pragma unroll
            for (int x = 0; x < 9; x++) pd[(size_t)x * 5 * SF_C + k * SF_C] = __float2bfloat16_rn(ds[k][x]);
          }
        }
      }
      tc::fence_before_sync();
      __syncthreads();   // the accumulators are free for the next 16 nodes (after the last: the tiles for the next nodes)
    }
  }
  if (!ok && tid == 0 && P.status != nullptr) atomicOr(P.status, LD_FLAG_TIMEOUT);
  // the weight copies were waited for before the first MMA; a block without tiles waits for them here (bounded)
  if (tid == 0 && !have_w) tc::mbar_wait(&bar_w, 0, wl);
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem_base, 512);
}

}  // namespace

// x_a [Nt][da], x_v [Nt][dv][3], x_d [Nt][dd][3][3] FP32 contiguous; LR0p, LR1p, LR2p from ld_pack_weights_bf16 for the
// stacked weight matrices [2*128][da], [2*128][dv], [2*128][dd] (left rows first). chan = 128; da, dv, dd multiples of 16
// with da + 3 dv + 9 dd <= 640. Outputs as ld_bee_self_products with out_bf16 = 1. BF16 operands, FP32 accumulation
// and FP32 products: the values of the three tensor-core linears followed by ld_bee_self_products.
extern "C" int ld_bee_self_front_bf16_tc(const float* x_a, const float* x_v, const float* x_d, long long Nt, int da, int dv, int dd,
                                         int chan, const void* LR0p, const void* LR1p, const void* LR2p, float* P_a, void* P_v,
                                         void* P_d, int* status_dev, void* stream) {
  if (Nt < 0 || da <= 0 || dv <= 0 || dd <= 0) return LD_ERR_SHAPE;
  if (chan != SF_C || da % 16 || dv % 16 || dd % 16 || da + 3 * dv + 9 * dd > 640) {
    ld_set_last_message("node-local products in one launch: chan = 128, widths multiples of 16, da + 3 dv + 9 dd <= 640");
    return LD_ERR_UNSUPPORTED;
  }
  if ((((uintptr_t)x_a | (uintptr_t)x_v | (uintptr_t)x_d | (uintptr_t)LR0p | (uintptr_t)LR1p | (uintptr_t)LR2p) % 16) != 0) return LD_ERR_SHAPE;
  if (Nt == 0) return LD_OK;
  SelfFrontParams P;
  P.xa = x_a; P.xv = x_v; P.xd = x_d; P.Nt = Nt; P.da = da; P.dv = dv; P.dd = dd;
  P.w0 = (const __nv_bfloat16*)LR0p; P.w1 = (const __nv_bfloat16*)LR1p; P.w2 = (const __nv_bfloat16*)LR2p;
  P.P_a = P_a; P.P_v = (__nv_bfloat16*)P_v; P.P_d = (__nv_bfloat16*)P_d; P.status = status_dev; P.wait_limit = tc::TC_WAIT_LIMIT;
  const size_t smem = (size_t)(da / 8 + 3 * (dv / 8) + 9 * (dd / 8)) * SF_PANEL + (size_t)(da / 8 + dv / 8 + dd / 8) * SF_WPANEL + 1024;
  LD_CUDA_TRY(cudaFuncSetAttribute(bee_self_front_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long ntiles = (Nt + SF_NODES - 1) / SF_NODES;
  bee_self_front_kernel<<<(int)(ntiles < sms ? ntiles : sms), SF_THREADS, smem, (cudaStream_t)stream>>>(P);
  LD_LAUNCH_CHECK();
  return LD_OK;
}
