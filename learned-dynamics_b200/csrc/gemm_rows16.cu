// Channel mixing of BF16 rows on the Blackwell tensor cores, as a streaming kernel:
//   y[(r,s), o] = act( sum_i W[o,i] * x16[(r,s), i] + b[o] ),   x16 [rows_outer][S][K] BF16 (K contiguous), y [rows_outer][N][S] FP32
// (the reference's tensor_linear, extensions/tensor_ops/tensor_ops_kern.cu:6-42, for activations kept component-major
// in BF16: the per-node product sums of the l<=2 layers, K = 5 * chan, N = dim_v or dim_d).
//
// These are tall, thin matrices (millions of rows, K = 640, N = 32..128): the work is reading x16 once, 1280 bytes
// per row against 2 K N flops. One persistent block per SM keeps the whole packed weight matrix in shared memory
// (loaded once by a bulk copy) and streams 128-row tiles through a ring of 128-wide K chunks:
//   warps 4..7   one thread per row issues sixteen 16-byte cp.async copies per chunk straight into the K-major operand
//                layout (a row's eight K values are exactly one 16-byte piece of it) and lets the chunk's mbarrier
//                count their completion: three or four chunks (96 or 128 KB per SM) are in flight without a register holding data;
//   warp 8       one thread waits for a chunk, issues its eight MMAs (128 x N x 16) and commits the chunk back to the
//                loaders; the accumulators of two tiles alternate in tensor memory;
//   warps 0..3   read a finished tile's accumulators (a thread = a row = a tensor-memory lane), add the bias, apply the
//                activation and store, while the next tile is already being multiplied.
// BF16 operands, FP32 accumulation: the same products and sums as ld_linear_bf16_tc_in16's general kernel.
// Every wait is bounded; a wait that runs out sets LD_FLAG_TIMEOUT and all roles leave.
#include "common.cuh"
#include "tc05.cuh"
#include "tp_math.h"

namespace {

constexpr int GR_ROWS = 128;
constexpr int GR_KC = 128;                       // K per chunk of the activation ring (the packed weights come in 64-wide chunks)
constexpr int GR_STAGE_BYTES = GR_ROWS * GR_KC * 2;   // 32768
constexpr int GR_STAGES = 4;
constexpr int GR_EPI_WARPS = 4, GR_LOAD_WARPS = 4;
constexpr int GR_MMA_WARP = GR_EPI_WARPS + GR_LOAD_WARPS;          // 8
constexpr int GR_THREADS = (GR_MMA_WARP + 1) * 32;                 // 288
constexpr int GR_MAX_W_BYTES = 94 * 1024;

struct RowsParams {
  const __nv_bfloat16* x; float* y;
  const __nv_bfloat16* wp;   // packed weights [nchunks][8 panels][N][8]
  const float* bias;
  const float* res;          // optional residual, laid out like y: y = res + act(...)
  long long rows;            // GEMM rows = rows_outer * S
  int K, N, S, act;
  int stages;                // chunks of the ring in use (<= GR_STAGES)
  int* status;
  uint32_t wait_limit;
};

__device__ __forceinline__ float gr_act(float v, int act) {
  if (act == 1) return silu_f(v);
  if (act == 2) return v > 0.f ? v : 0.1f * v;
  return v;
}

// 16 bytes global -> shared without a register in between; src_bytes = 0 writes zeros. A thread's consecutive copies
// take the two halves of every 32-byte sector: through L1 (.ca) the second half is a hit, which halves the L2 -> SM
// traffic, as long as the block's shared memory leaves L1 room for the lines in flight (the launch sizes the ring for it).
__device__ __forceinline__ void gr_cp_async16(void* dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(tc::smem_u32(dst)), "l"(src), "r"(src_bytes) : "memory");
}
// the mbarrier receives one arrival from this thread once all its cp.async copies issued so far have landed
__device__ __forceinline__ void gr_cp_async_arrive(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(tc::smem_u32(bar)) : "memory");
}

__global__ void __launch_bounds__(GR_THREADS, 1)
gemm_rows16_kernel(const __grid_constant__ RowsParams P) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t bar_full[GR_STAGES], bar_empty[GR_STAGES], bar_acc_full[2], bar_acc_empty[2], bar_w;
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int s_fail;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int N = P.N, K = P.K, S = P.S;
  const int nchunks = K / GR_KC;
  const uint32_t w_bytes = (uint32_t)K * N * 2;
  unsigned char* w_smem = smem;
  unsigned char* ring = smem + ((w_bytes + 1023u) & ~1023u);
  const uint32_t wl = P.wait_limit, nst = (uint32_t)P.stages;
  uint32_t acc_cols = 32;
  while (acc_cols < (uint32_t)N) acc_cols <<= 1;
  const uint32_t ncols = 2 * acc_cols;

  if (tid == 0) {
    for (int s = 0; s < GR_STAGES; s++) { tc::mbar_init(&bar_full[s], GR_LOAD_WARPS * 32); tc::mbar_init(&bar_empty[s], 1); }
    for (int s = 0; s < 2; s++) { tc::mbar_init(&bar_acc_full[s], 1); tc::mbar_init(&bar_acc_empty[s], GR_EPI_WARPS); }
    tc::mbar_init(&bar_w, 1);
    tc::mbar_init_fence();
    // every stage and both accumulators start out free: complete the first phase of their "empty" barriers, so that
    // the n-th use always waits for phase n
    for (int s = 0; s < GR_STAGES; s++) tc::mbar_arrive(&bar_empty[s]);
    s_fail = 0;
  }
  if (warp == 0) { tc::tmem_alloc(&tmem_slot, ncols); tc::tmem_relinquish(); }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  if (tid == 0) {
    for (int s = 0; s < 2; s++)
      for (int i = 0; i < GR_EPI_WARPS; i++) tc::mbar_arrive(&bar_acc_empty[s]);
  }
  const uint32_t tmem_base = tmem_slot;
  const long long ntiles = (P.rows + GR_ROWS - 1) / GR_ROWS;
  int fail = 0;

  if (warp == GR_MMA_WARP) {
    // ===== weights once, then the MMAs of every chunk ===============================================================
    if (lane == 0) {
      tc::mbar_expect_tx(&bar_w, w_bytes);
      tc::bulk_g2s(w_smem, P.wp, w_bytes, &bar_w);
      if (!tc::mbar_wait(&bar_w, 0, wl)) fail = 1;
      tc::fence_after_sync();
      const uint32_t ring_base = tc::smem_u32(ring), w_base = tc::smem_u32(w_smem);
      const uint32_t idesc = tc::idesc_bf16(GR_ROWS, N);
      const uint64_t a_desc0 = tc::smem_desc(ring_base, GR_ROWS * 16, 128), b_desc0 = tc::smem_desc(w_base, N * 16, 128);
      const uint64_t b_step = (uint64_t)((2 * N * 16) >> 4);   // the address field of a descriptor counts 16-byte units
      uint32_t g = 0, tile_it = 0;
      for (long long tile = blockIdx.x; tile < ntiles && !fail; tile += gridDim.x, tile_it++) {
        const uint32_t b = tile_it & 1;
        if (s_fail || !tc::mbar_wait(&bar_acc_empty[b], (tile_it >> 1) & 1, wl)) { fail = 1; break; }
        tc::fence_after_sync();
        for (int c = 0; c < nchunks; c++, g++) {
          const uint32_t st = g % nst, use = g / nst;
          if (!tc::mbar_wait(&bar_full[st], use & 1, wl)) { fail = 1; break; }
          tc::fence_async_smem();      // the copies went through the generic proxy, the tensor cores read through the async one
          tc::fence_after_sync();
          // panel p of the chunk (eight K values of all rows) lies at p * 2 KB in the stage; the packed weights hold
          // K panel kp of all N outputs at kp * N * 16 bytes
          uint64_t ad = a_desc0 + (uint64_t)((st * GR_STAGE_BYTES) >> 4);
          uint64_t bd = b_desc0 + (uint64_t)(((uint32_t)c * (GR_KC / 8) * N * 16) >> 4);
#pragma unroll
          for (int ks = 0; ks < GR_KC / 16; ks++) {
            tc::mma_bf16(tmem_base + b * acc_cols, ad, bd, idesc, (c > 0 || ks > 0) ? 1u : 0u);
            ad += (uint64_t)((2 * GR_ROWS * 16) >> 4);
            bd += b_step;
          }
          tc::mma_commit(&bar_empty[st]);
        }
        if (fail) break;
        tc::mma_commit(&bar_acc_full[b]);
      }
      if (fail) s_fail = 1;
    }
  } else if (warp >= GR_EPI_WARPS) {
    // ===== loaders: a thread per row, sixteen 16-byte asynchronous copies per chunk ===================================
    // (eight lanes per row, so that a request reads whole 128-byte lines, measured 15 % slower: the eight pieces of a
    // line go to eight panels 2 KB apart, which all map to the same shared-memory banks)
    const int r = tid - GR_EPI_WARPS * 32;
    uint32_t g = 0;
    for (long long tile = blockIdx.x; tile < ntiles && !fail; tile += gridDim.x) {
      const long long row = tile * GR_ROWS + r;
      const bool row_ok = row < P.rows;
      const __nv_bfloat16* xrow = P.x + (row_ok ? row : 0) * K;
      const uint32_t nbytes = row_ok ? 16u : 0u;
      for (int c = 0; c < nchunks; c++, g++) {
        const uint32_t st = g % nst, use = g / nst;
        // the MMAs that read this stage's previous content are done (every thread polls: no warp-wide handshake)
        if (s_fail || !tc::mbar_wait(&bar_empty[st], use & 1, wl)) { fail = 1; break; }
        unsigned char* dst = ring + (size_t)st * GR_STAGE_BYTES + r * 16;
        const __nv_bfloat16* src = xrow + c * GR_KC;
#pragma unroll
        for (int p = 0; p < GR_KC / 8; p++) gr_cp_async16(dst + p * (GR_ROWS * 16), src + p * 8, nbytes);
        gr_cp_async_arrive(&bar_full[st]);
      }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");   // nothing of this thread is in flight when the block ends
    if (fail) s_fail = 1;
  } else {
    // ===== epilogue: a thread per row =================================================================================
    uint32_t tile_it = 0;
    for (long long tile = blockIdx.x; tile < ntiles && !fail; tile += gridDim.x, tile_it++) {
      const uint32_t b = tile_it & 1;
      const long long row = tile * GR_ROWS + tid;
      const bool row_ok = row < P.rows;
      const long long ro = row_ok ? row / S : 0;
      const int rs = row_ok ? (int)(row - ro * S) : 0;
      float* yrow = P.y + (ro * N) * S + rs;
      const float* rrow = P.res != nullptr && row_ok ? P.res + (ro * N) * S + rs : nullptr;
      // the residuals of the first 32 columns are fetched before the accumulator is waited for, those of the next 32
      // beside the tensor-memory load: 32 independent loads in flight instead of a load in front of every store
      float r[32];
      auto fetch_res = [&](int cb) {
        if (rrow != nullptr) {
#pragma unroll
          for (int j = 0; j < 32; j++) r[j] = __ldg(rrow + (size_t)(cb + j) * S);
        }
      };
      fetch_res(0);
      {
        int ok = 1;
        if (lane == 0) ok = (!s_fail && tc::mbar_wait(&bar_acc_full[b], (tile_it >> 1) & 1, wl)) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) { fail = 1; break; }
      }
      tc::fence_after_sync();
      for (int cb = 0; cb < N; cb += 32) {
        float v[32];
        if (cb > 0) fetch_res(cb);
        tc::tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + b * acc_cols + cb, v);
        if (row_ok) {
#pragma unroll
          for (int j = 0; j < 32; j++) {
            const float t = gr_act(v[j] + (P.bias != nullptr ? __ldg(P.bias + cb + j) : 0.f), P.act);
            yrow[(size_t)(cb + j) * S] = rrow != nullptr ? r[j] + t : t;
          }
        }
      }
      tc::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&bar_acc_empty[b]);
    }
    if (fail) s_fail = 1;
  }
  if (fail && lane == 0 && P.status != nullptr) atomicOr(P.status, LD_FLAG_TIMEOUT);
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem_base, ncols);
}

}  // namespace

// true when the streaming kernel applies: whole 64-wide K chunks, at most 128 outputs, and a packed weight matrix that
// stays in shared memory beside the ring
bool ld_gemm_rows16_applies(int K, int N) {
  return K % GR_KC == 0 && N % 32 == 0 && N <= 128 && (long long)K * N * 2 <= GR_MAX_W_BYTES &&
         (long long)K * N * 2 + GR_STAGES * GR_STAGE_BYTES + 2048 <= 226 * 1024;
}

int ld_gemm_rows16_launch(const void* x16, long long rows, int K, int S, const void* wp, const float* bias, int N, int act, float* y,
                          int* status_dev, void* stream, unsigned wait_limit, const float* res) {
  RowsParams P;
  P.res = res;
  P.x = (const __nv_bfloat16*)x16; P.y = y; P.wp = (const __nv_bfloat16*)wp; P.bias = bias; P.rows = rows; P.K = K; P.N = N; P.S = S;
  P.act = act; P.status = status_dev; P.wait_limit = wait_limit;
  const size_t w_bytes = (size_t)K * N * 2;
  const size_t smem = ((w_bytes + 1023) & ~(size_t)1023) + (size_t)(w_bytes <= 48 * 1024 ? GR_STAGES : GR_STAGES - 1) * GR_STAGE_BYTES + 1024;
  // L1 needs room for the lines in flight: with large weights the ring gives up a chunk for it
  P.stages = w_bytes <= 48 * 1024 ? GR_STAGES : GR_STAGES - 1;
  LD_CUDA_TRY(cudaFuncSetAttribute(gemm_rows16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long ntiles = (rows + GR_ROWS - 1) / GR_ROWS;
  const int grid = (int)(ntiles < sms ? ntiles : sms);
  gemm_rows16_kernel<<<grid, GR_THREADS, smem, (cudaStream_t)stream>>>(P);
  LD_LAUNCH_CHECK();
  return LD_OK;
}
