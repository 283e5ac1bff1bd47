// Error bookkeeping and the int32 prefix sum shared by the graph kernels.
#include "common.cuh"
#include <stdio.h>
#include <string.h>
#include <mutex>

static thread_local char g_last_error[512] = "";

void ld_set_last_error(cudaError_t e, const char* file, int line) {
  snprintf(g_last_error, sizeof(g_last_error), "CUDA error %d (%s) at %s:%d", (int)e,
           cudaGetErrorString(e), file, line);
}

void ld_set_last_message(const char* msg) {
  strncpy(g_last_error, msg, sizeof(g_last_error) - 1);
  g_last_error[sizeof(g_last_error) - 1] = 0;
}

extern "C" const char* ld_last_error(void) { return g_last_error; }

namespace {
constexpr int WC_MAX_DEVICES = 64;
std::mutex g_wc_mutex;
int* g_wc_ring[WC_MAX_DEVICES] = {};
unsigned g_wc_next[WC_MAX_DEVICES] = {};
}  // namespace

int ld_work_counter(cudaStream_t stream, int** counter) {
  int dev = 0;
  LD_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= WC_MAX_DEVICES) { ld_set_last_message("work counter: device index out of range"); return LD_ERR_UNSUPPORTED; }
  int* slot = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_wc_mutex);
    if (g_wc_ring[dev] == nullptr) {
      int* ring = nullptr;
      LD_CUDA_TRY(cudaMalloc(&ring, sizeof(int) * LD_WORK_COUNTERS));
      g_wc_ring[dev] = ring;
    }
    slot = g_wc_ring[dev] + (g_wc_next[dev]++ % LD_WORK_COUNTERS);
  }
  LD_CUDA_TRY(cudaMemsetAsync(slot, 0, sizeof(int), stream));
  *counter = slot;
  return LD_OK;
}

extern "C" const char* ld_status_string(int status) {
  switch (status) {
    case LD_OK: return "ok";
    case LD_ERR_SHAPE: return "shape or argument error";
    case LD_ERR_CAPACITY: return "output capacity too small";
    case LD_ERR_BOX_TOO_SMALL: return "box dimension must be greater than 2*cutoff";
    case LD_ERR_NONFINITE: return "non-finite input";
    case LD_ERR_TIMEOUT: return "device-side wait ran out";
    case LD_ERR_CUDA: return "CUDA runtime error";
    case LD_ERR_WORKSPACE: return "workspace too small";
    case LD_ERR_UNSUPPORTED: return "unsupported size for this kernel";
    default: return "unknown status";
  }
}

// ---------------------------------------------------------------------------------------------
// Exclusive scan: three phases (tile sums, scan of tile sums by one block, tile-local scan).
// Sizes here are node / cell counts (at most a few million), so one block for the middle phase.
// ---------------------------------------------------------------------------------------------
namespace {

constexpr int SCAN_THREADS = 512;
constexpr int SCAN_ITEMS = 8;
constexpr int SCAN_TILE = SCAN_THREADS * SCAN_ITEMS;

__device__ __forceinline__ int warp_incl_scan(int v) {
  const unsigned lane = threadIdx.x & 31;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    int t = __shfl_up_sync(0xffffffffu, v, d);
    if (lane >= (unsigned)d) v += t;
  }
  return v;
}

// block-wide exclusive scan of one value per thread; returns exclusive prefix, total in *total.
__device__ __forceinline__ int block_excl_scan(int v, int* total) {
  __shared__ int warp_tot[32];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int nw = (blockDim.x + 31) >> 5;
  int inc = warp_incl_scan(v);
  if (lane == 31) warp_tot[w] = inc;
  __syncthreads();
  if (w == 0) {
    int t = lane < nw ? warp_tot[lane] : 0;
    int ti = warp_incl_scan(t);
    warp_tot[lane] = ti - t;  // exclusive warp offsets
    if (lane == 31) warp_tot[31] = ti - t;  // keep layout simple
    if (lane == nw - 1) *total = ti;
  }
  __syncthreads();
  int res = inc - v + warp_tot[w];
  __syncthreads();
  return res;
}

__global__ void scan_tile_sums(const int* __restrict__ in, long long n, int* __restrict__ tile_sums) {
  __shared__ int tot;
  long long base = (long long)blockIdx.x * SCAN_TILE + (long long)threadIdx.x * SCAN_ITEMS;
  int s = 0;
#pragma unroll
  for (int k = 0; k < SCAN_ITEMS; k++) {
    long long i = base + k;
    if (i < n) s += in[i];
  }
  (void)block_excl_scan(s, &tot);
  if (threadIdx.x == 0) tile_sums[blockIdx.x] = tot;
}

__global__ void scan_tile_offsets(int* __restrict__ tile_sums, int ntiles) {
  __shared__ int tot;
  int carry = 0;
  for (int base = 0; base < ntiles; base += blockDim.x) {
    int i = base + threadIdx.x;
    int v = i < ntiles ? tile_sums[i] : 0;
    int ex = block_excl_scan(v, &tot);
    if (i < ntiles) tile_sums[i] = ex + carry;
    carry += tot;
    __syncthreads();
  }
}

__global__ void scan_tiles(const int* __restrict__ in, int* __restrict__ out, long long n,
                           const int* __restrict__ tile_offsets) {
  __shared__ int tot;
  long long base = (long long)blockIdx.x * SCAN_TILE + (long long)threadIdx.x * SCAN_ITEMS;
  int v[SCAN_ITEMS];
  int s = 0;
#pragma unroll
  for (int k = 0; k < SCAN_ITEMS; k++) {
    long long i = base + k;
    v[k] = (i < n) ? in[i] : 0;
    s += v[k];
  }
  int ex = block_excl_scan(s, &tot) + tile_offsets[blockIdx.x];
#pragma unroll
  for (int k = 0; k < SCAN_ITEMS; k++) {
    long long i = base + k;
    if (i <= n) out[i] = ex;  // out[n] = grand total
    ex += v[k];
  }
}

}  // namespace

size_t ld_scan_scratch_ints(long long n) { return (size_t)((n + 1 + SCAN_TILE - 1) / SCAN_TILE) + 1; }

int ld_scan_exclusive(const int* in, int* out, long long n, int* scratch, cudaStream_t stream) {
  if (n < 0) return LD_ERR_SHAPE;
  int ntiles = (int)((n + 1 + SCAN_TILE - 1) / SCAN_TILE);
  scan_tile_sums<<<ntiles, SCAN_THREADS, 0, stream>>>(in, n, scratch);
  LD_LAUNCH_CHECK();
  scan_tile_offsets<<<1, SCAN_THREADS, 0, stream>>>(scratch, ntiles);
  LD_LAUNCH_CHECK();
  scan_tiles<<<ntiles, SCAN_THREADS, 0, stream>>>(in, out, n, scratch);
  LD_LAUNCH_CHECK();
  return LD_OK;
}
