// Shared helpers for the hot-path CUDA library (sm_100a).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>

// Status codes returned by every extern "C" entry point (0 = success).
#define LD_OK 0
#define LD_ERR_SHAPE -1
#define LD_ERR_CAPACITY -2
#define LD_ERR_BOX_TOO_SMALL -3
#define LD_ERR_NONFINITE -4
#define LD_ERR_TIMEOUT -5
#define LD_ERR_CUDA -6
#define LD_ERR_WORKSPACE -7
#define LD_ERR_UNSUPPORTED -8

// Bits that kernels OR into the caller's device status word.
#define LD_FLAG_CAPACITY 1
#define LD_FLAG_NONFINITE 2
#define LD_FLAG_TIMEOUT 4
#define LD_FLAG_OVERFLOW 8

#define LD_CUDA_TRY(expr)                          \
  do {                                             \
    cudaError_t _e = (expr);                       \
    if (_e != cudaSuccess) { ld_set_last_error(_e, __FILE__, __LINE__); return LD_ERR_CUDA; } \
  } while (0)

#define LD_LAUNCH_CHECK() LD_CUDA_TRY(cudaGetLastError())

void ld_set_last_error(cudaError_t e, const char* file, int line);
void ld_set_last_message(const char* msg);

static inline size_t ld_align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
static inline int ld_cdiv(long long a, long long b) { return (int)((a + b - 1) / b); }
// Nodes per segment when the edge kernels walk the node range in segments of about `want` nodes (so that the rows a
// segment gathers stay in L2): the segments are made equal, since a short last segment gives every block a sliver of work
static inline int ld_even_segments(long long Nt, long long want) {
  if (want < 1024) want = 1024;
  if (Nt <= want) return (int)(Nt > 0 ? Nt : 1);
  const long long nseg = (Nt + want - 1) / want;
  return (int)((Nt + nseg - 1) / nseg);
}

// A zeroed int32 in device memory for one launch that hands out work through an atomic counter: taken from a ring of
// LD_WORK_COUNTERS per device (allocated at the first call on that device, which therefore must not be inside a stream
// capture) and cleared in stream order before the launch. A counter is handed out again after LD_WORK_COUNTERS later
// calls, far more launches than a stream holds in flight.
#define LD_WORK_COUNTERS 4096
int ld_work_counter(cudaStream_t stream, int** counter);

// exclusive prefix sum of n int32 values; out[n] receives the total (out has n+1 entries).
// scratch must hold ld_scan_scratch_ints(n) ints.
size_t ld_scan_scratch_ints(long long n);
int ld_scan_exclusive(const int* in, int* out, long long n, int* scratch, cudaStream_t stream);
