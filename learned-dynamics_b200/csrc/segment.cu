// Edge <-> node data movement on a graph whose edges are sorted by source node.
//   ld_row_ptr_from_sorted : CSR offsets from a sorted src array (binary search per node)
//   ld_segment_sum         : edges -> src nodes sum; replaces torch_scatter.segment_coo at the
//                            call site managan/graph_layers.py:54-59 (edges_reduce_src)
//   ld_gather_rows         : nodes -> edges read; managan/graph_layers.py:37-52 (edges_read*)
// All three are HBM bound. One warp owns one output row and moves it with 16-byte accesses, so
// no atomics are needed and the summation order (ascending edge id) is fixed.
#include "common.cuh"

namespace {

template <typename IndexT>
__global__ void row_ptr_kernel(const IndexT* __restrict__ src, long long E, int Nt, int* __restrict__ row_ptr) {
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v > Nt) return;
  long long lo = 0, hi = E;  // first e with src[e] >= v
  while (lo < hi) {
    long long mid = (lo + hi) >> 1;
    if ((long long)src[mid] < v) lo = mid + 1; else hi = mid;
  }
  row_ptr[v] = (int)lo;
}

constexpr int SEG_WARPS = 8;

// F4 = F/4 float4 columns per row
__global__ void __launch_bounds__(SEG_WARPS * 32)
segment_sum_vec4(const float4* __restrict__ x, const int* __restrict__ row_ptr, int Nt, int F4, float4* __restrict__ out) {
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int row = blockIdx.x * SEG_WARPS + w; row < Nt; row += gridDim.x * SEG_WARPS) {
    const int e0 = row_ptr[row], e1 = row_ptr[row + 1];
    for (int c = lane; c < F4; c += 32) {
      float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
      int e = e0;
      for (; e + 1 < e1; e += 2) {
        const float4 u = __ldg(&x[(size_t)e * F4 + c]);
        const float4 v = __ldg(&x[(size_t)(e + 1) * F4 + c]);
        a0.x += u.x; a0.y += u.y; a0.z += u.z; a0.w += u.w;
        a1.x += v.x; a1.y += v.y; a1.z += v.z; a1.w += v.w;
      }
      if (e < e1) {
        const float4 u = __ldg(&x[(size_t)e * F4 + c]);
        a0.x += u.x; a0.y += u.y; a0.z += u.z; a0.w += u.w;
      }
      out[(size_t)row * F4 + c] = make_float4(a0.x + a1.x, a0.y + a1.y, a0.z + a1.z, a0.w + a1.w);
    }
  }
}

__global__ void __launch_bounds__(SEG_WARPS * 32)
segment_sum_scalar(const float* __restrict__ x, const int* __restrict__ row_ptr, int Nt, int F, float* __restrict__ out) {
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int row = blockIdx.x * SEG_WARPS + w; row < Nt; row += gridDim.x * SEG_WARPS) {
    const int e0 = row_ptr[row], e1 = row_ptr[row + 1];
    if (F >= 32) {
      for (int c = lane; c < F; c += 32) {
        float a = 0.f;
        for (int e = e0; e < e1; e++) a += __ldg(&x[(size_t)e * F + c]);
        out[(size_t)row * F + c] = a;
      }
    } else {
      // narrow rows: lanes split the edges, then reduce across lanes per column
      for (int c = 0; c < F; c++) {
        float a = 0.f;
        for (int e = e0 + lane; e < e1; e += 32) a += __ldg(&x[(size_t)e * F + c]);
        for (int d = 16; d > 0; d >>= 1) a += __shfl_xor_sync(0xffffffffu, a, d);
        if (lane == 0) out[(size_t)row * F + c] = a;
      }
    }
  }
}

template <typename IndexT>
__global__ void __launch_bounds__(SEG_WARPS * 32)
gather_rows_vec4(const float4* __restrict__ x, const IndexT* __restrict__ idx, long long E, int F4, float4* __restrict__ out) {
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (long long e = (long long)blockIdx.x * SEG_WARPS + w; e < E; e += (long long)gridDim.x * SEG_WARPS) {
    const size_t r = (size_t)idx[e];
    for (int c = lane; c < F4; c += 32) out[(size_t)e * F4 + c] = __ldg(&x[r * F4 + c]);
  }
}

template <typename IndexT>
__global__ void __launch_bounds__(SEG_WARPS * 32)
gather_rows_scalar(const float* __restrict__ x, const IndexT* __restrict__ idx, long long E, int F, float* __restrict__ out) {
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (long long e = (long long)blockIdx.x * SEG_WARPS + w; e < E; e += (long long)gridDim.x * SEG_WARPS) {
    const size_t r = (size_t)idx[e];
    for (int c = lane; c < F; c += 32) out[(size_t)e * F + c] = __ldg(&x[r * F + c]);
  }
}

// ---- legacy padded neighbour lists (extensions/neighbour_grid/neighbour_grid_kern.cu:226-306) ----------------
// One warp per (node, slot) row of the padded table; lanes run over the channels, so reads and writes are coalesced.
__global__ void __launch_bounds__(SEG_WARPS * 32)
padded_read_kernel(const int* __restrict__ neighbours, const int* __restrict__ counts, const float* __restrict__ x,
                   float* __restrict__ out, long long slots, int nodes, int nmax, int chan) {
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (long long s = (long long)blockIdx.x * SEG_WARPS + w; s < slots; s += (long long)gridDim.x * SEG_WARPS) {
    const long long i = s / nmax;
    const int j = (int)(s - i * nmax);
    float* o = out + (size_t)s * chan;
    if (j < counts[i]) {
      const float* r = x + ((size_t)(i / nodes) * nodes + (size_t)neighbours[s]) * chan;
      for (int c = lane; c < chan; c += 32) o[c] = __ldg(&r[c]);
    } else {
      for (int c = lane; c < chan; c += 32) o[c] = 0.f;
    }
  }
}

// One warp per node; each lane owns channels and adds the slots in ascending order, as the reference's loop does.
__global__ void __launch_bounds__(SEG_WARPS * 32)
padded_reduce_kernel(const int* __restrict__ counts, const float* __restrict__ x, float* __restrict__ out,
                     long long Nt, int nmax, int chan) {
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (long long i = (long long)blockIdx.x * SEG_WARPS + w; i < Nt; i += (long long)gridDim.x * SEG_WARPS) {
    const int n = min(counts[i], nmax);
    const float* r = x + (size_t)i * nmax * chan;
    for (int c = lane; c < chan; c += 32) {
      float a = 0.f;
      for (int j = 0; j < n; j++) a += __ldg(&r[(size_t)j * chan + c]);
      out[(size_t)i * chan + c] = a;
    }
  }
}

// CSR edge list -> padded per-node lists of in-system neighbour indices (what getNeighbours returns,
// neighbour_grid_kern.cu:62-133). A node with more than nmax neighbours raises LD_FLAG_CAPACITY.
__global__ void padded_lists_kernel(const int* __restrict__ row_ptr, const int* __restrict__ dst, long long Nt, int nodes,
                                    int nmax, int* __restrict__ lists, int* __restrict__ counts, int* __restrict__ status) {
  const long long s = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= Nt * nmax) return;
  const long long i = s / nmax;
  const int j = (int)(s - i * nmax);
  const int e0 = row_ptr[i], n = row_ptr[i + 1] - e0;
  if (j == 0) {
    counts[i] = n;
    if (n > nmax) atomicOr(status, LD_FLAG_CAPACITY);
  }
  lists[s] = j < n ? dst[e0 + j] - (int)(i / nodes) * nodes : 0;
}

inline int rows_grid(long long rows) {
  long long b = (rows + SEG_WARPS - 1) / SEG_WARPS;
  const long long cap = 148LL * 16;
  return (int)(b < cap ? (b > 0 ? b : 1) : cap);
}

}  // namespace

// index_bytes: 4 (int32) or 8 (int64) element size of src
extern "C" int ld_row_ptr_from_sorted(const void* src, int index_bytes, long long E, int Nt, int* row_ptr, void* stream) {
  if (E < 0 || Nt < 0 || (index_bytes != 4 && index_bytes != 8)) return LD_ERR_SHAPE;
  const int nb = ld_cdiv((long long)Nt + 1, 256);
  if (index_bytes == 4) row_ptr_kernel<int><<<nb, 256, 0, (cudaStream_t)stream>>>((const int*)src, E, Nt, row_ptr);
  else row_ptr_kernel<long long><<<nb, 256, 0, (cudaStream_t)stream>>>((const long long*)src, E, Nt, row_ptr);
  LD_LAUNCH_CHECK();
  return LD_OK;
}

// out[v, :] = sum over e in [row_ptr[v], row_ptr[v+1]) of x_edge[e, :]; rows without edges get 0.
extern "C" int ld_segment_sum(const float* x_edge, const int* row_ptr, int Nt, int F, float* out, void* stream) {
  if (Nt < 0 || F < 0) return LD_ERR_SHAPE;
  if (Nt == 0 || F == 0) return LD_OK;
  const bool vec = (F % 4 == 0) && (((uintptr_t)x_edge | (uintptr_t)out) % 16 == 0);
  if (vec) segment_sum_vec4<<<rows_grid(Nt), SEG_WARPS * 32, 0, (cudaStream_t)stream>>>((const float4*)x_edge, row_ptr, Nt, F / 4, (float4*)out);
  else segment_sum_scalar<<<rows_grid(Nt), SEG_WARPS * 32, 0, (cudaStream_t)stream>>>(x_edge, row_ptr, Nt, F, out);
  LD_LAUNCH_CHECK();
  return LD_OK;
}

// out[e, :] = x_node[idx[e], :]
extern "C" int ld_gather_rows(const float* x_node, const void* idx, int index_bytes, long long E, int F, float* out, void* stream) {
  if (E < 0 || F < 0 || (index_bytes != 4 && index_bytes != 8)) return LD_ERR_SHAPE;
  if (E == 0 || F == 0) return LD_OK;
  const bool vec = (F % 4 == 0) && (((uintptr_t)x_node | (uintptr_t)out) % 16 == 0);
  cudaStream_t st = (cudaStream_t)stream;
  const int g = rows_grid(E);
  if (vec) {
    if (index_bytes == 4) gather_rows_vec4<int><<<g, SEG_WARPS * 32, 0, st>>>((const float4*)x_node, (const int*)idx, E, F / 4, (float4*)out);
    else gather_rows_vec4<long long><<<g, SEG_WARPS * 32, 0, st>>>((const float4*)x_node, (const long long*)idx, E, F / 4, (float4*)out);
  } else {
    if (index_bytes == 4) gather_rows_scalar<int><<<g, SEG_WARPS * 32, 0, st>>>(x_node, (const int*)idx, E, F, out);
    else gather_rows_scalar<long long><<<g, SEG_WARPS * 32, 0, st>>>(x_node, (const long long*)idx, E, F, out);
  }
  LD_LAUNCH_CHECK();
  return LD_OK;
}

// Legacy dense interface of the reference extension (neighbour_grid.cpp:105-168): padded tables
// [batch, nodes, neighboursmax(, chan)]. neighbours holds in-system node indices.
extern "C" int ld_edges_read_padded(const int* neighbours, const int* counts, const float* x, int batch, int nodes, int nmax,
                                    int chan, float* out, void* stream) {
  if (batch < 0 || nodes < 0 || nmax < 0 || chan < 0) return LD_ERR_SHAPE;
  const long long slots = (long long)batch * nodes * nmax;
  if (slots == 0 || chan == 0) return LD_OK;
  padded_read_kernel<<<rows_grid(slots), SEG_WARPS * 32, 0, (cudaStream_t)stream>>>(neighbours, counts, x, out, slots, nodes, nmax, chan);
  LD_LAUNCH_CHECK();
  return LD_OK;
}

extern "C" int ld_edges_reduce_padded(const int* counts, const float* x, int batch, int nodes, int nmax, int chan, float* out,
                                      void* stream) {
  if (batch < 0 || nodes < 0 || nmax < 0 || chan < 0) return LD_ERR_SHAPE;
  const long long Nt = (long long)batch * nodes;
  if (Nt == 0 || chan == 0) return LD_OK;
  padded_reduce_kernel<<<rows_grid(Nt), SEG_WARPS * 32, 0, (cudaStream_t)stream>>>(counts, x, out, Nt, nmax, chan);
  LD_LAUNCH_CHECK();
  return LD_OK;
}

extern "C" int ld_neighbour_lists_from_csr(const int* row_ptr, const int* dst, int batch, int nodes, int nmax, int* lists,
                                           int* counts, int* status_dev, void* stream) {
  if (batch < 0 || nodes < 0 || nmax <= 0) return LD_ERR_SHAPE;
  const long long total = (long long)batch * nodes * nmax;
  if (total == 0) return LD_OK;
  padded_lists_kernel<<<(unsigned)ld_cdiv(total, 256), 256, 0, (cudaStream_t)stream>>>(row_ptr, dst, (long long)batch * nodes, nodes,
                                                                                nmax, lists, counts, status_dev);
  LD_LAUNCH_CHECK();
  return LD_OK;
}
