// Group norms of the node-level activations, per system and channel group:
//   ScalGroupNorm (managan/layers_common.py:201-223): y = beta + gamma * (x - mean) / sqrt(eps + var), mean and
//     variance over (nodes, channels of the group);
//   TensGroupNorm (managan/tensor_products.py:215-232): y = gamma * x / sqrt(eps + m2), m2 = mean over (nodes, channels
//     of the group) of the squared norm over the 3^inds Cartesian components; no mean is subtracted.
// x: [B][N][C][S] float32 (S = 3^inds; S = 1 for scalars). Blocks per (system, group, chunk of nodes) compute partial
// statistics (two passes over the chunk for the squared deviations), a small kernel joins them, a third applies them.
#include <cuda_runtime.h>
#include <cstdint>
#include "common.cuh"

namespace {

constexpr int GN_THREADS = 256;

__device__ __forceinline__ float gn_block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();   // red may still be read from the previous use
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < GN_THREADS / 32; i++) t += red[i];   // same order in every thread
  return t;
}

// One block per (system, group, chunk of nodes): count, mean and sum of squared deviations from that mean of the chunk
// (two passes over the chunk; not centred: mean = 0). part[((b*G + g)*nchunks + k)*3 + {0,1,2}].
// cm != 0: x is component-major, [B][N][S][C]: a node holds S runs of cpg contiguous floats of the group, C apart
__global__ void __launch_bounds__(GN_THREADS) gn_partial_kernel(const float* __restrict__ x, int N, int C, int S, int G, int center,
                                                               int nchunks, int cm, float* __restrict__ part) {
  __shared__ float red[GN_THREADS / 32];
  const int bg = blockIdx.x, b = bg / G, g = bg % G, kc = blockIdx.y;
  const int cpg = C / G, slab = cpg * S;            // floats of the group per node
  const int run = cm ? cpg : slab, run_stride = cm ? C : 0;   // contiguous run, distance between the runs of a node
  const int per = (N + nchunks - 1) / nchunks;
  const int n0 = kc * per, n1 = min(N, n0 + per);
  const long long total = (long long)max(n1 - n0, 0) * slab;
  const float* base = cm ? x + ((size_t)b * N + n0) * C * S + (size_t)g * cpg : x + (((size_t)b * N + n0) * C + (size_t)g * cpg) * S;
  auto at = [&](long long i) -> float {
    const long long n = i / slab;
    const int rem = (int)(i - n * slab), r = rem / run;
    return base[(size_t)n * C * S + (size_t)r * run_stride + (rem - r * run)];
  };
  float mean = 0.f;
  if (center && total > 0) {
    float s = 0.f;
    for (long long i = threadIdx.x; i < total; i += GN_THREADS) s += at(i);
    mean = gn_block_sum(s, red) / (float)total;
  }
  float q = 0.f;
  for (long long i = threadIdx.x; i < total; i += GN_THREADS) {
    const float d = at(i) - mean;
    q = fmaf(d, d, q);
  }
  q = gn_block_sum(q, red);
  if (threadIdx.x == 0) {
    float* o = part + ((size_t)bg * nchunks + kc) * 3;
    o[0] = (float)total; o[1] = mean; o[2] = q;
  }
}

// Joins the chunks of a (system, group) in a fixed order (pairwise update of mean and squared deviations):
// stats[(b*G + g)*2] = mean (0 when not centred), [.. + 1] = 1/sqrt(eps + second moment)
__global__ void gn_finalize_kernel(const float* __restrict__ part, int BG, int nchunks, int center, long long norm_count, float eps,
                                   float* __restrict__ stats) {
  const int bg = blockIdx.x * blockDim.x + threadIdx.x;
  if (bg >= BG) return;
  float n = 0.f, mean = 0.f, m2 = 0.f;
  for (int k = 0; k < nchunks; k++) {
    const float* p = part + ((size_t)bg * nchunks + k) * 3;
    const float nk = p[0];
    if (nk <= 0.f) continue;
    const float delta = p[1] - mean, nn = n + nk;
    mean += delta * (nk / nn);
    m2 += p[2] + delta * delta * (n * nk / nn);
    n = nn;
  }
  // centred: variance over all elements; else: mean over (node, channel) of the squared norm over the S components
  const float second = m2 / (float)(center ? (long long)n : norm_count);
  stats[(size_t)bg * 2] = center ? mean : 0.f;
  stats[(size_t)bg * 2 + 1] = 1.0f / sqrtf(eps + second);
}

__global__ void __launch_bounds__(256) gn_apply_kernel(const float* __restrict__ x, long long total, int N, int C, int S, int G, int cm,
                                                       const float* __restrict__ stats, const float* __restrict__ gamma,
                                                       const float* __restrict__ beta, const float* __restrict__ res,
                                                       float* __restrict__ y) {
  const int cpg = C / G;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int c = cm ? (int)(i % C) : (int)((i / S) % C);
    const long long b = i / ((long long)N * C * S);
    const float* st = stats + ((size_t)b * G + c / cpg) * 2;
    float v = (x[i] - st[0]) * st[1] * gamma[c];
    if (beta != nullptr) v += beta[c];
    y[i] = res != nullptr ? res[i] + v : v;
  }
}

// ---- row-wise variants: a block owns (system, chunk of nodes) and all channel groups ------------------------------
// A node's features are one contiguous row of L = C * S floats. The block has k * L/4 threads: thread t always reads
// the same four consecutive floats (column t % (L/4)) of every k-th node, so its channel group, gamma and beta are
// fixed, loads are 16 bytes and coalesced over whole rows, and no index arithmetic is left in the loops. Four
// consecutive floats never straddle a group (cpg * S and cpg are multiples of 4 on this path). The partial sums of the
// threads of a group are added by one thread in thread order: deterministic, and dependent on N alone.
constexpr int GN_ROW_MAX_THREADS = 256;

// group of the four floats at row position e
__device__ __forceinline__ int gn_group_of(int e, int C, int S, int cpg, int cm) { return cm ? (e % C) / cpg : e / (cpg * S); }

__global__ void __launch_bounds__(GN_ROW_MAX_THREADS)
gn_partial_rows_kernel(const float* __restrict__ x, int N, int C, int S, int G, int center, int nchunks, int cm, int k,
                       float* __restrict__ part) {
  __shared__ float s_part[GN_ROW_MAX_THREADS];
  __shared__ int s_gid[GN_ROW_MAX_THREADS];
  __shared__ float s_mean[64];
  const int L = C * S, L4 = L / 4, cpg = C / G;
  const int b = blockIdx.x, kc = blockIdx.y, tid = threadIdx.x;
  const int col = tid % L4, off = tid / L4;
  const int per = (N + nchunks - 1) / nchunks;
  const int n0 = kc * per, n1 = min(N, n0 + per);
  const int g = gn_group_of(col * 4, C, S, cpg, cm);
  s_gid[tid] = g;
  const float4* base = reinterpret_cast<const float4*>(x + ((size_t)b * N) * L) + col;
  const float total = (float)((long long)max(n1 - n0, 0) * cpg * S);
  // the threads of group `grp` in thread order
  auto group_sum = [&](int grp) {
    float t = 0.f;
    for (int i = 0; i < (int)blockDim.x; i++) if (s_gid[i] == grp) t += s_part[i];
    return t;
  };
  float mean = 0.f;
  if (center) {
    float sm = 0.f;
    for (int n = n0 + off; n < n1; n += k) { const float4 v = __ldg(base + (size_t)n * L4); sm += (v.x + v.y) + (v.z + v.w); }
    s_part[tid] = sm;
    __syncthreads();
    if (tid < G) s_mean[tid] = total > 0.f ? group_sum(tid) / total : 0.f;
    __syncthreads();
    mean = s_mean[g];
  }
  float q = 0.f;
  for (int n = n0 + off; n < n1; n += k) {
    const float4 v = __ldg(base + (size_t)n * L4);
    const float d0 = v.x - mean, d1 = v.y - mean, d2 = v.z - mean, d3 = v.w - mean;
    q = fmaf(d0, d0, q); q = fmaf(d1, d1, q); q = fmaf(d2, d2, q); q = fmaf(d3, d3, q);
  }
  __syncthreads();
  s_part[tid] = q;
  __syncthreads();
  if (tid < G) {
    float* o = part + (((size_t)b * G + tid) * nchunks + kc) * 3;
    o[0] = total; o[1] = center ? s_mean[tid] : 0.f; o[2] = group_sum(tid);
  }
}

__global__ void __launch_bounds__(GN_ROW_MAX_THREADS)
gn_apply_rows_kernel(const float* __restrict__ x, int N, int C, int S, int G, int nchunks, int cm, int k, const float* __restrict__ stats,
                     const float* __restrict__ gamma, const float* __restrict__ beta, const float* __restrict__ res,
                     float* __restrict__ y) {
  const int L = C * S, L4 = L / 4, cpg = C / G;
  const int b = blockIdx.x, kc = blockIdx.y, tid = threadIdx.x;
  const int col = tid % L4, off = tid / L4;
  const int per = (N + nchunks - 1) / nchunks;
  const int n0 = kc * per, n1 = min(N, n0 + per);
  const int e = col * 4;
  const float* st = stats + ((size_t)b * G + gn_group_of(e, C, S, cpg, cm)) * 2;
  const float mean = st[0], rstd = st[1];
  float ga[4], be[4];
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const int c = cm ? (e + j) % C : (e + j) / S;
    ga[j] = gamma[c] * rstd;
    be[j] = beta != nullptr ? beta[c] : 0.f;
  }
  const float4* xin = reinterpret_cast<const float4*>(x + ((size_t)b * N) * L) + col;
  float4* yout = reinterpret_cast<float4*>(y + ((size_t)b * N) * L) + col;
  const float4* rin = res != nullptr ? reinterpret_cast<const float4*>(res + ((size_t)b * N) * L) + col : nullptr;
  for (int n = n0 + off; n < n1; n += k) {
    const float4 v = __ldg(xin + (size_t)n * L4);
    float4 r;
    r.x = fmaf(v.x - mean, ga[0], be[0]); r.y = fmaf(v.y - mean, ga[1], be[1]);
    r.z = fmaf(v.z - mean, ga[2], be[2]); r.w = fmaf(v.w - mean, ga[3], be[3]);
    if (rin != nullptr) {   // the residual the caller would add next: res + norm, the same sum a separate add forms
      const float4 q = __ldg(rin + (size_t)n * L4);
      r.x = q.x + r.x; r.y = q.y + r.y; r.z = q.z + r.z; r.w = q.w + r.w;
    }
    yout[(size_t)n * L4] = r;
  }
}

}  // namespace

// x, y: [B][N][C][S]; gamma [C]; beta [C] or NULL; center != 0 subtracts the group mean (ScalGroupNorm, S = 1).
// workspace: 98 * B * groups floats of device memory (statistics per system and group + up to 32 chunk partials).
// ld_group_norm_cm: the same for component-major activations, x and y [B][N][S][C].
static int group_norm_launch(const float* x, int B, int N, int C, int S, int groups, int center, float eps, const float* gamma,
                             const float* beta, float* y, void* workspace, void* stream, int cm, const float* res = nullptr) {
  if (B < 0 || N <= 0 || C <= 0 || S <= 0 || groups <= 0 || C % groups != 0) return LD_ERR_SHAPE;
  if (center && S != 1) { ld_set_last_message("group norm: the centred form is defined for scalars (S = 1)"); return LD_ERR_SHAPE; }
  if (B == 0) return LD_OK;
  if (workspace == nullptr) return LD_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  float* stats = (float*)workspace;
  float* part = stats + (size_t)2 * B * groups;
  // the nodes of a (system, group) are split into chunks of about 64 so that a few large systems still fill the device.
  // The split depends on the system size alone, never on the batch: the statistics of a system are then bit-identical
  // whatever batch it is part of (a batch sharded over several GPUs gives the results of the whole batch on one).
  int nchunks = (N + 63) / 64;
  if (nchunks > 32) nchunks = 32;
  if (nchunks > N) nchunks = N;
  if (nchunks < 1) nchunks = 1;
  // rows of whole 16-byte pieces that never straddle a channel group, short enough for one block: the row-wise kernels
  const int L = C * S, cpg = C / groups;
  const bool rows = L % 4 == 0 && cpg % 4 == 0 && L / 4 <= GN_ROW_MAX_THREADS && groups <= 64 && B <= 65535 &&
                    ((uintptr_t)x % 16 == 0) && ((uintptr_t)y % 16 == 0) && ((uintptr_t)res % 16 == 0);
  const int k = rows ? (GN_ROW_MAX_THREADS / (L / 4) > 0 ? GN_ROW_MAX_THREADS / (L / 4) : 1) : 0;
  if (rows) gn_partial_rows_kernel<<<dim3(B, nchunks), k * (L / 4), 0, st>>>(x, N, C, S, groups, center, nchunks, cm, k, part);
  else gn_partial_kernel<<<dim3(B * groups, nchunks), GN_THREADS, 0, st>>>(x, N, C, S, groups, center, nchunks, cm, part);
  LD_LAUNCH_CHECK();
  gn_finalize_kernel<<<(B * groups + 127) / 128, 128, 0, st>>>(part, B * groups, nchunks, center, (long long)N * (C / groups), eps, stats);
  LD_LAUNCH_CHECK();
  if (rows) {
    gn_apply_rows_kernel<<<dim3(B, nchunks), k * (L / 4), 0, st>>>(x, N, C, S, groups, nchunks, cm, k, stats, gamma, beta, res, y);
  } else {
    const long long total = (long long)B * N * C * S;
    long long blocks = (total + 255) / 256;
    if (blocks > 148LL * 32) blocks = 148LL * 32;
    gn_apply_kernel<<<(unsigned)blocks, 256, 0, st>>>(x, total, N, C, S, groups, cm, stats, gamma, beta, res, y);
  }
  LD_LAUNCH_CHECK();
  return LD_OK;
}

extern "C" int ld_group_norm(const float* x, int B, int N, int C, int S, int groups, int center, float eps, const float* gamma,
                             const float* beta, float* y, void* workspace, void* stream) {
  return group_norm_launch(x, B, N, C, S, groups, center, eps, gamma, beta, y, workspace, stream, 0);
}

extern "C" int ld_group_norm_cm(const float* x, int B, int N, int C, int S, int groups, int center, float eps, const float* gamma,
                                const float* beta, float* y, void* workspace, void* stream) {
  return group_norm_launch(x, B, N, C, S, groups, center, eps, gamma, beta, y, workspace, stream, 1);
}

// ld_group_norm with a residual: y = residual + norm(x), residual laid out like x (the sum a caller's separate add would
// form, without the extra pass over the tensor). residual may be NULL.
extern "C" int ld_group_norm_res(const float* x, const float* residual, int B, int N, int C, int S, int groups, int center, float eps,
                                 const float* gamma, const float* beta, float* y, void* workspace, void* stream) {
  return group_norm_launch(x, B, N, C, S, groups, center, eps, gamma, beta, y, workspace, stream, 0, residual);
}
