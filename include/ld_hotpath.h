/* C ABI of libld_hotpath.so: the equivariant message-passing hot path of learned-dynamics as
 * sm_100a CUDA kernels. Plain pointers and sizes only; every pointer named "device" below is a
 * device address owned by the caller, every call is asynchronous on `stream` (a cudaStream_t
 * passed as void*), nothing is allocated or freed inside the library, and the return value is a
 * status code (0 = LD_OK). Citations name the reference interface each entry point replaces
 * (paths inside pb1729/learned-dynamics).
 */
#ifndef LD_HOTPATH_H
#define LD_HOTPATH_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  LD_OK = 0,
  LD_ERR_SHAPE = -1,          /* bad sizes / null where a pointer is required */
  LD_ERR_CAPACITY = -2,       /* caller-provided output too small */
  LD_ERR_BOX_TOO_SMALL = -3,  /* periodic box not > 2*cutoff on some axis (reference: TORCH_CHECK ndiv>=3) */
  LD_ERR_NONFINITE = -4,
  LD_ERR_TIMEOUT = -5,        /* a bounded device-side wait ran out */
  LD_ERR_CUDA = -6,           /* CUDA runtime error; text in ld_last_error() */
  LD_ERR_WORKSPACE = -7,
  LD_ERR_UNSUPPORTED = -8
};

/* bits OR-ed by kernels into the caller's device status word */
enum { LD_FLAG_CAPACITY = 1, LD_FLAG_NONFINITE = 2, LD_FLAG_TIMEOUT = 4, LD_FLAG_OVERFLOW = 8 };

/* activation codes for the dense layers */
enum { LD_ACT_NONE = 0, LD_ACT_SILU = 1, LD_ACT_LEAKY01 = 2 };

const char* ld_last_error(void);           /* thread-local text of the last failure */
const char* ld_status_string(int status);

/* ---- radius graph ---------------------------------------------------------------------------
 * Replaces neighbour_grid_cuda.get_neighbours / get_edges
 * (extensions/neighbour_grid/neighbour_grid.cpp:59-103, 170-195; kernels
 * extensions/neighbour_grid/neighbour_grid_kern.cu:57-150, 334-352) and the boxwrap of
 * graph_setup (managan/graph_layers.py:62-66, archs/meanflow_painn8.py:167-172).
 * pos: device float32 [batch, nodes, 3]. periodic != 0: box = 3 HOST floats; periodic == 0: open
 * boundary (no counterpart in the reference, which emulates it with a large box).
 * mode 0: every pair within the cutoff. mode 1: the reference's ceil(box/cutoff) cell grid, which
 * misses pairs two cells apart when box/cutoff is not an integer (periodic only).
 * open_cells_cap: cells reserved per system for open boundaries (0 = default).
 * Two calls: _count fills row_ptr[batch*nodes+1] (CSR offsets over global node id b*nodes+i) and
 * edge_counts[batch] (cumulative, as the reference's third return value); the caller sizes the
 * edge arrays (or keeps a fixed capacity) and _fill writes them. src ascending; order within a
 * node is deterministic. shift/rij may be NULL. */
int ld_radius_graph_workspace_size(int batch, int nodes, int periodic, float cutoff, const float* box, int mode,
                                   int open_cells_cap, size_t* bytes);
int ld_radius_graph_count(const float* pos, int batch, int nodes, int periodic, float cutoff, const float* box, int mode,
                          int open_cells_cap, void* workspace, size_t workspace_bytes, int* row_ptr, int* edge_counts,
                          int* status_dev, void* stream);
int ld_radius_graph_fill(const float* pos, int batch, int nodes, int periodic, float cutoff, const float* box, int mode,
                         int open_cells_cap, void* workspace, size_t workspace_bytes, const int* row_ptr,
                         long long capacity, int* src, int* dst, int* shift, float* rij, int* status_dev, void* stream);

/* Allocation-free variant. It has no counterpart in the reference. Count + fill in one call with the
 * scratch space in a fixed 8 MiB device array inside the library, for callers that may not allocate
 * device memory where they need the graph (a plugin called from inside an engine's time-step loop, a
 * service whose allocator is frozen after start-up). Refuses larger problems with LD_ERR_WORKSPACE. The first
 * call per device resolves the array's address and should precede any stream capture; calls that
 * overlap on one device race on the shared array. */
int ld_radius_graph_build_noalloc(const float* pos, int batch, int nodes, int periodic, float cutoff, const float* box,
                                  int mode, int open_cells_cap, int* row_ptr, int* edge_counts, long long capacity,
                                  int* src, int* dst, int* shift, float* rij, int* status_dev, void* stream);

/* ---- edge <-> node movement -----------------------------------------------------------------
 * ld_segment_sum replaces torch_scatter.segment_coo at managan/graph_layers.py:54-59;
 * ld_gather_rows replaces the index reads of managan/graph_layers.py:37-52;
 * ld_row_ptr_from_sorted turns a sorted src array (int32 or int64) into CSR offsets. */
int ld_row_ptr_from_sorted(const void* src, int index_bytes, long long E, int Nt, int* row_ptr, void* stream);
int ld_segment_sum(const float* x_edge, const int* row_ptr, int Nt, int F, float* out, void* stream);
int ld_gather_rows(const float* x_node, const void* idx, int index_bytes, long long E, int F, float* out, void* stream);

/* Legacy padded tables of the reference extension: get_neighbours, edges_read, edges_reduce
 * (extensions/neighbour_grid/neighbour_grid.cpp:69-168, neighbour_grid_kern.cu:62-133, 226-306).
 * lists / neighbours int32 [batch, nodes, nmax] hold in-system node indices, counts int32 [batch, nodes].
 * ld_neighbour_lists_from_csr pads the CSR edge list (entries past a node's count are 0; a node with more than nmax
 * neighbours raises LD_FLAG_CAPACITY in *status_dev). ld_edges_read_padded: out [batch, nodes, nmax, chan] = x of the
 * neighbour, 0 past the count. ld_edges_reduce_padded: out [batch, nodes, chan] = sum over the first count slots,
 * added in ascending slot order. */
int ld_neighbour_lists_from_csr(const int* row_ptr, const int* dst, int batch, int nodes, int nmax, int* lists, int* counts,
                                int* status_dev, void* stream);
int ld_edges_read_padded(const int* neighbours, const int* counts, const float* x, int batch, int nodes, int nmax, int chan,
                         float* out, void* stream);
int ld_edges_reduce_padded(const int* counts, const float* x, int batch, int nodes, int nmax, int chan, float* out,
                           void* stream);

/* ---- channel mixing -------------------------------------------------------------------------
 * Replaces tensor_ops_cuda.tensor_linear forward and backward
 * (extensions/tensor_ops/tensor_ops.cpp:31-170, tensor_ops_kern.cu:6-71).
 * y[r,o,s] = sum_i W[o,i] x[r,i,s], s < 3^inds. W element strides sw0, sw1 (dx uses W transposed). */
int ld_tensor_linear(int inds, const float* W, long long sw0, long long sw1, const float* x, float* y, long long rows,
                     int dim_in, int dim_out, void* stream);
int ld_tensor_linear_dw_workspace(int inds, long long rows, int dim_in, int dim_out, size_t* bytes);
int ld_tensor_linear_dw(int inds, const float* dy, const float* x, float* dW, long long rows, int dim_in, int dim_out,
                        void* workspace, size_t workspace_bytes, void* stream);

/* ---- l<=2 tensor products ---------------------------------------------------------------------
 * Replace codegen_tensops_cuda.bee_fwd_cuda / bee_bwl_cuda / bee_bwr_cuda
 * (extensions/codegen_tensops/codegen_tensops.cpp:1519-1769) and cow_o0_* / cow_o1_*
 * (codegen_tensops.cpp:1771-1979). Operands contiguous [rows, chan, (3,)^l]. out13/grads13 are
 * HOST arrays of 13 device pointers in the order 000,110,220,011,101,121,211,022,202,112,222,111,212. */
int ld_bee_fwd(const float* l0, const float* l1, const float* l2, const float* r0, const float* r1, const float* r2,
               long long rows, int chan, float* const* out13, void* stream);
/* Node-local products of SelfTensProds (archs/diffuser_atoms15.py:59-95) for ONE channel mixing per rank on either
 * side: inputs lr0 [rows][2*chan], lr1 [rows][2*chan][3], lr2 [rows][2*chan][3][3] hold the left operands in channels
 * [0, chan) and the right operands in [chan, 2*chan) (one linear per rank with 2*chan outputs); outputs are the 13
 * Bee products concatenated per rank, P_a [rows][3*chan] = (000|110|220), P_v [rows][5*chan][3] =
 * (011|101|121|211|111), P_d [rows][5*chan][3][3] = (022|202|112|222|212), the K dimension of the concatenated Y maps.
 * chan a multiple of 32. Same arithmetic as ld_bee_fwd. out_bf16: P_v and P_d are stored as BF16. */
int ld_bee_self_products(const float* lr0, const float* lr1, const float* lr2, long long rows, int chan, float* P_a,
                         void* P_v, void* P_d, int out_bf16, void* stream);
int ld_bee_bw(int left, const float* o0, const float* o1, const float* o2, const float* const* grads13, long long rows,
              int chan, float* d0, float* d1, float* d2, void* stream);
int ld_cow_o0_fwd(const float* l0, const float* l1, const float* r0, const float* r1, long long rows, int chan,
                  float* y000, float* y110, void* stream);
int ld_cow_o0_bw(const float* o0, const float* o1, const float* g000, const float* g110, long long rows, int chan,
                 float* d0, float* d1, void* stream);
int ld_cow_o1_fwd(const float* l0, const float* l1, const float* r0, const float* r1, long long rows, int chan,
                  float* y011, float* y101, float* y111, void* stream);
int ld_cow_o1_bw(int left, const float* o0, const float* o1, const float* g011, const float* g101, const float* g111,
                 long long rows, int chan, float* d0, float* d1, void* stream);

/* ---- dense layers and the fused PaiNN message ----------------------------------------------------
 * ld_mlp3_rows: the three-layer MLPs applied per node (archs/meanflow_painn8.py:38-51;
 * archs/diffuser_atoms15.py:98-110 with the direct term Wdt). Weights are "packed":
 * Wkt = nn.Linear.weight.t().contiguous(), [in][out].
 * ld_painn_message_f32: Message.forward (archs/meanflow_painn8.py:77-100) fused with the edge
 * gather and edges_reduce_src; FP32 arithmetic throughout. */
int ld_mlp3_rows(const float* x, long long rows, int k0, const float* W1t, const float* b1, int n1, const float* W2t,
                 const float* b2, int n2, const float* W3t, const float* b3, int n3, int act, const float* Wdt,
                 float* out, void* stream);
int ld_painn_message_f32(const int* row_ptr, const int* dst, const float* rij, int Nt, int n, int n_rbf, int radial_kind,
                         float rmax, float eps, const float* W1t, const float* b1, const float* W2t, const float* b2,
                         const float* W3t, const float* b3, const float* actv, const float* x_v, const float* res_a,
                         const float* res_v, float* out_a, float* out_v, long long* edge_counter, void* stream);

/* ---- tensor-core dense layers (tcgen05, BF16 operands, FP32 accumulation) ------------------------
 * ld_linear_bf16_tc: y = act(x W^T + b) with the Cartesian index folded into the rows; the
 * tensor-core counterpart of tensor_ops_cuda.tensor_linear (extensions/tensor_ops/tensor_ops_kern.cu:6-42)
 * and of nn.Linear inside the reference's MLPs (archs/meanflow_painn8.py:38-51). 2e-2 relative.
 * Weights are packed once with ld_pack_weights_bf16 (ld_packed_weight_elems BF16 values). */
long long ld_packed_weight_elems(int N, int K);
int ld_pack_weights_bf16(const float* W, long long sw0, long long sw1, int N, int K, void* out, void* stream);
int ld_linear_bf16_tc(const float* x, long long rows_outer, int K, int S, const void* wp, const float* bias, int N, int act,
                      float* y, int* status_dev, void* stream);
/* same with the activations already stored as BF16 ([rows_outer, K, S] contiguous); the MMA operands are BF16 in
 * any case, so the result equals that of the same values passed as FP32 */
int ld_linear_bf16_tc_in16(const void* x_bf16, long long rows_outer, int K, int S, const void* wp, const float* bias, int N,
                           int act, float* y, int* status_dev, void* stream);
/* The same with a residual, y = residual + act(x W^T + b), residual laid out like y. Only for the shapes of the streaming
 * kernel (K a multiple of 128, N <= 128, packed weights up to 94 KB); LD_ERR_UNSUPPORTED otherwise. */
int ld_linear_bf16_tc_in16_res(const void* x_bf16, const float* residual, long long rows_outer, int K, int S, const void* wp,
                               const float* bias, int N, int act, float* y, int* status_dev, void* stream);
/* same with a BF16 result written to y_bf16[r*ld_row + o*ld_col + s + off] (plain layout: ld_row = N*S,
 * ld_col = S, off = 0); used to interleave the left operands of the l<=2 message layer per channel */
int ld_linear_bf16_tc_out16(const float* x, long long rows_outer, int K, int S, const void* wp, const float* bias, int N,
                            int act, void* y_bf16, long long ld_row, long long ld_col, int off, int* status_dev, void* stream);

/* ld_linear_bf16_tc_out16 with a two-piece component axis (components s >= s_split land s_jump elements further on) and,
 * with in_cm != 0, component-major FP32 activations x [rows_outer][S][K]. Writes the gather layouts of the fused l<=2
 * edge kernels; same reference operator as ld_linear_bf16_tc. */
int ld_linear_bf16_tc_out16_split(const float* x, long long rows_outer, int K, int S, const void* wp, const float* bias, int N,
                                  int act, void* y_bf16, long long ld_row, long long ld_col, int off, int s_split,
                                  long long s_jump, int in_cm, int* status_dev, void* stream);
/* The three channel mixings L0, L1, L2 of an l<=2 message layer (archs/diffuser_atoms15.py:244-246) in one launch that
 * writes whole neighbour rows: rows [Nt][128][16] BF16 = (L0 x_a, L1 x_v [3], L2 x_d [9], 0, 0, 0) per (node, channel),
 * the same values as three ld_linear_bf16_tc_out16 launches into that buffer, without their partially written sectors.
 * x_a [Nt][da], x_v [Nt][dv][3], x_d [Nt][dd][3][3] FP32; W*p from ld_pack_weights_bf16 ([128][da|dv|dd]); chan = 128,
 * widths multiples of 16 with da + 3 dv + 9 dd <= 640. LD_FLAG_TIMEOUT in *status_dev if a wait runs out. */
int ld_bee_left_rows_bf16_tc(const float* x_a, const float* x_v, const float* x_d, long long Nt, int da, int dv, int dd, int chan,
                             const void* W0p, const void* W1p, const void* W2p, void* rows, int* status_dev, void* stream);

/* Self-test of the bounded waits (no counterpart in the reference): ld_linear_bf16_tc (S = 1, no bias) on a launch
 * whose weight panels are never requested and whose waits give up after 64 polls. Every block leaves through the
 * failure path: *status_dev receives LD_FLAG_TIMEOUT, tensor memory is released, y stays unwritten, the device stays
 * usable. rows_outer <= 1024. */
int ld_linear_bf16_tc_selftest_timeout(const float* x, long long rows_outer, int K, const void* wp, int N, float* y,
                                       int* status_dev, void* stream);

/* ---- edge radial encodings as an operator of their own: r [rows, 3] (kind 3: r [rows]) -> out [rows, n] -------
 * kind 0: radial_encode of archs/meanflow_painn8.py:25-35; kind 1: Gaussian basis x cosine cutoff (benchmark spec,
 * not in the reference); kind 2: radial_encode_edge of archs/diffuser_atoms5.py:25-30; kind 3: radial_encode of
 * managan/layers_common.py:122-126 (rmax unused); kind 4: radial_encode_8 of managan/jacobi_radenc.py:27-33
 * (n = 8, coeff = its 8x9 coefficient matrix; NULL for the other kinds). */
int ld_radial_encode(int kind, const float* r, long long rows, int n, float rmax, const float* coeff, float* out,
                     void* stream);

/* Counter-based Gaussian noise for sharded rollouts (the reference draws torch.randn_like per step,
 * archs/meanflow_painn8.py:302-310, whose stream depends on how the batch is split): out[i] = base[i] + scale *
 * z(seed, step, first_element + i), z ~ N(0,1) a pure function of its three arguments (splitmix64 hash + Box-Muller),
 * so a rank owning systems [b0, b1) draws what a single GPU draws for them. base may be NULL. */
int ld_counter_noise(float* out, const float* base, float scale, long long first_element, long long count,
                     unsigned long long seed, unsigned long long step, void* stream);

/* ld_painn_message_bf16_tc: ld_painn_message_f32 with the per-edge distance MLP on tcgen05
 * (BF16 operands, FP32 accumulation in tensor memory); same reference lines
 * (archs/meanflow_painn8.py:77-100). Weights packed by ld_pack_weights_bf16. 2e-2 relative.
 * gather16 (optional, else NULL): the node features of the neighbours as BF16 records made by
 * ld_painn_pack_gather from actv [Nt][4n] and x_v [Nt][n][3]; [Nt][n/8][64] BF16, per 8 channels the four
 * actv planes, the 24 vector components and 8 unused values (128 bytes, four 32-byte loads per thread).
 * With gather16 the kernel does not read actv / x_v. */
int ld_painn_pack_gather(const float* actv, const float* x_v, int Nt, int n, void* out_bf16, void* stream);
int ld_painn_message_bf16_tc(const int* row_ptr, const int* dst, const float* rij, int Nt, int n, int n_rbf, int radial_kind,
                             float rmax, float eps, const void* w1p, const float* b1, const void* w2p, const float* b2,
                             const void* w3p, const float* b3, const float* actv, const float* x_v, const void* gather16,
                             const float* res_a, const float* res_v, float* out_a, float* out_v, long long* edge_counter,
                             int* status_dev, void* stream);

/* ---- fused l<=2 message layer ------------------------------------------------------------------------
 * Messages.forward (archs/diffuser_atoms15.py:227-253) without edge-sized tensors: the radial
 * read-in (managan/jacobi_radenc.py:27-33), the Bee products (managan/codegen_tensor_products.py:64-75)
 * and edges_reduce_src (managan/graph_layers.py:54-59) in one pass over the CSR.
 * _vd: per-node sums of the five rank-1 and five rank-2 products (the Y maps are linear, so the
 * caller applies them per node with ld_tensor_linear over 5*chan inputs). _scalar: per-edge Y maps
 * and mlp_a, summed per node. `jacobi` = 8x9 coefficients of the shifted Jacobi(1,0) polynomials.
 * feat_bf16: 0 = L0/L1/L2 FP32; 1 = BF16; 2 = L0 alone points to the interleaved BF16 form
 * [node][chan][16] = (l0, l1[3], l2[9], 3 unused) written by ld_linear_bf16_tc_out16.
 * out_bf16 (vd): S_v / S_d are stored as BF16 (same shapes), the input form of ld_linear_bf16_tc_in16. */
int ld_bee_messages_vd_f32(const int* row_ptr, const int* dst, const float* rij, int Nt, int chan, float r0, const float* L0,
                           const float* L1, const float* L2, const float* enc_w, const float* enc_b, const float* jacobi,
                           float scale, void* S_v, void* S_d, int feat_bf16, int out_bf16, void* stream);
/* The same sums for chan = 128 on the tensor cores: one tcgen05 MMA per edge (the neighbour's row scaled by the radial
 * weight, times a 16 x 64 matrix of monomials of the unit vector), accumulated over a node's edges in tensor memory.
 * rows [Nt][128][16] BF16 interleaved per channel (l0, l1[3], l2[9], 3 unused; written by ld_linear_bf16_tc_out16);
 * S_v [Nt][3][640], S_d [Nt][9][640] BF16 component-major, times scale. BF16 operands, FP32 accumulation: 2e-2.
 * A wait that runs out raises LD_FLAG_TIMEOUT in *status_dev. */
int ld_bee_messages_vd_bf16_tc(const int* row_ptr, const int* dst, const float* rij, int Nt, int chan, float r0, const void* rows,
                               const float* enc_w, const float* enc_b, const float* jacobi, float scale, void* S_v, void* S_d,
                               int* status_dev, void* stream);
int ld_bee_messages_scalar_f32(const int* row_ptr, const int* dst, const float* rij, int Nt, int chan, int dim_a, float r0,
                               const float* L0, const float* L1, const float* L2, const float* enc_w, const float* enc_b,
                               const float* jacobi, const float* Yt, const float* W1t, const float* b1, const float* W2t,
                               const float* b2, const float* W3t, const float* b3, const float* Wdt, float scale,
                               float* out_a, void* stream);

/* Tensor-core variant of ld_bee_messages_scalar_f32 (tcgen05, BF16 operands, 2e-2 relative); weights
 * packed by ld_pack_weights_bf16: Yp [a][3*chan], W1p [2a][a], W2p [2a][2a], W3p [a][3a] = (W3 | W_direct + I). */
int ld_bee_messages_scalar_bf16_tc(const int* row_ptr, const int* dst, const float* rij, int Nt, int chan, int dim_a, float r0,
                                   const float* L0, const float* L1, const float* L2, const float* enc_w, const float* enc_b,
                                   const float* jacobi, const void* Yp, const void* W1p, const float* b1, const void* W2p,
                                   const float* b2, const void* W3p, const float* b3, float scale, float* out_a,
                                   int feat_bf16, int* status_dev, void* stream);

/* ---- group norms of node-level activations ----------------------------------------------------------
 * Replace ScalGroupNorm (managan/layers_common.py:201-223; center = 1, S = 1: y = beta + gamma (x - mean) /
 * sqrt(eps + var), statistics over the nodes of a system and the channels of a group) and TensGroupNorm
 * (managan/tensor_products.py:215-232; center = 0, beta = NULL: y = gamma x / sqrt(eps + m2), m2 = mean over
 * nodes and group channels of the squared norm over the S = 3^inds components). x, y: [B][N][C][S] float32.
 * workspace: 98 * B * groups floats of device memory (statistics and chunk partials). */
int ld_group_norm(const float* x, int B, int N, int C, int S, int groups, int center, float eps, const float* gamma,
                  const float* beta, float* y, void* workspace, void* stream);

/* ---- dense proximity attention ---------------------------------------------------------------------
 * Replace the Triton operators proxattn (managan/triton_kernels/proxattn.py:239-311: _fwd_kernel :30-83,
 * _bwd_kernel_kvy :86-164, _bwd_kernel_qx :167-236) and proxattn_periodic (proxattn_periodic.py, same layout plus
 * the box), defined by refimpl_proxattn (proxattn.py:9-27, proxattn_periodic.py:9-28):
 *   out[z,m,:] = sum_n r0sq[z % heads] / (r0sq[z % heads] + dist2(X[z,m], Y[z,n])) * (Q[z,m] . K[z,n]) * V[z,n,:]
 * Q, K, V, out, d_out, dQ, dK, dV: [Z][N][dim] float32, dim in {16, 32, 64, 128}; X, Y, dX, dY: [Z][N][3];
 * r0sq: [heads] on the device, Z a multiple of heads (r0sq receives no gradient, as in the reference).
 * periodic = 0: dist2 = |x - y|^2; periodic = 1: sum_a (1 - cos(2 pi (x_a - y_a) / box_a)) box_a^2 / (2 pi^2).
 * ld_proxattn_bwd writes all five gradients (two kernels: one per key tile, one per query tile). */
int ld_proxattn_fwd(const float* Q, const float* K, const float* V, const float* X, const float* Y, const float* r0sq,
                    int heads, int Z, int N, int dim, int periodic, float box_x, float box_y, float box_z, float* out,
                    void* stream);
/* The same forward on the tensor cores in TF32 (tcgen05.mma kind::tf32, accumulators in TMEM) - the precision of the
 * Triton kernel's tl.dot on FP32 inputs. status_dev: optional device word, LD_FLAG_TIMEOUT if a bounded wait ran out. */
int ld_proxattn_fwd_tf32_tc(const float* Q, const float* K, const float* V, const float* X, const float* Y, const float* r0sq,
                            int heads, int Z, int N, int dim, int periodic, float box_x, float box_y, float box_z, float* out,
                            int* status_dev, void* stream);
int ld_proxattn_bwd(const float* Q, const float* K, const float* V, const float* X, const float* Y, const float* r0sq,
                    int heads, int Z, int N, int dim, int periodic, float box_x, float box_y, float box_z,
                    const float* d_out, float* dQ, float* dK, float* dV, float* dX, float* dY, void* stream);

/* ---- dense-weight l<=2 products (Ant16) and the bare channel-wise product --------------------------
 * Replace codegen_tensops_cuda.ant16_{o0,o1,o2,oc}_cuda and their _backward / _backleft / _wtsback
 * companions (extensions/codegen_tensops/codegen_tensops.cpp:610-1517; einsum definitions
 * managan/codegen_tensor_products.py:112-133) and the einsum of TensorProdBare
 * (managan/tensor_products.py:91-108).
 * product = position in 000,110,220,011,101,121,211,022,202,112,222,111,212. With
 * U[b,(o,l),J] = sum_r P[o,l,r] x[b,r,J] (ld_tensor_linear with P viewed as [(o l), r]):
 *   contract_left: y[b,o,K] (+)= sum_l c_IJK left[b,l,I] U[b,o,l,J]            (forward)
 *   expand:        dU[b,o,l,J] = c_IJK left[b,l,I] dy[b,o,K]                    (dx = ld_tensor_linear(dU, P^T);
 *                                                                               dP = ld_tensor_linear_dw(dU, x))
 *   contract_out:  dleft[b,l,I] = sum_o c_IJK U[b,o,l,J] dy[b,o,K]
 * c = the product's constant coupling (Kronecker deltas and the Levi-Civita symbol).
 * ld_tensor_prod_bare: y[n, keep_l + keep_r] = sum_c a[n, keep_l + c] b[n, keep_r + c] with
 * (inds_l + inds_r - inds_o) / 2 trailing indices contracted (mode 0); mode 1: a = dy, b = x_r -> dx_l;
 * mode 2: a = dy, b = x_l -> dx_r. n counts (row, channel) pairs. */
int ld_ant16_contract_left(int product, const float* left, const float* U, long long rows, int dim_o, int dim_l, float* y,
                           int accumulate, void* stream);
int ld_ant16_expand(int product, const float* left, const float* dy, long long rows, int dim_o, int dim_l, float* dU,
                    void* stream);
int ld_ant16_contract_out(int product, const float* U, const float* dy, long long rows, int dim_o, int dim_l, float* dleft,
                          void* stream);
int ld_tensor_prod_bare(int mode, int inds_l, int inds_r, int inds_o, const float* a, const float* b, long long n, float* out,
                        void* stream);

/* ---- the l<=2 message layer as ONE edge kernel (chan = 128, dim_a = 128; BF16 tensor-core path, 2e-2 relative) ------
 * Messages.forward (archs/diffuser_atoms15.py:227-253) with every neighbour row gathered once: rows [Nt][2][128][8] BF16
 * (per node and channel l0, l1[3], l2[0..3] | l2[4..8], three zeros; written by ld_linear_bf16_tc_out16 / _split), the
 * per-node sums of the rank-1 / rank-2 products accumulated by tcgen05 MMAs in tensor memory. out_a [Nt][128] FP32;
 * S_v [Nt][3][640], S_d [Nt][9][640] BF16 as from ld_bee_messages_vd_f32 (out_bf16). Other arguments as
 * ld_bee_messages_scalar_bf16_tc. Measured slower than the two-kernel path on B200; kept as an option.
 * ld_bee_gamma_table: the (column, left component, monomial, sign) table of the products as a matrix product, for host
 * checks against the reference's einsum definitions (managan/codegen_tensor_products.py:235-249); returns the count. */
int ld_bee_messages_fused_bf16_tc(const int* row_ptr, const int* dst, const float* rij, int Nt, int chan, int dim_a, float r0,
                                  const void* rows, const float* enc_w, const float* enc_b, const float* jacobi, const void* Yp,
                                  const void* W1p, const float* b1, const void* W2p, const float* b2, const void* W3p,
                                  const float* b3, float scale, float* out_a, void* S_v, void* S_d, int* status_dev,
                                  void* stream);
int ld_bee_gamma_table(int* out);

/* ---- component-major activations (no counterpart in the reference, whose tensors are [.., chan, 3^l]) -------------
 * Between fused stages the vector / rank-2 node features can be kept as [node][component][chan]: every (node,
 * component) pair is then a plain GEMM row, and the channel mixings above take them without strided access:
 * ld_linear_bf16_tc_out16_split (in_cm = 1) reads them, ld_linear_bf16_tc / _in16 with S = 1 over rows*3^l rows write
 * them. The two operators below are the node-local ones in that layout: TensGroupNorm (managan/tensor_products.py:215-232)
 * and the Bee products of SelfTensProds (archs/diffuser_atoms15.py:59-95), results identical to their
 * [.., chan, 3^l] forms element for element. */
int ld_group_norm_cm(const float* x, int B, int N, int C, int S, int groups, int center, float eps, const float* gamma,
                     const float* beta, float* y, void* workspace, void* stream);
/* ld_group_norm with a residual: y = residual + norm(x), residual laid out like x (may be NULL). */
int ld_group_norm_res(const float* x, const float* residual, int B, int N, int C, int S, int groups, int center, float eps,
                      const float* gamma, const float* beta, float* y, void* workspace, void* stream);
int ld_bee_self_products_cm(const float* lr0, const float* lr1, const float* lr2, long long rows, int chan, float* P_a,
                            void* P_v, void* P_d, void* stream);
/* The six channel mixings in front of the node-local products and the products themselves in one launch (chan = 128;
 * archs/diffuser_atoms15.py:59-95): x_a [Nt][da], x_v [Nt][dv][3], x_d [Nt][dd][3][3] FP32; LR*p = ld_pack_weights_bf16 of
 * the stacked (left | right) weight matrices [256][da|dv|dd]; outputs as ld_bee_self_products with out_bf16 = 1. Widths
 * multiples of 16 with da + 3 dv + 9 dd <= 640. BF16 operands, FP32 accumulation and products. LD_FLAG_TIMEOUT in
 * *status_dev if a wait runs out. */
int ld_bee_self_front_bf16_tc(const float* x_a, const float* x_v, const float* x_d, long long Nt, int da, int dv, int dd, int chan,
                              const void* LR0p, const void* LR1p, const void* LR2p, float* P_a, void* P_v, void* P_d,
                              int* status_dev, void* stream);

#ifdef __cplusplus
}
#endif
#endif
