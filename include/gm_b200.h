/* libgmb200 -- C ABI of the B200 (sm_100a) fused neighbourhood kernels.
 *
 * Every entry point takes plain device pointers and sizes, launches on the
 * given CUDA stream (a cudaStream_t passed as void*; NULL = the legacy default
 * stream), never synchronises, never throws, and returns a status code:
 *
 *    0  GM_OK
 *   -1  GM_ERR_ARGUMENT     a null pointer, a negative size, a shape the layout forbids
 *   -2  GM_ERR_UNSUPPORTED  a dtype / head count / width outside the kernels' bounds
 *   -3  GM_ERR_CUDA         the launch (or a CUDA call around it) failed
 *   -4  GM_ERR_LIMIT        a documented fixed capacity was exceeded
 *
 * gm_last_error() returns the calling thread's last message.  Unless stated
 * otherwise the caller owns every buffer; outputs documented as "accumulated"
 * must be zeroed by the caller before the call (the Python host layer does it
 * with one cudaMemsetAsync on the same stream).
 *
 * Element types: GM_F32, GM_F64 store and compute in that type; GM_BF16 stores
 * node fields as bfloat16 and computes / accumulates in fp32 (per-edge tables
 * are then fp32).
 *
 * Citations name files of the reference project masonfaldet/gm-attention by
 * their path inside that project.
 */
#ifndef GM_B200_H
#define GM_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { GM_OK = 0, GM_ERR_ARGUMENT = -1, GM_ERR_UNSUPPORTED = -2, GM_ERR_CUDA = -3, GM_ERR_LIMIT = -4 };
enum { GM_F32 = 0, GM_F64 = 1, GM_BF16 = 2 };

/* Library identity: ABI version (bumped on any signature change) and the last
 * error message of the calling thread. */
int gm_abi_version(void);
const char* gm_last_error(void);

/* ------------------------------------------------------------------------
 * Scores + neighbourhood softmax (drop-in for the reference extension's
 * softmax_forward / softmax_backward:
 * src/gm_attention/nn/fused/attention_cpu.cpp:197-252, arithmetic
 * src/gm_attention/nn/fused/attention.h:295-348).
 *
 *   q, k        (n_nodes, D)            node fields, flat layout
 *   transport   (n_edges, orders, 2)    (cos k*gamma, sin k*gamma), k = 0..orders-1
 *   bias        (n_edges)               log window + log quadrature weight
 *   inside      (n_edges) uint8         window > 0
 *   desc        (F, 5) int64            rows (n, a_n per head, flat offset, coeff offset, dim)
 *   row_ptr     (n_nodes + 1) int64, source (n_edges) int64   target-major CSR
 *   alpha       (n_edges, H)            out
 *   dq          (n_nodes, D)            out (written)
 *   dk          (n_nodes, D)            out, ACCUMULATED (zero it first)
 *   max_mult    the largest a_n among desc's rows if the host knows it (desc lives on the device), else 0:
 *               lets the forward pick the kernel that splits a warp's lanes over the heads
 * dtype: GM_F32 or GM_F64.
 * ------------------------------------------------------------------------ */
int gm_softmax_forward(const void* q, const void* k, const void* transport, const void* bias, const uint8_t* inside,
                       const int64_t* desc, const int64_t* row_ptr, const int64_t* source, int64_t n_nodes,
                       int64_t n_edges, int D, int F, int orders, int H, double scale, int64_t deg_max, int max_mult,
                       int dtype, void* alpha, void* stream);

int gm_softmax_backward(const void* dalpha, const void* q, const void* k, const void* transport, const void* bias,
                        const uint8_t* inside, const int64_t* desc, const int64_t* row_ptr, const int64_t* source,
                        const void* alpha, int64_t n_nodes, int64_t n_edges, int D, int F, int orders, int H,
                        double scale, int64_t deg_max, int dtype, void* dq, void* dk, void* stream);

/* ------------------------------------------------------------------------
 * Depthwise steerable convolution under given per-edge weights (drop-in for
 * conv_forward / conv_backward: attention_cpu.cpp:94-145, arithmetic
 * attention.h:174-232, 265-287).
 *
 *   v          (n_nodes, D)
 *   rc         (n_edges, A0)   scalar coefficients R (may be NULL when A0 == 0)
 *   cc         (n_edges, W)    per frequency n >= 1: A (a_n, 2) then B (a_n, 2) at the row's coeff offset
 *   transport, angular (n_edges, orders, 2); rho (n_edges) = r / cutoff; weights (n_edges)
 *   out        (n_nodes, D)    out
 *   dv         (n_nodes, D)    out, ACCUMULATED (zero it first)
 *   drc, dcc   shaped as rc, cc; every entry written
 * dtype: GM_F32 or GM_F64.
 * ------------------------------------------------------------------------ */
int gm_conv_forward(const void* v, const void* rc, const void* cc, const void* transport, const void* angular,
                    const void* rho, const void* weights, const int64_t* desc, const int64_t* row_ptr,
                    const int64_t* source, int64_t n_nodes, int64_t n_edges, int D, int F, int orders, int A0, int W,
                    int dtype, void* out, void* stream);

int gm_conv_backward(const void* g, const void* v, const void* rc, const void* cc, const void* transport,
                     const void* angular, const void* rho, const void* weights, const int64_t* desc,
                     const int64_t* row_ptr, const int64_t* source, int64_t n_nodes, int64_t n_edges, int D, int F,
                     int orders, int A0, int W, int dtype, void* dv, void* drc, void* dcc, void* stream);

/* ------------------------------------------------------------------------
 * Fully fused gauge attention on a general CSR neighbourhood graph:
 *
 *   out_i = sum_e softmax_e( scale <q_i, tau(e) k_j> + bias_e ) * tau_n(e) v_j
 *
 * = the reference's scores+softmax op (attention.h:145-165, 295-316) followed
 * by its eager value path: transport_field (nn/kernels.py:156-189), weighting
 * by alpha, scatter_add_to_nodes (nn/_scatter.py:36-46) -- with alpha and every
 * per-edge field kept in registers.  The reference documents such a fused op
 * (attention.h:1-39) but exports no entry point for it.
 *
 * The geometry (row_ptr, source, tables) describes ONE sample of n_nodes
 * points; q, k, v, out hold `batch` samples back to back, (batch * n_nodes, D),
 * and share it (pass batch = 1 with a tiled geometry for the reference's
 * disjoint-union batching, edge_geometry.py:216-252).
 *
 *   desc_host   (F, 5) int64 in HOST memory (rows as above)
 *   transport   (n_edges, orders, 2), bias (n_edges): fp32 for GM_F32 / GM_BF16, fp64 for GM_F64
 *   lse         (batch * n_nodes, H)   fp32 (fp64 for GM_F64): log-sum-exp of each row's logits
 *   H must be 1, 2, 4 or 8.
 * Backward: dq, dk, dv are fully written (zero-initialised inside).  With
 * GM_BF16 the source-side sums accumulate in fp32 in `scratch`
 * (gm_attention_backward_scratch_bytes bytes, caller-provided, contents
 * undefined on return); other dtypes ignore it.
 * ------------------------------------------------------------------------ */
int gm_attention_forward(const void* q, const void* k, const void* v, const void* transport, const void* bias,
                         const uint8_t* inside, const int64_t* desc_host, const int64_t* row_ptr, const int64_t* source,
                         int64_t n_nodes, int64_t n_edges, int64_t batch, int D, int F, int orders, int H, double scale,
                         int dtype, void* out, void* lse, void* stream);

int64_t gm_attention_backward_scratch_bytes(int64_t n_nodes, int64_t batch, int D, int dtype);

int gm_attention_backward(const void* dout, const void* q, const void* k, const void* v, const void* out, const void* lse,
                          const void* transport, const void* bias, const uint8_t* inside, const int64_t* desc_host,
                          const int64_t* row_ptr, const int64_t* source, int64_t n_nodes, int64_t n_edges, int64_t batch,
                          int D, int F, int orders, int H, double scale, int dtype, void* dq, void* dk, void* dv,
                          void* scratch, void* stream);

/* ------------------------------------------------------------------------
 * Neighbourhood geometry built on the device (replaces the reference's CPU
 * KD-tree search + table derivation: discretization/edge_geometry.py:320-396
 * compute_edge_geometry, :506-619 edge_geometry_from_index, :622-653 row_ptr).
 *
 *   nodes      (n_nodes, 3) float64 unit vectors; frames (n_nodes, 3, 2) float64;
 *   weights    (n_nodes) float64 spherical quadrature weights
 *   cand_lo/hi (n_nodes) int64 or both NULL: target i only examines sources in [lo[i], hi[i])
 * gm_geometry_count writes each target's degree (pairs with float64 geodesic
 * distance <= radius + 1e-10, self-loop included).  The caller forms
 * row_ptr = [0, cumsum(degree)] and allocates E = row_ptr[n_nodes] entries;
 * gm_geometry_fill then writes the CSR (target, source ascending within a row)
 * and the per-edge tables in `dtype` (GM_F32 / GM_F64):
 *   distances, polar_angles, transport_angles, tangent_weights (E);
 *   log_coordinates (E, 2); angular_phases, transport_phases (E, max_frequency + 1, 2)
 *   as (cos, sin) pairs of k * angle.
 * ------------------------------------------------------------------------ */
int gm_geometry_count(const double* nodes, int64_t n_nodes, const int64_t* cand_lo, const int64_t* cand_hi, double radius,
                      int64_t* degree, void* stream);

int gm_geometry_fill(const double* nodes, const double* frames, const double* weights, int64_t n_nodes,
                     const int64_t* cand_lo, const int64_t* cand_hi, double radius, const int64_t* row_ptr,
                     int max_frequency, int dtype, int64_t* target, int64_t* source, void* distances,
                     void* log_coordinates, void* polar_angles, void* transport_angles, void* tangent_weights,
                     void* angular_phases, void* transport_phases, void* stream);

/* ------------------------------------------------------------------------
 * gm_attention_backward without any device allocation (no counterpart in the
 * reference, which allocates through ATen).  For embedders that own all device
 * memory themselves -- a runtime that commits the whole budget to its own
 * arena at start-up, a latency-bound loop that must stay off the driver's
 * allocator -- and so cannot obtain the fp32 accumulation buffer the bf16
 * backward needs.  The buffer is a fixed array inside the library image
 * (gm_attention_backward_static_capacity() bytes, held by every GPU that loads
 * the library until the process ends); bigger problems
 * (2 * batch * n_nodes * D * 4 bytes > capacity) return GM_ERR_LIMIT.
 * Same arguments as gm_attention_backward minus `scratch`.  The first call on
 * a device resolves the array's device address: issue it before any stream
 * capture, and before the embedder claims the rest of the device's memory (the
 * driver sets the array aside when the library's image is loaded onto the
 * device).  The resolved address is valid for the life of the device's primary
 * context.  Calls on one device share the array; it is cleared at the start of
 * each call, and calls that overlap on the GPU race on it.
 * ------------------------------------------------------------------------ */
int64_t gm_attention_backward_static_capacity(void);

int gm_attention_backward_static(const void* dout, const void* q, const void* k, const void* v, const void* out,
                                 const void* lse, const void* transport, const void* bias, const uint8_t* inside,
                                 const int64_t* desc_host, const int64_t* row_ptr, const int64_t* source, int64_t n_nodes,
                                 int64_t n_edges, int64_t batch, int D, int F, int orders, int H, double scale, int dtype,
                                 void* dq, void* dk, void* dv, void* stream);

/* ------------------------------------------------------------------------
 * The fused layer on an equiangular lattice with longitude-equivariant frames
 * (fast path of gm_attention_forward / gm_attention_backward; same arithmetic).
 * Every per-edge quantity depends on (target row, source row, longitude offset)
 * only, so the per-edge tables collapse to compact ones:
 *
 *   win_cnt/win_lo/win_off (rows, 2W + 1) int32: for target row i and source row
 *       j = i + dj (dj in [-W, W]) the neighbours are the cnt longitudes
 *       t + lo .. t + lo + cnt - 1 (mod nlon) of a target at longitude t, and their
 *       entries start at entry win_off; cnt = 0: none
 *   entries (n_entries, ES) fp32: (cos, sin) of n * gamma for n = 1..NORD, then the
 *       bias (-inf for a pair outside the window's support) at index 2 * NORD
 *   row_order (n_order_rows) int32: the rows that own targets, heaviest first
 *   t_*: the same tables transposed (owner = source row, neighbours = the targets
 *       that see it), used by the backward's source-major pass
 *
 * Node fields are (batch, rows, nlon, D), fp32 or bf16 (fp32 arithmetic); head
 * layouts: an optional scalar block plus complex frequencies sharing one
 * multiplicity (else GM_ERR_UNSUPPORTED: use the general entry points).
 * The backward is deterministic (no atomics): dq from a target-major pass, dk
 * and dv from a source-major pass; rows outside row_order / t_row_order are not
 * written.  `delta` is caller-provided workspace, (batch * rows * nlon, H) fp32.
 * ------------------------------------------------------------------------ */
int gm_lattice_attention_forward(const void* q, const void* k, const void* v, const int* win_cnt, const int* win_lo,
                                 const int* win_off, const float* entries, const int* row_order, int n_order_rows,
                                 const int64_t* desc_host, int F, int rows, int nlon, int64_t batch, int D, int H, int W, int ES,
                                 int NORD, double scale, int dtype, void* out, float* lse, void* stream);

int gm_lattice_attention_backward(const void* dout, const void* q, const void* k, const void* v, const void* out, const float* lse,
                                  const int* win_cnt, const int* win_lo, const int* win_off, const float* entries,
                                  const int* row_order, int n_order_rows, const int* t_win_cnt, const int* t_win_lo,
                                  const int* t_win_off, const float* t_entries, const int* t_row_order, int t_n_order_rows,
                                  const int64_t* desc_host, int F, int rows, int nlon, int64_t batch, int D, int H, int W, int ES,
                                  int NORD, double scale, int dtype, void* dq, void* dk, void* dv, float* delta, void* stream);

/* ------------------------------------------------------------------------
 * Factored steerable kernel (drop-in for the reference extension's forward /
 * aggregate / backward / backward_aggregated: factored_cpu.cpp:77-219,
 * arithmetic factored.h:118-347).
 *
 *   h          (n_edges, k - 1)       trunk features; h~ = (1, h)
 *   zc         (n_nodes, k, wc, 2), zr (n_nodes, k, wr)   node-side mixes
 *   angular, transport (n_edges, n_f, 2); rho (n_edges)
 *   desc       (n_blocks, 8) int32    rows (kind, z_off, b_m, ang, trn, power, out_off, take_real),
 *                                     sorted by out_off
 *   order (n_edges), group_ptr (n_groups + 1), group_source (n_groups) int64:
 *              the edges sorted by source, each source's run, the sources
 *   out / rows (n_edges, d_out)
 * gm_factored_backward: g is (n_edges, d_out), or -- the aggregated form, when
 * `target` is non-NULL -- (n_targets, d_out) read through target[e] and scaled
 * by weights[e], with dweights[e] = <g[target[e]], rows[e]> also written.
 * dh (n_edges, k - 1) is written; dzc, dzr are written for every source that has
 * edges (zero them first: nodes without edges keep zero).
 * The packed width 2 wc + wr is bounded by k * (2 wc + wr) <= 8192 (the
 * reference stops at 320).  dtype: GM_F32 or GM_F64.
 * ------------------------------------------------------------------------ */
int gm_factored_forward(const void* h, const void* zc, const void* zr, const void* angular, const void* transport,
                        const void* rho, const int32_t* desc, const int64_t* source, const int64_t* order,
                        const int64_t* group_ptr, const int64_t* group_source, int64_t n_edges, int64_t n_groups, int k, int wc,
                        int wr, int n_f, int n_blocks, int d_out, int dtype, void* out, void* stream);

int gm_factored_aggregate(const void* rows, const void* weights, const int64_t* row_ptr, int64_t n_targets, int64_t n_edges,
                          int d_out, int dtype, void* out, void* stream);

int gm_factored_backward(const void* g, const int64_t* target, const void* weights, const void* rows, const void* h,
                         const void* zc, const void* zr, const void* angular, const void* transport, const void* rho,
                         const int32_t* desc, const int64_t* source, const int64_t* order, const int64_t* group_ptr,
                         const int64_t* group_source, int64_t n_edges, int64_t n_groups, int k, int wc, int wr, int n_f,
                         int n_blocks, int d_out, int dtype, void* dh, void* dzc, void* dzr, void* dweights, void* stream);

/* ------------------------------------------------------------------------
 * Pair term of the general steerable kernel (drop-in for the reference
 * extension's forward / backward: pairs_cpu.cpp:88-136, arithmetic
 * pairs.h:201-365).  out(e) += post(e) f(M(e) (pre(e) u~(e))), M = W h(e) + b.
 *
 *   hidden (n_edges, trunk); weight (width, trunk), bias (width) or NULL,
 *       width = (MATRIX_COMPLEX ? 2 : 1) * a * b
 *   u      (n_edges, a) real (U_REAL) or (n_edges, a, 2) complex
 *   pre, post (n_edges, 2) complex or NULL; scale (n_edges) or NULL
 *   out    (n_edges, b) real (OUT_REAL) or (n_edges, b, 2); ACCUMULATED
 *   grad_u, grad_hidden: ACCUMULATED in place; grad_k (width, n_edges) written
 *   flags: MATRIX_COMPLEX = 1, U_REAL = 2, CONJ_U = 4, OUT_REAL = 8; a, b, trunk in 1..16
 * dtype: GM_F32 or GM_F64.
 * ------------------------------------------------------------------------ */
int gm_pairs_forward(const void* hidden, const void* weight, const void* bias, const void* u, const void* pre, const void* post,
                     const void* scale, void* out, int64_t n_edges, int a, int b, int trunk, int flags, int dtype, void* stream);

int gm_pairs_backward(const void* hidden, const void* weight, const void* bias, const void* u, const void* pre, const void* post,
                      const void* scale, const void* grad_out, void* grad_u, void* grad_hidden, void* grad_k, int64_t n_edges,
                      int a, int b, int trunk, int flags, int dtype, void* stream);

/* ------------------------------------------------------------------------
 * Tensor-core variants of the lattice fast path for bf16 node fields (same
 * tables, same results within bf16 rounding of the attention weights): the
 * per-frequency Gram blocks and the (alpha o tau) V sums run as m16n8k16 bf16
 * matrix products on (16 source positions x 8 targets) tiles of the longitude
 * band; neighbour rows are staged with TMA tensor copies where the head's
 * blocks are exactly 16 / 32 columns wide, with per-thread copies otherwise
 * (environment GM_LATTICE_TMA=0 forces the latter; same results bit for bit).
 * Head layouts: an optional scalar block of <= 16 copies and one to three complex
 * frequencies of orders 1, 2, 3 sharing one multiplicity <= 16; otherwise
 * GM_ERR_UNSUPPORTED (use gm_lattice_attention_forward).
 * ------------------------------------------------------------------------ */
int gm_lattice_attention_backward_tc(const void* dout, const void* q, const void* k, const void* v, const void* out, const float* lse,
                                     const int* win_cnt, const int* win_lo, const int* win_off, const float* entries,
                                     const int* row_order, int n_order_rows, const int* t_win_cnt, const int* t_win_lo,
                                     const int* t_win_off, const float* t_entries, const int* t_row_order, int t_n_order_rows,
                                     const int64_t* desc_host, int F, int rows, int nlon, int64_t batch, int D, int H, int W, int ES,
                                     int NORD, double scale, void* dq, void* dk, void* dv, float* delta, void* stream);

/* The same with a pass mask (bit 0: Delta = <dO, O>; bit 1: target-major pass -> dq; bit 2: source-major pass ->
 * dk, dv).  The band-parallel layer uses it to run the source-major pass of its halo rows first (their sums are sent
 * to the owners while the pass over its own rows runs); the benchmark uses it to time the passes one by one.  With bits 0 and 1 both set the target-major pass forms Delta itself and
 * writes it to `delta` (no separate launch); bit 0 alone runs the stand-alone Delta kernel; passes 2 and 4 without bit 0
 * read the Delta an earlier call left in `delta`. */
int gm_lattice_attention_backward_tc_passes(const void* dout, const void* q, const void* k, const void* v, const void* out,
                                            const float* lse, const int* win_cnt, const int* win_lo, const int* win_off,
                                            const float* entries, const int* row_order, int n_order_rows, const int* t_win_cnt,
                                            const int* t_win_lo, const int* t_win_off, const float* t_entries, const int* t_row_order,
                                            int t_n_order_rows, const int64_t* desc_host, int F, int rows, int nlon, int64_t batch,
                                            int D, int H, int W, int ES, int NORD, double scale, void* dq, void* dk, void* dv,
                                            float* delta, int passes, void* stream);

/* Health flag of the tensor-core lattice kernels (no counterpart in the reference).  Their waits on the
 * completion barriers of the TMA copies are bounded; a wait that runs out sets a per-device flag and the
 * launch's results are invalid.  Writes the flag of the current device to *expired (0: never happened);
 * synchronises the device. */
int gm_lattice_attention_tc_wait_expired(int* expired);

int gm_lattice_attention_forward_tc(const void* q, const void* k, const void* v, const int* win_cnt, const int* win_lo,
                                    const int* win_off, const float* entries, const int* row_order, int n_order_rows,
                                    const int64_t* desc_host, int F, int rows, int nlon, int64_t batch, int D, int H, int W, int ES,
                                    int NORD, double scale, void* out, float* lse, void* stream);

/* ------------------------------------------------------------------------
 * The tensor-core lattice kernels with ALL FOUR HEADS of an owner tile in one
 * CTA (no counterpart in the reference).  Same arithmetic; a neighbour row
 * reaches shared memory as five tensor copies of 128-byte rows (four heads'
 * scalar blocks; two heads' complex blocks) instead of three copies of 32- and
 * 64-byte rows per head, which is what bounds the one-head kernels.  One
 * persistent CTA per SM: twelve consumer warps (head x group of 8 owners) and
 * four producer warps that keep a ring of three stages and the next item's
 * owner rows filled; bounded waits, results poisoned with NaN if one runs out
 * (gm_lattice_attention_tc4_wait_expired reads the device's flag).
 * Serves: 4 heads of 16 scalar + 16 complex copies of each of the orders
 * 1 .. n, n <= 3, every block on a 16-byte boundary, D a multiple of 8, at most
 * 32 neighbour rows, nlon >= 40, fields on 16-byte boundaries; otherwise
 * GM_ERR_UNSUPPORTED (use the one-head entry points above).
 *
 * These entry points read their OWN entry table, ES = 12 (orders <= 2) or 20
 * words per longitude offset x of a row pair (win_off / t_win_off index it):
 *   [0..3] fp32 cos, sin of 1 * gamma and 2 * gamma
 *   [4..7] the same rounded to bf16 and packed in pairs, entry x in the low and
 *          entry x - 1 in the high half of a word
 *   [8] bias * log2(e); with order 3: [9..10] its cos, sin, [12..13] their pairs
 * Every row pair's run of cnt entries must be preceded by 8 and followed by 24
 * padding entries whose bias is -inf (phases 0): the kernels read the entry of
 * every (position, owner) pair of a 16 x 8 tile without a bounds test, and the
 * padding's bias is what gives pairs outside an owner's window the logit -inf.
 * (gm_attention_b200.attention.tensor_core_entries builds the table.)
 * `passes` as in gm_lattice_attention_backward_tc_passes, except that bit 0
 * always runs the stand-alone Delta kernel.
 * ------------------------------------------------------------------------ */
int gm_lattice_attention_forward_tc4(const void* q, const void* k, const void* v, const int* win_cnt, const int* win_lo,
                                     const int* win_off, const float* entries, const int* row_order, int n_order_rows,
                                     const int64_t* desc_host, int F, int rows, int nlon, int64_t batch, int D, int H, int W, int ES,
                                     int NORD, double scale, void* out, float* lse, void* stream);

int gm_lattice_attention_backward_tc4_passes(const void* dout, const void* q, const void* k, const void* v, const void* out,
                                             const float* lse, const int* win_cnt, const int* win_lo, const int* win_off,
                                             const float* entries, const int* row_order, int n_order_rows, const int* t_win_cnt,
                                             const int* t_win_lo, const int* t_win_off, const float* t_entries, const int* t_row_order,
                                             int t_n_order_rows, const int64_t* desc_host, int F, int rows, int nlon, int64_t batch,
                                             int D, int H, int W, int ES, int NORD, double scale, void* dq, void* dk, void* dv,
                                             float* delta, int passes, void* stream);

int gm_lattice_attention_tc4_wait_expired(int* expired);

/* ------------------------------------------------------------------------
 * Halo exchange of the latitude-band decomposition (no counterpart in the
 * reference, which has no distributed code).  One process per GPU; a rank
 * holds its band of lattice rows plus the rows either side that its
 * neighbourhoods reach.  An exchange is a list of point-to-point operations
 * (peer rank, send or receive, device pointer, bytes), issued as ONE NCCL
 * group on `stream`: sends read field memory in place, receives land in this
 * GPU's own memory; nothing blocks the host.  NCCL is looked up at run time in
 * the libnccl.so.2 the process has loaded (GM_ERR_UNSUPPORTED if there is none).
 *
 *   gm_halo_unique_id    rank 0 creates the 128-byte id every rank passes to
 *   gm_halo_comm_create  (collective over the ranks; binds to the current device)
 *   gm_halo_comm_error   NCCL's asynchronous error state of the communicator
 *                        (0: none), for a host-side watchdog
 *   gm_halo_move         packs the rows a neighbour needs into one buffer, unpacks
 *                        or adds a received buffer (one launch each way): NCCL
 *                        costs ~10 us per point-to-point operation, so a
 *                        neighbour gets ONE message per direction
 *   gm_halo_accumulate   dst slab s += src slab s for `slabs` slabs of
 *                        slab_elems elements, dst_stride / src_stride elements
 *                        apart: adds the partial sums a neighbour sent for this
 *                        rank's rows (dtype GM_F32, GM_F64 or GM_BF16)
 * ------------------------------------------------------------------------ */
int gm_halo_unique_id(void* id128);
int gm_halo_comm_create(const void* id128, int rank, int world, void** comm);
int gm_halo_comm_destroy(void* comm);
int gm_halo_comm_error(void* comm, int* async_error);
int gm_halo_exchange(void* comm, int n_ops, const int* peers, const int* sends, void* const* pointers, const int64_t* nbytes,
                     void* stream);
int gm_halo_accumulate(void* dst, const void* src, int64_t slabs, int64_t slab_elems, int64_t dst_stride, int64_t src_stride,
                       int dtype, void* stream);
/* Slabs of up to 4 fields <-> one packed buffer laid out (field, sample, slab): mode 0 packs, 1 unpacks, 2 adds the
 * buffer to the fields (GM_BF16 or GM_F32).  fields[i]: sample 0's slab of field i; samples sample_bytes apart;
 * slab_bytes each; everything in 16-byte units.  One launch. */
int gm_halo_move(int mode, void* const* fields, int n_fields, int64_t batch, int64_t slab_bytes, int64_t sample_bytes, void* packed,
                 int dtype, void* stream);

/* ---------------------------------------------------------------------------
 * Depthwise steerable convolution on a longitude-symmetric lattice with the
 * per-edge coefficient stream of gm_conv_forward replaced by a table per
 * (target row, source row, longitude offset).
 *
 * Replaces, for lattices, the reference's depthwise op fed by its per-edge radial
 * network: nn/depthwise.py:206-238 (stacked_coefficients) ->
 * nn/fused_attention.py:309-321 (forward_depthwise) -> nn/fused/attention.h:174-206,
 * 265-287.  The caller folds every entry's coefficients, transport phase,
 * (r/c)^{2n} e^{2 i n phi} and aggregation weight into
 *   table (entries, table_width) float32:  one factor per scalar channel (padded
 *   to a multiple of 4 columns), then per complex copy the row-major 2 x 2 matrix
 *   of  z -> w (A tau z + omega B conj(tau z))  acting on (re z, im z)
 * (gm_attention_b200/nn/lattice_depthwise.py: fold).  Windows as in
 * gm_lattice_attention_forward: win_cnt / win_lo / win_off (rows, 2 * halo + 1),
 * win_off counting table entries.
 *
 *   items (n_items, 3) int32: kind (0: complex copy, 1: two scalar channels), the
 *       item's first column in the field (even), its first column in the table.
 *   x, y: (batch, rows * nlon, width) GM_F32 or GM_BF16 (fp32 arithmetic); nlon a
 *       multiple of 8; width even.
 *
 * gm_lattice_conv_apply: y[target] = sum over the target's entries of
 *   table[entry] x[source], for the target rows listed in order[0 .. n_order)
 *   (other rows of y are left untouched).  transpose != 0 applies the transposed
 *   matrices: with the transposed windows and the table gathered into their entry
 *   order this is the gradient with respect to x.  Only true neighbours are read.
 * gm_lattice_conv_table_grad: dtable[entry] = sum over the longitudes and samples
 *   of g[target] (x) x[source]  (scalar channels: the products; complex copies:
 *   the 2 x 2 outer product).  blocks (n_blocks, 2) int32 = (window index =
 *   target row * (2 * halo + 1) + source row - target row + halo, first offset):
 *   8 consecutive offsets per block; entries no block covers are left untouched.
 * No atomics: results do not depend on the launch geometry.
 * ------------------------------------------------------------------------ */
int gm_lattice_conv_apply(const void* x, const float* table, const int32_t* items, int n_items, const int32_t* win_cnt,
                          const int32_t* win_lo, const int32_t* win_off, const int32_t* order, int n_order, int rows, int nlon,
                          int batch, int width, int halo, int table_width, int transpose, int dtype, void* y, void* stream);
int gm_lattice_conv_table_grad(const void* g, const void* x, const int32_t* items, int n_items, const int32_t* win_cnt,
                               const int32_t* win_lo, const int32_t* win_off, const int32_t* blocks, int64_t n_blocks, int rows,
                               int nlon, int batch, int width, int halo, int table_width, int dtype, float* dtable, void* stream);

/* ---------------------------------------------------------------------------
 * Halo exchange through peer memory (machines whose GPUs can map each other's
 * memory; one process per GPU).  No reference counterpart.
 *
 * Every rank allocates one zeroed block (gm_peer_alloc) holding its receive
 * buffers and flag words and publishes its 64-byte IPC handle; neighbours map
 * it (gm_peer_open) and only ever STORE into it.  Per (neighbour, kind of
 * exchange) and step = 1, 2, ...:
 *   gm_peer_send  waits (bounded) until *local_ack >= step - 1, copies the rows
 *                 of up to 4 fields into remote_buffer (layout (field, sample,
 *                 slab)), then stores step to *remote_data_flag;
 *   gm_peer_land  waits (bounded) until *local_data_flag >= step, copies
 *                 (add == 0) or adds (add != 0, GM_BF16 / GM_F32) local_buffer
 *                 into the fields' rows, then stores step to *remote_ack.
 * fields[i]: sample 0's slab of field i; batch slabs sample_bytes apart,
 * slab_bytes each; 16-byte units.  local_ticket: a zeroed 4-byte word of the
 * caller's own block, private to the (neighbour, kind, direction).  A rank
 * sends to all neighbours before it lands; a wait that runs out (about one
 * second) sets the word gm_peer_error reads (1: a send's, 2: a landing's),
 * moves nothing and returns.  One launch per call, on `stream`.
 * ------------------------------------------------------------------------ */
int gm_peer_alloc(int64_t bytes, void** block, void* handle64);
int gm_peer_free(void* block);
int gm_peer_open(const void* handle64, void** mapped);
int gm_peer_close(void* mapped);
int gm_peer_send(void* const* fields, int n_fields, int64_t batch, int64_t slab_bytes, int64_t sample_bytes, void* remote_buffer,
                 const uint32_t* local_ack, uint32_t* local_ticket, uint32_t* remote_data_flag, uint32_t step, void* stream);
int gm_peer_land(void* const* fields, int n_fields, int64_t batch, int64_t slab_bytes, int64_t sample_bytes, void* local_buffer,
                 int add, int dtype, const uint32_t* local_data_flag, uint32_t* local_ticket, uint32_t* remote_ack, uint32_t step,
                 void* stream);
/* The same for n_lanes (1 or 2) neighbours in ONE launch (the transfers to / from both sides of a band overlap): every
 * per-neighbour argument is an array of n_lanes; fields holds n_lanes * n_fields pointers, neighbour-major. */
int gm_peer_send_many(int n_lanes, void* const* fields, int n_fields, int64_t batch, const int64_t* slab_bytes, int64_t sample_bytes,
                      void* const* remote_buffers, const uint32_t* const* local_acks, uint32_t* const* local_tickets,
                      uint32_t* const* remote_data_flags, const uint32_t* steps, void* stream);
int gm_peer_land_many(int n_lanes, void* const* fields, int n_fields, int64_t batch, const int64_t* slab_bytes, int64_t sample_bytes,
                      void* const* local_buffers, int add, int dtype, const uint32_t* const* local_data_flags,
                      uint32_t* const* local_tickets, uint32_t* const* remote_acks, const uint32_t* steps, void* stream);
int gm_peer_error(int* code);

#ifdef __cplusplus
}
#endif
#endif /* GM_B200_H */
