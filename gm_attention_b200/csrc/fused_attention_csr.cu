// Fully fused gauge attention on an arbitrary target-major CSR neighbourhood
// graph with per-edge tables:
//
//   s_e,h  = scale * sum_n <q_i, tau_n(e) k_j>_h + bias_e       (in-window edges only)
//   alpha  = softmax over the target's edges
//   out_i  = sum_e alpha_e,h * tau_n(e) v_j                      per head h, frequency n
//
// i.e. the reference's scores+softmax op (src/gm_attention/nn/fused/attention.h:145-165,
// 295-316) composed with its eager value path "transport, weight, segment-sum"
// (src/gm_attention/nn/kernels.py:156-189, src/gm_attention/nn/_scatter.py:36-46),
// without ever materialising alpha or any per-edge field.
//
// One warp owns one (target, sample).  The 32 lanes are split into H groups of
// L = 32 / H lanes, one group per head; a lane owns the head's copies
// u = s, s + L, ... of every frequency ("slots": a real for n = 0, an (re, im)
// pair for n >= 1) in registers for q, the output accumulator and (backward)
// dO / dq.  Per edge the group reduces its partial dot products with log2(L)
// xor-shuffles, so all heads' logits appear at once; the softmax is online
// (running max / sum), the transport rho(n theta) is applied in registers.
//
// The geometry (row_ptr, source, tables) describes ONE sample of n_nodes
// points; the node fields hold `batch` samples back to back and every sample
// shares the tables.
//
// Backward: per (target, sample) warp again, with the row's log-sum-exp saved
// by the forward and Delta = <dO_i, O_i> per head: dq_i in registers, dk_j and
// dv_j by atomic adds (fp32 accumulators for bf16 storage).
#include <mutex>

#include "common.cuh"

namespace gmb {
namespace {

constexpr int MAX_SLOTS = 16;  // slots a lane can own
constexpr int MAX_F = 8;

struct SlotPlan {
  int n_slots;
  int off[MAX_SLOTS];    // flat offset of the slot's frequency block (all heads)
  int mult[MAX_SLOTS];   // a_n per head
  int order[MAX_SLOTS];  // n (0: scalar)
  int round[MAX_SLOTS];  // r: the lane owns copy u = s + L * r
};

template <typename S>
struct FusedArgs {
  using C = typename Compute<S>::type;
  const S *q, *k, *v, *out_in, *dout;
  const C *transport, *bias, *lse_in;
  const uint8_t* inside;
  const int64_t *row_ptr, *source;
  S *out, *dq;
  C *lse;
  void *dk, *dv;  // S*, or float* accumulators when S is bf16
  int64_t n_nodes, batch;
  int D, orders, H;
  C scale;
  SlotPlan plan;
};

template <typename T>
__device__ __forceinline__ T group_sum(T v, int L) {
  for (int o = L >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename S, int NS>
__global__ void __launch_bounds__(256) fused_forward_kernel(FusedArgs<S> a) {
  using C = typename Compute<S>::type;
  const int lane = threadIdx.x & 31;
  const int64_t gw = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (gw >= a.n_nodes * a.batch) return;
  const int64_t i = gw / a.batch, b = gw % a.batch;
  const int L = 32 / a.H, h = lane / L, s = lane % L;
  const int64_t base = b * a.n_nodes;

  int col[NS];
  C qr[NS], qi[NS], accr[NS], acci[NS];
  const S* q_i = a.q + (base + i) * a.D;
#pragma unroll
  for (int t = 0; t < NS; ++t) {
    col[t] = -1;
    qr[t] = qi[t] = accr[t] = acci[t] = C(0);
    if (t < a.plan.n_slots) {
      const int u = s + L * a.plan.round[t], a_n = a.plan.mult[t];
      if (u < a_n) {
        const int dim = a.plan.order[t] == 0 ? 1 : 2;
        col[t] = a.plan.off[t] + dim * (h * a_n + u);
        qr[t] = ld<C>(q_i + col[t]);
        if (dim == 2) qi[t] = ld<C>(q_i + col[t] + 1);
      }
    }
  }
  C m = neg_inf<C>(), l = C(0);
  const int64_t e0 = a.row_ptr[i], e1 = a.row_ptr[i + 1];
  for (int64_t e = e0; e < e1; ++e) {
    if (!a.inside[e]) continue;
    const int64_t j = base + a.source[e];
    const S* k_j = a.k + j * a.D;
    const S* v_j = a.v + j * a.D;
    const C* tau = a.transport + e * a.orders * 2;
    C part = C(0);
    C tvr[NS], tvi[NS];
#pragma unroll
    for (int t = 0; t < NS; ++t) {
      tvr[t] = tvi[t] = C(0);
      if (col[t] >= 0) {
        const int n = a.plan.order[t];
        if (n == 0) {
          part += qr[t] * ld<C>(k_j + col[t]);
          tvr[t] = ld<C>(v_j + col[t]);
        } else {
          const C tr = tau[2 * n], ti = tau[2 * n + 1];
          const C kr = ld<C>(k_j + col[t]), ki = ld<C>(k_j + col[t] + 1);
          part += qr[t] * (tr * kr - ti * ki) + qi[t] * (tr * ki + ti * kr);
          const C vr = ld<C>(v_j + col[t]), vi = ld<C>(v_j + col[t] + 1);
          tvr[t] = tr * vr - ti * vi;
          tvi[t] = tr * vi + ti * vr;
        }
      }
    }
    const C logit = a.scale * group_sum(part, L) + a.bias[e];
    if (logit > m) {
      const C corr = gm_exp(m - logit);
      l *= corr;
#pragma unroll
      for (int t = 0; t < NS; ++t) { accr[t] *= corr; acci[t] *= corr; }
      m = logit;
    }
    const C p = gm_exp(logit - m);
    l += p;
#pragma unroll
    for (int t = 0; t < NS; ++t) { accr[t] += p * tvr[t]; acci[t] += p * tvi[t]; }
  }
  const C inv = l > C(0) ? C(1) / l : C(0);
  S* out_i = a.out + (base + i) * a.D;
#pragma unroll
  for (int t = 0; t < NS; ++t) {
    if (col[t] >= 0) {
      st<S>(out_i + col[t], accr[t] * inv);
      if (a.plan.order[t] != 0) st<S>(out_i + col[t] + 1, acci[t] * inv);
    }
  }
  if (s == 0) a.lse[(base + i) * a.H + h] = l > C(0) ? m + gm_log(l) : neg_inf<C>();
}

template <typename A, typename C>
__device__ __forceinline__ void accumulate(A* p, C v) { atomicAdd(p, (A)v); }

template <typename S, int NS>
__global__ void __launch_bounds__(256) fused_backward_kernel(FusedArgs<S> a) {
  using C = typename Compute<S>::type;
  using A = typename std::conditional<std::is_same<S, __nv_bfloat16>::value, float, S>::type;
  const int lane = threadIdx.x & 31;
  const int64_t gw = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (gw >= a.n_nodes * a.batch) return;
  const int64_t i = gw / a.batch, b = gw % a.batch;
  const int L = 32 / a.H, h = lane / L, s = lane % L;
  const int64_t base = b * a.n_nodes;
  A* dk = reinterpret_cast<A*>(a.dk);
  A* dv = reinterpret_cast<A*>(a.dv);

  int col[NS];
  C qr[NS], qi[NS], gr[NS], gi[NS], dqr[NS], dqi[NS];
  const S* q_i = a.q + (base + i) * a.D;
  const S* g_i = a.dout + (base + i) * a.D;
  const S* o_i = a.out_in + (base + i) * a.D;
  C delta = C(0);
#pragma unroll
  for (int t = 0; t < NS; ++t) {
    col[t] = -1;
    qr[t] = qi[t] = gr[t] = gi[t] = dqr[t] = dqi[t] = C(0);
    if (t < a.plan.n_slots) {
      const int u = s + L * a.plan.round[t], a_n = a.plan.mult[t];
      if (u < a_n) {
        const int dim = a.plan.order[t] == 0 ? 1 : 2;
        col[t] = a.plan.off[t] + dim * (h * a_n + u);
        qr[t] = ld<C>(q_i + col[t]);
        gr[t] = ld<C>(g_i + col[t]);
        delta += gr[t] * ld<C>(o_i + col[t]);
        if (dim == 2) {
          qi[t] = ld<C>(q_i + col[t] + 1);
          gi[t] = ld<C>(g_i + col[t] + 1);
          delta += gi[t] * ld<C>(o_i + col[t] + 1);
        }
      }
    }
  }
  delta = group_sum(delta, L);
  const C lse = a.lse_in[(base + i) * a.H + h];
  const int64_t e0 = a.row_ptr[i], e1 = a.row_ptr[i + 1];
  for (int64_t e = e0; e < e1; ++e) {
    if (!a.inside[e]) continue;
    const int64_t j = base + a.source[e];
    const S* k_j = a.k + j * a.D;
    const S* v_j = a.v + j * a.D;
    const C* tau = a.transport + e * a.orders * 2;
    C part = C(0), dpart = C(0);
    C tkr[NS], tki[NS];
#pragma unroll
    for (int t = 0; t < NS; ++t) {
      tkr[t] = tki[t] = C(0);
      if (col[t] >= 0) {
        const int n = a.plan.order[t];
        if (n == 0) {
          tkr[t] = ld<C>(k_j + col[t]);
          part += qr[t] * tkr[t];
          dpart += gr[t] * ld<C>(v_j + col[t]);
        } else {
          const C tr = tau[2 * n], ti = tau[2 * n + 1];
          const C kr = ld<C>(k_j + col[t]), ki = ld<C>(k_j + col[t] + 1);
          tkr[t] = tr * kr - ti * ki;
          tki[t] = tr * ki + ti * kr;
          part += qr[t] * tkr[t] + qi[t] * tki[t];
          const C vr = ld<C>(v_j + col[t]), vi = ld<C>(v_j + col[t] + 1);
          dpart += gr[t] * (tr * vr - ti * vi) + gi[t] * (tr * vi + ti * vr);
        }
      }
    }
    // one shuffle tree for both sums
    for (int o = L >> 1; o > 0; o >>= 1) {
      part += __shfl_xor_sync(0xffffffffu, part, o);
      dpart += __shfl_xor_sync(0xffffffffu, dpart, o);
    }
    const C p = gm_exp(a.scale * part + a.bias[e] - lse);
    const C ds = a.scale * p * (dpart - delta);
    A* dk_j = dk + j * a.D;
    A* dv_j = dv + j * a.D;
#pragma unroll
    for (int t = 0; t < NS; ++t) {
      if (col[t] >= 0) {
        const int n = a.plan.order[t];
        dqr[t] += ds * tkr[t];
        if (n == 0) {
          accumulate(dk_j + col[t], ds * qr[t]);
          accumulate(dv_j + col[t], p * gr[t]);
        } else {
          dqi[t] += ds * tki[t];
          const C tr = tau[2 * n], ti = tau[2 * n + 1];
          // conj(tau) x = (tr xr + ti xi, tr xi - ti xr)
          accumulate(dk_j + col[t], ds * (tr * qr[t] + ti * qi[t]));
          accumulate(dk_j + col[t] + 1, ds * (tr * qi[t] - ti * qr[t]));
          accumulate(dv_j + col[t], p * (tr * gr[t] + ti * gi[t]));
          accumulate(dv_j + col[t] + 1, p * (tr * gi[t] - ti * gr[t]));
        }
      }
    }
  }
  S* dq_i = a.dq + (base + i) * a.D;
#pragma unroll
  for (int t = 0; t < NS; ++t) {
    if (col[t] >= 0) {
      st<S>(dq_i + col[t], dqr[t]);
      if (a.plan.order[t] != 0) st<S>(dq_i + col[t] + 1, dqi[t]);
    }
  }
}

__global__ void narrow_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int64_t n) {
  for (int64_t x = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; x < n; x += (int64_t)gridDim.x * blockDim.x)
    dst[x] = __float2bfloat16_rn(src[x]);
}

int make_plan(const int64_t* desc_host, int F, int H, int D, SlotPlan& plan) {
  GM_REQUIRE(H == 1 || H == 2 || H == 4 || H == 8, GM_ERR_UNSUPPORTED, "gm_attention: heads must be 1, 2, 4 or 8 (got %d)", H);
  GM_REQUIRE(F >= 1 && F <= MAX_F, GM_ERR_ARGUMENT, "gm_attention: 1 <= F <= %d descriptor rows", MAX_F);
  const int L = 32 / H;
  plan.n_slots = 0;
  for (int f = 0; f < F; ++f) {
    const int n = (int)desc_host[f * 5 + 0], a_n = (int)desc_host[f * 5 + 1], off = (int)desc_host[f * 5 + 2];
    const int dim = n == 0 ? 1 : 2;
    GM_REQUIRE(n >= 0 && a_n >= 1 && off >= 0 && off + H * a_n * dim <= D, GM_ERR_ARGUMENT,
               "gm_attention: descriptor row %d (n=%d, a_n=%d, off=%d) leaves the width D=%d", f, n, a_n, off, D);
    for (int r = 0; r * L < a_n; ++r) {
      GM_REQUIRE(plan.n_slots < MAX_SLOTS, GM_ERR_LIMIT, "gm_attention: a lane would own more than %d slots (D=%d, H=%d)", MAX_SLOTS, D, H);
      plan.off[plan.n_slots] = off;
      plan.mult[plan.n_slots] = a_n;
      plan.order[plan.n_slots] = n;
      plan.round[plan.n_slots] = r;
      ++plan.n_slots;
    }
  }
  return GM_OK;
}

template <typename S>
int fill_args(FusedArgs<S>& a, const void* q, const void* k, const void* v, const void* transport, const void* bias,
              const uint8_t* inside, const int64_t* desc_host, const int64_t* row_ptr, const int64_t* source,
              int64_t n_nodes, int64_t batch, int D, int F, int orders, int H, double scale) {
  using C = typename Compute<S>::type;
  a.q = (const S*)q; a.k = (const S*)k; a.v = (const S*)v;
  a.transport = (const C*)transport; a.bias = (const C*)bias; a.inside = inside;
  a.row_ptr = row_ptr; a.source = source;
  a.n_nodes = n_nodes; a.batch = batch; a.D = D; a.orders = orders; a.H = H; a.scale = (C)scale;
  int status = make_plan(desc_host, F, H, D, a.plan);
  if (status != GM_OK) return status;
  for (int t = 0; t < a.plan.n_slots; ++t)
    GM_REQUIRE(a.plan.order[t] < orders, GM_ERR_ARGUMENT, "gm_attention: transport table has %d orders, frequency %d needs more", orders, a.plan.order[t]);
  return GM_OK;
}

int check_common(const void* q, const void* k, const void* v, const void* transport, const void* bias, const uint8_t* inside,
                 const int64_t* desc_host, const int64_t* row_ptr, const int64_t* source, int64_t n_nodes, int64_t n_edges,
                 int64_t batch, int D, int orders, int dtype) {
  GM_REQUIRE(n_nodes >= 0 && n_edges >= 0 && batch >= 1, GM_ERR_ARGUMENT, "gm_attention: bad sizes");
  GM_REQUIRE(D >= 1 && orders >= 1, GM_ERR_ARGUMENT, "gm_attention: D and orders must be positive");
  GM_REQUIRE(dtype == GM_F32 || dtype == GM_F64 || dtype == GM_BF16, GM_ERR_UNSUPPORTED, "gm_attention: unknown dtype %d", dtype);
  GM_REQUIRE(desc_host, GM_ERR_ARGUMENT, "gm_attention: null descriptor");
  if (n_nodes == 0) return GM_OK;
  GM_REQUIRE(q && k && v && row_ptr, GM_ERR_ARGUMENT, "gm_attention: null pointer");
  GM_REQUIRE(n_edges == 0 || (transport && bias && inside && source), GM_ERR_ARGUMENT, "gm_attention: null edge table");
  return GM_OK;
}

template <typename S, template <typename, int> class Launcher>
int dispatch_slots(const FusedArgs<S>& a, cudaStream_t stream) {
  const int64_t warps = a.n_nodes * a.batch;
  const int threads = 256, per_block = threads / 32;
  const int64_t blocks = (warps + per_block - 1) / per_block;
  GM_REQUIRE(blocks < ((int64_t)1 << 31), GM_ERR_LIMIT, "gm_attention: too many (node, sample) pairs");
  if (a.plan.n_slots <= 4) Launcher<S, 4>::run(a, (int)blocks, threads, stream);
  else if (a.plan.n_slots <= 8) Launcher<S, 8>::run(a, (int)blocks, threads, stream);
  else Launcher<S, 16>::run(a, (int)blocks, threads, stream);
  return launch_status("gm_attention");
}

template <typename S, int NS> struct ForwardLauncher {
  static void run(const FusedArgs<S>& a, int blocks, int threads, cudaStream_t stream) {
    fused_forward_kernel<S, NS><<<blocks, threads, 0, stream>>>(a);
  }
};
template <typename S, int NS> struct BackwardLauncher {
  static void run(const FusedArgs<S>& a, int blocks, int threads, cudaStream_t stream) {
    fused_backward_kernel<S, NS><<<blocks, threads, 0, stream>>>(a);
  }
};

}  // namespace
}  // namespace gmb

using namespace gmb;

extern "C" int gm_attention_forward(const void* q, const void* k, const void* v, const void* transport, const void* bias,
                                    const uint8_t* inside, const int64_t* desc_host, const int64_t* row_ptr,
                                    const int64_t* source, int64_t n_nodes, int64_t n_edges, int64_t batch, int D, int F,
                                    int orders, int H, double scale, int dtype, void* out, void* lse, void* stream) {
  int status = check_common(q, k, v, transport, bias, inside, desc_host, row_ptr, source, n_nodes, n_edges, batch, D, orders, dtype);
  if (status != GM_OK || n_nodes == 0) return status;
  GM_REQUIRE(out && lse, GM_ERR_ARGUMENT, "gm_attention_forward: null output");
  auto run = [&](auto tag) {
    using S = decltype(tag);
    using C = typename Compute<S>::type;
    FusedArgs<S> a{};
    int st = fill_args<S>(a, q, k, v, transport, bias, inside, desc_host, row_ptr, source, n_nodes, batch, D, F, orders, H, scale);
    if (st != GM_OK) return st;
    a.out = (S*)out; a.lse = (C*)lse;
    return dispatch_slots<S, ForwardLauncher>(a, (cudaStream_t)stream);
  };
  if (dtype == GM_F32) return run(float());
  if (dtype == GM_F64) return run(double());
  return run(__nv_bfloat16());
}

extern "C" int64_t gm_attention_backward_scratch_bytes(int64_t n_nodes, int64_t batch, int D, int dtype) {
  return dtype == GM_BF16 ? 2 * n_nodes * batch * (int64_t)D * (int64_t)sizeof(float) : 0;
}

extern "C" int gm_attention_backward(const void* dout, const void* q, const void* k, const void* v, const void* out,
                                     const void* lse, const void* transport, const void* bias, const uint8_t* inside,
                                     const int64_t* desc_host, const int64_t* row_ptr, const int64_t* source,
                                     int64_t n_nodes, int64_t n_edges, int64_t batch, int D, int F, int orders, int H,
                                     double scale, int dtype, void* dq, void* dk, void* dv, void* scratch, void* stream) {
  int status = check_common(q, k, v, transport, bias, inside, desc_host, row_ptr, source, n_nodes, n_edges, batch, D, orders, dtype);
  if (status != GM_OK || n_nodes == 0) return status;
  GM_REQUIRE(dout && out && lse && dq && dk && dv, GM_ERR_ARGUMENT, "gm_attention_backward: null pointer");
  GM_REQUIRE(dtype != GM_BF16 || scratch, GM_ERR_ARGUMENT, "gm_attention_backward: bf16 storage needs the fp32 scratch buffer");
  cudaStream_t cs = (cudaStream_t)stream;
  const int64_t count = n_nodes * batch * (int64_t)D;
  auto run = [&](auto tag) {
    using S = decltype(tag);
    using C = typename Compute<S>::type;
    FusedArgs<S> a{};
    int st = fill_args<S>(a, q, k, v, transport, bias, inside, desc_host, row_ptr, source, n_nodes, batch, D, F, orders, H, scale);
    if (st != GM_OK) return st;
    a.dout = (const S*)dout; a.out_in = (const S*)out; a.lse_in = (const C*)lse; a.dq = (S*)dq;
    if (std::is_same<S, __nv_bfloat16>::value) {
      a.dk = scratch; a.dv = (float*)scratch + count;
      GM_CUDA(cudaMemsetAsync(scratch, 0, 2 * count * sizeof(float), cs));
    } else {
      a.dk = dk; a.dv = dv;
      GM_CUDA(cudaMemsetAsync(dk, 0, count * sizeof(S), cs));
      GM_CUDA(cudaMemsetAsync(dv, 0, count * sizeof(S), cs));
    }
    return dispatch_slots<S, BackwardLauncher>(a, cs);
  };
  if (dtype == GM_F32) return run(float());
  if (dtype == GM_F64) return run(double());
  status = run(__nv_bfloat16());
  if (status != GM_OK) return status;
  const int blocks = (int)((count + 255) / 256 < 148 * 16 ? (count + 255) / 256 : 148 * 16);
  narrow_to_bf16_kernel<<<blocks, 256, 0, cs>>>((const float*)scratch, (__nv_bfloat16*)dk, count);
  narrow_to_bf16_kernel<<<blocks, 256, 0, cs>>>((const float*)scratch + count, (__nv_bfloat16*)dv, count);
  return launch_status("gm_attention_backward (narrow)");
}

// ---------------------------------------------------------------------------
// gm_attention_backward_static: the backward above for callers that cannot
// allocate device memory.
//
// Some embedders hand the whole device-memory budget to an arena of their own
// when they start (a serving runtime with a fixed memory plan, a host loop
// with a hard latency bound that may not take the driver's allocator lock or
// the device-wide synchronisation cudaMalloc can imply).  They can pass inputs
// and outputs carved from that arena, but they have nowhere to get the fp32
// accumulation buffer the bf16 backward wants.  For them the buffer lives
// inside the library image: a file-scope device array of a fixed size that
// every GPU loading the library holds until the process exits.
//
// The array's name is only a host-side handle; its device address is looked
// up once per device with cudaGetSymbolAddress (with that device current) and
// kept.  That lookup happens on the FIRST call made on a device, so make that
// first call outside any stream capture.  No cudaMalloc, cudaFree or other
// allocating routine is called.  All calls on a device share the one array:
// it still holds the previous call's sums, so each call clears it first, and
// two calls that overlap on the GPU (different streams) race on it -- order
// them.  Problems larger than the array are refused with GM_ERR_LIMIT.
// The array is part of the library's device image: the driver sets its 32 MiB
// aside when the image is loaded onto a device (with lazy module loading, at
// the first kernel launch or symbol lookup of this library there), so an
// embedder that claims all remaining memory for its arena must make one call
// into this library on each device BEFORE it does so.
// ---------------------------------------------------------------------------
namespace gmb {
namespace {

constexpr int64_t STATIC_SCRATCH_BYTES = 32ll << 20;  // 32 MiB: batch * n_nodes * D <= 4 Mi elements
constexpr int MAX_DEVICES = 64;

static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];

// Device address of the array per device ordinal, looked up under a lock (two host threads may make their first calls
// at once).  An address stays valid for the life of the device's primary context: a process that destroys the context
// (cudaDeviceReset) must not call this entry point again.
void* g_static_scratch_address[MAX_DEVICES] = {nullptr};
std::mutex g_static_scratch_lock;

int static_scratch(void** out) {
  int device = -1;
  GM_CUDA(cudaGetDevice(&device));
  GM_REQUIRE(device >= 0 && device < MAX_DEVICES, GM_ERR_LIMIT, "gm_attention_backward_static: device index %d beyond %d", device, MAX_DEVICES);
  std::lock_guard<std::mutex> guard(g_static_scratch_lock);
  if (g_static_scratch_address[device] == nullptr) {
    void* address = nullptr;
    GM_CUDA(cudaGetSymbolAddress(&address, g_static_scratch));
    g_static_scratch_address[device] = address;
  }
  *out = g_static_scratch_address[device];
  return GM_OK;
}

}  // namespace
}  // namespace gmb

extern "C" int64_t gm_attention_backward_static_capacity(void) { return gmb::STATIC_SCRATCH_BYTES; }

extern "C" int gm_attention_backward_static(const void* dout, const void* q, const void* k, const void* v, const void* out,
                                            const void* lse, const void* transport, const void* bias, const uint8_t* inside,
                                            const int64_t* desc_host, const int64_t* row_ptr, const int64_t* source,
                                            int64_t n_nodes, int64_t n_edges, int64_t batch, int D, int F, int orders, int H,
                                            double scale, int dtype, void* dq, void* dk, void* dv, void* stream) {
  GM_REQUIRE(n_nodes >= 0 && batch >= 1 && D >= 1, GM_ERR_ARGUMENT, "gm_attention_backward_static: bad sizes");
  // sizes whose product would overflow 64 bits must not slip under the limit: bound the factors by division first
  const int64_t element_limit = STATIC_SCRATCH_BYTES / 8;
  const bool representable = n_nodes <= element_limit / D / batch || dtype != GM_BF16;
  const int64_t need = representable ? gm_attention_backward_scratch_bytes(n_nodes, batch, D, dtype) : INT64_MAX;
  GM_REQUIRE(need <= STATIC_SCRATCH_BYTES, GM_ERR_LIMIT,
             "gm_attention_backward_static: this problem needs %lld bytes of accumulation space, the built-in buffer holds %lld "
             "(batch * n_nodes * D <= %lld); use gm_attention_backward with a caller-provided buffer",
             (long long)need, (long long)STATIC_SCRATCH_BYTES, (long long)(STATIC_SCRATCH_BYTES / 8));
  void* scratch = nullptr;
  int status = static_scratch(&scratch);
  if (status != GM_OK) return status;
  return gm_attention_backward(dout, q, k, v, out, lse, transport, bias, inside, desc_host, row_ptr, source, n_nodes, n_edges, batch,
                               D, F, orders, H, scale, dtype, dq, dk, dv, scratch, stream);
}
