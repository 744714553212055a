// Op-level kernels behind the reference extension's four attention entry
// points: scores + neighbourhood softmax (forward, backward) and the depthwise
// steerable convolution under given weights (forward, backward).
//
// Semantics follow src/gm_attention/nn/fused/attention.h of the reference
// (scores :145-165, softmax :295-316, softmax backward :320-348, depthwise
// message :174-206, its backward :211-232); the kernels themselves are new:
//
//  * scores, head-grouped (H a power of two, the usual case): one warp per target, the lanes split into H head
//    groups, every lane owning a few copies of every frequency; four edges' gathers of k_j are in flight; the raw
//    logits go to alpha and the same warp normalises the row in place.
//  * scores, general: one block per target, one WARP per edge with the lanes striding the key row (coalesced
//    128-byte reads of k_j), per-head sums by warp shuffle; the row's logits live in shared memory (or, for very
//    large neighbourhoods, in the alpha output itself) and are normalised there.
//  * softmax backward, conv forward / backward: one warp per target and one LANE per work item -- a (head,
//    frequency, copy) or (frequency, copy): a scalar column or a (re, im) column pair -- listed once per CTA in
//    shared memory; a lane walks the node's edges in order (sequential sums per output) with four edges' loads in
//    flight, 8-byte accesses for the pairs where the address allows, atomics only for the scattered dk / dv.
#include "common.cuh"

namespace gmb {
namespace {

constexpr int MAX_H = 8;
constexpr int MAX_F = 8;
constexpr int DESC = 5;

// ------------------------------------------------------------------ softmax

template <typename T>
struct SoftmaxArgs {
  const T *q, *k, *transport, *bias, *alpha_in, *dalpha;
  const uint8_t* inside;
  const int64_t *desc, *row_ptr, *source;
  T *alpha, *dq, *dk;
  int64_t n_nodes;
  int D, F, orders, H;
  int slots;  // shared-memory logit slots per block (0: keep the logits in alpha)
  T scale;
};

constexpr int SM_THREADS = 128;

template <typename T>
__global__ void __launch_bounds__(SM_THREADS) softmax_forward_kernel(SoftmaxArgs<T> a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* q_s = reinterpret_cast<T*>(smem_raw);
  T* logit_s = q_s + a.D;
  __shared__ int d_n[MAX_F], d_mult[MAX_F], d_off[MAX_F];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = SM_THREADS / 32;
  if (threadIdx.x < a.F) {
    d_n[threadIdx.x] = (int)a.desc[threadIdx.x * DESC + 0];
    d_mult[threadIdx.x] = (int)a.desc[threadIdx.x * DESC + 1];
    d_off[threadIdx.x] = (int)a.desc[threadIdx.x * DESC + 2];
  }
  for (int64_t i = blockIdx.x; i < a.n_nodes; i += gridDim.x) {
    const int64_t e0 = a.row_ptr[i], e1 = a.row_ptr[i + 1];
    const int deg = (int)(e1 - e0);
    __syncthreads();  // the previous node's reads of q_s / logit_s are done (and d_* are written)
    if (deg == 0) continue;
    for (int c = threadIdx.x; c < a.D; c += SM_THREADS) q_s[c] = a.q[i * a.D + c];
    T* logits = (deg * a.H <= a.slots) ? logit_s : a.alpha + e0 * a.H;
    __syncthreads();
    for (int t = warp; t < deg; t += n_warps) {
      const int64_t e = e0 + t, j = a.source[e];
      const T* k_j = a.k + j * a.D;
      const T* tau_e = a.transport + e * a.orders * 2;
      const T bias = a.bias[e];
      for (int h = 0; h < a.H; ++h) {
        T acc = T(0);
        for (int f = 0; f < a.F; ++f) {
          const int n = d_n[f], a_n = d_mult[f];
          if (n == 0) {
            const int base = d_off[f] + h * a_n;
            for (int u = lane; u < a_n; u += 32) acc += q_s[base + u] * k_j[base + u];
          } else {
            const T tr = tau_e[2 * n], ti = tau_e[2 * n + 1];
            const int base = d_off[f] + 2 * h * a_n;
            for (int u = lane; u < a_n; u += 32) {
              const T kr = k_j[base + 2 * u], ki = k_j[base + 2 * u + 1];
              acc += q_s[base + 2 * u] * (tr * kr - ti * ki) + q_s[base + 2 * u + 1] * (tr * ki + ti * kr);
            }
          }
        }
        acc = warp_sum(acc);
        if (lane == 0) logits[t * a.H + h] = a.scale * acc + bias;
      }
    }
    __syncthreads();
    for (int h = warp; h < a.H; h += n_warps) {
      T m = neg_inf<T>();
      for (int t = lane; t < deg; t += 32) {
        const T lw = logits[t * a.H + h];
        if (a.inside[e0 + t] && lw > m) m = lw;  // masked edges never set the shift
      }
      m = warp_max(m);
      T sum = T(0);
      for (int t = lane; t < deg; t += 32) {
        const T u = a.inside[e0 + t] ? gm_exp(logits[t * a.H + h] - m) : T(0);
        logits[t * a.H + h] = u;
        sum += u;
      }
      sum = warp_sum(sum);
      for (int t = lane; t < deg; t += 32) a.alpha[(e0 + t) * a.H + h] = logits[t * a.H + h] / sum;
    }
  }
}


// Scores + softmax with the lanes of a warp split into H head groups (H a power of two): one warp per target,
// a group of L = 32 / H lanes owns a head and each lane the copies u = s, s + L, ... of every frequency (at most
// R per frequency).  Per edge every lane reads its own columns of k_j (the groups together read the whole row once),
// the group reduces with log2(L) xor-shuffles, and all H logits of the edge appear at once.  The raw logits go to
// alpha, the row is then normalised in place by the same warp (masked edges never enter the shift or the sum).
// NF: the number of descriptor rows when known at compile time (3 or 4 frequencies: the usual head types), 0 = up to MAX_F
template <typename T, int R, int NF>
__global__ void __launch_bounds__(128) softmax_forward_grouped_kernel(SoftmaxArgs<T> a) {
  constexpr int FN = NF ? NF : MAX_F;
  const int lane = threadIdx.x & 31;
  const int64_t i = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= a.n_nodes) return;
  const int L = 32 / a.H, h = lane / L, s = lane % L;
  int col[FN][R], order[FN];
  T qr[FN][R], qi[FN][R];
#pragma unroll
  for (int f = 0; f < FN; ++f) {
    order[f] = -1;
#pragma unroll
    for (int r = 0; r < R; ++r) { col[f][r] = -1; qr[f][r] = qi[f][r] = T(0); }
    if (NF || f < a.F) {
      const int n = (int)a.desc[f * DESC], a_n = (int)a.desc[f * DESC + 1], off = (int)a.desc[f * DESC + 2];
      order[f] = n;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int u = s + L * r;
        if (u < a_n) {
          col[f][r] = off + (n == 0 ? 1 : 2) * (h * a_n + u);
          qr[f][r] = a.q[i * a.D + col[f][r]];
          if (n != 0) qi[f][r] = a.q[i * a.D + col[f][r] + 1];
        }
      }
    }
  }
  const int64_t e0 = a.row_ptr[i], e1 = a.row_ptr[i + 1];
  T m = neg_inf<T>();
  // this lane's share of <q_i, tau k_j> for one edge
  auto dot = [&](const T* k_j, const T* tau) -> T {
    T part = T(0);
#pragma unroll
    for (int f = 0; f < FN; ++f) {
      if (!NF && order[f] < 0) continue;
      const T tr = order[f] ? tau[2 * order[f]] : T(1), ti = order[f] ? tau[2 * order[f] + 1] : T(0);
#pragma unroll
      for (int r = 0; r < R; ++r) {
        if (col[f][r] < 0) continue;
        if (order[f] == 0) {
          part += qr[f][r] * k_j[col[f][r]];
        } else {
          const T kr = k_j[col[f][r]], ki = k_j[col[f][r] + 1];
          part += qr[f][r] * (tr * kr - ti * ki) + qi[f][r] * (tr * ki + ti * kr);
        }
      }
    }
    return part;
  };
  auto finish = [&](int64_t e, T part) {
    const T lw = a.scale * part + a.bias[e];
    if (a.inside[e] && lw > m) m = lw;
    if (s == 0) a.alpha[e * a.H + h] = lw;
  };
  constexpr int U = 4;  // edges in flight: their gathers of k_j are issued together
  int64_t e = e0;
  for (; e + U <= e1; e += U) {
    const T* k_j[U];
    T part[U];
#pragma unroll
    for (int u = 0; u < U; ++u) k_j[u] = a.k + a.source[e + u] * a.D;
#pragma unroll
    for (int u = 0; u < U; ++u) part[u] = dot(k_j[u], a.transport + (e + u) * a.orders * 2);
    for (int o = L >> 1; o > 0; o >>= 1) {
#pragma unroll
      for (int u = 0; u < U; ++u) part[u] += __shfl_xor_sync(0xffffffffu, part[u], o);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) finish(e + u, part[u]);
  }
  for (; e < e1; ++e) {
    T part = dot(a.k + a.source[e] * a.D, a.transport + e * a.orders * 2);
    for (int o = L >> 1; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    finish(e, part);
  }
  __syncwarp();
  // normalise: the group's lanes stride the row's edges for their head
  T sum = T(0);
  for (int64_t e = e0 + s; e < e1; e += L) {
    const T u = a.inside[e] ? gm_exp(a.alpha[e * a.H + h] - m) : T(0);
    a.alpha[e * a.H + h] = u;
    sum += u;
  }
  for (int o = L >> 1; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  for (int64_t e = e0 + s; e < e1; e += L) a.alpha[e * a.H + h] /= sum;
}

// ------------------------------------------------------------------ depthwise conv

template <typename T>
struct ConvArgs {
  const T *v, *rc, *cc, *transport, *angular, *rho, *weights, *g;
  const int64_t *desc, *row_ptr, *source;
  T *out, *dv, *drc, *dcc;
  int64_t n_nodes;
  int D, F, orders, A0, W;
};

template <typename T>
__device__ __forceinline__ T rho_power(T rho, int n) {  // (r / c)^{2n} by repeated multiplication from 1
  T s = T(1);
  for (int i = 0; i < 2 * n; ++i) s *= rho;
  return s;
}

// One work item of the depthwise conv = one copy of one frequency: a scalar column, or a (re, im) column pair.
struct ConvItem {
  int col;    // flat column (of the real part)
  int order;  // frequency n
  int coef;   // index into a row of rc (n = 0) / of cc: A at coef, B at coef + 2 mult (n > 0)
  int mult;
};

template <typename T> struct Pair;
template <> struct Pair<float> { using type = float2; };
template <> struct Pair<double> { using type = double2; };

// (x, y) at p: one vector access when the address allows it (decided from the address itself), two scalar ones otherwise
template <typename T>
__device__ __forceinline__ void load_pair(const T* p, T& x, T& y) {
  if ((reinterpret_cast<uintptr_t>(p) & (2 * sizeof(T) - 1)) == 0) {
    const typename Pair<T>::type t = *reinterpret_cast<const typename Pair<T>::type*>(p);
    x = t.x; y = t.y;
  } else {
    x = p[0]; y = p[1];
  }
}
template <typename T>
__device__ __forceinline__ void store_pair(T* p, T x, T y) {
  if ((reinterpret_cast<uintptr_t>(p) & (2 * sizeof(T) - 1)) == 0) {
    typename Pair<T>::type t;
    t.x = x; t.y = y;
    *reinterpret_cast<typename Pair<T>::type*>(p) = t;
  } else {
    p[0] = x; p[1] = y;
  }
}

// One (head, frequency, copy) of the scores' backward: a scalar column or a (re, im) column pair of one head
struct ScoreItem {
  int col, order, head, pad;
};

// Backward of scores + softmax: a warp per target node.  The lanes first reduce sum_e alpha dalpha per head, then
// every lane owns one item and walks the node's edges in order (dq is a sequential sum per column), four edges'
// gathers in flight; dk is accumulated atomically.
template <typename T>
__global__ void softmax_backward_kernel(SoftmaxArgs<T> a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  ScoreItem* items_s = reinterpret_cast<ScoreItem*>(smem_raw);
  int n_items = 0, n_real = 0;
  for (int f = 0; f < a.F; ++f) {
    const int n = (int)a.desc[f * DESC], a_n = (int)a.desc[f * DESC + 1], off = (int)a.desc[f * DESC + 2], dim = (int)a.desc[f * DESC + 4];
    for (int x = threadIdx.x; x < a.H * a_n; x += blockDim.x) items_s[n_items + x] = ScoreItem{off + dim * x, n, x / a_n, 0};
    n_items += a.H * a_n;
    if (n == 0) n_real = n_items;  // items are in column order: the scalar block first
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  constexpr int U = 4;
  for (int64_t i = (int64_t)blockIdx.x * warps + (threadIdx.x >> 5); i < a.n_nodes; i += (int64_t)gridDim.x * warps) {
    const int64_t e0 = a.row_ptr[i], e1 = a.row_ptr[i + 1];
    T total_of_lane = T(0);  // lane h < H ends up with sum_e alpha[e, h] dalpha[e, h]
    for (int h = 0; h < a.H; ++h) {
      T total = T(0);
      for (int64_t e = e0 + lane; e < e1; e += 32) total += a.alpha_in[e * a.H + h] * a.dalpha[e * a.H + h];
      total = warp_sum(total);
      if (lane == h) total_of_lane = total;
    }
    for (int t0 = 0; t0 < n_items; t0 += 32) {
      // a block of 32 items never mixes scalar and complex items unless it straddles the boundary: split it there
      const int t1 = (t0 < n_real && t0 + 32 > n_real) ? n_real : min(t0 + 32, n_items);
      const bool active = t0 + lane < t1;
      const ScoreItem it = items_s[active ? t0 + lane : t0];
      const T total = __shfl_sync(0xffffffffu, total_of_lane, it.head);
      if (active && it.order == 0) {
        const T q_c = a.q[i * a.D + it.col];
        T dq = T(0);
        int64_t e = e0;
        for (; e + U <= e1; e += U) {
          int64_t j[U];
          T al[U], da[U], kc[U];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            j[u] = a.source[e + u];
            al[u] = a.alpha_in[(e + u) * a.H + it.head];
            da[u] = a.dalpha[(e + u) * a.H + it.head];
            kc[u] = a.k[j[u] * a.D + it.col];
          }
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const T ds = a.scale * al[u] * (da[u] - total);
            dq += ds * kc[u];
            atomicAdd(a.dk + j[u] * a.D + it.col, ds * q_c);
          }
        }
        for (; e < e1; ++e) {
          const int64_t j = a.source[e];
          const T ds = a.scale * a.alpha_in[e * a.H + it.head] * (a.dalpha[e * a.H + it.head] - total);
          dq += ds * a.k[j * a.D + it.col];
          atomicAdd(a.dk + j * a.D + it.col, ds * q_c);
        }
        a.dq[i * a.D + it.col] = dq;
      } else if (active) {
        T q_r, q_i;
        load_pair(a.q + i * a.D + it.col, q_r, q_i);
        T dq_r = T(0), dq_i = T(0);
        auto edge = [&](int64_t j, T al, T da, T tr, T ti, T kr, T ki) {
          const T ds = a.scale * al * (da - total);
          dq_r += ds * (tr * kr - ti * ki);  // (tau k)
          dq_i += ds * (tr * ki + ti * kr);
          atomicAdd(a.dk + j * a.D + it.col, ds * (tr * q_r + ti * q_i));  // conj(tau) q
          atomicAdd(a.dk + j * a.D + it.col + 1, ds * (tr * q_i - ti * q_r));
        };
        int64_t e = e0;
        for (; e + U <= e1; e += U) {
          int64_t j[U];
          T al[U], da[U], tr[U], ti[U], kr[U], ki[U];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            j[u] = a.source[e + u];
            al[u] = a.alpha_in[(e + u) * a.H + it.head];
            da[u] = a.dalpha[(e + u) * a.H + it.head];
            load_pair(a.transport + ((e + u) * a.orders + it.order) * 2, tr[u], ti[u]);
            load_pair(a.k + j[u] * a.D + it.col, kr[u], ki[u]);
          }
#pragma unroll
          for (int u = 0; u < U; ++u) edge(j[u], al[u], da[u], tr[u], ti[u], kr[u], ki[u]);
        }
        for (; e < e1; ++e) {
          const int64_t j = a.source[e];
          T tr, ti, kr, ki;
          load_pair(a.transport + (e * a.orders + it.order) * 2, tr, ti);
          load_pair(a.k + j * a.D + it.col, kr, ki);
          edge(j, a.alpha_in[e * a.H + it.head], a.dalpha[e * a.H + it.head], tr, ti, kr, ki);
        }
        store_pair(a.dq + i * a.D + it.col, dq_r, dq_i);
      }
      if (t1 != min(t0 + 32, n_items)) t0 = t1 - 32;  // resume at the boundary
    }
  }
}

// The items of the (single-head) descriptor, in column order, into shared memory; returns their number.
__device__ __forceinline__ int build_conv_items(const int64_t* desc, int F, ConvItem* items_s) {
  int total = 0;
  for (int f = 0; f < F; ++f) {
    const int64_t* row = desc + f * DESC;
    const int n = (int)row[0], a_n = (int)row[1], off = (int)row[2], coff = (int)row[3], dim = (int)row[4];
    for (int x = threadIdx.x; x < a_n; x += blockDim.x)
      items_s[total + x] = ConvItem{off + dim * x, n, n == 0 ? x : coff + 2 * x, a_n};
    total += a_n;
  }
  return total;
}

// Depthwise conv, forward: a warp per target node, a lane per item (scalar items and complex items in separate
// passes, so a pass never diverges); the node's edges are walked in order -- same summation order per output as a
// sequential loop -- four at a time, with the four edges' loads issued before their arithmetic.
constexpr int CONV_UNROLL = 4;

template <typename T>
__global__ void conv_forward_kernel(ConvArgs<T> a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  ConvItem* items_s = reinterpret_cast<ConvItem*>(smem_raw);
  const int n_items = build_conv_items(a.desc, a.F, items_s);
  __syncthreads();
  int n_real = 0;  // items are in column order: the scalar block (frequency 0) first
  while (n_real < n_items && items_s[n_real].order == 0) ++n_real;
  const int lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  for (int64_t i = (int64_t)blockIdx.x * warps + (threadIdx.x >> 5); i < a.n_nodes; i += (int64_t)gridDim.x * warps) {
    const int64_t e0 = a.row_ptr[i], e1 = a.row_ptr[i + 1];
    for (int t0 = 0; t0 < n_real; t0 += 32) {
      if (t0 + lane >= n_real) continue;
      const ConvItem it = items_s[t0 + lane];
      T y = T(0);
      int64_t e = e0;
      for (; e + CONV_UNROLL <= e1; e += CONV_UNROLL) {
        T w[CONV_UNROLL], r[CONV_UNROLL], x[CONV_UNROLL];
#pragma unroll
        for (int u = 0; u < CONV_UNROLL; ++u) {
          w[u] = a.weights[e + u];
          r[u] = a.rc[(e + u) * a.A0 + it.coef];
          x[u] = a.v[a.source[e + u] * a.D + it.col];
        }
#pragma unroll
        for (int u = 0; u < CONV_UNROLL; ++u) y += w[u] * (r[u] * x[u]);
      }
      for (; e < e1; ++e) y += a.weights[e] * (a.rc[e * a.A0 + it.coef] * a.v[a.source[e] * a.D + it.col]);
      a.out[i * a.D + it.col] = y;
    }
    for (int t0 = n_real; t0 < n_items; t0 += 32) {
      if (t0 + lane >= n_items) continue;
      const ConvItem it = items_s[t0 + lane];
      const int n = it.order;
      T yr = T(0), yi = T(0);
      auto message = [&](T w_e, T rho, T tr, T ti, T vr, T vi, T Ar, T Ai, T Br, T Bi, T ar, T ai) {
        const T zr = tr * vr - ti * vi, zi = tr * vi + ti * vr;  // z = tau v
        const T p = rho_power(rho, n);
        const T wr = p * ar, wi = p * ai;
        // m = A z + w (B conj z)
        const T bzr = Br * zr + Bi * zi, bzi = Bi * zr - Br * zi;
        const T mr = (Ar * zr - Ai * zi) + (wr * bzr - wi * bzi);
        const T mi = (Ar * zi + Ai * zr) + (wr * bzi + wi * bzr);
        yr += w_e * mr;
        yi += w_e * mi;
      };
      int64_t e = e0;
      for (; e + CONV_UNROLL <= e1; e += CONV_UNROLL) {
        T w[CONV_UNROLL], rho[CONV_UNROLL], tr[CONV_UNROLL], ti[CONV_UNROLL], vr[CONV_UNROLL], vi[CONV_UNROLL];
        T Ar[CONV_UNROLL], Ai[CONV_UNROLL], Br[CONV_UNROLL], Bi[CONV_UNROLL], ar[CONV_UNROLL], ai[CONV_UNROLL];
#pragma unroll
        for (int u = 0; u < CONV_UNROLL; ++u) {
          const int64_t eu = e + u;
          w[u] = a.weights[eu];
          rho[u] = a.rho[eu];
          load_pair(a.v + a.source[eu] * a.D + it.col, vr[u], vi[u]);
          load_pair(a.transport + (eu * a.orders + n) * 2, tr[u], ti[u]);
          load_pair(a.angular + (eu * a.orders + 2 * n) * 2, ar[u], ai[u]);
          const T* co = a.cc + eu * a.W + it.coef;
          load_pair(co, Ar[u], Ai[u]);
          load_pair(co + 2 * it.mult, Br[u], Bi[u]);
        }
#pragma unroll
        for (int u = 0; u < CONV_UNROLL; ++u) message(w[u], rho[u], tr[u], ti[u], vr[u], vi[u], Ar[u], Ai[u], Br[u], Bi[u], ar[u], ai[u]);
      }
      for (; e < e1; ++e) {
        T tr, ti, vr, vi, Ar, Ai, Br, Bi, ar, ai;
        load_pair(a.transport + (e * a.orders + n) * 2, tr, ti);
        load_pair(a.v + a.source[e] * a.D + it.col, vr, vi);
        const T* co = a.cc + e * a.W + it.coef;
        load_pair(co, Ar, Ai);
        load_pair(co + 2 * it.mult, Br, Bi);
        load_pair(a.angular + (e * a.orders + 2 * n) * 2, ar, ai);
        message(a.weights[e], a.rho[e], tr, ti, vr, vi, Ar, Ai, Br, Bi, ar, ai);
      }
      store_pair(a.out + i * a.D + it.col, yr, yi);
    }
  }
}

// Backward: same walk and grouping; the edge-owned coefficient gradients are written once, dv is accumulated atomically.
template <typename T>
__global__ void conv_backward_kernel(ConvArgs<T> a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  ConvItem* items_s = reinterpret_cast<ConvItem*>(smem_raw);
  const int n_items = build_conv_items(a.desc, a.F, items_s);
  __syncthreads();
  int n_real = 0;
  while (n_real < n_items && items_s[n_real].order == 0) ++n_real;
  const int lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  for (int64_t i = (int64_t)blockIdx.x * warps + (threadIdx.x >> 5); i < a.n_nodes; i += (int64_t)gridDim.x * warps) {
    const int64_t e0 = a.row_ptr[i], e1 = a.row_ptr[i + 1];
    for (int t0 = 0; t0 < n_real; t0 += 32) {
      if (t0 + lane >= n_real) continue;
      const ConvItem it = items_s[t0 + lane];
      const T dy = a.g[i * a.D + it.col];
      int64_t e = e0;
      for (; e + CONV_UNROLL <= e1; e += CONV_UNROLL) {
        T w[CONV_UNROLL], r[CONV_UNROLL], x[CONV_UNROLL];
        int64_t j[CONV_UNROLL];
#pragma unroll
        for (int u = 0; u < CONV_UNROLL; ++u) {
          j[u] = a.source[e + u];
          w[u] = a.weights[e + u];
          r[u] = a.rc[(e + u) * a.A0 + it.coef];
          x[u] = a.v[j[u] * a.D + it.col];
        }
#pragma unroll
        for (int u = 0; u < CONV_UNROLL; ++u) {
          const T dm = w[u] * dy;
          a.drc[(e + u) * a.A0 + it.coef] = dm * x[u];
          atomicAdd(a.dv + j[u] * a.D + it.col, dm * r[u]);
        }
      }
      for (; e < e1; ++e) {
        const int64_t j = a.source[e];
        const T dm = a.weights[e] * dy;
        a.drc[e * a.A0 + it.coef] = dm * a.v[j * a.D + it.col];
        atomicAdd(a.dv + j * a.D + it.col, dm * a.rc[e * a.A0 + it.coef]);
      }
    }
    for (int t0 = n_real; t0 < n_items; t0 += 32) {
      if (t0 + lane >= n_items) continue;
      const ConvItem it = items_s[t0 + lane];
      const int n = it.order;
      T dyr, dyi;
      load_pair(a.g + i * a.D + it.col, dyr, dyi);
      auto edge = [&](int64_t e, int64_t j, T w_e, T rho, T tr, T ti, T vr, T vi, T Ar, T Ai, T Br, T Bi, T ar, T ai) {
        const T zr = tr * vr - ti * vi, zi = tr * vi + ti * vr;
        const T p = rho_power(rho, n);
        const T wr = p * ar, wi = p * ai;
        const T dmr = w_e * dyr, dmi = w_e * dyi;
        // dA = dm conj(z); dB = (dm conj(w)) z
        const T dAr = dmr * zr + dmi * zi, dAi = dmi * zr - dmr * zi;
        const T cr = dmr * wr + dmi * wi, ci2 = dmi * wr - dmr * wi;
        const T dBr = cr * zr - ci2 * zi, dBi = cr * zi + ci2 * zr;
        const int64_t ci = e * a.W + it.coef;
        store_pair(a.dcc + ci, dAr, dAi);
        store_pair(a.dcc + ci + 2 * it.mult, dBr, dBi);
        // dz = conj(A) dm + w (B conj(dm)); dv = conj(tau) dz
        const T bdr = Br * dmr + Bi * dmi, bdi = Bi * dmr - Br * dmi;
        const T dzr = (Ar * dmr + Ai * dmi) + (wr * bdr - wi * bdi);
        const T dzi = (Ar * dmi - Ai * dmr) + (wr * bdi + wi * bdr);
        atomicAdd(a.dv + j * a.D + it.col, tr * dzr + ti * dzi);
        atomicAdd(a.dv + j * a.D + it.col + 1, tr * dzi - ti * dzr);
      };
      int64_t e = e0;
      for (; e + CONV_UNROLL <= e1; e += CONV_UNROLL) {
        T w[CONV_UNROLL], rho[CONV_UNROLL], tr[CONV_UNROLL], ti[CONV_UNROLL], vr[CONV_UNROLL], vi[CONV_UNROLL];
        T Ar[CONV_UNROLL], Ai[CONV_UNROLL], Br[CONV_UNROLL], Bi[CONV_UNROLL], ar[CONV_UNROLL], ai[CONV_UNROLL];
        int64_t j[CONV_UNROLL];
#pragma unroll
        for (int u = 0; u < CONV_UNROLL; ++u) {
          const int64_t eu = e + u;
          j[u] = a.source[eu];
          w[u] = a.weights[eu];
          rho[u] = a.rho[eu];
          load_pair(a.v + j[u] * a.D + it.col, vr[u], vi[u]);
          load_pair(a.transport + (eu * a.orders + n) * 2, tr[u], ti[u]);
          load_pair(a.angular + (eu * a.orders + 2 * n) * 2, ar[u], ai[u]);
          const T* co = a.cc + eu * a.W + it.coef;
          load_pair(co, Ar[u], Ai[u]);
          load_pair(co + 2 * it.mult, Br[u], Bi[u]);
        }
#pragma unroll
        for (int u = 0; u < CONV_UNROLL; ++u)
          edge(e + u, j[u], w[u], rho[u], tr[u], ti[u], vr[u], vi[u], Ar[u], Ai[u], Br[u], Bi[u], ar[u], ai[u]);
      }
      for (; e < e1; ++e) {
        const int64_t j = a.source[e];
        T tr, ti, vr, vi, Ar, Ai, Br, Bi, ar, ai;
        load_pair(a.transport + (e * a.orders + n) * 2, tr, ti);
        load_pair(a.v + j * a.D + it.col, vr, vi);
        const T* co = a.cc + e * a.W + it.coef;
        load_pair(co, Ar, Ai);
        load_pair(co + 2 * it.mult, Br, Bi);
        load_pair(a.angular + (e * a.orders + 2 * n) * 2, ar, ai);
        edge(e, j, a.weights[e], a.rho[e], tr, ti, vr, vi, Ar, Ai, Br, Bi, ar, ai);
      }
    }
  }
}

constexpr int CONV_THREADS = 128;  // 4 target nodes per CTA

int conv_grid(int64_t n_nodes) {  // a few CTAs per SM, each striding the nodes: the item table is built once per CTA
  const int64_t want = (n_nodes + CONV_THREADS / 32 - 1) / (CONV_THREADS / 32);
  const int64_t cap = (int64_t)sm_count() * 16;
  return (int)(want < cap ? (want < 1 ? 1 : want) : cap);
}

int grid_for(int64_t n_nodes) { return (int)(n_nodes < (int64_t)1 << 30 ? n_nodes : (int64_t)1 << 30); }

template <typename T>
int softmax_forward_t(SoftmaxArgs<T> a, int64_t deg_max, int max_mult, cudaStream_t stream) {
  // head-group kernel when the heads split a warp evenly and every lane owns at most 4 copies per frequency
  if ((a.H == 1 || a.H == 2 || a.H == 4 || a.H == 8) && max_mult > 0 && max_mult <= 4 * (32 / a.H)) {
    const int per_lane = (max_mult + 32 / a.H - 1) / (32 / a.H);
    const unsigned blocks = (unsigned)((a.n_nodes + 3) / 4);
    if (per_lane <= 1 && a.F == 3) softmax_forward_grouped_kernel<T, 1, 3><<<blocks, 128, 0, stream>>>(a);
    else if (per_lane <= 1 && a.F == 4) softmax_forward_grouped_kernel<T, 1, 4><<<blocks, 128, 0, stream>>>(a);
    else if (per_lane <= 1) softmax_forward_grouped_kernel<T, 1, 0><<<blocks, 128, 0, stream>>>(a);
    else if (per_lane <= 2 && a.F == 3) softmax_forward_grouped_kernel<T, 2, 3><<<blocks, 128, 0, stream>>>(a);
    else if (per_lane <= 2) softmax_forward_grouped_kernel<T, 2, 0><<<blocks, 128, 0, stream>>>(a);
    else softmax_forward_grouped_kernel<T, 4, 0><<<blocks, 128, 0, stream>>>(a);
    return launch_status("gm_softmax_forward");
  }
  // Logits in shared memory when the largest neighbourhood fits ~96 KiB; else kept in alpha.
  const size_t budget = 96 * 1024;
  size_t want = (size_t)deg_max * a.H;
  if ((want + a.D) * sizeof(T) > budget) want = 0;
  a.slots = (int)want;
  const size_t smem = (a.D + want) * sizeof(T);
  int status = allow_smem(softmax_forward_kernel<T>, smem, "gm_softmax_forward");
  if (status != GM_OK) return status;
  softmax_forward_kernel<T><<<grid_for(a.n_nodes), SM_THREADS, smem, stream>>>(a);
  return launch_status("gm_softmax_forward");
}

template <typename T>
int softmax_backward_t(SoftmaxArgs<T> a, cudaStream_t stream) {
  softmax_backward_kernel<T><<<conv_grid(a.n_nodes), CONV_THREADS, a.D * sizeof(ScoreItem), stream>>>(a);
  return launch_status("gm_softmax_backward");
}

int check_softmax(const void* q, const void* k, const void* transport, const void* bias, const uint8_t* inside,
                  const int64_t* desc, const int64_t* row_ptr, const int64_t* source, int64_t n_nodes, int64_t n_edges,
                  int D, int F, int orders, int H, int dtype) {
  GM_REQUIRE(n_nodes >= 0 && n_edges >= 0, GM_ERR_ARGUMENT, "gm_softmax: negative size");
  GM_REQUIRE(D >= 1, GM_ERR_ARGUMENT, "gm_softmax: D must be positive");
  GM_REQUIRE(H >= 1 && H <= MAX_H, GM_ERR_ARGUMENT, "gm_softmax: at most %d heads", MAX_H);
  GM_REQUIRE(F >= 0 && F <= MAX_F, GM_ERR_ARGUMENT, "gm_softmax: desc must be int64 (F <= %d, %d)", MAX_F, DESC);
  GM_REQUIRE(orders >= 1, GM_ERR_ARGUMENT, "gm_softmax: transport must be (n_edges, orders, 2)");
  GM_REQUIRE(dtype == GM_F32 || dtype == GM_F64, GM_ERR_UNSUPPORTED, "gm_softmax: dtype must be float32 or float64");
  if (n_nodes == 0) return GM_OK;
  GM_REQUIRE(q && k && desc && row_ptr, GM_ERR_ARGUMENT, "gm_softmax: null pointer");
  GM_REQUIRE(n_edges == 0 || (transport && bias && inside && source), GM_ERR_ARGUMENT, "gm_softmax: null edge table");
  return GM_OK;
}

}  // namespace
}  // namespace gmb

using namespace gmb;

extern "C" int gm_softmax_forward(const void* q, const void* k, const void* transport, const void* bias,
                                  const uint8_t* inside, const int64_t* desc, const int64_t* row_ptr,
                                  const int64_t* source, int64_t n_nodes, int64_t n_edges, int D, int F, int orders,
                                  int H, double scale, int64_t deg_max, int max_mult, int dtype, void* alpha, void* stream) {
  int status = check_softmax(q, k, transport, bias, inside, desc, row_ptr, source, n_nodes, n_edges, D, F, orders, H, dtype);
  if (status != GM_OK || n_nodes == 0 || n_edges == 0) return status;
  GM_REQUIRE(alpha, GM_ERR_ARGUMENT, "gm_softmax_forward: null alpha");
  GM_REQUIRE(deg_max >= 1, GM_ERR_ARGUMENT, "gm_softmax_forward: deg_max must be positive");
  auto run = [&](auto tag) {
    using T = decltype(tag);
    SoftmaxArgs<T> a{};
    a.q = (const T*)q; a.k = (const T*)k; a.transport = (const T*)transport; a.bias = (const T*)bias;
    a.inside = inside; a.desc = desc; a.row_ptr = row_ptr; a.source = source; a.alpha = (T*)alpha;
    a.n_nodes = n_nodes; a.D = D; a.F = F; a.orders = orders; a.H = H; a.scale = (T)scale;
    return softmax_forward_t<T>(a, deg_max, max_mult, (cudaStream_t)stream);
  };
  return dtype == GM_F32 ? run(float()) : run(double());
}

extern "C" int gm_softmax_backward(const void* dalpha, const void* q, const void* k, const void* transport,
                                   const void* bias, const uint8_t* inside, const int64_t* desc, const int64_t* row_ptr,
                                   const int64_t* source, const void* alpha, int64_t n_nodes, int64_t n_edges, int D,
                                   int F, int orders, int H, double scale, int64_t deg_max, int dtype, void* dq,
                                   void* dk, void* stream) {
  (void)deg_max;
  int status = check_softmax(q, k, transport, bias, inside, desc, row_ptr, source, n_nodes, n_edges, D, F, orders, H, dtype);
  if (status != GM_OK || n_nodes == 0) return status;
  GM_REQUIRE(dq && dk, GM_ERR_ARGUMENT, "gm_softmax_backward: null output");
  GM_REQUIRE(n_edges == 0 || (alpha && dalpha), GM_ERR_ARGUMENT, "gm_softmax_backward: null alpha / dalpha");
  auto run = [&](auto tag) {
    using T = decltype(tag);
    SoftmaxArgs<T> a{};
    a.q = (const T*)q; a.k = (const T*)k; a.transport = (const T*)transport; a.bias = (const T*)bias;
    a.inside = inside; a.desc = desc; a.row_ptr = row_ptr; a.source = source;
    a.alpha_in = (const T*)alpha; a.dalpha = (const T*)dalpha; a.dq = (T*)dq; a.dk = (T*)dk;
    a.n_nodes = n_nodes; a.D = D; a.F = F; a.orders = orders; a.H = H; a.scale = (T)scale;
    return softmax_backward_t<T>(a, (cudaStream_t)stream);
  };
  return dtype == GM_F32 ? run(float()) : run(double());
}

namespace {

int check_conv(const void* v, const void* rc, const void* cc, const void* transport, const void* angular, const void* rho,
               const void* weights, const int64_t* desc, const int64_t* row_ptr, const int64_t* source, int64_t n_nodes,
               int64_t n_edges, int D, int F, int orders, int A0, int W, int dtype) {
  GM_REQUIRE(n_nodes >= 0 && n_edges >= 0, GM_ERR_ARGUMENT, "gm_conv: negative size");
  GM_REQUIRE(D >= 1, GM_ERR_ARGUMENT, "gm_conv: D must be positive");
  GM_REQUIRE(F >= 0 && F <= MAX_F, GM_ERR_ARGUMENT, "gm_conv: desc must be int64 (F <= %d, %d)", MAX_F, DESC);
  GM_REQUIRE(A0 >= 0 && W >= 0 && orders >= 1, GM_ERR_ARGUMENT, "gm_conv: bad widths");
  GM_REQUIRE(dtype == GM_F32 || dtype == GM_F64, GM_ERR_UNSUPPORTED, "gm_conv: dtype must be float32 or float64");
  if (n_nodes == 0) return GM_OK;
  GM_REQUIRE(v && desc && row_ptr, GM_ERR_ARGUMENT, "gm_conv: null pointer");
  if (n_edges > 0) {
    GM_REQUIRE(transport && angular && rho && weights && source, GM_ERR_ARGUMENT, "gm_conv: null edge table");
    GM_REQUIRE(A0 == 0 || rc, GM_ERR_ARGUMENT, "gm_conv: rc must hold (1, n_edges, a_0) entries");
    GM_REQUIRE(W == 0 || cc, GM_ERR_ARGUMENT, "gm_conv: cc must hold (1, n_edges, W) entries");
  }
  return GM_OK;
}

template <typename T>
ConvArgs<T> conv_args(const void* v, const void* rc, const void* cc, const void* transport, const void* angular,
                      const void* rho, const void* weights, const int64_t* desc, const int64_t* row_ptr,
                      const int64_t* source, int64_t n_nodes, int D, int F, int orders, int A0, int W) {
  ConvArgs<T> a{};
  a.v = (const T*)v; a.rc = (const T*)rc; a.cc = (const T*)cc; a.transport = (const T*)transport;
  a.angular = (const T*)angular; a.rho = (const T*)rho; a.weights = (const T*)weights;
  a.desc = desc; a.row_ptr = row_ptr; a.source = source;
  a.n_nodes = n_nodes; a.D = D; a.F = F; a.orders = orders; a.A0 = A0; a.W = W;
  return a;
}

}  // namespace

extern "C" int gm_conv_forward(const void* v, const void* rc, const void* cc, const void* transport, const void* angular,
                               const void* rho, const void* weights, const int64_t* desc, const int64_t* row_ptr,
                               const int64_t* source, int64_t n_nodes, int64_t n_edges, int D, int F, int orders, int A0,
                               int W, int dtype, void* out, void* stream) {
  int status = check_conv(v, rc, cc, transport, angular, rho, weights, desc, row_ptr, source, n_nodes, n_edges, D, F, orders, A0, W, dtype);
  if (status != GM_OK || n_nodes == 0) return status;
  GM_REQUIRE(out, GM_ERR_ARGUMENT, "gm_conv_forward: null out");
  auto run = [&](auto tag) {
    using T = decltype(tag);
    auto a = conv_args<T>(v, rc, cc, transport, angular, rho, weights, desc, row_ptr, source, n_nodes, D, F, orders, A0, W);
    a.out = (T*)out;
    conv_forward_kernel<T><<<conv_grid(n_nodes), CONV_THREADS, D * sizeof(ConvItem), (cudaStream_t)stream>>>(a);
    return launch_status("gm_conv_forward");
  };
  return dtype == GM_F32 ? run(float()) : run(double());
}

extern "C" int gm_conv_backward(const void* g, const void* v, const void* rc, const void* cc, const void* transport,
                                const void* angular, const void* rho, const void* weights, const int64_t* desc,
                                const int64_t* row_ptr, const int64_t* source, int64_t n_nodes, int64_t n_edges, int D,
                                int F, int orders, int A0, int W, int dtype, void* dv, void* drc, void* dcc, void* stream) {
  int status = check_conv(v, rc, cc, transport, angular, rho, weights, desc, row_ptr, source, n_nodes, n_edges, D, F, orders, A0, W, dtype);
  if (status != GM_OK || n_nodes == 0 || n_edges == 0) return status;
  GM_REQUIRE(g && dv, GM_ERR_ARGUMENT, "gm_conv_backward: null g / dv");
  GM_REQUIRE((A0 == 0 || drc) && (W == 0 || dcc), GM_ERR_ARGUMENT, "gm_conv_backward: null coefficient gradient");
  auto run = [&](auto tag) {
    using T = decltype(tag);
    auto a = conv_args<T>(v, rc, cc, transport, angular, rho, weights, desc, row_ptr, source, n_nodes, D, F, orders, A0, W);
    a.g = (const T*)g; a.dv = (T*)dv; a.drc = (T*)drc; a.dcc = (T*)dcc;
    conv_backward_kernel<T><<<conv_grid(n_nodes), CONV_THREADS, D * sizeof(ConvItem), (cudaStream_t)stream>>>(a);
    return launch_status("gm_conv_backward");
  };
  return dtype == GM_F32 ? run(float()) : run(double());
}
