// The fused pair term of a steerable kernel, per edge -- the reference
// extension's forward / backward (src/gm_attention/nn/fused/pairs_cpu.cpp:88-136,
// arithmetic src/gm_attention/nn/fused/pairs.h:201-365):
//
//   out(e) += post(e) * f( M(e) (pre(e) u~(e)) ),   M(e) = W h(e) + b  (B x A, formed in registers)
//
// u~ = u or conj(u) (u real or complex), pre / post unit phases, post also
// carries the real per-edge scale, f = identity or real part.  The backward
// recomputes M, accumulates grad_u and grad_hidden in place and writes this
// term's coefficient gradient grad_k (width, n_edges), coefficient-major.
//
// One thread per edge.  The input side (A <= 16) and the trunk (T <= 16) are
// unrolled to their bounds with predicates so that every per-edge vector stays
// in registers; the output side (B) is a runtime loop.  W (rows padded to 16
// trunk columns) and b are staged in shared memory once per CTA and read with
// 16-byte loads: every thread of a warp reads the same address (broadcast).
#include "common.cuh"

namespace gmb {
namespace {

constexpr int PMAX = 16;
enum { MATRIX_COMPLEX = 1, U_REAL = 2, CONJ_U = 4, OUT_REAL = 8 };

template <typename T>
struct PArgs {
  int64_t n_edges;
  int a, b, trunk, flags;
  const T *hidden, *weight, *bias, *u, *pre, *post, *scale;
  T* out;
  const T* grad_out;
  T *grad_u, *grad_hidden, *grad_k;
};

// n consecutive values at p into v[0..n) (n <= N): 16-byte loads when the address and n allow it
template <typename T, int N>
__device__ __forceinline__ void load_run(const T* p, int n, T (&v)[N]) {
  constexpr int V = 16 / sizeof(T);
  if ((reinterpret_cast<uintptr_t>(p) & 15) == 0 && n % V == 0) {
#pragma unroll
    for (int k0 = 0; k0 < N; k0 += V)
      if (k0 < n) *reinterpret_cast<uint4*>(&v[k0]) = *reinterpret_cast<const uint4*>(p + k0);
  } else {
#pragma unroll
    for (int k = 0; k < N; ++k)
      if (k < n) v[k] = p[k];
  }
}
// p[0..n) += v[0..n), same access pattern
template <typename T, int N>
__device__ __forceinline__ void add_run(T* p, int n, const T (&v)[N]) {
  constexpr int V = 16 / sizeof(T);
  if ((reinterpret_cast<uintptr_t>(p) & 15) == 0 && n % V == 0) {
#pragma unroll
    for (int k0 = 0; k0 < N; k0 += V)
      if (k0 < n) {
        T q[V];
        *reinterpret_cast<uint4*>(q) = *reinterpret_cast<const uint4*>(p + k0);
#pragma unroll
        for (int x = 0; x < V; ++x) q[x] += v[k0 + x];
        *reinterpret_cast<uint4*>(p + k0) = *reinterpret_cast<const uint4*>(q);
      }
  } else {
#pragma unroll
    for (int k = 0; k < N; ++k)
      if (k < n) p[k] += v[k];
  }
}
// (x, y) added at p: one 2-element access when the address allows it
template <typename T>
__device__ __forceinline__ void add_pair(T* p, T x, T y) {
  if ((reinterpret_cast<uintptr_t>(p) & (2 * sizeof(T) - 1)) == 0) {
    T q[2];
    if (sizeof(T) == 4) *reinterpret_cast<uint2*>(q) = *reinterpret_cast<const uint2*>(p);
    else *reinterpret_cast<uint4*>(q) = *reinterpret_cast<const uint4*>(p);
    q[0] += x; q[1] += y;
    if (sizeof(T) == 4) *reinterpret_cast<uint2*>(p) = *reinterpret_cast<const uint2*>(q);
    else *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(q);
  } else {
    p[0] += x; p[1] += y;
  }
}

template <typename T>
__device__ __forceinline__ void load_edge(const PArgs<T>& p, int64_t e, T (&h)[PMAX], T (&ur)[PMAX], T (&ui)[PMAX], T& s, T& pr, T& pi, T& qr, T& qi) {
#pragma unroll
  for (int k = 0; k < PMAX; ++k) h[k] = T(0);
  load_run(p.hidden + e * p.trunk, p.trunk, h);
  pr = p.pre ? p.pre[2 * e] : T(1);
  pi = p.pre ? p.pre[2 * e + 1] : T(0);
  s = p.scale ? p.scale[e] : T(1);
  qr = (p.post ? p.post[2 * e] : T(1)) * s;
  qi = (p.post ? p.post[2 * e + 1] : T(0)) * s;
  T raw[2 * PMAX];
#pragma unroll
  for (int x = 0; x < 2 * PMAX; ++x) raw[x] = T(0);
  if (p.flags & U_REAL) load_run(p.u + e * p.a, p.a, raw);
  else load_run(p.u + 2 * e * p.a, 2 * p.a, raw);
#pragma unroll
  for (int x = 0; x < PMAX; ++x) {
    ur[x] = ui[x] = T(0);
    if (x < p.a) {
      T re, im;
      if (p.flags & U_REAL) {
        re = raw[x];
        im = T(0);
      } else {
        re = raw[2 * x];
        im = raw[2 * x + 1];
        if (p.flags & CONJ_U) im = -im;
      }
      ur[x] = pr * re - pi * im;  // uu = pre * u~
      ui[x] = pr * im + pi * re;
    }
  }
}

// Weights and bias of the term in shared memory: w_s (rows, PMAX) zero-padded beyond the trunk width, b_s (rows);
// rows = a b (real matrix) or 2 a b (complex: real row, then imaginary row of every entry).
template <typename T>
__device__ __forceinline__ void stage_weights(const PArgs<T>& p, T* w_s, T* b_s) {
  const int rows = ((p.flags & MATRIX_COMPLEX) ? 2 : 1) * p.a * p.b;
  for (int x = threadIdx.x; x < rows * PMAX; x += blockDim.x) {
    const int r = x / PMAX, k = x - r * PMAX;
    w_s[x] = k < p.trunk ? p.weight[(int64_t)r * p.trunk + k] : T(0);
  }
  for (int r = threadIdx.x; r < rows; r += blockDim.x) b_s[r] = p.bias ? p.bias[r] : T(0);
  __syncthreads();
}

// <row r of W, v> over the trunk, four (fp32) / two (fp64) weights per shared-memory load
template <typename T>
__device__ __forceinline__ T row_dot(const T* w_s, int r, int trunk, const T (&v)[PMAX]) {
  constexpr int V = 16 / sizeof(T);
  const T* w = w_s + r * PMAX;
  T acc = T(0);
#pragma unroll
  for (int k0 = 0; k0 < PMAX; k0 += V)
    if (k0 < trunk) {
      T q[V];
      *reinterpret_cast<uint4*>(q) = *reinterpret_cast<const uint4*>(w + k0);
#pragma unroll
      for (int x = 0; x < V; ++x) acc += q[x] * v[k0 + x];
    }
  return acc;
}

// v += s * (row r of W), same access pattern
template <typename T>
__device__ __forceinline__ void row_axpy(const T* w_s, int r, int trunk, T s, T (&v)[PMAX]) {
  constexpr int V = 16 / sizeof(T);
  const T* w = w_s + r * PMAX;
#pragma unroll
  for (int k0 = 0; k0 < PMAX; k0 += V)
    if (k0 < trunk) {
      T q[V];
      *reinterpret_cast<uint4*>(q) = *reinterpret_cast<const uint4*>(w + k0);
#pragma unroll
      for (int x = 0; x < V; ++x) v[k0 + x] += q[x] * s;
    }
}

// M_idx = <W rows, h> + b
template <typename T>
__device__ __forceinline__ void entry(const PArgs<T>& p, const T* w_s, const T* b_s, int trunk, int idx, const T (&h)[PMAX], T& mr, T& mi) {
  if (p.flags & MATRIX_COMPLEX) {
    mr = b_s[2 * idx] + row_dot(w_s, 2 * idx, trunk, h);
    mi = b_s[2 * idx + 1] + row_dot(w_s, 2 * idx + 1, trunk, h);
  } else {
    mr = b_s[idx] + row_dot(w_s, idx, trunk, h);
    mi = T(0);
  }
}

// FULL: the trunk is exactly PMAX wide (the usual 16): the trunk loops carry no bound checks
template <typename T, bool FULL>
__global__ void pairs_forward_kernel(PArgs<T> p) {
  const int trunk = FULL ? PMAX : p.trunk;
  extern __shared__ __align__(16) unsigned char pairs_smem[];
  T* w_s = reinterpret_cast<T*>(pairs_smem);
  T* b_s = w_s + ((p.flags & MATRIX_COMPLEX) ? 2 : 1) * p.a * p.b * PMAX;
  stage_weights(p, w_s, b_s);
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < p.n_edges; e += (int64_t)gridDim.x * blockDim.x) {
    T h[PMAX], ur[PMAX], ui[PMAX], s, pr, pi, qr, qi;
    load_edge(p, e, h, ur, ui, s, pr, pi, qr, qi);
    for (int bi = 0; bi < p.b; ++bi) {
      T accr = T(0), acci = T(0);
#pragma unroll
      for (int x = 0; x < PMAX; ++x)
        if (x < p.a) {
          T mr, mi;
          entry(p, w_s, b_s, trunk, bi * p.a + x, h, mr, mi);
          accr += mr * ur[x] - mi * ui[x];
          acci += mr * ui[x] + mi * ur[x];
        }
      if (p.flags & OUT_REAL) {
        p.out[e * p.b + bi] += accr * s;
      } else {
        add_pair(p.out + 2 * (e * p.b + bi), qr * accr - qi * acci, qr * acci + qi * accr);
      }
    }
  }
}

// FULL: the trunk is exactly PMAX wide (the usual 16): the trunk loops carry no bound checks
template <typename T, bool FULL>
__global__ void pairs_backward_kernel(PArgs<T> p) {
  const int trunk = FULL ? PMAX : p.trunk;
  extern __shared__ __align__(16) unsigned char pairs_smem[];
  T* w_s = reinterpret_cast<T*>(pairs_smem);
  T* b_s = w_s + ((p.flags & MATRIX_COMPLEX) ? 2 : 1) * p.a * p.b * PMAX;
  stage_weights(p, w_s, b_s);
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < p.n_edges; e += (int64_t)gridDim.x * blockDim.x) {
    T h[PMAX], ur[PMAX], ui[PMAX], s, pr, pi, qr, qi;
    load_edge(p, e, h, ur, ui, s, pr, pi, qr, qi);
    T gur[PMAX], gui[PMAX], gh[PMAX];
#pragma unroll
    for (int x = 0; x < PMAX; ++x) gur[x] = gui[x] = gh[x] = T(0);
    for (int bi = 0; bi < p.b; ++bi) {
      // gq = dL/dq for q = M uu: conj(post) g, or (g s, 0) for a real output
      T gqr, gqi;
      if (p.flags & OUT_REAL) {
        gqr = p.grad_out[e * p.b + bi] * s;
        gqi = T(0);
      } else {
        const T gr = p.grad_out[2 * (e * p.b + bi)], gi = p.grad_out[2 * (e * p.b + bi) + 1];
        gqr = qr * gr + qi * gi;
        gqi = qr * gi - qi * gr;
      }
#pragma unroll
      for (int x = 0; x < PMAX; ++x)
        if (x < p.a) {
          const int idx = bi * p.a + x;
          const T gmr = gqr * ur[x] + gqi * ui[x], gmi = gqi * ur[x] - gqr * ui[x];  // gm = gq conj(uu)
          T mr, mi;
          entry(p, w_s, b_s, trunk, idx, h, mr, mi);
          gur[x] += mr * gqr + mi * gqi;  // guu += conj(m) gq
          gui[x] += mr * gqi - mi * gqr;
          if (p.flags & MATRIX_COMPLEX) {
            row_axpy(w_s, 2 * idx, trunk, gmr, gh);
            row_axpy(w_s, 2 * idx + 1, trunk, gmi, gh);
            p.grad_k[(int64_t)(2 * idx) * p.n_edges + e] = gmr;
            p.grad_k[(int64_t)(2 * idx + 1) * p.n_edges + e] = gmi;
          } else {
            row_axpy(w_s, idx, trunk, gmr, gh);
            p.grad_k[(int64_t)idx * p.n_edges + e] = gmr;
          }
        }
    }
    // through uu = pre * u~ (and u~ = conj(u), or u real)
#pragma unroll
    for (int x = 0; x < PMAX; ++x)
      if (x < p.a) {
        const T gr = pr * gur[x] + pi * gui[x];  // conj(pre) guu
        T gi = pr * gui[x] - pi * gur[x];
        if (p.flags & U_REAL) {
          p.grad_u[e * p.a + x] += gr;
        } else {
          if (p.flags & CONJ_U) gi = -gi;
          add_pair(p.grad_u + 2 * (e * p.a + x), gr, gi);
        }
      }
    add_run(p.grad_hidden + e * p.trunk, p.trunk, gh);
  }
}

int check_pairs(int64_t n_edges, int a, int b, int trunk, int flags, int dtype, const void* hidden, const void* weight, const void* u) {
  GM_REQUIRE(n_edges >= 0, GM_ERR_ARGUMENT, "gm_pairs: negative size");
  GM_REQUIRE(a >= 1 && a <= PMAX && b >= 1 && b <= PMAX, GM_ERR_ARGUMENT, "gm_pairs: block dimensions must be in 1..16");
  GM_REQUIRE(trunk >= 1 && trunk <= PMAX, GM_ERR_ARGUMENT, "gm_pairs: trunk width must be in 1..16");
  GM_REQUIRE(flags >= 0 && flags < 16, GM_ERR_ARGUMENT, "gm_pairs: unknown flags");
  GM_REQUIRE(dtype == GM_F32 || dtype == GM_F64, GM_ERR_UNSUPPORTED, "gm_pairs: dtype must be float32 or float64");
  if (n_edges == 0) return GM_OK;
  GM_REQUIRE(hidden && weight && u, GM_ERR_ARGUMENT, "gm_pairs: null pointer");
  return GM_OK;
}

}  // namespace
}  // namespace gmb

using namespace gmb;

extern "C" int gm_pairs_forward(const void* hidden, const void* weight, const void* bias, const void* u, const void* pre,
                                const void* post, const void* scale, void* out, int64_t n_edges, int a, int b, int trunk, int flags,
                                int dtype, void* stream) {
  int status = check_pairs(n_edges, a, b, trunk, flags, dtype, hidden, weight, u);
  if (status != GM_OK || n_edges == 0) return status;
  GM_REQUIRE(out, GM_ERR_ARGUMENT, "gm_pairs_forward: null out");
  auto run = [&](auto tag) {
    using T = decltype(tag);
    PArgs<T> p{n_edges, a, b, trunk, flags, (const T*)hidden, (const T*)weight, (const T*)bias, (const T*)u, (const T*)pre,
               (const T*)post, (const T*)scale, (T*)out, nullptr, nullptr, nullptr, nullptr};
    const int rows = ((flags & MATRIX_COMPLEX) ? 2 : 1) * a * b;
    const size_t smem = (size_t)rows * (PMAX + 1) * sizeof(T);
    int st = trunk == PMAX ? allow_smem(pairs_forward_kernel<T, true>, smem, "gm_pairs_forward") : allow_smem(pairs_forward_kernel<T, false>, smem, "gm_pairs_forward");
    if (st != GM_OK) return st;
    const int64_t want = (n_edges + 127) / 128, cap = (int64_t)sm_count() * 8;  // each CTA stages the weights once and strides the edges
    if (trunk == PMAX) pairs_forward_kernel<T, true><<<(unsigned)(want < cap ? want : cap), 128, smem, (cudaStream_t)stream>>>(p);
    else pairs_forward_kernel<T, false><<<(unsigned)(want < cap ? want : cap), 128, smem, (cudaStream_t)stream>>>(p);
    return launch_status("gm_pairs_forward");
  };
  return dtype == GM_F32 ? run(float()) : run(double());
}

extern "C" int gm_pairs_backward(const void* hidden, const void* weight, const void* bias, const void* u, const void* pre,
                                 const void* post, const void* scale, const void* grad_out, void* grad_u, void* grad_hidden,
                                 void* grad_k, int64_t n_edges, int a, int b, int trunk, int flags, int dtype, void* stream) {
  int status = check_pairs(n_edges, a, b, trunk, flags, dtype, hidden, weight, u);
  if (status != GM_OK || n_edges == 0) return status;
  GM_REQUIRE(grad_out && grad_u && grad_hidden && grad_k, GM_ERR_ARGUMENT, "gm_pairs_backward: null pointer");
  auto run = [&](auto tag) {
    using T = decltype(tag);
    PArgs<T> p{n_edges, a, b, trunk, flags, (const T*)hidden, (const T*)weight, (const T*)bias, (const T*)u, (const T*)pre,
               (const T*)post, (const T*)scale, nullptr, (const T*)grad_out, (T*)grad_u, (T*)grad_hidden, (T*)grad_k};
    const int rows = ((flags & MATRIX_COMPLEX) ? 2 : 1) * a * b;
    const size_t smem = (size_t)rows * (PMAX + 1) * sizeof(T);
    int st = trunk == PMAX ? allow_smem(pairs_backward_kernel<T, true>, smem, "gm_pairs_backward") : allow_smem(pairs_backward_kernel<T, false>, smem, "gm_pairs_backward");
    if (st != GM_OK) return st;
    const int64_t want = (n_edges + 127) / 128, cap = (int64_t)sm_count() * 8;  // each CTA stages the weights once and strides the edges
    if (trunk == PMAX) pairs_backward_kernel<T, true><<<(unsigned)(want < cap ? want : cap), 128, smem, (cudaStream_t)stream>>>(p);
    else pairs_backward_kernel<T, false><<<(unsigned)(want < cap ? want : cap), 128, smem, (cudaStream_t)stream>>>(p);
    return launch_status("gm_pairs_backward");
  };
  return dtype == GM_F32 ? run(float()) : run(double());
}
