// The factored steerable kernel behind the reference extension's entry points
// forward / aggregate / backward / backward_aggregated
// (src/gm_attention/nn/fused/factored_cpu.cpp:77-219; arithmetic
// src/gm_attention/nn/fused/factored.h:118-347).
//
// Per edge e with source j:  row_e = sum over blocks of F_b(e) * sum_t h~_t(e) Z_{t,b}(j),
// h~ = (1, h), F_b = e^{i ang phi} e^{i trn gamma} (r / c)^p (negative orders conjugate,
// the power by repeated multiplication), blocks that share an output offset summed
// before the write, rows n -> 0 keep the real part.
//
// Forward: one CTA per source node (the caller's grouping order / group_ptr /
// group_source), Z(j) staged once in shared memory, one thread per edge of the
// source with h~ in registers; all threads read the same Z address at the same
// time (broadcast).  The packed width 2 wc + wr is bounded only by shared memory
// (the reference stops at 320).
//
// Backward: one CTA per source again, so dZ(j) needs no atomics.  Edges are taken
// in tiles of 32; each lane of the first warp... every thread of the tile builds its
// edge's packed row W(e) = scale * G conj(F) and h~(e) in shared memory, then the CTA
// forms dh(e, t) = <W(e), Z_t(j)> (one thread per (edge, t)) and accumulates
// dZ(t, c) += h~_t(e) W_c(e) with patches of 4 (fp32) / 2 (fp64) consecutive columns of one t
// owned by fixed threads in registers; both read shared memory 16 bytes at a time.
#include "common.cuh"

namespace gmb {
namespace {

constexpr int FMAX_K = 20;
constexpr int FDESC = 8;
constexpr int FTHREADS = 128;
constexpr int TILE = 32;           // edges per backward tile
constexpr int MAX_OWNED = 64;      // (t, c) pairs a thread can own in the backward: K * C <= 64 * 256

template <typename T>
struct FArgs {
  int64_t n_edges, n_groups;
  int k, wc, wr, n_f, n_blocks, d_out;
  const T *h, *zc, *zr, *angular, *transport, *rho;
  const int32_t* desc;
  const int64_t *source, *order, *group_ptr, *group_source;
  T* out;
  // backward
  const T* g;
  const int64_t* target;
  const T *weights, *rows;
  T *dh, *dzc, *dzr, *dweights;
};

// The block's per-edge factor (factored.h:118-144).
template <typename T>
__device__ __forceinline__ void block_factor(const FArgs<T>& a, int64_t e, const int32_t* d, T& fr, T& fi) {
  fr = T(1);
  fi = T(0);
  const int ang = d[3], trn = d[4], power = d[5];
  if (ang != 0) {
    const int o = ang < 0 ? -ang : ang;
    const T pr = a.angular[(e * a.n_f + o) * 2], pi = ang < 0 ? -a.angular[(e * a.n_f + o) * 2 + 1] : a.angular[(e * a.n_f + o) * 2 + 1];
    const T nr = fr * pr - fi * pi, ni = fr * pi + fi * pr;
    fr = nr;
    fi = ni;
  }
  if (trn != 0) {
    const int o = trn < 0 ? -trn : trn;
    const T pr = a.transport[(e * a.n_f + o) * 2], pi = trn < 0 ? -a.transport[(e * a.n_f + o) * 2 + 1] : a.transport[(e * a.n_f + o) * 2 + 1];
    const T nr = fr * pr - fi * pi, ni = fr * pi + fi * pr;
    fr = nr;
    fi = ni;
  }
  const T r = a.rho[e];
  T s = T(1);
  for (int x = 0; x < power; ++x) s *= r;
  fr *= s;
  fi *= s;
}

// Z(j) of one node into shared memory: zc (k, wc, 2) then zr (k, wr).
template <typename T>
__device__ __forceinline__ void stage_node(const FArgs<T>& a, int64_t j, T* zc_s, T* zr_s) {
  const int nc = a.k * a.wc * 2, nr = a.k * a.wr;
  for (int x = threadIdx.x; x < nc; x += blockDim.x) zc_s[x] = a.zc[j * nc + x];
  for (int x = threadIdx.x; x < nr; x += blockDim.x) zr_s[x] = a.zr[j * nr + x];
}

// KT: the trunk width + 1 when it is known at compile time (17: the reference's default radial trunk), 0 = any k <= FMAX_K
template <typename T, int KT>
__global__ void __launch_bounds__(FTHREADS) factored_forward_kernel(FArgs<T> a, int pitch) {
  constexpr int KMAX = KT ? KT : FMAX_K;
  extern __shared__ __align__(16) unsigned char raw[];
  T* zc_s = reinterpret_cast<T*>(raw);
  T* zr_s = zc_s + a.k * a.wc * 2;
  // every thread builds its edge's row in shared memory (odd pitch: no bank conflicts); the warp then writes its 32 rows
  // to global memory one row per store instruction (contiguous) instead of 32 scattered elements per instruction
  T* row = zr_s + ((a.k * a.wr + 3) / 4) * 4 + (size_t)threadIdx.x * pitch;
  const int lane = threadIdx.x & 31;
  for (int64_t grp = blockIdx.x; grp < a.n_groups; grp += gridDim.x) {
    const int64_t j = a.group_source[grp], first = a.group_ptr[grp], last = a.group_ptr[grp + 1];
    __syncthreads();
    stage_node(a, j, zc_s, zr_s);
    __syncthreads();
    for (int64_t x0 = first; x0 < last; x0 += blockDim.x) {  // x0: uniform, so that whole warps take part in the row hand-over
      const int64_t x = x0 + threadIdx.x;
      const bool mine = x < last;
      const int64_t e = mine ? a.order[x] : -1;
      if (mine) {
        T hh[KMAX];
        hh[0] = T(1);
#pragma unroll
        for (int t = 1; t < KMAX; ++t) hh[t] = (KT || t < a.k) ? a.h[e * (a.k - 1) + t - 1] : T(0);
        // Blocks are sorted by output offset; blocks of one offset add into the same columns.  The
        // first block of a group writes, the following ones add to the edge's row.
        int open_offset = -1;
        for (int b = 0; b < a.n_blocks; ++b) {
          const int32_t* d = a.desc + b * FDESC;
          const int kind = d[0], zoff = d[1], bm = d[2], ooff = d[6];
          const bool take_real = d[7] != 0;
          const bool first_of_group = ooff != open_offset;
          open_offset = ooff;
          if (kind == 0) {
            for (int c = 0; c < bm; ++c) {
              T s = T(0);
#pragma unroll
              for (int t = 0; t < KMAX; ++t)
                if (KT || t < a.k) s += hh[t] * zr_s[t * a.wr + zoff + c];
              row[ooff + c] = first_of_group ? s : row[ooff + c] + s;
            }
            continue;
          }
          T fr, fi;
          block_factor(a, e, d, fr, fi);
          auto emit = [&](int c, T ur, T ui) {
            const T vr = fr * ur - fi * ui, vi = fr * ui + fi * ur;
            if (take_real) {
              row[ooff + c] = first_of_group ? vr : row[ooff + c] + vr;
            } else {
              row[ooff + 2 * c] = first_of_group ? vr : row[ooff + 2 * c] + vr;
              row[ooff + 2 * c + 1] = first_of_group ? vi : row[ooff + 2 * c + 1] + vi;
            }
          };
          int c = 0;
          if (sizeof(T) == 4 && (a.wc % 2) == 0 && (zoff % 2) == 0) {
            // two complex columns per 16-byte shared-memory load: (re, im, re, im) of columns c, c + 1 for one t
            for (; c + 2 <= bm; c += 2) {
              T ur0 = T(0), ui0 = T(0), ur1 = T(0), ui1 = T(0);
#pragma unroll
              for (int t = 0; t < KMAX; ++t)
                if (KT || t < a.k) {
                  const float4 z = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(zc_s) + (t * a.wc + zoff + c) * 2);
                  ur0 += hh[t] * (T)z.x; ui0 += hh[t] * (T)z.y;
                  ur1 += hh[t] * (T)z.z; ui1 += hh[t] * (T)z.w;
                }
              emit(c, ur0, ui0);
              emit(c + 1, ur1, ui1);
            }
          }
          for (; c < bm; ++c) {
            T ur = T(0), ui = T(0);
#pragma unroll
            for (int t = 0; t < KMAX; ++t)
              if (KT || t < a.k) {
                ur += hh[t] * zc_s[(t * a.wc + zoff + c) * 2];
                ui += hh[t] * zc_s[(t * a.wc + zoff + c) * 2 + 1];
              }
            emit(c, ur, ui);
          }
        }
      }
      __syncwarp();
      const T* warp_rows = row - (size_t)lane * pitch;
      for (int r = 0; r < 32; ++r) {
        const int64_t e_r = __shfl_sync(0xffffffffu, e, r);
        if (e_r < 0) break;  // lanes take consecutive x: the first idle lane ends the warp's rows
        for (int c = lane; c < a.d_out; c += 32) a.out[e_r * a.d_out + c] = warp_rows[(size_t)r * pitch + c];
      }
      __syncwarp();
    }
  }
}

// out_i = sum over the target's edges of w_e * row_e  (factored.h:337-347): a warp per target, lanes over columns.
template <typename T>
__global__ void aggregate_kernel(const T* __restrict__ rows, const T* __restrict__ weights, const int64_t* __restrict__ row_ptr,
                                 int64_t n_targets, int d_out, T* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t i = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= n_targets) return;
  const int64_t e0 = row_ptr[i], e1 = row_ptr[i + 1];
  for (int c = lane; c < d_out; c += 32) {
    T acc = T(0);
    for (int64_t e = e0; e < e1; ++e) acc += weights[e] * rows[e * d_out + c];
    out[i * d_out + c] = acc;
  }
}

// Backward.  C = 2 wc + wr packed columns, CP = C rounded up to a whole number of 16-byte vectors (the padding
// columns of Z and W stay zero), so that both small products run on 16-byte shared-memory loads:
//   dh(e, t)   = <W(e), Z_t>           one thread per (edge, t), V columns per pair of loads
//   dZ(t, c)  += h~_t(e) W_c(e)        a thread owns patches of V consecutive columns of one t, in registers
template <typename T>
__global__ void __launch_bounds__(FTHREADS) factored_backward_kernel(FArgs<T> a, int C, int CP) {
  constexpr int V = 16 / sizeof(T);
  constexpr int MAX_PATCH = MAX_OWNED / V;
  extern __shared__ __align__(16) unsigned char raw[];
  const int K = a.k;
  T* z_s = reinterpret_cast<T*>(raw);  // (K, CP): packed per t as [zc (wc, 2) | zr (wr) | 0]
  T* w_s = z_s + K * CP;               // (TILE, CP)
  T* h_s = w_s + TILE * CP;            // (TILE, K)
  const int wc2 = 2 * a.wc, patches = K * (CP / V);
  for (int x = threadIdx.x; x < TILE * CP; x += blockDim.x) w_s[x] = T(0);  // the padding columns are never written again
  for (int64_t grp = blockIdx.x; grp < a.n_groups; grp += gridDim.x) {
    const int64_t j = a.group_source[grp], first = a.group_ptr[grp], last = a.group_ptr[grp + 1];
    __syncthreads();
    for (int x = threadIdx.x; x < K * CP; x += blockDim.x) {
      const int t = x / CP, c = x - t * CP;
      z_s[x] = c < wc2 ? a.zc[(j * K + t) * wc2 + c] : (c < C ? a.zr[(j * K + t) * a.wr + (c - wc2)] : T(0));
    }
    T acc[MAX_PATCH][V];
#pragma unroll
    for (int o = 0; o < MAX_PATCH; ++o)
#pragma unroll
      for (int v = 0; v < V; ++v) acc[o][v] = T(0);
    for (int64_t base = first; base < last; base += TILE) {
      const int n_tile = (int)min((int64_t)TILE, last - base);
      __syncthreads();
      // build W(e) and h~(e): threads split (edge, block) pairs
      for (int x = threadIdx.x; x < n_tile * a.n_blocks; x += blockDim.x) {
        const int le = x / a.n_blocks, b = x - le * a.n_blocks;
        const int64_t e = a.order[base + le];
        const int32_t* d = a.desc + b * FDESC;
        const int kind = d[0], zoff = d[1], bm = d[2], ooff = d[6];
        const bool take_real = d[7] != 0;
        const T scale = a.weights ? a.weights[e] : T(1);
        const T* g = a.target ? a.g + a.target[e] * a.d_out : a.g + e * a.d_out;
        T* w = w_s + le * CP;
        if (kind == 0) {
          for (int c = 0; c < bm; ++c) w[wc2 + zoff + c] = scale * g[ooff + c];
        } else {
          T fr, fi;
          block_factor(a, e, d, fr, fi);
          for (int c = 0; c < bm; ++c) {
            const T gr = scale * (take_real ? g[ooff + c] : g[ooff + 2 * c]);
            const T gi = take_real ? T(0) : scale * g[ooff + 2 * c + 1];
            w[(zoff + c) * 2] = gr * fr + gi * fi;  // W = G conj(F)
            w[(zoff + c) * 2 + 1] = gi * fr - gr * fi;
          }
        }
      }
      for (int x = threadIdx.x; x < n_tile * K; x += blockDim.x) {
        const int le = x / K, t = x - le * K;
        const int64_t e = a.order[base + le];
        h_s[le * K + t] = t == 0 ? T(1) : a.h[e * (K - 1) + t - 1];
      }
      if (a.dweights) {  // dweights_e = <g_i, row_e>
        for (int le = threadIdx.x; le < n_tile; le += blockDim.x) {
          const int64_t e = a.order[base + le];
          const T* g = a.g + a.target[e] * a.d_out;
          T s = T(0);
          for (int c = 0; c < a.d_out; ++c) s += g[c] * a.rows[e * a.d_out + c];
          a.dweights[e] = s;
        }
      }
      __syncthreads();
      // dh(e, t) = <W(e), Z_t>, t >= 1
      for (int x = threadIdx.x; x < n_tile * (K - 1); x += blockDim.x) {
        const int le = x / (K - 1), t = x - le * (K - 1) + 1;
        const T* w = w_s + le * CP;
        const T* z = z_s + t * CP;
        T s = T(0);
        for (int c = 0; c < CP; c += V) {
          T wv[V], zv[V];
          *reinterpret_cast<uint4*>(wv) = *reinterpret_cast<const uint4*>(w + c);
          *reinterpret_cast<uint4*>(zv) = *reinterpret_cast<const uint4*>(z + c);
#pragma unroll
          for (int v = 0; v < V; ++v) s += wv[v] * zv[v];
        }
        a.dh[a.order[base + le] * (K - 1) + t - 1] = s;
      }
      // dZ(t, c) += h~_t(e) W_c(e): patch x = threadIdx.x + o * blockDim.x stays with this thread
#pragma unroll
      for (int o = 0; o < MAX_PATCH; ++o) {
        const int x = threadIdx.x + o * FTHREADS;
        if (x < patches) {
          const int t = x / (CP / V), c = (x - t * (CP / V)) * V;
          for (int le = 0; le < n_tile; ++le) {
            const T hv = h_s[le * K + t];
            T wv[V];
            *reinterpret_cast<uint4*>(wv) = *reinterpret_cast<const uint4*>(w_s + le * CP + c);
#pragma unroll
            for (int v = 0; v < V; ++v) acc[o][v] += hv * wv[v];
          }
        }
      }
    }
#pragma unroll
    for (int o = 0; o < MAX_PATCH; ++o) {
      const int x = threadIdx.x + o * FTHREADS;
      if (x < patches) {
        const int t = x / (CP / V), c0 = (x - t * (CP / V)) * V;
#pragma unroll
        for (int v = 0; v < V; ++v) {
          const int c = c0 + v;
          if (c < wc2) a.dzc[(j * K + t) * wc2 + c] = acc[o][v];
          else if (c < C) a.dzr[(j * K + t) * a.wr + (c - wc2)] = acc[o][v];
        }
      }
    }
  }
}

int check_factored(const void* h, const void* zc, const void* zr, const void* angular, const void* transport, const void* rho,
                   const int32_t* desc, const int64_t* source, int64_t n_edges, int k, int wc, int wr, int n_f, int n_blocks, int d_out,
                   int dtype) {
  GM_REQUIRE(n_edges >= 0 && wc >= 0 && wr >= 0 && n_f >= 1 && n_blocks >= 0, GM_ERR_ARGUMENT, "gm_factored: bad sizes");
  GM_REQUIRE(k >= 1 && k <= FMAX_K, GM_ERR_ARGUMENT, "gm_factored: k exceeds MAX_K");
  GM_REQUIRE(d_out >= 1 && d_out <= 128, GM_ERR_ARGUMENT, "gm_factored: d_out must be in [1, MAX_OUT]");
  GM_REQUIRE(dtype == GM_F32 || dtype == GM_F64, GM_ERR_UNSUPPORTED, "gm_factored: dtype must be float32 or float64");
  if (n_edges == 0) return GM_OK;
  GM_REQUIRE(h || k == 1, GM_ERR_ARGUMENT, "gm_factored: null h");
  GM_REQUIRE((zc || wc == 0) && (zr || wr == 0) && angular && transport && rho && desc && source, GM_ERR_ARGUMENT, "gm_factored: null pointer");
  return GM_OK;
}

}  // namespace
}  // namespace gmb

using namespace gmb;

extern "C" int gm_factored_forward(const void* h, const void* zc, const void* zr, const void* angular, const void* transport,
                                   const void* rho, const int32_t* desc, const int64_t* source, const int64_t* order,
                                   const int64_t* group_ptr, const int64_t* group_source, int64_t n_edges, int64_t n_groups, int k,
                                   int wc, int wr, int n_f, int n_blocks, int d_out, int dtype, void* out, void* stream) {
  int status = check_factored(h, zc, zr, angular, transport, rho, desc, source, n_edges, k, wc, wr, n_f, n_blocks, d_out, dtype);
  if (status != GM_OK || n_edges == 0) return status;
  GM_REQUIRE(order && group_ptr && group_source && out && n_groups >= 1, GM_ERR_ARGUMENT, "gm_factored_forward: null grouping / output");
  auto run = [&](auto tag) {
    using T = decltype(tag);
    FArgs<T> a{};
    a.n_edges = n_edges; a.n_groups = n_groups; a.k = k; a.wc = wc; a.wr = wr; a.n_f = n_f; a.n_blocks = n_blocks; a.d_out = d_out;
    a.h = (const T*)h; a.zc = (const T*)zc; a.zr = (const T*)zr; a.angular = (const T*)angular; a.transport = (const T*)transport;
    a.rho = (const T*)rho; a.desc = desc; a.source = source; a.order = order; a.group_ptr = group_ptr; a.group_source = group_source;
    a.out = (T*)out;
    const int pitch = d_out | 1;  // per-thread output rows in shared memory, odd pitch
    const size_t smem = ((size_t)k * 2 * wc + ((size_t)k * wr + 3) / 4 * 4 + (size_t)FTHREADS * pitch) * sizeof(T);
    int st = k == 17 ? allow_smem(factored_forward_kernel<T, 17>, smem, "gm_factored_forward")
                     : allow_smem(factored_forward_kernel<T, 0>, smem, "gm_factored_forward");
    if (st != GM_OK) return st;
    const unsigned blocks = (unsigned)(n_groups < (1 << 20) ? n_groups : (1 << 20));
    if (k == 17) factored_forward_kernel<T, 17><<<blocks, FTHREADS, smem, (cudaStream_t)stream>>>(a, pitch);
    else factored_forward_kernel<T, 0><<<blocks, FTHREADS, smem, (cudaStream_t)stream>>>(a, pitch);
    return launch_status("gm_factored_forward");
  };
  return dtype == GM_F32 ? run(float()) : run(double());
}

extern "C" int gm_factored_aggregate(const void* rows, const void* weights, const int64_t* row_ptr, int64_t n_targets, int64_t n_edges,
                                     int d_out, int dtype, void* out, void* stream) {
  GM_REQUIRE(n_targets >= 0 && n_edges >= 0 && d_out >= 1 && d_out <= 128, GM_ERR_ARGUMENT, "gm_factored_aggregate: bad sizes");
  GM_REQUIRE(dtype == GM_F32 || dtype == GM_F64, GM_ERR_UNSUPPORTED, "gm_factored_aggregate: dtype must be float32 or float64");
  if (n_targets == 0) return GM_OK;
  GM_REQUIRE(row_ptr && out && (n_edges == 0 || (rows && weights)), GM_ERR_ARGUMENT, "gm_factored_aggregate: null pointer");
  const unsigned blocks = (unsigned)((n_targets + 7) / 8);
  if (dtype == GM_F32)
    aggregate_kernel<float><<<blocks, 256, 0, (cudaStream_t)stream>>>((const float*)rows, (const float*)weights, row_ptr, n_targets, d_out, (float*)out);
  else
    aggregate_kernel<double><<<blocks, 256, 0, (cudaStream_t)stream>>>((const double*)rows, (const double*)weights, row_ptr, n_targets, d_out, (double*)out);
  return launch_status("gm_factored_aggregate");
}

extern "C" int gm_factored_backward(const void* g, const int64_t* target, const void* weights, const void* rows, const void* h,
                                    const void* zc, const void* zr, const void* angular, const void* transport, const void* rho,
                                    const int32_t* desc, const int64_t* source, const int64_t* order, const int64_t* group_ptr,
                                    const int64_t* group_source, int64_t n_edges, int64_t n_groups, int k, int wc, int wr, int n_f,
                                    int n_blocks, int d_out, int dtype, void* dh, void* dzc, void* dzr, void* dweights, void* stream) {
  int status = check_factored(h, zc, zr, angular, transport, rho, desc, source, n_edges, k, wc, wr, n_f, n_blocks, d_out, dtype);
  if (status != GM_OK || n_edges == 0) return status;
  GM_REQUIRE(g && order && group_ptr && group_source && n_groups >= 1, GM_ERR_ARGUMENT, "gm_factored_backward: null pointer");
  GM_REQUIRE((dh || k == 1) && (dzc || wc == 0) && (dzr || wr == 0), GM_ERR_ARGUMENT, "gm_factored_backward: null output");
  const bool aggregated = target != nullptr;
  GM_REQUIRE(!aggregated || (weights && rows && dweights), GM_ERR_ARGUMENT, "gm_factored_backward: the aggregated form needs weights, rows and dweights");
  const int C = 2 * wc + wr;
  GM_REQUIRE(k * ((C + 3) / 4 * 4) <= MAX_OWNED * FTHREADS, GM_ERR_LIMIT, "gm_factored_backward: k * (2 wc + wr) = %d exceeds %d", k * C, MAX_OWNED * FTHREADS);
  auto run = [&](auto tag) {
    using T = decltype(tag);
    FArgs<T> a{};
    a.n_edges = n_edges; a.n_groups = n_groups; a.k = k; a.wc = wc; a.wr = wr; a.n_f = n_f; a.n_blocks = n_blocks; a.d_out = d_out;
    a.h = (const T*)h; a.zc = (const T*)zc; a.zr = (const T*)zr; a.angular = (const T*)angular; a.transport = (const T*)transport;
    a.rho = (const T*)rho; a.desc = desc; a.source = source; a.order = order; a.group_ptr = group_ptr; a.group_source = group_source;
    a.g = (const T*)g; a.target = target; a.weights = aggregated ? (const T*)weights : nullptr; a.rows = aggregated ? (const T*)rows : nullptr;
    a.dh = (T*)dh; a.dzc = (T*)dzc; a.dzr = (T*)dzr; a.dweights = aggregated ? (T*)dweights : nullptr;
    const int V = 16 / (int)sizeof(T), CP = (C + V - 1) / V * V;  // packed columns padded to whole 16-byte vectors
    const size_t smem = ((size_t)k * CP + (size_t)TILE * CP + (size_t)TILE * k) * sizeof(T);
    int st = allow_smem(factored_backward_kernel<T>, smem, "gm_factored_backward");
    if (st != GM_OK) return st;
    const unsigned blocks = (unsigned)(n_groups < (1 << 20) ? n_groups : (1 << 20));
    factored_backward_kernel<T><<<blocks, FTHREADS, smem, (cudaStream_t)stream>>>(a, C, CP);
    return launch_status("gm_factored_backward");
  };
  return dtype == GM_F32 ? run(float()) : run(double());
}
