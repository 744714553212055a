// Depthwise steerable convolution on a longitude-symmetric lattice with the per-edge coefficients replaced by a
// per-(row pair, longitude offset) table.
//
// The reference's depthwise op (nn/fused/attention.h:174-206, 265-287) streams E * (a_0 + W) coefficients: per edge a
// real factor R per scalar channel and complex A, B per complex copy, applied as  m = A z + w B conj(z),  z = tau_n v_j,
// w = (r/c)^{2n} e^{2 i n phi}, and summed with the edge's aggregation weight.  On a lattice whose frames turn with the
// longitude every one of those quantities depends on (target row, source row, longitude offset) only, and
// z -> A z + w B conj(z) is a real-linear map of the plane, so the whole edge collapses into ONE real 2 x 2 matrix per
// (table entry, complex copy) and one real factor per (entry, scalar channel); the caller folds the coefficients into
// that table (gm_attention_b200/nn/lattice_depthwise.py: fold; plain tensor algebra on ~45 000 entries, differentiable), and the
// kernels here are
//
//   apply       y[i, l] = sum over entries (j, d) of row i   M[entry] x[j, l + lo + d]      (forward; with the transposed
//               windows and M^T it is the gradient with respect to the node field)
//   table_grad  dM[entry] = sum over longitudes l and samples  dy[i, l] (x) x[j, l + lo + d]
//
// Both are FMA-bound, not HBM-bound (4 multiply-adds per complex copy, edge and sample against 0.01 bytes of compulsory
// traffic), and neither has a contraction over channels, so there is nothing for the tensor cores here.  A thread owns
// one item -- a complex copy, or a pair of scalar channels -- so a warp reads 32 neighbouring items of a node as one
// 128-byte line; it keeps 8 longitudes x 2 samples of accumulators in registers and slides a register window of 8
// source longitudes (apply) or 8 target longitudes (table_grad) past them, so every loaded value is used for 8 x 4
// multiply-adds and nothing is staged in shared memory.  Results do not depend on the launch geometry: no atomics.
#include "common.cuh"

namespace gmb {
namespace {

constexpr int LON = 8;  // longitudes (apply) / longitude offsets (table_grad) per thread
constexpr int THREADS = 160;  // at most; three CTAs per SM (136 registers per thread); more items than threads are looped over

struct ConvArgs {
  const void* x;        // (batch, rows * nlon, width) node field
  const void* g;        // table_grad: the output gradient, same layout
  const float* table;   // (entries, table_width)
  const int* items;     // (n_items, 3): kind (0 complex copy, 1 pair of scalar channels), field column, table column
  const int* win_cnt;   // (rows, 2 * halo + 1)
  const int* win_lo;
  const int* win_off;
  const int* order;     // apply: target rows, heaviest first; table_grad: (blocks, 2) = window index, first offset
  void* y;              // apply: (batch, rows * nlon, width)
  float* dtable;        // table_grad: (entries, table_width)
  int n_items, rows, nlon, batch, width, halo, table_width, transpose;
};

// Two neighbouring elements of a node's row: loaded as one word (bf16) or two (float), unpacked when used, so that a
// value in flight between its load and its use costs one register per bf16 pair.
template <typename S> struct Pair;
template <> struct Pair<float> {
  using Raw = float2;
  static __device__ __forceinline__ Raw load(const float* p) { return __ldg(reinterpret_cast<const float2*>(p)); }
  static __device__ __forceinline__ Raw zero() { return make_float2(0.f, 0.f); }
  static __device__ __forceinline__ float2 unpack(Raw r) { return r; }
  static __device__ __forceinline__ void store(float* p, float2 v) { *reinterpret_cast<float2*>(p) = v; }
};
template <> struct Pair<__nv_bfloat16> {
  using Raw = unsigned;
  static __device__ __forceinline__ Raw load(const __nv_bfloat16* p) { return __ldg(reinterpret_cast<const unsigned*>(p)); }
  static __device__ __forceinline__ Raw zero() { return 0u; }
  static __device__ __forceinline__ float2 unpack(Raw r) { return make_float2(__uint_as_float(r << 16), __uint_as_float(r & 0xffff0000u)); }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float2 v) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v.x, v.y);
  }
};

// ---------------------------------------------------------------------------------------------------------------- apply
// TL targets (consecutive longitudes) x NB samples per thread.
template <typename S, int NB, int TL>
__global__ void __launch_bounds__(THREADS, 3) conv_apply_kernel(const ConvArgs a) {
  constexpr int PF = 4;  // steps in flight (a power of two <= 8)
  const int row = a.order[blockIdx.y];
  const int l0 = blockIdx.x * TL;
  const int b0 = blockIdx.z * NB;
  const int span = 2 * a.halo + 1;
  const size_t sample = (size_t)a.rows * a.nlon * a.width;
  const S* x = static_cast<const S*>(a.x) + (size_t)b0 * sample;
  S* y = static_cast<S*>(a.y) + (size_t)b0 * sample;
  const int nb = min(NB, a.batch - b0);

  for (int item = threadIdx.x; item < a.n_items; item += blockDim.x) {
    const int kind = a.items[3 * item], col = a.items[3 * item + 1], fcol = a.items[3 * item + 2];
    float2 acc[TL][NB];
#pragma unroll
    for (int l = 0; l < TL; ++l)
#pragma unroll
      for (int b = 0; b < NB; ++b) acc[l][b] = make_float2(0.f, 0.f);

    for (int c = 0; c < span; ++c) {
      const int j = row + c - a.halo;
      if (j < 0 || j >= a.rows) continue;
      const int cnt = a.win_cnt[row * span + c];
      if (cnt == 0) continue;
      const int lo = a.win_lo[row * span + c];
      const float* table = a.table + (size_t)a.win_off[row * span + c] * a.table_width + fcol;
      const S* xrow = x + (size_t)j * a.nlon * a.width + col;
      int p = (l0 + lo) % a.nlon;
      if (p < 0) p += a.nlon;
      // Position t of the source row is longitude l0 + lo + t; under offset d the block's target l sees position d + l.
      // A register window holds the 8 most recent positions and slides by one per offset, so every offset is 8 targets x
      // NB samples of multiply-adds on true neighbours only: no ramp, no validity tests.
      auto matrix = [&](int d) {
        const float* f = table + (size_t)d * a.table_width;
        if (kind == 0) {
          const float4 m = __ldg(reinterpret_cast<const float4*>(f));
          return a.transpose ? make_float4(m.x, m.z, m.y, m.w) : m;
        }
        const float2 m = __ldg(reinterpret_cast<const float2*>(f));
        return make_float4(m.x, 0.f, 0.f, m.y);
      };
      int ahead = p;  // longitude of the next position to load
      auto source = [&](int b) { return b < nb ? Pair<S>::load(xrow + b * sample + (size_t)ahead * a.width) : Pair<S>::zero(); };
      auto advance = [&]() { ahead = ahead + 1 == a.nlon ? 0 : ahead + 1; };
      float2 xs[TL][NB];  // xs[t % 8] = position t
#pragma unroll
      for (int t = 0; t < TL - 1; ++t) {
#pragma unroll
        for (int b = 0; b < NB; ++b) xs[t][b] = Pair<S>::unpack(source(b));
        advance();
      }
      // ring of PF offsets in flight: matrix d + PF and position d + 7 + PF are loaded when offset d is consumed
      typename Pair<S>::Raw ring_v[PF][NB];
      float4 ring_m[PF];
#pragma unroll
      for (int t = 0; t < PF; ++t) {
        if (t < cnt) {
          ring_m[t] = matrix(t);
#pragma unroll
          for (int b = 0; b < NB; ++b) ring_v[t][b] = source(b);
          advance();
        }
      }
      for (int d0 = 0; d0 < cnt; d0 += TL) {
#pragma unroll
        for (int u = 0; u < TL; ++u) {
          const int d = d0 + u;
          if (d >= cnt) break;
          const float4 m = ring_m[u % PF];
#pragma unroll
          for (int b = 0; b < NB; ++b) xs[(u + TL - 1) & (TL - 1)][b] = Pair<S>::unpack(ring_v[u % PF][b]);
          if (d + PF < cnt) {
            ring_m[u % PF] = matrix(d + PF);
#pragma unroll
            for (int b = 0; b < NB; ++b) ring_v[u % PF][b] = source(b);
            advance();
          }
          if (kind == 0) {
#pragma unroll
            for (int l = 0; l < TL; ++l)
#pragma unroll
              for (int b = 0; b < NB; ++b) {
                const float2 v = xs[(u + l) & (TL - 1)][b];
                acc[l][b].x = fmaf(m.x, v.x, fmaf(m.y, v.y, acc[l][b].x));
                acc[l][b].y = fmaf(m.z, v.x, fmaf(m.w, v.y, acc[l][b].y));
              }
          } else {  // two independent scalar channels: no cross terms, so a non-finite value stays in its channel
#pragma unroll
            for (int l = 0; l < TL; ++l)
#pragma unroll
              for (int b = 0; b < NB; ++b) {
                const float2 v = xs[(u + l) & (TL - 1)][b];
                acc[l][b].x = fmaf(m.x, v.x, acc[l][b].x);
                acc[l][b].y = fmaf(m.w, v.y, acc[l][b].y);
              }
          }
        }
      }
    }
#pragma unroll
    for (int l = 0; l < TL; ++l) {
      if (l0 + l >= a.nlon) break;
#pragma unroll
      for (int b = 0; b < NB; ++b)
        if (b < nb) Pair<S>::store(y + b * sample + ((size_t)row * a.nlon + l0 + l) * a.width + col, acc[l][b]);
    }
  }
}

// ----------------------------------------------------------------------------------------------------------- table_grad
// One CTA: one window (target row, source row) and 8 consecutive offsets d0 .. d0 + 7 of it; it walks once around the
// source row.  Step u brings the source at longitude u + lo + d0; offset d0 + k pairs it with the target u - k (cyclic),
// whose gradient row sits in a register window of the 8 most recent targets.
template <typename S, int NB>
__global__ void __launch_bounds__(THREADS, 3) conv_table_grad_kernel(const ConvArgs a) {
  constexpr int PF = 4;  // steps in flight (a power of two <= 8; nlon >= 8)
  const int w = a.order[2 * blockIdx.x], d0 = a.order[2 * blockIdx.x + 1];
  const int span = 2 * a.halo + 1;
  const int row = w / span, j = row + w % span - a.halo;
  const int cnt = a.win_cnt[w], lo = a.win_lo[w];
  const size_t sample = (size_t)a.rows * a.nlon * a.width;
  const int valid = min(LON, cnt - d0);

  for (int item = threadIdx.x; item < a.n_items; item += blockDim.x) {
    const int kind = a.items[3 * item], col = a.items[3 * item + 1], fcol = a.items[3 * item + 2];
    float4 acc[LON];
#pragma unroll
    for (int k = 0; k < LON; ++k) acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int b0 = 0; b0 < a.batch; b0 += NB) {
      const int nb = min(NB, a.batch - b0);
      const S* xrow = static_cast<const S*>(a.x) + (size_t)b0 * sample + (size_t)j * a.nlon * a.width + col;
      const S* grow = static_cast<const S*>(a.g) + (size_t)b0 * sample + (size_t)row * a.nlon * a.width + col;
      float2 window[LON][NB];  // window[t % 8] = gradient of target t
#pragma unroll
      for (int t = 1; t < LON; ++t)  // targets -7 .. -1 (cyclic) are seen by the first steps
#pragma unroll
        for (int b = 0; b < NB; ++b)
          window[(LON - t) & (LON - 1)][b] = b < nb ? Pair<S>::unpack(Pair<S>::load(grow + b * sample + (size_t)(a.nlon - t) * a.width)) : make_float2(0.f, 0.f);
      int p = (lo + d0) % a.nlon;
      if (p < 0) p += a.nlon;
      // ring of PF steps in flight: the source and the target of step u + PF are loaded when step u is consumed
      typename Pair<S>::Raw ring_v[PF][NB], ring_g[PF][NB];
      int ahead = p;
#pragma unroll
      for (int t = 0; t < PF; ++t) {
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          ring_v[t][b] = b < nb ? Pair<S>::load(xrow + b * sample + (size_t)ahead * a.width) : Pair<S>::zero();
          ring_g[t][b] = b < nb ? Pair<S>::load(grow + b * sample + (size_t)t * a.width) : Pair<S>::zero();
        }
        ahead = ahead + 1 == a.nlon ? 0 : ahead + 1;
      }
      for (int u0 = 0; u0 < a.nlon; u0 += LON) {  // nlon is a multiple of 8 (checked by the host)
#pragma unroll
        for (int u = 0; u < LON; ++u) {
          float2 v[NB];
#pragma unroll
          for (int b = 0; b < NB; ++b) {
            v[b] = Pair<S>::unpack(ring_v[u % PF][b]);
            window[u][b] = Pair<S>::unpack(ring_g[u % PF][b]);
          }
          if (u0 + u + PF < a.nlon) {
#pragma unroll
            for (int b = 0; b < NB; ++b) {
              ring_v[u % PF][b] = b < nb ? Pair<S>::load(xrow + b * sample + (size_t)ahead * a.width) : Pair<S>::zero();
              ring_g[u % PF][b] = b < nb ? Pair<S>::load(grow + b * sample + (size_t)(u0 + u + PF) * a.width) : Pair<S>::zero();
            }
            ahead = ahead + 1 == a.nlon ? 0 : ahead + 1;
          }
#pragma unroll
          for (int k = 0; k < LON; ++k) {
            if (k >= valid) break;  // offsets beyond the window: their pairs are not edges
#pragma unroll
            for (int b = 0; b < NB; ++b) {
              const float2 g = window[(u - k) & (LON - 1)][b];
              acc[k].x = fmaf(g.x, v[b].x, acc[k].x);
              acc[k].y = fmaf(g.x, v[b].y, acc[k].y);
              acc[k].z = fmaf(g.y, v[b].x, acc[k].z);
              acc[k].w = fmaf(g.y, v[b].y, acc[k].w);
            }
          }
        }
      }
    }
    float* out = a.dtable + (size_t)(a.win_off[w] + d0) * a.table_width + fcol;
#pragma unroll
    for (int k = 0; k < LON; ++k) {
      if (k >= valid) break;
      if (kind == 0) *reinterpret_cast<float4*>(out + (size_t)k * a.table_width) = acc[k];
      else *reinterpret_cast<float2*>(out + (size_t)k * a.table_width) = make_float2(acc[k].x, acc[k].w);
    }
  }
}

int check_common(const char* what, const void* x, const float* table, const int* items, int n_items, const int* win_cnt, const int* win_lo,
                 const int* win_off, int rows, int nlon, int batch, int width, int halo, int table_width, int dtype) {
  GM_REQUIRE(dtype == GM_F32 || dtype == GM_BF16, GM_ERR_UNSUPPORTED, "%s: node fields are float32 or bfloat16", what);
  GM_REQUIRE(x && table && items && win_cnt && win_lo && win_off, GM_ERR_ARGUMENT, "%s: null pointer", what);
  GM_REQUIRE(rows > 0 && nlon > 0 && batch > 0 && width > 0 && halo >= 0 && n_items > 0, GM_ERR_ARGUMENT, "%s: empty or negative sizes", what);
  GM_REQUIRE(nlon % LON == 0, GM_ERR_UNSUPPORTED, "%s: the number of longitudes must be a multiple of %d", what, LON);
  GM_REQUIRE(width % 2 == 0 && table_width % 4 == 0, GM_ERR_UNSUPPORTED,
             "%s: the field width must be even and the table width a multiple of 4 (8- and 16-byte accesses)", what);
  GM_REQUIRE(reinterpret_cast<uintptr_t>(x) % 8 == 0 && reinterpret_cast<uintptr_t>(table) % 16 == 0, GM_ERR_ARGUMENT,
             "%s: the field must sit on an 8-byte and the table on a 16-byte boundary", what);
  return GM_OK;
}

}  // namespace
}  // namespace gmb

using namespace gmb;

// y = table applied along the windows.  order: n_order target rows (any subset, any order).  transpose != 0 applies the
// transposed matrices (the windows and the table are then the transposed ones: gradient with respect to the field).
extern "C" int gm_lattice_conv_apply(const void* x, const float* table, const int32_t* items, int n_items, const int32_t* win_cnt,
                                     const int32_t* win_lo, const int32_t* win_off, const int32_t* order, int n_order, int rows, int nlon,
                                     int batch, int width, int halo, int table_width, int transpose, int dtype, void* y, void* stream) {
  if (n_order == 0) return GM_OK;
  if (int status = check_common("gm_lattice_conv_apply", x, table, items, n_items, win_cnt, win_lo, win_off, rows, nlon, batch, width, halo,
                                table_width, dtype))
    return status;
  GM_REQUIRE(order && y && n_order > 0 && n_order <= 65535, GM_ERR_ARGUMENT, "gm_lattice_conv_apply: bad row list");
  ConvArgs a{};
  a.x = x; a.table = table; a.items = items; a.win_cnt = win_cnt; a.win_lo = win_lo; a.win_off = win_off; a.order = order; a.y = y;
  a.n_items = n_items; a.rows = rows; a.nlon = nlon; a.batch = batch; a.width = width; a.halo = halo; a.table_width = table_width;
  a.transpose = transpose;
  const int threads = min(THREADS, (n_items + 31) / 32 * 32);
  // 32 accumulators + a window of as many sources + 4 steps in flight stay under 128 registers: three CTAs per SM (four
  // samples x 8 targets measured one CTA per SM and half the speed)
  // (16 targets x 1 sample per thread -- the same registers -- measured the same 8.05 ms in bf16 and 4 % slower in float32)
  const int nb = batch >= 2 ? 2 : 1, tl = LON;
  GM_REQUIRE((batch + nb - 1) / nb <= 65535, GM_ERR_LIMIT, "gm_lattice_conv_apply: batch too large");
  dim3 grid(nlon / tl, n_order, (batch + nb - 1) / nb);
  cudaStream_t cs = (cudaStream_t)stream;
#define GM_APPLY(S, NB) conv_apply_kernel<S, NB, LON><<<grid, threads, 0, cs>>>(a)
  if (dtype == GM_F32) {
    if (nb == 2) GM_APPLY(float, 2); else GM_APPLY(float, 1);
  } else {
    if (nb == 2) GM_APPLY(__nv_bfloat16, 2); else GM_APPLY(__nv_bfloat16, 1);
  }
#undef GM_APPLY
  return launch_status("gm_lattice_conv_apply");
}

// dtable[entry] = sum over longitudes and samples of g (target) (x) x (source).  blocks: (n_blocks, 2) int32 = (window
// index = target row * (2 * halo + 1) + source row - target row + halo, first offset), 8 offsets each; entries no block
// covers are left untouched.
extern "C" int gm_lattice_conv_table_grad(const void* g, const void* x, const int32_t* items, int n_items, const int32_t* win_cnt,
                                          const int32_t* win_lo, const int32_t* win_off, const int32_t* blocks, int64_t n_blocks, int rows,
                                          int nlon, int batch, int width, int halo, int table_width, int dtype, float* dtable, void* stream) {
  if (n_blocks == 0) return GM_OK;
  if (int status = check_common("gm_lattice_conv_table_grad", x, dtable, items, n_items, win_cnt, win_lo, win_off, rows, nlon, batch, width,
                                halo, table_width, dtype))
    return status;
  GM_REQUIRE(g && blocks && n_blocks > 0 && n_blocks < (int64_t)1 << 31, GM_ERR_ARGUMENT, "gm_lattice_conv_table_grad: bad block list");
  ConvArgs a{};
  a.x = x; a.g = g; a.items = items; a.win_cnt = win_cnt; a.win_lo = win_lo; a.win_off = win_off; a.order = blocks; a.dtable = dtable;
  a.n_items = n_items; a.rows = rows; a.nlon = nlon; a.batch = batch; a.width = width; a.halo = halo; a.table_width = table_width;
  const int threads = min(THREADS, (n_items + 31) / 32 * 32);
  const int nb = batch >= 2 ? 2 : 1;  // four samples' windows would take every register a thread can have
  cudaStream_t cs = (cudaStream_t)stream;
#define GM_GRAD(S, NB) conv_table_grad_kernel<S, NB><<<(unsigned)n_blocks, threads, 0, cs>>>(a)
  if (dtype == GM_F32) {
    if (nb == 2) GM_GRAD(float, 2); else GM_GRAD(float, 1);
  } else {
    if (nb == 2) GM_GRAD(__nv_bfloat16, 2); else GM_GRAD(__nv_bfloat16, 1);
  }
#undef GM_GRAD
  return launch_status("gm_lattice_conv_table_grad");
}
