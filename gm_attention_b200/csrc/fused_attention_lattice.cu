// Fused gauge attention on an equiangular lattice with longitude-equivariant
// frames: the fast path of gm_attention_forward / backward.
//
// On such a lattice every per-edge quantity depends on (target row, source
// row, longitude offset) only, so the per-edge tables of the general kernel
// (8 + 8 * orders + 5 bytes per edge, per-edge index) collapse to one entry per
// (row pair, offset) -- ~26 k entries for the 256 x 512 lattice instead of
// 13.5 M edges -- and the neighbours of a target in one source row are a
// contiguous (cyclic) run of longitudes.  Same arithmetic as the general kernel
// (reference semantics: src/gm_attention/nn/fused/attention.h:145-165, 295-316
// for the scores and softmax, src/gm_attention/nn/kernels.py:156-189 for the
// transported values).
//
// Work split: one CTA = (tile of TL consecutive longitudes of one row) x (one
// sample) x (one head).  The "owner" rows (targets in the forward) live in
// registers: a group of L lanes shares an owner pair (TT = 2 adjacent
// longitudes), each lane holding a contiguous run of the head's copies of
// every frequency.  The "neighbour" rows (sources) of one lattice row are
// staged once per CTA into shared memory as fp32, head-local and padded to an
// odd multiple of 8 floats so that the groups' 16/32-byte reads spread over the
// banks; every staged value is used for both owners of the pair.  Logits are
// reduced over the L lanes with xor-shuffles, the softmax is online, the
// transport phase is applied in registers.
//
// The backward is deterministic and atomic-free: pass T (owners = targets)
// recomputes the logits from the saved log-sum-exp and accumulates dq; pass S
// (owners = SOURCES, neighbours = targets, transposed tables) recomputes them
// again and accumulates dk and dv, each element written exactly once.
#include "common.cuh"

namespace gmb {
namespace {

constexpr int LAT_MAX_CF = 4;   // complex frequencies per head
constexpr int LAT_THREADS = 128;
constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;
enum { MODE_FWD = 0, MODE_BWD_T = 1, MODE_BWD_S = 2 };

// A head's layout: optionally a_0 scalar copies, then n_cf complex frequencies of a_c copies each.
// Head-local order (the order rows are staged in): [a_0 reals][f = 0: a_c pairs][f = 1: a_c pairs]...
struct LatPlan {
  int a0, ac, n_cf, d_head, pitch, L;
  int real_off;               // flat offset of the scalar block (all heads)
  int cf_off[LAT_MAX_CF];     // flat offset of each complex frequency's block (all heads)
  int cf_order[LAT_MAX_CF];   // its frequency n >= 1
  int aligned;                // 1: every run a lane reads from shared memory starts on a 16-byte boundary
  int stage_vec;              // 1: every head segment starts / ends on a 16-byte boundary of the stored element type
};

template <typename S>
struct LatArgs {
  const S *f1, *f2;   // neighbour-side fields staged in shared memory (k, v | k, v | q, dO)
  const S *o1, *o2;   // owner-side fields held in registers          (q, - | q, dO | k, v)
  const float *lse, *delta;  // (batch * rows * nlon, H)
  S *r1, *r2;         // results: out | dq | dk, dv
  float* lse_out;
  const int *win_cnt, *win_lo, *win_off;  // (rows, 2W + 1)
  const float* entries;                   // (n_entries, ES): (cos, sin) of orders 1..NORD, then bias
  const int* row_order;                   // owner rows, heaviest first
  int rows, nlon, D, H, W, ES, NORD;
  int SC;                                 // neighbour rows staged per chunk
  float scale;
  LatPlan plan;
};

__device__ __forceinline__ int wrap(int x, int n) {
  x %= n;
  return x < 0 ? x + n : x;
}

// N consecutive floats from shared memory; 16- / 8-byte loads when the run is known to be aligned.
template <int N, bool ALIGNED>
__device__ __forceinline__ void load_run(const float* __restrict__ p, float (&dst)[N]) {
  if constexpr (ALIGNED && N % 4 == 0) {
#pragma unroll
    for (int x = 0; x < N; x += 4) {
      const float4 v = *reinterpret_cast<const float4*>(p + x);
      dst[x] = v.x; dst[x + 1] = v.y; dst[x + 2] = v.z; dst[x + 3] = v.w;
    }
  } else if constexpr (ALIGNED && N % 2 == 0) {
#pragma unroll
    for (int x = 0; x < N; x += 2) {
      const float2 v = *reinterpret_cast<const float2*>(p + x);
      dst[x] = v.x; dst[x + 1] = v.y;
    }
  } else {
#pragma unroll
    for (int x = 0; x < N; ++x) dst[x] = p[x];
  }
}

// One row's slice owned by a lane: NR scalars and NCF * UC complex numbers.
template <int NR, int NC>
struct Slice {
  float re[NR > 0 ? NR : 1];
  float cr[NC > 0 ? NC : 1], ci[NC > 0 ? NC : 1];
};

template <typename S, int NR, int NCF, int UC, int TT, int MODE, bool ALIGNED>
__global__ void __launch_bounds__(LAT_THREADS) lattice_kernel(LatArgs<S> a) {
  constexpr int NC = NCF * UC;
  extern __shared__ __align__(16) float smem[];
  const LatPlan& P = a.plan;
  const int L = P.L, groups_per_warp = 32 / L, pitch = P.pitch;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ls = lane % L;
  const int group = warp * groups_per_warp + lane / L;  // owner pair inside the CTA
  const int TL = (LAT_THREADS / L) * TT;                // owners per CTA
  const int tiles = (a.nlon + TL - 1) / TL;
  const int row = a.row_order[blockIdx.x / tiles];
  const int c0 = (blockIdx.x % tiles) * TL;
  const int h = blockIdx.y;
  const int64_t b = blockIdx.z;
  const int64_t node0 = (b * a.rows + row) * (int64_t)a.nlon;
  const int SC = a.SC;
  float* s1 = smem;
  float* s2 = smem + (size_t)SC * pitch;
  float* sstat = s2 + (size_t)SC * pitch;  // (SC, 2): lse, delta of the staged rows (pass S)
  float* sent = sstat + 2 * (size_t)SC;     // (SC + TL, ES): table entries of the offsets a chunk can meet

  // The lane's runs: scalars u = ls * NR + x (valid below a0), complex copies u = ls * UC + x (valid below ac,
  // frequency below n_cf).  An invalid slot keeps zero owner values, reads a clamped (valid, finite) staged
  // element so that it contributes exactly nothing, and is never written.  With ALIGNED the host guarantees
  // that every slot of every lane is valid and every run starts on its vector boundary.
  const int real_u0 = ls * NR, cx_u0 = ls * UC;
  auto real_valid = [&](int x) { return ALIGNED || real_u0 + x < P.a0; };
  auto cx_valid = [&](int f, int x) { return ALIGNED || (f < P.n_cf && cx_u0 + x < P.ac); };
  auto real_at = [&](int x) { return ALIGNED ? real_u0 + x : min(real_u0 + x, max(P.a0 - 1, 0)); };
  auto cx_at = [&](int f, int x) {
    return ALIGNED ? P.a0 + 2 * (P.ac * f + cx_u0 + x) : P.a0 + 2 * (P.ac * min(f, max(P.n_cf - 1, 0)) + min(cx_u0 + x, max(P.ac - 1, 0)));
  };

  Slice<NR, NC> o1[TT], o2[TT], acc1[TT], acc2[TT];
  float own_lse[TT], own_delta[TT], m[TT], l[TT];
  bool own_ok[TT];
#pragma unroll
  for (int tt = 0; tt < TT; ++tt) {
    const int t = c0 + group * TT + tt;
    own_ok[tt] = t < a.nlon;
    m[tt] = -1e30f;
    l[tt] = 0.f;
    own_lse[tt] = own_delta[tt] = 0.f;
    if (MODE == MODE_BWD_T && own_ok[tt]) {
      own_lse[tt] = a.lse[(node0 + t) * a.H + h];
      own_delta[tt] = a.delta[(node0 + t) * a.H + h];
    }
    const int64_t base = (node0 + (own_ok[tt] ? t : 0)) * a.D;
#pragma unroll
    for (int x = 0; x < NR; ++x) {
      const bool ok = own_ok[tt] && real_valid(x);
      const int64_t g = base + P.real_off + h * P.a0 + real_u0 + x;
      o1[tt].re[x] = ok ? ld<float>(a.o1 + g) : 0.f;
      o2[tt].re[x] = (MODE != MODE_FWD && ok) ? ld<float>(a.o2 + g) : 0.f;
      acc1[tt].re[x] = acc2[tt].re[x] = 0.f;
    }
#pragma unroll
    for (int f = 0; f < NCF; ++f)
#pragma unroll
      for (int x = 0; x < UC; ++x) {
        const bool ok = own_ok[tt] && cx_valid(f, x);
        const int64_t g = base + P.cf_off[f < P.n_cf ? f : 0] + 2 * (h * P.ac + cx_u0 + x);
        const int s = f * UC + x;
        o1[tt].cr[s] = ok ? ld<float>(a.o1 + g) : 0.f;
        o1[tt].ci[s] = ok ? ld<float>(a.o1 + g + 1) : 0.f;
        o2[tt].cr[s] = (MODE != MODE_FWD && ok) ? ld<float>(a.o2 + g) : 0.f;
        o2[tt].ci[s] = (MODE != MODE_FWD && ok) ? ld<float>(a.o2 + g + 1) : 0.f;
        acc1[tt].cr[s] = acc1[tt].ci[s] = acc2[tt].cr[s] = acc2[tt].ci[s] = 0.f;
      }
  }

  // ---- walk the lattice rows that hold neighbours
  for (int dj = -a.W; dj <= a.W; ++dj) {
    const int j = row + dj;
    if (j < 0 || j >= a.rows) continue;
    const int widx = row * (2 * a.W + 1) + dj + a.W;
    const int cnt = a.win_cnt[widx];
    if (cnt == 0) continue;
    const int lo = a.win_lo[widx];
    const float* ent = a.entries + (size_t)a.win_off[widx] * a.ES;
    const int64_t nrow0 = (b * a.rows + j) * (int64_t)a.nlon;
    const int window = TL + cnt - 1;  // staged position p <-> longitude c0 + lo + p
    for (int p0 = 0; p0 < window; p0 += SC) {
      const int np = min(SC, window - p0);
      __syncthreads();
      // stage np neighbour rows (the head's columns of both fields) as fp32
      if (P.stage_vec) {
        // 16-byte global loads: EV elements per vector, V vectors per row; a lane keeps one vector slot for every row
        constexpr int EV = 16 / (int)sizeof(S);
        const int V = P.d_head / EV;
        const int lanes_per_row = V <= 8 ? 8 : (V <= 16 ? 16 : 32);
        const int rows_per_pass = (32 / lanes_per_row) * (LAT_THREADS / 32);
        const int sub = lane / lanes_per_row, vec = lane % lanes_per_row;
        const int c = vec * EV;  // head-local column of the vector
        int g = 0;
        if (c < P.a0) {
          g = P.real_off + h * P.a0 + c;
        } else if (P.ac > 0) {
          const int f = min((c - P.a0) / (2 * P.ac), P.n_cf - 1);
          g = P.cf_off[f] + 2 * h * P.ac + (c - P.a0 - 2 * P.ac * f);
        }
        for (int pp = warp * (32 / lanes_per_row) + sub; pp < np; pp += rows_per_pass) {
          if (vec < V) {
            const int64_t nb = (nrow0 + wrap(c0 + lo + p0 + pp, a.nlon)) * a.D + g;
            const uint4 raw1 = __ldg(reinterpret_cast<const uint4*>(a.f1 + nb));
            const uint4 raw2 = __ldg(reinterpret_cast<const uint4*>(a.f2 + nb));
            float* d1 = s1 + pp * pitch + c;
            float* d2 = s2 + pp * pitch + c;
            if constexpr (sizeof(S) == 4) {
              *reinterpret_cast<uint4*>(d1) = raw1;
              *reinterpret_cast<uint4*>(d2) = raw2;
            } else {  // 8 bf16 -> 8 floats: a bf16 is the upper half of the fp32 with the same value
              const unsigned w1[4] = {raw1.x, raw1.y, raw1.z, raw1.w}, w2[4] = {raw2.x, raw2.y, raw2.z, raw2.w};
#pragma unroll
              for (int x = 0; x < 4; x += 2) {
                *reinterpret_cast<float4*>(d1 + 2 * x) = make_float4(__uint_as_float(w1[x] << 16), __uint_as_float(w1[x] & 0xffff0000u),
                                                                     __uint_as_float(w1[x + 1] << 16), __uint_as_float(w1[x + 1] & 0xffff0000u));
                *reinterpret_cast<float4*>(d2 + 2 * x) = make_float4(__uint_as_float(w2[x] << 16), __uint_as_float(w2[x] & 0xffff0000u),
                                                                     __uint_as_float(w2[x + 1] << 16), __uint_as_float(w2[x + 1] & 0xffff0000u));
              }
            }
          }
          if (MODE == MODE_BWD_S && vec == 0) {
            const int64_t nn = (nrow0 + wrap(c0 + lo + p0 + pp, a.nlon)) * a.H + h;
            sstat[2 * pp] = a.lse[nn];
            sstat[2 * pp + 1] = a.delta[nn];
          }
        }
      } else {
        for (int p = warp; p < np; p += LAT_THREADS / 32) {
          const int64_t nb = (nrow0 + wrap(c0 + lo + p0 + p, a.nlon)) * a.D;
          for (int c = lane; c < P.d_head; c += 32) {
            int g;
            if (c < P.a0) {
              g = P.real_off + h * P.a0 + c;
            } else {
              const int f = (c - P.a0) / (2 * P.ac);
              g = P.cf_off[f] + 2 * h * P.ac + (c - P.a0 - 2 * P.ac * f);
            }
            s1[p * pitch + c] = ld<float>(a.f1 + nb + g);
            s2[p * pitch + c] = ld<float>(a.f2 + nb + g);
          }
          if (MODE == MODE_BWD_S && lane == 0) {
            const int64_t nn = (nrow0 + wrap(c0 + lo + p0 + p, a.nlon)) * a.H + h;
            sstat[2 * p] = a.lse[nn];
            sstat[2 * p + 1] = a.delta[nn];
          }
        }
      }
      // the table entries of the offsets x = p - (tile offset) this chunk can meet, clamped (validity is decided from x)
      for (int idx = threadIdx.x; idx < (np + TL) * a.ES; idx += LAT_THREADS) {
        const int xi = idx / a.ES, w = idx - xi * a.ES;
        const int x = min(max(xi + p0 - (TL - 1), 0), cnt - 1);
        sent[idx] = __ldg(ent + (size_t)x * a.ES + w);
      }
      __syncthreads();
      // Owner tt of pair `group` sits at tile offset q0 + tt and reads positions p = q0 + tt + x, x in [0, cnt).
      // The walk is over r = p - q0, the SAME r for every lane of the warp (the shuffles below need all 32
      // lanes in step); lanes whose p falls outside this chunk idle through the step.
      const int q0 = group * TT;
      const int qw_lo = warp * groups_per_warp * TT, qw_hi = qw_lo + (groups_per_warp - 1) * TT;
      const int r_begin = max(0, p0 - qw_hi), r_end = min(TT - 1 + cnt, p0 + np - qw_lo);
      for (int r = r_begin; r < r_end; ++r) {
        const int p = q0 + r;
        const bool staged = p >= p0 && p < p0 + np;
        const int pl = staged ? p - p0 : 0;
        Slice<NR, NC> n1, n2;
        const float* row1 = s1 + pl * pitch;
        const float* row2 = s2 + pl * pitch;
        if constexpr (ALIGNED) {
          if constexpr (NR > 0) {
            load_run<NR, true>(row1 + real_u0, n1.re);
            load_run<NR, true>(row2 + real_u0, n2.re);
          }
#pragma unroll
          for (int f = 0; f < NCF; ++f) {
            float t1[2 * UC], t2[2 * UC];
            load_run<2 * UC, true>(row1 + cx_at(f, 0), t1);
            load_run<2 * UC, true>(row2 + cx_at(f, 0), t2);
#pragma unroll
            for (int x = 0; x < UC; ++x) {
              n1.cr[f * UC + x] = t1[2 * x]; n1.ci[f * UC + x] = t1[2 * x + 1];
              n2.cr[f * UC + x] = t2[2 * x]; n2.ci[f * UC + x] = t2[2 * x + 1];
            }
          }
        } else {
#pragma unroll
          for (int x = 0; x < NR; ++x) {
            n1.re[x] = row1[real_at(x)];
            n2.re[x] = row2[real_at(x)];
          }
#pragma unroll
          for (int f = 0; f < NCF; ++f)
#pragma unroll
            for (int x = 0; x < UC; ++x) {
              const int at = cx_at(f, x);
              n1.cr[f * UC + x] = row1[at]; n1.ci[f * UC + x] = row1[at + 1];
              n2.cr[f * UC + x] = row2[at]; n2.ci[f * UC + x] = row2[at + 1];
            }
        }
#pragma unroll
        for (int tt = 0; tt < TT; ++tt) {
          const int x = r - tt;
          const bool valid = staged && own_ok[tt] && x >= 0 && x < cnt;
          const float* e = sent + (size_t)(valid ? (p - p0) - (q0 + tt) + (TL - 1) : 0) * a.ES;
          float tr[NCF > 0 ? NCF : 1], ti[NCF > 0 ? NCF : 1];
          float part = 0.f, dpart = 0.f;
#pragma unroll
          for (int s = 0; s < NR; ++s) {
            part += o1[tt].re[s] * n1.re[s];
            if (MODE != MODE_FWD) dpart += o2[tt].re[s] * n2.re[s];
          }
#pragma unroll
          for (int f = 0; f < NCF; ++f) {
            const int n = P.cf_order[f < P.n_cf ? f : 0];
            tr[f] = e[2 * (n - 1)];
            ti[f] = e[2 * (n - 1) + 1];
            // G = sum over copies of conj(q) k  (q on the owner side in passes FWD / T, on the neighbour side in pass S)
            float gr = 0.f, gi = 0.f, hr = 0.f, hi = 0.f;
#pragma unroll
            for (int u = 0; u < UC; ++u) {
              const int s = f * UC + u;
              if (MODE == MODE_BWD_S) {
                gr += n1.cr[s] * o1[tt].cr[s] + n1.ci[s] * o1[tt].ci[s];
                gi += n1.cr[s] * o1[tt].ci[s] - n1.ci[s] * o1[tt].cr[s];
                hr += n2.cr[s] * o2[tt].cr[s] + n2.ci[s] * o2[tt].ci[s];
                hi += n2.cr[s] * o2[tt].ci[s] - n2.ci[s] * o2[tt].cr[s];
              } else {
                gr += o1[tt].cr[s] * n1.cr[s] + o1[tt].ci[s] * n1.ci[s];
                gi += o1[tt].cr[s] * n1.ci[s] - o1[tt].ci[s] * n1.cr[s];
                if (MODE == MODE_BWD_T) {
                  hr += o2[tt].cr[s] * n2.cr[s] + o2[tt].ci[s] * n2.ci[s];
                  hi += o2[tt].cr[s] * n2.ci[s] - o2[tt].ci[s] * n2.cr[s];
                }
              }
            }
            part += tr[f] * gr - ti[f] * gi;  // Re(tau G)
            if (MODE != MODE_FWD) dpart += tr[f] * hr - ti[f] * hi;
          }
          for (int o = L >> 1; o > 0; o >>= 1) {
            part += __shfl_xor_sync(0xffffffffu, part, o);
            if (MODE != MODE_FWD) dpart += __shfl_xor_sync(0xffffffffu, dpart, o);
          }
          // logits are kept in base 2 (scale and bias carry log2 e), so the exponentials are single ex2 instructions
          const float bias = valid ? e[2 * a.NORD] : -INFINITY;
          const float logit = LOG2E * (a.scale * part + bias);
          if (MODE == MODE_FWD) {
            if (logit > m[tt]) {
              const float corr = exp2f(m[tt] - logit);
              l[tt] *= corr;
#pragma unroll
              for (int s = 0; s < NR; ++s) acc1[tt].re[s] *= corr;
#pragma unroll
              for (int s = 0; s < NC; ++s) { acc1[tt].cr[s] *= corr; acc1[tt].ci[s] *= corr; }
              m[tt] = logit;
            }
            const float pr = exp2f(logit - m[tt]);  // 2^(-inf) = 0 for masked or out-of-window pairs
            l[tt] += pr;
#pragma unroll
            for (int s = 0; s < NR; ++s) acc1[tt].re[s] += pr * n2.re[s];
#pragma unroll
            for (int f = 0; f < NCF; ++f) {
              const float ar = pr * tr[f], ai = pr * ti[f];  // alpha * tau
#pragma unroll
              for (int u = 0; u < UC; ++u) {
                const int s = f * UC + u;
                acc1[tt].cr[s] += ar * n2.cr[s] - ai * n2.ci[s];
                acc1[tt].ci[s] += ar * n2.ci[s] + ai * n2.cr[s];
              }
            }
          } else {
            const float lse = MODE == MODE_BWD_T ? own_lse[tt] : sstat[2 * pl];
            const float delta = MODE == MODE_BWD_T ? own_delta[tt] : sstat[2 * pl + 1];
            const float pr = valid ? exp2f(logit - LOG2E * lse) : 0.f;
            const float ds = a.scale * pr * (dpart - delta);
#pragma unroll
            for (int s = 0; s < NR; ++s) {
              acc1[tt].re[s] += ds * n1.re[s];                              // dq += ds k   | dk += ds q
              if (MODE == MODE_BWD_S) acc2[tt].re[s] += pr * n2.re[s];      //               dv += p dO
            }
#pragma unroll
            for (int f = 0; f < NCF; ++f) {
              const float ar = ds * tr[f], ai = ds * ti[f], cr = pr * tr[f], ci = pr * ti[f];
#pragma unroll
              for (int u = 0; u < UC; ++u) {
                const int s = f * UC + u;
                if (MODE == MODE_BWD_T) {  // dq += ds tau k
                  acc1[tt].cr[s] += ar * n1.cr[s] - ai * n1.ci[s];
                  acc1[tt].ci[s] += ar * n1.ci[s] + ai * n1.cr[s];
                } else {                   // dk += ds conj(tau) q ; dv += p conj(tau) dO
                  acc1[tt].cr[s] += ar * n1.cr[s] + ai * n1.ci[s];
                  acc1[tt].ci[s] += ar * n1.ci[s] - ai * n1.cr[s];
                  acc2[tt].cr[s] += cr * n2.cr[s] + ci * n2.ci[s];
                  acc2[tt].ci[s] += cr * n2.ci[s] - ci * n2.cr[s];
                }
              }
            }
          }
        }
      }
    }
  }

  // ---- write the owners' results
#pragma unroll
  for (int tt = 0; tt < TT; ++tt) {
    if (!own_ok[tt]) continue;
    const int64_t node = node0 + c0 + group * TT + tt;
    const float inv = MODE == MODE_FWD ? (l[tt] > 0.f ? 1.f / l[tt] : 0.f) : 1.f;
    const int64_t base = node * a.D;
#pragma unroll
    for (int x = 0; x < NR; ++x) {
      if (!real_valid(x)) continue;
      const int64_t g = base + P.real_off + h * P.a0 + real_u0 + x;
      st<S>(a.r1 + g, acc1[tt].re[x] * inv);
      if (MODE == MODE_BWD_S) st<S>(a.r2 + g, acc2[tt].re[x]);
    }
#pragma unroll
    for (int f = 0; f < NCF; ++f)
#pragma unroll
      for (int x = 0; x < UC; ++x) {
        if (!cx_valid(f, x)) continue;
        const int64_t g = base + P.cf_off[f] + 2 * (h * P.ac + cx_u0 + x);
        const int s = f * UC + x;
        st<S>(a.r1 + g, acc1[tt].cr[s] * inv);
        st<S>(a.r1 + g + 1, acc1[tt].ci[s] * inv);
        if (MODE == MODE_BWD_S) {
          st<S>(a.r2 + g, acc2[tt].cr[s]);
          st<S>(a.r2 + g + 1, acc2[tt].ci[s]);
        }
      }
    if (MODE == MODE_FWD && ls == 0) a.lse_out[node * a.H + h] = l[tt] > 0.f ? (m[tt] + log2f(l[tt])) * LN2 : -INFINITY;
  }
}

// delta[node, h] = sum over the head's columns of dO * O
template <typename S>
__global__ void lattice_delta_kernel(const S* __restrict__ dout, const S* __restrict__ out, float* __restrict__ delta, int64_t n_rows,
                                     int D, int H, LatPlan P) {
  const int lane = threadIdx.x & 31;
  const int64_t w = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= n_rows * H) return;
  const int64_t node = w / H;
  const int h = (int)(w % H);
  float acc = 0.f;
  for (int c = lane; c < P.a0; c += 32) {
    const int64_t g = node * D + P.real_off + h * P.a0 + c;
    acc += ld<float>(dout + g) * ld<float>(out + g);
  }
  for (int f = 0; f < P.n_cf; ++f)
    for (int c = lane; c < 2 * P.ac; c += 32) {
      const int64_t g = node * D + P.cf_off[f] + 2 * h * P.ac + c;
      acc += ld<float>(dout + g) * ld<float>(out + g);
    }
  acc = warp_sum(acc);
  if (lane == 0) delta[node * H + h] = acc;
}

// The layouts the lattice kernels serve: an optional scalar block and complex frequencies that share one
// multiplicity.  Anything else is GM_ERR_UNSUPPORTED (callers then use the general CSR kernels).
int make_lat_plan(const int64_t* desc_host, int F, int H, int D, int L, LatPlan& P) {
  GM_REQUIRE(F >= 1 && F <= LAT_MAX_CF + 1, GM_ERR_UNSUPPORTED, "gm_lattice_attention: at most %d frequencies per head", LAT_MAX_CF + 1);
  P = LatPlan{};
  P.L = L;
  for (int f = 0; f < F; ++f) {
    const int n = (int)desc_host[5 * f], a_n = (int)desc_host[5 * f + 1], off = (int)desc_host[5 * f + 2];
    const int dim = n == 0 ? 1 : 2;
    GM_REQUIRE(n >= 0 && a_n >= 1 && off >= 0 && off + H * a_n * dim <= D, GM_ERR_ARGUMENT,
               "gm_lattice_attention: descriptor row %d leaves the width D=%d", f, D);
    if (n == 0) {
      GM_REQUIRE(P.a0 == 0, GM_ERR_ARGUMENT, "gm_lattice_attention: two scalar rows");
      P.a0 = a_n;
      P.real_off = off;
    } else {
      GM_REQUIRE(P.n_cf < LAT_MAX_CF, GM_ERR_UNSUPPORTED, "gm_lattice_attention: more than %d complex frequencies", LAT_MAX_CF);
      GM_REQUIRE(P.ac == 0 || P.ac == a_n, GM_ERR_UNSUPPORTED, "gm_lattice_attention: complex frequencies must share one multiplicity");
      P.ac = a_n;
      P.cf_off[P.n_cf] = off;
      P.cf_order[P.n_cf] = n;
      ++P.n_cf;
    }
  }
  P.d_head = P.a0 + 2 * P.ac * P.n_cf;
  P.pitch = P.d_head + ((8 - P.d_head % 16) + 16) % 16;  // pitch = 8 (mod 16) floats
  // aligned: every lane owns full runs (a0 = NR * L, ac = UC * L) and every run starts on a 16-byte boundary
  const int nr = (P.a0 + L - 1) / L, uc = (P.ac + L - 1) / L;
  P.aligned = (P.a0 == nr * L) && (P.ac == uc * L) && (P.a0 % 4 == 0) && (P.ac % 2 == 0) &&
              (nr == 0 || nr == 1 || nr == 2 || nr == 4) && (uc == 0 || uc == 1 || uc == 2 || uc == 4);
  return GM_OK;
}

struct LatCall {
  const void *f1, *f2, *o1, *o2;
  const float *lse, *delta;
  void *r1, *r2;
  float* lse_out;
  const int *win_cnt, *win_lo, *win_off;
  const float* entries;
  const int* row_order;
  int n_order_rows;
};

template <typename S, int MODE>
int launch_lattice(const LatCall& c, const int64_t* desc_host, int F, int rows, int nlon, int64_t batch, int D, int H, int W, int ES,
                   int NORD, double scale, cudaStream_t stream) {
  LatArgs<S> a{};
  const int L = MODE == MODE_BWD_S ? 8 : 4;
  int status = make_lat_plan(desc_host, F, H, D, L, a.plan);
  if (status != GM_OK) return status;
  for (int f = 0; f < a.plan.n_cf; ++f)
    GM_REQUIRE(a.plan.cf_order[f] <= NORD, GM_ERR_ARGUMENT, "gm_lattice_attention: tables hold %d orders, frequency %d needs more", NORD, a.plan.cf_order[f]);
  a.f1 = (const S*)c.f1; a.f2 = (const S*)c.f2; a.o1 = (const S*)c.o1; a.o2 = (const S*)c.o2;
  a.lse = c.lse; a.delta = c.delta; a.r1 = (S*)c.r1; a.r2 = (S*)c.r2; a.lse_out = c.lse_out;
  a.win_cnt = c.win_cnt; a.win_lo = c.win_lo; a.win_off = c.win_off; a.entries = c.entries; a.row_order = c.row_order;
  a.rows = rows; a.nlon = nlon; a.D = D; a.H = H; a.W = W; a.ES = ES; a.NORD = NORD; a.scale = (float)scale;
  {
    const int ev = 16 / (int)sizeof(S);  // elements per 16-byte vector
    bool ok = D % ev == 0 && a.plan.a0 % ev == 0 && (2 * a.plan.ac) % ev == 0 && a.plan.real_off % ev == 0 && a.plan.pitch % 4 == 0;
    for (int f = 0; f < a.plan.n_cf; ++f) ok = ok && a.plan.cf_off[f] % ev == 0;
    for (const void* ptr : {c.f1, c.f2}) ok = ok && (reinterpret_cast<uintptr_t>(ptr) % 16 == 0);
    a.plan.stage_vec = ok ? 1 : 0;
  }
  constexpr int TT = 2;
  const int TL = (LAT_THREADS / L) * TT;
  const int tiles = (nlon + TL - 1) / TL;
  // rows staged per chunk: what ~48 KiB of shared memory hold (two fields + stats), at least TL + 8
  int SC = (44 * 1024) / ((2 * a.plan.pitch + 2 + ES) * (int)sizeof(float));
  if (SC < TL + 8) SC = TL + 8;
  if (SC > nlon + TL) SC = nlon + TL;
  a.SC = SC;
  const size_t smem = ((size_t)SC * (2 * a.plan.pitch + 2) + (size_t)(SC + TL) * ES) * sizeof(float);
  dim3 grid((unsigned)(c.n_order_rows * tiles), (unsigned)H, (unsigned)batch);
  auto go = [&](auto kernel) {
    int st = allow_smem(kernel, smem, "gm_lattice_attention");
    if (st != GM_OK) return st;
    kernel<<<grid, LAT_THREADS, smem, stream>>>(a);
    return launch_status("gm_lattice_attention");
  };
  const int nr = (a.plan.a0 + L - 1) / L, uc = (a.plan.ac + L - 1) / L, ncf = a.plan.n_cf;
#define GM_LAT_CASE(NR_, NCF_, UC_)                                                                 \
  if (nr <= NR_ && ncf <= NCF_ && uc <= UC_) {                                                      \
    if (a.plan.aligned && nr == NR_ && uc == UC_ && ncf == NCF_) return go(lattice_kernel<S, NR_, NCF_, UC_, TT, MODE, true>); \
    return go(lattice_kernel<S, NR_, NCF_, UC_, TT, MODE, false>);                                   \
  }
  GM_LAT_CASE(1, 2, 1)
  GM_LAT_CASE(2, 2, 2)
  GM_LAT_CASE(2, 3, 2)
  GM_LAT_CASE(4, 2, 4)
  GM_LAT_CASE(4, 4, 4)
#undef GM_LAT_CASE
  return fail(GM_ERR_UNSUPPORTED, "gm_lattice_attention: no kernel for %d scalar / %d x %d complex copies per lane", nr, ncf, uc);
}

int check_lattice(int rows, int nlon, int64_t batch, int D, int H, int W, int ES, int NORD, int dtype) {
  GM_REQUIRE(rows >= 1 && nlon >= 1 && batch >= 1 && D >= 1, GM_ERR_ARGUMENT, "gm_lattice_attention: bad sizes");
  GM_REQUIRE(H >= 1 && H <= 65535 && batch <= 65535, GM_ERR_LIMIT, "gm_lattice_attention: heads and batch must fit a grid dimension");
  GM_REQUIRE(W >= 0 && NORD >= 0 && ES >= 2 * NORD + 1, GM_ERR_ARGUMENT, "gm_lattice_attention: entry stride %d too small for %d orders", ES, NORD);
  GM_REQUIRE(dtype == GM_F32 || dtype == GM_BF16, GM_ERR_UNSUPPORTED, "gm_lattice_attention: float32 or bfloat16 node fields (fp32 arithmetic)");
  return GM_OK;
}

}  // namespace
}  // namespace gmb

using namespace gmb;

extern "C" int gm_lattice_attention_forward(const void* q, const void* k, const void* v, const int* win_cnt, const int* win_lo,
                                            const int* win_off, const float* entries, const int* row_order, int n_order_rows,
                                            const int64_t* desc_host, int F, int rows, int nlon, int64_t batch, int D, int H, int W,
                                            int ES, int NORD, double scale, int dtype, void* out, float* lse, void* stream) {
  int status = check_lattice(rows, nlon, batch, D, H, W, ES, NORD, dtype);
  if (status != GM_OK) return status;
  GM_REQUIRE(q && k && v && win_cnt && win_lo && win_off && entries && row_order && desc_host && out && lse, GM_ERR_ARGUMENT,
             "gm_lattice_attention_forward: null pointer");
  if (n_order_rows == 0) return GM_OK;
  LatCall c{k, v, q, nullptr, nullptr, nullptr, out, nullptr, lse, win_cnt, win_lo, win_off, entries, row_order, n_order_rows};
  if (dtype == GM_F32)
    return launch_lattice<float, MODE_FWD>(c, desc_host, F, rows, nlon, batch, D, H, W, ES, NORD, scale, (cudaStream_t)stream);
  return launch_lattice<__nv_bfloat16, MODE_FWD>(c, desc_host, F, rows, nlon, batch, D, H, W, ES, NORD, scale, (cudaStream_t)stream);
}

extern "C" int gm_lattice_attention_backward(const void* dout, const void* q, const void* k, const void* v, const void* out,
                                             const float* lse, const int* win_cnt, const int* win_lo, const int* win_off,
                                             const float* entries, const int* row_order, int n_order_rows, const int* t_win_cnt,
                                             const int* t_win_lo, const int* t_win_off, const float* t_entries,
                                             const int* t_row_order, int t_n_order_rows, const int64_t* desc_host, int F, int rows,
                                             int nlon, int64_t batch, int D, int H, int W, int ES, int NORD, double scale, int dtype,
                                             void* dq, void* dk, void* dv, float* delta, void* stream) {
  int status = check_lattice(rows, nlon, batch, D, H, W, ES, NORD, dtype);
  if (status != GM_OK) return status;
  GM_REQUIRE(dout && q && k && v && out && lse && win_cnt && win_lo && win_off && entries && row_order && t_win_cnt && t_win_lo &&
                 t_win_off && t_entries && t_row_order && desc_host && dq && dk && dv && delta,
             GM_ERR_ARGUMENT, "gm_lattice_attention_backward: null pointer");
  cudaStream_t cs = (cudaStream_t)stream;
  const int64_t n_rows = batch * rows * (int64_t)nlon;
  auto run = [&](auto tag) {
    using S = decltype(tag);
    LatPlan plan{};
    int st = make_lat_plan(desc_host, F, H, D, 4, plan);
    if (st != GM_OK) return st;
    const int64_t warps = n_rows * H;
    lattice_delta_kernel<S><<<(unsigned)((warps + 7) / 8), 256, 0, cs>>>((const S*)dout, (const S*)out, delta, n_rows, D, H, plan);
    st = launch_status("gm_lattice_attention_backward (delta)");
    if (st != GM_OK) return st;
    if (n_order_rows > 0) {
      LatCall t{k, v, q, dout, lse, delta, dq, nullptr, nullptr, win_cnt, win_lo, win_off, entries, row_order, n_order_rows};
      st = launch_lattice<S, MODE_BWD_T>(t, desc_host, F, rows, nlon, batch, D, H, W, ES, NORD, scale, cs);
      if (st != GM_OK) return st;
    }
    if (t_n_order_rows > 0) {
      LatCall s{q, dout, k, v, lse, delta, dk, dv, nullptr, t_win_cnt, t_win_lo, t_win_off, t_entries, t_row_order, t_n_order_rows};
      st = launch_lattice<S, MODE_BWD_S>(s, desc_host, F, rows, nlon, batch, D, H, W, ES, NORD, scale, cs);
    }
    return st;
  };
  return dtype == GM_F32 ? run(float()) : run(__nv_bfloat16());
}
