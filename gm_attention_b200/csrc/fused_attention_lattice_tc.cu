// Tensor-core version of the lattice fast path for bf16 node fields.
//
// Same layer, same compact tables as fused_attention_lattice.cu.  The identity
// that makes the contraction a matrix product: the transport phase commutes
// with the sum over copies,
//
//   <q_i, tau k_j> = G0 + sum_n Re( tau_n(i, j) * G_n ),   G_n = sum_c conj(q_{i,c}) k_{j,c},
//   sum_j alpha_ij tau_n v_j = ((alpha o tau_n) V)_i,
//
// so for a tile of 16 consecutive targets of one lattice row and 16 consecutive
// source longitudes of one neighbour row the Gram blocks G0, Re G_n, Im G_n are
// plain bf16 x bf16 -> fp32 products (Re: Q K^T with the (re, im) interleave of
// the flat layout as the contraction index; Im: the same Q against K with each
// pair swapped and one sign flipped), the phases / bias / window enter
// elementwise on the 16 x 16 tile in registers, and the value sums are
// (P o tau) V products with P in registers as the A operand.  Pairs outside a
// target's cyclic window are masked by staging their table entry with bias
// -inf; only the longitude band of a row pair is visited, so the tiles are
// dense in the polar rows (whole rows are neighbours) and ~20-40 % dense at the
// equator.
//
// One CTA = 64 targets x one head x one sample; a warp owns 16 targets.  Source
// rows are staged in shared memory as raw bf16 (row pitch an odd number of
// 16-byte chunks: conflict-free ldmatrix), together with a pair-swapped copy of
// V for the imaginary phase part.  Tensor-core instruction: mma.sync m16n8k16
// (bf16 inputs, fp32 accumulate); fragments via ldmatrix.
#include "common.cuh"

namespace gmb {
namespace {

constexpr int TC_THREADS = 128;
constexpr int TC_TL = 64;  // targets per CTA
constexpr float TC_LOG2E = 1.4426950408889634f, TC_LN2 = 0.6931471805599453f;
constexpr int TC_MAX_CF = 3;

struct TcPlan {
  int a0, ac, n_cf;
  int real_off;
  int cf_off[TC_MAX_CF];
  int cf_order[TC_MAX_CF];
};

struct TcArgs {
  const __nv_bfloat16 *q, *k, *v;
  __nv_bfloat16* out;
  float* lse_out;
  const int *win_cnt, *win_lo, *win_off;
  const float* entries;
  const int* row_order;
  int rows, nlon, D, H, W, ES, NORD;
  int SC;  // staged positions per chunk (multiple of 16)
  float scale;
  TcPlan plan;
};

__device__ __forceinline__ int tc_wrap(int x, int n) {
  x %= n;
  return x < 0 ? x + n : x;
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void ldsm_x4(unsigned (&r)[4], const void* p) {
  const unsigned addr = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(unsigned (&r)[4], const void* p) {
  const unsigned addr = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// (re, im) -> (im, -re): the B operand of the imaginary Gram part
__device__ __forceinline__ unsigned swap_neg(unsigned w) { return __byte_perm(w, 0, 0x1032) ^ 0x80000000u; }
// (re, im) -> (-im, re): the value operand multiplied by the imaginary phase part
__device__ __forceinline__ unsigned swap_neg_lo(unsigned w) { return __byte_perm(w, 0, 0x1032) ^ 0x00008000u; }

__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const unsigned*>(&v);
}

// Head-local PADDED column layout: the scalar block (KS0 k-steps of 16 columns), then each complex
// frequency (KSC k-steps).  Padding columns are zero on both operands.  Returns the flat column of a
// padded head-local column, or -1 for padding.
template <int KS0, int NCF, int KSC>
__device__ __forceinline__ int flat_column(const TcPlan& P, int h, int c) {
  if (c < 16 * KS0) return c < P.a0 ? P.real_off + h * P.a0 + c : -1;
  const int cc = c - 16 * KS0, f = cc / (16 * KSC), r = cc - f * 16 * KSC;
  return (f < P.n_cf && r < 2 * P.ac) ? P.cf_off[f] + 2 * h * P.ac + r : -1;
}

template <int KS0, int NCF, int KSC>
__global__ void __launch_bounds__(TC_THREADS) lattice_tc_forward_kernel(TcArgs a) {
  constexpr int KQ = KS0 + NCF * KSC;   // k-steps across a head's padded width
  constexpr int DP = 16 * KQ;           // padded head width
  constexpr int CH = DP / 8;            // 16-byte chunks per staged row
  constexpr int PITCH = (CH % 2 == 0 ? CH + 1 : CH) * 8;  // bf16 elements; odd number of chunks
  constexpr int NT = 2 * KQ;            // output n-tiles of 8 columns
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const TcPlan& P = a.plan;
  const int SC = a.SC;
  __nv_bfloat16* k_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // (SC, PITCH)
  __nv_bfloat16* v_s = k_s + (size_t)SC * PITCH;                      // (SC, PITCH)
  __nv_bfloat16* w_s = v_s + (size_t)SC * PITCH;                      // (SC, PITCH): V with complex pairs as (-im, re)
  float* e_s = reinterpret_cast<float*>(w_s + (size_t)SC * PITCH);   // (SC + TC_TL, 8): tau(f = 0..2), bias * log2 e, pad

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, c = lane & 3;
  const int tiles = (a.nlon + TC_TL - 1) / TC_TL;
  const int row = a.row_order[blockIdx.x / tiles];
  const int c0 = (blockIdx.x % tiles) * TC_TL;
  const int h = blockIdx.y;
  const int64_t b = blockIdx.z;
  const int64_t node0 = (b * a.rows + row) * (int64_t)a.nlon;
  const int tl_a = 16 * warp + g, tl_b = tl_a + 8;  // the two target rows this thread sees in every fragment
  const float cscale = a.scale * TC_LOG2E;

  // ---- Q fragments (A operand), all k-steps
  unsigned qa[KQ][4];
#pragma unroll
  for (int ks = 0; ks < KQ; ++ks)
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int tl = (r & 1) ? tl_b : tl_a;
      const int col = 16 * ks + 2 * c + ((r & 2) ? 8 : 0);
      const int t = c0 + tl;
      float lo = 0.f, hi = 0.f;
      if (t < a.nlon) {
        const __nv_bfloat16* src = a.q + (node0 + t) * a.D;
        const int g0 = flat_column<KS0, NCF, KSC>(P, h, col), g1 = flat_column<KS0, NCF, KSC>(P, h, col + 1);
        if (g0 >= 0) lo = __bfloat162float(src[g0]);
        if (g1 >= 0) hi = __bfloat162float(src[g1]);
      }
      qa[ks][r] = pack_bf16(lo, hi);
    }

  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
  float m_a = -1e30f, m_b = -1e30f, l_a = 0.f, l_b = 0.f;  // running max (base-2 logits) and partial row sums

  for (int dj = -a.W; dj <= a.W; ++dj) {
    const int j = row + dj;
    if (j < 0 || j >= a.rows) continue;
    const int widx = row * (2 * a.W + 1) + dj + a.W;
    const int cnt = a.win_cnt[widx];
    if (cnt == 0) continue;
    const int lo = a.win_lo[widx];
    const float* ent = a.entries + (size_t)a.win_off[widx] * a.ES;
    const int64_t nrow0 = (b * a.rows + j) * (int64_t)a.nlon;
    const int window = TC_TL + cnt - 1;
    for (int p0 = 0; p0 < window; p0 += SC) {
      __syncthreads();
      // ---- stage positions p0 .. p0 + SC - 1 (zero beyond the window), 16-byte chunks
      for (int idx = threadIdx.x; idx < SC * CH; idx += TC_THREADS) {
        const int pl = idx / CH, ch = idx - pl * CH;
        uint4 kv = make_uint4(0, 0, 0, 0), vv = kv, wv = kv;
        if (p0 + pl < window) {
          const int64_t nb = (nrow0 + tc_wrap(c0 + lo + p0 + pl, a.nlon)) * a.D;
          const int g0 = flat_column<KS0, NCF, KSC>(P, h, 8 * ch);
          const int g7 = flat_column<KS0, NCF, KSC>(P, h, 8 * ch + 7);
          const bool whole = g0 >= 0 && g7 == g0 + 7 && ((nb + g0) % 8 == 0);
          if (whole) {
            kv = __ldg(reinterpret_cast<const uint4*>(a.k + nb + g0));
            vv = __ldg(reinterpret_cast<const uint4*>(a.v + nb + g0));
          } else {
            unsigned short kk[8], vs[8];
#pragma unroll
            for (int x = 0; x < 8; ++x) {
              const int gx = flat_column<KS0, NCF, KSC>(P, h, 8 * ch + x);
              kk[x] = gx >= 0 ? __bfloat16_as_ushort(a.k[nb + gx]) : (unsigned short)0;
              vs[x] = gx >= 0 ? __bfloat16_as_ushort(a.v[nb + gx]) : (unsigned short)0;
            }
            kv = make_uint4(kk[0] | (kk[1] << 16), kk[2] | (kk[3] << 16), kk[4] | (kk[5] << 16), kk[6] | (kk[7] << 16));
            vv = make_uint4(vs[0] | (vs[1] << 16), vs[2] | (vs[3] << 16), vs[4] | (vs[5] << 16), vs[6] | (vs[7] << 16));
          }
          wv = make_uint4(swap_neg_lo(vv.x), swap_neg_lo(vv.y), swap_neg_lo(vv.z), swap_neg_lo(vv.w));
        }
        *reinterpret_cast<uint4*>(k_s + pl * PITCH + 8 * ch) = kv;
        *reinterpret_cast<uint4*>(v_s + pl * PITCH + 8 * ch) = vv;
        *reinterpret_cast<uint4*>(w_s + pl * PITCH + 8 * ch) = wv;
      }
      // ---- stage the table entries the chunk can need: x = p - tl, p in the chunk, tl in [0, 64)
      for (int xi = threadIdx.x; xi < SC + TC_TL; xi += TC_THREADS) {
        const int x = xi + p0 - (TC_TL - 1);
        float4 t0 = make_float4(0.f, 0.f, 0.f, 0.f), t1 = make_float4(0.f, 0.f, -INFINITY, 0.f);
        if (x >= 0 && x < cnt) {
          const float* e = ent + (size_t)x * a.ES;
          if (NCF > 0) { t0.x = e[2 * (P.cf_order[0] - 1)]; t0.y = e[2 * (P.cf_order[0] - 1) + 1]; }
          if (NCF > 1 && P.n_cf > 1) { t0.z = e[2 * (P.cf_order[1] - 1)]; t0.w = e[2 * (P.cf_order[1] - 1) + 1]; }
          if (NCF > 2 && P.n_cf > 2) { t1.x = e[2 * (P.cf_order[2] - 1)]; t1.y = e[2 * (P.cf_order[2] - 1) + 1]; }
          t1.z = e[2 * a.NORD] * TC_LOG2E;
        }
        reinterpret_cast<float4*>(e_s)[2 * xi] = t0;
        reinterpret_cast<float4*>(e_s)[2 * xi + 1] = t1;
      }
      __syncthreads();

      // ---- this warp's 16-position steps inside the chunk
      const int p_lo = max(p0, 16 * warp), p_hi = min(min(p0 + SC, window), 16 * warp + 15 + cnt);
      for (int p = p_lo; p < p_hi; p += 16) {
        const int pl = p - p0;
        // S phase: five Gram accumulators for each of the two 8-position halves
        float s0[2][4], sr[NCF > 0 ? NCF : 1][2][4], si[NCF > 0 ? NCF : 1][2][4];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            s0[half][x] = 0.f;
#pragma unroll
            for (int f = 0; f < NCF; ++f) sr[f][half][x] = si[f][half][x] = 0.f;
          }
          // B fragments of this half: positions pl + 8 half + (lane % 8), k-chunks in ldmatrix.x4 groups of two k-steps
#pragma unroll
          for (int ks = 0; ks < KQ; ks += 2) {
            unsigned bf[4];
            const int mi = lane >> 3, rr = lane & 7;
            const int kcol = 16 * ks + 8 * mi;  // matrices: (ks, lo), (ks, hi), (ks + 1, lo), (ks + 1, hi)
            ldsm_x4(bf, k_s + (pl + 8 * half + rr) * PITCH + min(kcol, DP - 8));
#pragma unroll
            for (int sub = 0; sub < 2; ++sub) {
              const int kk = ks + sub;
              if (kk >= KQ) break;
              const unsigned b0 = bf[2 * sub], b1 = bf[2 * sub + 1];
              if (kk < KS0) {
                mma_bf16(s0[half], qa[kk], b0, b1);
              } else {
                const int f = (kk - KS0) / KSC;
                mma_bf16(sr[f][half], qa[kk], b0, b1);
                mma_bf16(si[f][half], qa[kk], swap_neg(b0), swap_neg(b1));
              }
            }
          }
        }
        // elementwise: logits (base 2), online softmax, P o tau fragments
        float lg[2][4];
        float tr[NCF > 0 ? NCF : 1][2][4], ti[NCF > 0 ? NCF : 1][2][4];
        float mx_a = m_a, mx_b = m_b;
#pragma unroll
        for (int half = 0; half < 2; ++half)
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            const int tl = (x & 2) ? tl_b : tl_a;
            const int pos = pl + 8 * half + 2 * c + (x & 1);
            const int xi = pos - tl + (TC_TL - 1);  // staged entry of offset x = p - tl
            const float4 t0 = reinterpret_cast<const float4*>(e_s)[2 * xi];
            const float4 t1 = reinterpret_cast<const float4*>(e_s)[2 * xi + 1];
            float sum = s0[half][x];
            if (NCF > 0) { tr[0][half][x] = t0.x; ti[0][half][x] = t0.y; sum += t0.x * sr[0][half][x] - t0.y * si[0][half][x]; }
            if (NCF > 1) { tr[1][half][x] = t0.z; ti[1][half][x] = t0.w; sum += t0.z * sr[1][half][x] - t0.w * si[1][half][x]; }
            if (NCF > 2) { tr[2][half][x] = t1.x; ti[2][half][x] = t1.y; sum += t1.x * sr[2][half][x] - t1.y * si[2][half][x]; }
            const float v = cscale * sum + t1.z;  // -inf outside the window
            lg[half][x] = v;
            if (x & 2) mx_b = fmaxf(mx_b, v); else mx_a = fmaxf(mx_a, v);
          }
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
        const float corr_a = exp2f(m_a - mx_a), corr_b = exp2f(m_b - mx_b);
        m_a = mx_a;
        m_b = mx_b;
        l_a *= corr_a;
        l_b *= corr_b;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          acc[nt][0] *= corr_a; acc[nt][1] *= corr_a;
          acc[nt][2] *= corr_b; acc[nt][3] *= corr_b;
        }
        unsigned pa[4], par[NCF > 0 ? NCF : 1][4], pai[NCF > 0 ? NCF : 1][4];  // A fragments: P, P tau_re, P tau_im
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          float pr[4];
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            pr[x] = exp2f(lg[half][x] - ((x & 2) ? m_b : m_a));
            if (x & 2) l_b += pr[x]; else l_a += pr[x];
          }
          // C-fragment (row g | g + 8, cols 2c, 2c + 1) of half -> A-fragment registers (2 half, 2 half + 1)
          pa[2 * half] = pack_bf16(pr[0], pr[1]);
          pa[2 * half + 1] = pack_bf16(pr[2], pr[3]);
#pragma unroll
          for (int f = 0; f < NCF; ++f) {
            par[f][2 * half] = pack_bf16(pr[0] * tr[f][half][0], pr[1] * tr[f][half][1]);
            par[f][2 * half + 1] = pack_bf16(pr[2] * tr[f][half][2], pr[3] * tr[f][half][3]);
            pai[f][2 * half] = pack_bf16(pr[0] * ti[f][half][0], pr[1] * ti[f][half][1]);
            pai[f][2 * half + 1] = pack_bf16(pr[2] * ti[f][half][2], pr[3] * ti[f][half][3]);
          }
        }
        // PV phase: k = the 16 positions, n-tiles over the head's padded columns (two per ldmatrix.x4.trans)
#pragma unroll
        for (int nt = 0; nt < NT; nt += 2) {
          const int mi = lane >> 3, rr = lane & 7;
          const int prow = pl + 8 * (mi & 1) + rr, pcol = 8 * (nt + (mi >> 1));
          unsigned vf[4];
          ldsm_x4_trans(vf, v_s + prow * PITCH + pcol);
          if (nt < 2 * KS0) {
            mma_bf16(acc[nt], pa, vf[0], vf[1]);
            mma_bf16(acc[nt + 1], pa, vf[2], vf[3]);
          } else {
            const int f = (nt - 2 * KS0) / (2 * KSC);
            unsigned wf[4];
            ldsm_x4_trans(wf, w_s + prow * PITCH + pcol);
            mma_bf16(acc[nt], par[f], vf[0], vf[1]);
            mma_bf16(acc[nt], pai[f], wf[0], wf[1]);
            mma_bf16(acc[nt + 1], par[f], vf[2], vf[3]);
            mma_bf16(acc[nt + 1], pai[f], wf[2], wf[3]);
          }
        }
      }
    }
  }

  // ---- epilogue: finish the row sums over the quad, normalise, write
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  const float inv_a = l_a > 0.f ? 1.f / l_a : 0.f, inv_b = l_b > 0.f ? 1.f / l_b : 0.f;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      const int tl = (x & 2) ? tl_b : tl_a;
      const int t = c0 + tl;
      const int gcol = flat_column<KS0, NCF, KSC>(P, h, 8 * nt + 2 * c + (x & 1));
      if (t < a.nlon && gcol >= 0) a.out[(node0 + t) * a.D + gcol] = __float2bfloat16_rn(acc[nt][x] * ((x & 2) ? inv_b : inv_a));
    }
  if (c == 0) {
    if (c0 + tl_a < a.nlon) a.lse_out[(node0 + c0 + tl_a) * a.H + h] = l_a > 0.f ? (m_a + log2f(l_a)) * TC_LN2 : -INFINITY;
    if (c0 + tl_b < a.nlon) a.lse_out[(node0 + c0 + tl_b) * a.H + h] = l_b > 0.f ? (m_b + log2f(l_b)) * TC_LN2 : -INFINITY;
  }
}

// ------------------------------------------------------------------------------------------------
// Backward on tensor cores, in two deterministic passes (no atomics), mirroring the FMA kernels:
//   pass T: owners = 16 targets per warp; neighbours (sources) staged.  Gram blocks of (q, k) and of (dO, v)
//           give the logits and d alpha; ds = scale p (d alpha - Delta) becomes the A operand of (ds o tau) K -> dq.
//   pass S: owners = 16 SOURCES per warp; neighbours (targets) staged with their lse / Delta, transposed tables.
//           The same Gram blocks (roles swapped), then (ds o conj tau) Q -> dk and (p o conj tau) dO -> dv.
// ------------------------------------------------------------------------------------------------

struct TcBwdArgs {
  const __nv_bfloat16 *own1, *own2;   // owners' fields: (q, dO) in pass T, (k, v) in pass S
  const __nv_bfloat16 *nb1, *nb2;     // neighbours' fields: (k, v) in pass T, (q, dO) in pass S
  const float *lse, *delta;           // (nodes, H)
  __nv_bfloat16 *res1, *res2;         // dq | dk, dv
  const int *win_cnt, *win_lo, *win_off;
  const float* entries;
  const int* row_order;
  int rows, nlon, D, H, W, ES, NORD, SC;
  float scale;
  TcPlan plan;
};

// A-operand fragments of 16 owner rows for every k-step of the padded head layout
template <int KS0, int NCF, int KSC>
__device__ __forceinline__ void load_owner_fragments(const TcPlan& P, const __nv_bfloat16* field, int64_t node0, int c0, int nlon, int D,
                                                     int h, int tl_a, int tl_b, int c, unsigned (&fa)[KS0 + NCF * KSC][4]) {
#pragma unroll
  for (int ks = 0; ks < KS0 + NCF * KSC; ++ks)
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int tl = (r & 1) ? tl_b : tl_a;
      const int col = 16 * ks + 2 * c + ((r & 2) ? 8 : 0);
      const int t = c0 + tl;
      float lo = 0.f, hi = 0.f;
      if (t < nlon) {
        const __nv_bfloat16* src = field + (node0 + t) * D;
        const int g0 = flat_column<KS0, NCF, KSC>(P, h, col), g1 = flat_column<KS0, NCF, KSC>(P, h, col + 1);
        if (g0 >= 0) lo = __bfloat162float(src[g0]);
        if (g1 >= 0) hi = __bfloat162float(src[g1]);
      }
      fa[ks][r] = pack_bf16(lo, hi);
    }
}

// Gram blocks of 16 owners x 8 staged rows (prow0 .. prow0 + 7): g0 (scalar block), gr / gi per complex frequency.
// OWNER_IS_Q: owners carry q (imaginary part uses (k_im, -k_re)); else owners carry k and the staged rows q
// (imaginary part uses (-q_im, q_re)).
template <int KS0, int NCF, int KSC, bool OWNER_IS_Q>
__device__ __forceinline__ void gram_half(const unsigned (&fa)[KS0 + NCF * KSC][4], const __nv_bfloat16* tile, int pitch, int prow0, int lane,
                                          float (&g0)[4], float (&gr)[NCF > 0 ? NCF : 1][4], float (&gi)[NCF > 0 ? NCF : 1][4]) {
  constexpr int KQ = KS0 + NCF * KSC, DP = 16 * KQ;
#pragma unroll
  for (int x = 0; x < 4; ++x) {
    g0[x] = 0.f;
#pragma unroll
    for (int f = 0; f < NCF; ++f) gr[f][x] = gi[f][x] = 0.f;
  }
#pragma unroll
  for (int ks = 0; ks < KQ; ks += 2) {
    unsigned bf[4];
    const int mi = lane >> 3, rr = lane & 7;
    ldsm_x4(bf, tile + (prow0 + rr) * pitch + min(16 * ks + 8 * mi, DP - 8));
#pragma unroll
    for (int sub = 0; sub < 2; ++sub) {
      const int kk = ks + sub;
      if (kk >= KQ) break;
      const unsigned b0 = bf[2 * sub], b1 = bf[2 * sub + 1];
      if (kk < KS0) {
        mma_bf16(g0, fa[kk], b0, b1);
      } else {
        const int f = (kk - KS0) / KSC;
        mma_bf16(gr[f], fa[kk], b0, b1);
        if (OWNER_IS_Q) mma_bf16(gi[f], fa[kk], swap_neg(b0), swap_neg(b1));
        else mma_bf16(gi[f], fa[kk], swap_neg_lo(b0), swap_neg_lo(b1));
      }
    }
  }
}

// acc (16 owners x padded head width) += A (16 x 16 staged rows) * tile, with the phase parts:
// scalar block: a0 * tile; complex frequency f: ar[f] * tile + ai[f] * tile_w (tile_w = pair-swapped copy).
template <int KS0, int NCF, int KSC>
__device__ __forceinline__ void accumulate_tiles(float (&acc)[2 * (KS0 + NCF * KSC)][4], const unsigned (&a0)[4],
                                                 const unsigned (&ar)[NCF > 0 ? NCF : 1][4], const unsigned (&ai)[NCF > 0 ? NCF : 1][4],
                                                 const __nv_bfloat16* tile, const __nv_bfloat16* tile_w, int pitch, int pl, int lane) {
  constexpr int NT = 2 * (KS0 + NCF * KSC);
#pragma unroll
  for (int nt = 0; nt < NT; nt += 2) {
    const int mi = lane >> 3, rr = lane & 7;
    const int prow = pl + 8 * (mi & 1) + rr, pcol = 8 * (nt + (mi >> 1));
    unsigned vf[4];
    ldsm_x4_trans(vf, tile + prow * pitch + pcol);
    if (nt < 2 * KS0) {
      mma_bf16(acc[nt], a0, vf[0], vf[1]);
      mma_bf16(acc[nt + 1], a0, vf[2], vf[3]);
    } else {
      const int f = (nt - 2 * KS0) / (2 * KSC);
      unsigned wf[4];
      ldsm_x4_trans(wf, tile_w + prow * pitch + pcol);
      mma_bf16(acc[nt], ar[f], vf[0], vf[1]);
      mma_bf16(acc[nt], ai[f], wf[0], wf[1]);
      mma_bf16(acc[nt + 1], ar[f], vf[2], vf[3]);
      mma_bf16(acc[nt + 1], ai[f], wf[2], wf[3]);
    }
  }
}

// PASS_S = false: pass T (dq).  PASS_S = true: pass S (dk, dv).
template <int KS0, int NCF, int KSC, bool PASS_S>
__global__ void __launch_bounds__(TC_THREADS) lattice_tc_backward_kernel(TcBwdArgs a) {
  constexpr int KQ = KS0 + NCF * KSC, DP = 16 * KQ, CH = DP / 8, PITCH = (CH % 2 == 0 ? CH + 1 : CH) * 8, NT = 2 * KQ;
  constexpr int NF = NCF > 0 ? NCF : 1;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const TcPlan& P = a.plan;
  const int SC = a.SC;
  // staged tiles: t1 = first neighbour field, t2 = second, w1 / w2 = their pair-swapped copies used as value operands
  __nv_bfloat16* t1 = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* t2 = t1 + (size_t)SC * PITCH;
  __nv_bfloat16* w1 = t2 + (size_t)SC * PITCH;
  __nv_bfloat16* w2 = w1 + (size_t)SC * PITCH;                        // pass S only
  float* e_s = reinterpret_cast<float*>(PASS_S ? w2 + (size_t)SC * PITCH : w2);  // (SC + TC_TL, 8)
  float* stat_s = e_s + (size_t)(SC + TC_TL) * 8;                     // pass S: (SC, 2) = lse * log2 e, Delta of staged targets

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, c = lane & 3;
  const int tiles = (a.nlon + TC_TL - 1) / TC_TL;
  const int row = a.row_order[blockIdx.x / tiles];
  const int c0 = (blockIdx.x % tiles) * TC_TL;
  const int h = blockIdx.y;
  const int64_t b = blockIdx.z;
  const int64_t node0 = (b * a.rows + row) * (int64_t)a.nlon;
  const int tl_a = 16 * warp + g, tl_b = tl_a + 8;
  const float cscale = a.scale * TC_LOG2E;

  unsigned f1[KQ][4], f2[KQ][4];
  load_owner_fragments<KS0, NCF, KSC>(P, a.own1, node0, c0, a.nlon, a.D, h, tl_a, tl_b, c, f1);
  load_owner_fragments<KS0, NCF, KSC>(P, a.own2, node0, c0, a.nlon, a.D, h, tl_a, tl_b, c, f2);
  float lse_a = 0.f, lse_b = 0.f, dl_a = 0.f, dl_b = 0.f;
  if (!PASS_S) {
    if (c0 + tl_a < a.nlon) { lse_a = a.lse[(node0 + c0 + tl_a) * a.H + h] * TC_LOG2E; dl_a = a.delta[(node0 + c0 + tl_a) * a.H + h]; }
    if (c0 + tl_b < a.nlon) { lse_b = a.lse[(node0 + c0 + tl_b) * a.H + h] * TC_LOG2E; dl_b = a.delta[(node0 + c0 + tl_b) * a.H + h]; }
  }
  float acc1[NT][4], acc2[PASS_S ? NT : 1][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    acc1[nt][0] = acc1[nt][1] = acc1[nt][2] = acc1[nt][3] = 0.f;
    if constexpr (PASS_S) acc2[nt][0] = acc2[nt][1] = acc2[nt][2] = acc2[nt][3] = 0.f;
  }

  for (int dj = -a.W; dj <= a.W; ++dj) {
    const int j = row + dj;
    if (j < 0 || j >= a.rows) continue;
    const int widx = row * (2 * a.W + 1) + dj + a.W;
    const int cnt = a.win_cnt[widx];
    if (cnt == 0) continue;
    const int lo = a.win_lo[widx];
    const float* ent = a.entries + (size_t)a.win_off[widx] * a.ES;
    const int64_t nrow0 = (b * a.rows + j) * (int64_t)a.nlon;
    const int window = TC_TL + cnt - 1;
    for (int p0 = 0; p0 < window; p0 += SC) {
      __syncthreads();
      for (int idx = threadIdx.x; idx < SC * CH; idx += TC_THREADS) {
        const int pl = idx / CH, ch = idx - pl * CH;
        uint4 x1 = make_uint4(0, 0, 0, 0), x2 = x1;
        if (p0 + pl < window) {
          const int64_t nb = (nrow0 + tc_wrap(c0 + lo + p0 + pl, a.nlon)) * a.D;
          const int g0 = flat_column<KS0, NCF, KSC>(P, h, 8 * ch);
          const int g7 = flat_column<KS0, NCF, KSC>(P, h, 8 * ch + 7);
          if (g0 >= 0 && g7 == g0 + 7 && ((nb + g0) % 8 == 0)) {
            x1 = __ldg(reinterpret_cast<const uint4*>(a.nb1 + nb + g0));
            x2 = __ldg(reinterpret_cast<const uint4*>(a.nb2 + nb + g0));
          } else {
            unsigned short u1[8], u2[8];
#pragma unroll
            for (int x = 0; x < 8; ++x) {
              const int gx = flat_column<KS0, NCF, KSC>(P, h, 8 * ch + x);
              u1[x] = gx >= 0 ? __bfloat16_as_ushort(a.nb1[nb + gx]) : (unsigned short)0;
              u2[x] = gx >= 0 ? __bfloat16_as_ushort(a.nb2[nb + gx]) : (unsigned short)0;
            }
            x1 = make_uint4(u1[0] | (u1[1] << 16), u1[2] | (u1[3] << 16), u1[4] | (u1[5] << 16), u1[6] | (u1[7] << 16));
            x2 = make_uint4(u2[0] | (u2[1] << 16), u2[2] | (u2[3] << 16), u2[4] | (u2[5] << 16), u2[6] | (u2[7] << 16));
          }
        }
        *reinterpret_cast<uint4*>(t1 + pl * PITCH + 8 * ch) = x1;
        *reinterpret_cast<uint4*>(t2 + pl * PITCH + 8 * ch) = x2;
        if (PASS_S) {  // value operands of conj(tau): (im, -re)
          *reinterpret_cast<uint4*>(w1 + pl * PITCH + 8 * ch) = make_uint4(swap_neg(x1.x), swap_neg(x1.y), swap_neg(x1.z), swap_neg(x1.w));
          *reinterpret_cast<uint4*>(w2 + pl * PITCH + 8 * ch) = make_uint4(swap_neg(x2.x), swap_neg(x2.y), swap_neg(x2.z), swap_neg(x2.w));
        } else {       // value operand of tau: (-im, re), of the keys only
          *reinterpret_cast<uint4*>(w1 + pl * PITCH + 8 * ch) = make_uint4(swap_neg_lo(x1.x), swap_neg_lo(x1.y), swap_neg_lo(x1.z), swap_neg_lo(x1.w));
        }
      }
      for (int xi = threadIdx.x; xi < SC + TC_TL; xi += TC_THREADS) {
        const int x = xi + p0 - (TC_TL - 1);
        float4 e0 = make_float4(0.f, 0.f, 0.f, 0.f), e1 = make_float4(0.f, 0.f, -INFINITY, 0.f);
        if (x >= 0 && x < cnt) {
          const float* e = ent + (size_t)x * a.ES;
          if (NCF > 0) { e0.x = e[2 * (P.cf_order[0] - 1)]; e0.y = e[2 * (P.cf_order[0] - 1) + 1]; }
          if (NCF > 1 && P.n_cf > 1) { e0.z = e[2 * (P.cf_order[1] - 1)]; e0.w = e[2 * (P.cf_order[1] - 1) + 1]; }
          if (NCF > 2 && P.n_cf > 2) { e1.x = e[2 * (P.cf_order[2] - 1)]; e1.y = e[2 * (P.cf_order[2] - 1) + 1]; }
          e1.z = e[2 * a.NORD] * TC_LOG2E;
        }
        reinterpret_cast<float4*>(e_s)[2 * xi] = e0;
        reinterpret_cast<float4*>(e_s)[2 * xi + 1] = e1;
      }
      if (PASS_S) {
        for (int pl = threadIdx.x; pl < SC; pl += TC_THREADS) {
          float ls = 0.f, dl = 0.f;
          if (p0 + pl < window) {
            const int64_t nn = (nrow0 + tc_wrap(c0 + lo + p0 + pl, a.nlon)) * a.H + h;
            ls = a.lse[nn] * TC_LOG2E;
            dl = a.delta[nn];
          }
          stat_s[2 * pl] = ls;
          stat_s[2 * pl + 1] = dl;
        }
      }
      __syncthreads();

      const int p_lo = max(p0, 16 * warp), p_hi = min(min(p0 + SC, window), 16 * warp + 15 + cnt);
      for (int p = p_lo; p < p_hi; p += 16) {
        const int pl = p - p0;
        unsigned da[4], dar[NF][4], dai[NF][4];   // ds, ds tau_re, ds tau_im
        unsigned pa[4], par[NF][4], pai[NF][4];   // p, p tau_re, p tau_im (pass S)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          float s0[4], sr[NF][4], si[NF][4], h0[4], hr[NF][4], hi[NF][4];
          gram_half<KS0, NCF, KSC, !PASS_S>(f1, t1, PITCH, pl + 8 * half, lane, s0, sr, si);
          gram_half<KS0, NCF, KSC, !PASS_S>(f2, t2, PITCH, pl + 8 * half, lane, h0, hr, hi);
          float ds[4], pr[4], tr[NF][4], ti[NF][4];
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            const int tl = (x & 2) ? tl_b : tl_a;
            const int pos = pl + 8 * half + 2 * c + (x & 1);
            const int xi = pos - tl + (TC_TL - 1);
            const float4 e0 = reinterpret_cast<const float4*>(e_s)[2 * xi];
            const float4 e1 = reinterpret_cast<const float4*>(e_s)[2 * xi + 1];
            float sum = s0[x], dal = h0[x];
            if (NCF > 0) { tr[0][x] = e0.x; ti[0][x] = e0.y; sum += e0.x * sr[0][x] - e0.y * si[0][x]; dal += e0.x * hr[0][x] - e0.y * hi[0][x]; }
            if (NCF > 1) { tr[1][x] = e0.z; ti[1][x] = e0.w; sum += e0.z * sr[1][x] - e0.w * si[1][x]; dal += e0.z * hr[1][x] - e0.w * hi[1][x]; }
            if (NCF > 2) { tr[2][x] = e1.x; ti[2][x] = e1.y; sum += e1.x * sr[2][x] - e1.y * si[2][x]; dal += e1.x * hr[2][x] - e1.y * hi[2][x]; }
            float lse, delta;
            if (PASS_S) { lse = stat_s[2 * pos]; delta = stat_s[2 * pos + 1]; }
            else { lse = (x & 2) ? lse_b : lse_a; delta = (x & 2) ? dl_b : dl_a; }
            pr[x] = exp2f(cscale * sum + e1.z - lse);  // 0 outside the window (bias -inf)
            ds[x] = a.scale * pr[x] * (dal - delta);
          }
          da[2 * half] = pack_bf16(ds[0], ds[1]);
          da[2 * half + 1] = pack_bf16(ds[2], ds[3]);
          if (PASS_S) {
            pa[2 * half] = pack_bf16(pr[0], pr[1]);
            pa[2 * half + 1] = pack_bf16(pr[2], pr[3]);
          }
#pragma unroll
          for (int f = 0; f < NCF; ++f) {
            dar[f][2 * half] = pack_bf16(ds[0] * tr[f][0], ds[1] * tr[f][1]);
            dar[f][2 * half + 1] = pack_bf16(ds[2] * tr[f][2], ds[3] * tr[f][3]);
            dai[f][2 * half] = pack_bf16(ds[0] * ti[f][0], ds[1] * ti[f][1]);
            dai[f][2 * half + 1] = pack_bf16(ds[2] * ti[f][2], ds[3] * ti[f][3]);
            if (PASS_S) {
              par[f][2 * half] = pack_bf16(pr[0] * tr[f][0], pr[1] * tr[f][1]);
              par[f][2 * half + 1] = pack_bf16(pr[2] * tr[f][2], pr[3] * tr[f][3]);
              pai[f][2 * half] = pack_bf16(pr[0] * ti[f][0], pr[1] * ti[f][1]);
              pai[f][2 * half + 1] = pack_bf16(pr[2] * ti[f][2], pr[3] * ti[f][3]);
            }
          }
        }
        // pass T: dq += (ds tau) k.  pass S: dk += (ds conj tau) q, dv += (p conj tau) dO.
        accumulate_tiles<KS0, NCF, KSC>(acc1, da, dar, dai, t1, w1, PITCH, pl, lane);
        if constexpr (PASS_S) accumulate_tiles<KS0, NCF, KSC>(acc2, pa, par, pai, t2, w2, PITCH, pl, lane);
      }
    }
  }

#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      const int t = c0 + ((x & 2) ? tl_b : tl_a);
      const int gcol = flat_column<KS0, NCF, KSC>(P, h, 8 * nt + 2 * c + (x & 1));
      if (t < a.nlon && gcol >= 0) {
        a.res1[(node0 + t) * a.D + gcol] = __float2bfloat16_rn(acc1[nt][x]);
        if constexpr (PASS_S) a.res2[(node0 + t) * a.D + gcol] = __float2bfloat16_rn(acc2[nt][x]);
      }
    }
}

// Delta[node, h] = <dO, O> over the head's columns
__global__ void tc_delta_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ out, float* __restrict__ delta,
                                int64_t n_nodes, int D, int H, TcPlan P) {
  const int lane = threadIdx.x & 31;
  const int64_t w = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= n_nodes * H) return;
  const int64_t node = w / H;
  const int h = (int)(w % H);
  float acc = 0.f;
  for (int x = lane; x < P.a0; x += 32) {
    const int64_t gidx = node * D + P.real_off + h * P.a0 + x;
    acc += __bfloat162float(dout[gidx]) * __bfloat162float(out[gidx]);
  }
  for (int f = 0; f < P.n_cf; ++f)
    for (int x = lane; x < 2 * P.ac; x += 32) {
      const int64_t gidx = node * D + P.cf_off[f] + 2 * h * P.ac + x;
      acc += __bfloat162float(dout[gidx]) * __bfloat162float(out[gidx]);
    }
  acc = warp_sum(acc);
  if (lane == 0) delta[node * H + h] = acc;
}

int make_tc_plan(const int64_t* desc_host, int F, int H, int D, TcPlan& P) {
  P = TcPlan{};
  GM_REQUIRE(F >= 1 && F <= TC_MAX_CF + 1, GM_ERR_UNSUPPORTED, "gm_lattice_attention (tensor cores): at most %d frequencies", TC_MAX_CF + 1);
  for (int f = 0; f < F; ++f) {
    const int n = (int)desc_host[5 * f], a_n = (int)desc_host[5 * f + 1], off = (int)desc_host[5 * f + 2];
    const int dim = n == 0 ? 1 : 2;
    GM_REQUIRE(n >= 0 && a_n >= 1 && off >= 0 && off + H * a_n * dim <= D, GM_ERR_ARGUMENT,
               "gm_lattice_attention: descriptor row %d leaves the width D=%d", f, D);
    if (n == 0) {
      GM_REQUIRE(P.a0 == 0 && a_n <= 16, GM_ERR_UNSUPPORTED, "gm_lattice_attention (tensor cores): one scalar block of at most 16 copies");
      P.a0 = a_n;
      P.real_off = off;
    } else {
      GM_REQUIRE(P.n_cf < TC_MAX_CF && a_n <= 16 && (P.ac == 0 || P.ac == a_n), GM_ERR_UNSUPPORTED,
                 "gm_lattice_attention (tensor cores): at most %d complex frequencies of one multiplicity <= 16", TC_MAX_CF);
      P.ac = a_n;
      P.cf_off[P.n_cf] = off;
      P.cf_order[P.n_cf] = n;
      ++P.n_cf;
    }
  }
  return GM_OK;
}

template <int KS0, int NCF, int KSC>
int launch_tc_forward(TcArgs& a, int n_order_rows, int64_t batch, cudaStream_t stream) {
  constexpr int KQ = KS0 + NCF * KSC, CH = 2 * KQ, PITCH = (CH % 2 == 0 ? CH + 1 : CH) * 8;
  int SC = 96;  // 64 targets + a window of up to 33 fit one chunk; wider windows take several
  if (SC > ((a.nlon + TC_TL + 15) / 16) * 16) SC = ((a.nlon + TC_TL + 15) / 16) * 16;
  a.SC = SC;
  const size_t smem = (size_t)SC * PITCH * 2 * 3 + (size_t)(SC + TC_TL) * 8 * sizeof(float);
  auto kernel = lattice_tc_forward_kernel<KS0, NCF, KSC>;
  int st = allow_smem(kernel, smem, "gm_lattice_attention_forward_tc");
  if (st != GM_OK) return st;
  const int tiles = (a.nlon + TC_TL - 1) / TC_TL;
  dim3 grid((unsigned)(n_order_rows * tiles), (unsigned)a.H, (unsigned)batch);
  kernel<<<grid, TC_THREADS, smem, stream>>>(a);
  return launch_status("gm_lattice_attention_forward_tc");
}

}  // namespace
}  // namespace gmb

using namespace gmb;

extern "C" int gm_lattice_attention_forward_tc(const void* q, const void* k, const void* v, const int* win_cnt, const int* win_lo,
                                               const int* win_off, const float* entries, const int* row_order, int n_order_rows,
                                               const int64_t* desc_host, int F, int rows, int nlon, int64_t batch, int D, int H, int W,
                                               int ES, int NORD, double scale, void* out, float* lse, void* stream) {
  GM_REQUIRE(rows >= 1 && nlon >= 1 && batch >= 1 && D >= 1 && H >= 1 && H <= 65535 && batch <= 65535, GM_ERR_ARGUMENT,
             "gm_lattice_attention_forward_tc: bad sizes");
  GM_REQUIRE(W >= 0 && NORD >= 0 && ES >= 2 * NORD + 1, GM_ERR_ARGUMENT, "gm_lattice_attention_forward_tc: entry stride too small");
  GM_REQUIRE(q && k && v && win_cnt && win_lo && win_off && entries && row_order && desc_host && out && lse, GM_ERR_ARGUMENT,
             "gm_lattice_attention_forward_tc: null pointer");
  if (n_order_rows == 0) return GM_OK;
  TcArgs a{};
  int status = make_tc_plan(desc_host, F, H, D, a.plan);
  if (status != GM_OK) return status;
  for (int f = 0; f < a.plan.n_cf; ++f)
    GM_REQUIRE(a.plan.cf_order[f] <= NORD, GM_ERR_ARGUMENT, "gm_lattice_attention_forward_tc: tables hold %d orders", NORD);
  a.q = (const __nv_bfloat16*)q; a.k = (const __nv_bfloat16*)k; a.v = (const __nv_bfloat16*)v; a.out = (__nv_bfloat16*)out; a.lse_out = lse;
  a.win_cnt = win_cnt; a.win_lo = win_lo; a.win_off = win_off; a.entries = entries; a.row_order = row_order;
  a.rows = rows; a.nlon = nlon; a.D = D; a.H = H; a.W = W; a.ES = ES; a.NORD = NORD; a.scale = (float)scale;
  const int ks0 = a.plan.a0 > 0 ? 1 : 0, ksc = a.plan.ac > 8 ? 2 : 1, ncf = a.plan.n_cf;
  cudaStream_t cs = (cudaStream_t)stream;
  if (ks0 == 1 && ncf == 2 && ksc == 2) return launch_tc_forward<1, 2, 2>(a, n_order_rows, batch, cs);
  if (ks0 == 1 && ncf == 2 && ksc == 1) return launch_tc_forward<1, 2, 1>(a, n_order_rows, batch, cs);
  if (ks0 == 1 && ncf == 3 && ksc == 1) return launch_tc_forward<1, 3, 1>(a, n_order_rows, batch, cs);
  if (ks0 == 1 && ncf == 1 && ksc <= 2) return ksc == 2 ? launch_tc_forward<1, 1, 2>(a, n_order_rows, batch, cs) : launch_tc_forward<1, 1, 1>(a, n_order_rows, batch, cs);
  if (ks0 == 0 && ncf == 2 && ksc == 1) return launch_tc_forward<0, 2, 1>(a, n_order_rows, batch, cs);
  return fail(GM_ERR_UNSUPPORTED, "gm_lattice_attention_forward_tc: no tensor-core kernel for this head layout (a0=%d, %d x %d complex)",
              a.plan.a0, ncf, a.plan.ac);
}

namespace gmb {
namespace {

template <int KS0, int NCF, int KSC, bool PASS_S>
int launch_tc_backward(TcBwdArgs& a, int n_order_rows, int64_t batch, cudaStream_t stream) {
  constexpr int KQ = KS0 + NCF * KSC, CH = 2 * KQ, PITCH = (CH % 2 == 0 ? CH + 1 : CH) * 8;
  int SC = 96;
  if (SC > ((a.nlon + TC_TL + 15) / 16) * 16) SC = ((a.nlon + TC_TL + 15) / 16) * 16;
  a.SC = SC;
  const size_t smem = (size_t)SC * PITCH * 2 * (PASS_S ? 4 : 3) + (size_t)(SC + TC_TL) * 8 * sizeof(float) + (PASS_S ? (size_t)SC * 2 * sizeof(float) : 0);
  auto kernel = lattice_tc_backward_kernel<KS0, NCF, KSC, PASS_S>;
  int st = allow_smem(kernel, smem, "gm_lattice_attention_backward_tc");
  if (st != GM_OK) return st;
  const int tiles = (a.nlon + TC_TL - 1) / TC_TL;
  dim3 grid((unsigned)(n_order_rows * tiles), (unsigned)a.H, (unsigned)batch);
  kernel<<<grid, TC_THREADS, smem, stream>>>(a);
  return launch_status("gm_lattice_attention_backward_tc");
}

template <bool PASS_S>
int dispatch_tc_backward(TcBwdArgs& a, int n_order_rows, int64_t batch, cudaStream_t cs) {
  const int ks0 = a.plan.a0 > 0 ? 1 : 0, ksc = a.plan.ac > 8 ? 2 : 1, ncf = a.plan.n_cf;
  if (ks0 == 1 && ncf == 2 && ksc == 2) return launch_tc_backward<1, 2, 2, PASS_S>(a, n_order_rows, batch, cs);
  if (ks0 == 1 && ncf == 2 && ksc == 1) return launch_tc_backward<1, 2, 1, PASS_S>(a, n_order_rows, batch, cs);
  if (ks0 == 1 && ncf == 3 && ksc == 1) return launch_tc_backward<1, 3, 1, PASS_S>(a, n_order_rows, batch, cs);
  if (ks0 == 1 && ncf == 1 && ksc == 2) return launch_tc_backward<1, 1, 2, PASS_S>(a, n_order_rows, batch, cs);
  if (ks0 == 1 && ncf == 1 && ksc == 1) return launch_tc_backward<1, 1, 1, PASS_S>(a, n_order_rows, batch, cs);
  if (ks0 == 0 && ncf == 2 && ksc == 1) return launch_tc_backward<0, 2, 1, PASS_S>(a, n_order_rows, batch, cs);
  return fail(GM_ERR_UNSUPPORTED, "gm_lattice_attention_backward_tc: no tensor-core kernel for this head layout (a0=%d, %d x %d complex)",
              a.plan.a0, ncf, a.plan.ac);
}

}  // namespace
}  // namespace gmb

extern "C" int gm_lattice_attention_backward_tc(const void* dout, const void* q, const void* k, const void* v, const void* out,
                                                const float* lse, const int* win_cnt, const int* win_lo, const int* win_off,
                                                const float* entries, const int* row_order, int n_order_rows, const int* t_win_cnt,
                                                const int* t_win_lo, const int* t_win_off, const float* t_entries,
                                                const int* t_row_order, int t_n_order_rows, const int64_t* desc_host, int F, int rows,
                                                int nlon, int64_t batch, int D, int H, int W, int ES, int NORD, double scale, void* dq,
                                                void* dk, void* dv, float* delta, void* stream) {
  GM_REQUIRE(rows >= 1 && nlon >= 1 && batch >= 1 && D >= 1 && H >= 1 && H <= 65535 && batch <= 65535, GM_ERR_ARGUMENT,
             "gm_lattice_attention_backward_tc: bad sizes");
  GM_REQUIRE(W >= 0 && NORD >= 0 && ES >= 2 * NORD + 1, GM_ERR_ARGUMENT, "gm_lattice_attention_backward_tc: entry stride too small");
  GM_REQUIRE(dout && q && k && v && out && lse && win_cnt && win_lo && win_off && entries && row_order && t_win_cnt && t_win_lo &&
                 t_win_off && t_entries && t_row_order && desc_host && dq && dk && dv && delta,
             GM_ERR_ARGUMENT, "gm_lattice_attention_backward_tc: null pointer");
  using B = __nv_bfloat16;
  cudaStream_t cs = (cudaStream_t)stream;
  TcBwdArgs a{};
  int status = make_tc_plan(desc_host, F, H, D, a.plan);
  if (status != GM_OK) return status;
  for (int f = 0; f < a.plan.n_cf; ++f)
    GM_REQUIRE(a.plan.cf_order[f] <= NORD, GM_ERR_ARGUMENT, "gm_lattice_attention_backward_tc: tables hold %d orders", NORD);
  const int64_t n_nodes = batch * rows * (int64_t)nlon;
  tc_delta_kernel<<<(unsigned)((n_nodes * H + 7) / 8), 256, 0, cs>>>((const B*)dout, (const B*)out, delta, n_nodes, D, H, a.plan);
  status = launch_status("gm_lattice_attention_backward_tc (delta)");
  if (status != GM_OK) return status;
  a.lse = lse; a.delta = delta; a.rows = rows; a.nlon = nlon; a.D = D; a.H = H; a.W = W; a.ES = ES; a.NORD = NORD; a.scale = (float)scale;
  if (n_order_rows > 0) {
    a.own1 = (const B*)q; a.own2 = (const B*)dout; a.nb1 = (const B*)k; a.nb2 = (const B*)v; a.res1 = (B*)dq; a.res2 = nullptr;
    a.win_cnt = win_cnt; a.win_lo = win_lo; a.win_off = win_off; a.entries = entries; a.row_order = row_order;
    status = dispatch_tc_backward<false>(a, n_order_rows, batch, cs);
    if (status != GM_OK) return status;
  }
  if (t_n_order_rows > 0) {
    a.own1 = (const B*)k; a.own2 = (const B*)v; a.nb1 = (const B*)q; a.nb2 = (const B*)dout; a.res1 = (B*)dk; a.res2 = (B*)dv;
    a.win_cnt = t_win_cnt; a.win_lo = t_win_lo; a.win_off = t_win_off; a.entries = t_entries; a.row_order = t_row_order;
    status = dispatch_tc_backward<true>(a, t_n_order_rows, batch, cs);
  }
  return status;
}
