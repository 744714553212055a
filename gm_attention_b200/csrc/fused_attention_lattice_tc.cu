// Tensor-core version of the lattice fast path for bf16 node fields.
//
// Same layer, same compact tables as fused_attention_lattice.cu.  The identity
// that makes the contraction a matrix product: the transport phase commutes
// with the sum over copies,
//
//   <q_i, tau k_j> = G0 + sum_n Re( tau_n(i, j) * G_n ),   G_n = sum_c conj(q_{i,c}) k_{j,c},
//   sum_j alpha_ij tau_n v_j = ((alpha o tau_n) V)_i,
//
// so for 8 consecutive owners (targets; sources in the backward's source-major
// pass) of one lattice row and 16 consecutive positions of one neighbour row the
// Gram blocks G0, Re G_n, Im G_n are plain bf16 x bf16 -> fp32 products, the
// phases / bias / window enter elementwise on the tile in registers, and the value
// sums are products with the weights as an operand.  The staged neighbour
// positions are the M dimension of the MMAs (16 per step) and a warp's owners the
// N dimension (8 per warp):
//
//   S^T   (16 positions x 8 owners)  = tile (positions x columns) * owners^T      A: shared memory, B: loop-invariant registers
//   out^T (16 columns   x 8 owners) += tile^T (columns x positions) * (P o tau)^T  A: shared memory (ldmatrix.trans), B: P^T
//
// * Only the longitude band of a row pair is visited; pairs outside an owner's cyclic window get logit -inf.  8 owners
//   see a window of 7 + cnt positions, so the narrow equatorial windows (cnt <= 9) take ONE step per neighbour row;
//   polar windows (whole rows) are dense.
// * Im G_n uses a pre-swapped copy of the OWNERS' fragments, (re, im) -> (-im, re) or (im, -re), made once per CTA.
// * The imaginary part of the phase accumulates into a second accumulator set; the multiplication by +-i (the pair
//   swap) is applied once in the epilogue, so the staged value tile is never swapped.
// * The weights P (accumulator layout: position rows, owner columns) become a B operand with movmatrix (8 x 8 b16
//   transpose in registers); the same instruction turns the result tiles into 4-byte stores per owner.
// * The softmax reference maximum of an owner moves only when it is exceeded by 2^8 (lazy rescaling).
//
// One CTA = 8 owners x WARPS warps x one head x one sample.  The neighbour rows of one lattice row and the table
// entries they need are copied into shared memory as raw bf16 / fp32, double-buffered: the copy of the next
// (row pair, chunk) runs while the current one is consumed.  A staged field is one sub-tile per frequency block
// (88 or 56 positions x 32 or 64 bytes) in the 32-byte / 64-byte shared-memory swizzle, so that ldmatrix is conflict-free
// without padding and a whole sub-tile is ONE TMA tensor copy (cp.async.bulk.tensor.3d over (column, longitude,
// sample * row), completion on an mbarrier, issued by one thread).  Chunks that wrap the longitude seam, and head
// layouts whose blocks are not exactly 16 / 32 columns, are staged with per-thread cp.async into the same swizzled
// layout.  Tensor-core instruction: mma.sync m16n8k16 (bf16 inputs, fp32 accumulate); fragments via ldmatrix.
//
// Backward, two deterministic passes (no atomics):
//   pass T: owners = targets.  Delta = <dO, O> per (target, head) from the owners' own rows (written out for pass S);
//           Gram blocks of (q, k) and of (dO, v) give the logits and d alpha; ds = scale p (d alpha - Delta)
//           weights (ds o tau) K -> dq.
//   pass S: owners = SOURCES, neighbours = the targets that see them (transposed tables, their lse / Delta
//           staged with them).  Same Gram blocks with the roles swapped, then (ds o conj tau) Q -> dk and
//           (p o conj tau) dO -> dv.
#include <cuda.h>
#include <cudaTypedefs.h>

#include "common.cuh"

namespace gmb {
namespace {

constexpr float TC_LOG2E = 1.4426950408889634f, TC_LN2 = 0.6931471805599453f;
constexpr int TC_MAX_CF = 3;
constexpr int TC_MAX_WIN = 33;  // 2 W + 1 neighbour rows at most
constexpr unsigned TC_WAIT_LIMIT = 1u << 22;  // polls of a copy barrier before the kernel gives up on it

// set when a wait on a TMA completion barrier ran out (never expected; the results of that launch are invalid)
__device__ int g_tc_wait_expired;

struct TcPlan {
  int a0, ac, n_cf;
  int real_off;
  int cf_off[TC_MAX_CF];
  int cf_order[TC_MAX_CF];
};

struct TcArgs {
  const __nv_bfloat16 *own1, *own2;   // owners' fields:     q, -  |  q, dO  |  k, v
  const __nv_bfloat16 *nb1, *nb2;     // neighbours' fields: k, v  |  k, v   |  q, dO
  const float *lse, *delta;           // (nodes, H), backward
  const __nv_bfloat16* out_fwd;       // pass T with delta_out: the forward's output, Delta = <dO, O> is formed here
  float* delta_out;                   // pass T: where Delta is written for the source-major pass (null: read `delta`)
  __nv_bfloat16 *res1, *res2;         // out | dq | dk, dv
  float* lse_out;                     // forward
  const int *win_cnt, *win_lo, *win_off;
  const float* entries;               // (n_entries, 8): (cos, sin) of orders 1..NORD, bias at 2 NORD
  const int* row_order;
  int rows, nlon, D, H, W, NORD;
  int exact;    // every block is exactly 16 (scalar) / 16 KSC (complex) columns wide and starts on an even column: no padding, 4-byte accesses
  int use_tma;  // the neighbours' fields have tensor maps (exact 16 / 32-column blocks, aligned, at least one chunk of longitudes)
  int aligned16;  // the neighbours' fields start on 16-byte boundaries (16-byte per-thread copies allowed)
  float scale;
  TcPlan plan;
  // tensor maps over the neighbours' fields as (D, nlon, batch * rows): [field][0 = 16-column box, 1 = complex-block box]
  alignas(64) CUtensorMap maps[2][2];
};

enum { TC_FWD = 0, TC_BWD_T = 1, TC_BWD_S = 2 };

__device__ __forceinline__ int tc_wrap(int x, int n) {
  x %= n;
  return x < 0 ? x + n : x;
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// ---- TMA + mbarrier (single CTA; no multicast)
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"((unsigned)__cvta_generic_to_shared(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"((unsigned)__cvta_generic_to_shared(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned parity) {
  unsigned done;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(done) : "r"((unsigned)__cvta_generic_to_shared(bar)), "r"(parity) : "memory");
  return done != 0;
}
// bounded wait: gives up after TC_WAIT_LIMIT polls, records it in the device-wide flag and returns false
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity) {
  for (unsigned tries = 0; tries < TC_WAIT_LIMIT; ++tries) {
    if (mbar_try_wait(bar, parity)) return true;
    if (tries > 64) __nanosleep(64);
  }
  atomicOr(&g_tc_wait_expired, 1);
  return false;
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, unsigned long long* bar, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n"
               ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(reinterpret_cast<unsigned long long>(map)),
                 "r"((unsigned)__cvta_generic_to_shared(bar)), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }

// 16-byte asynchronous copy global -> shared; src_bytes = 0 writes zeros
__device__ __forceinline__ void cp_async16(void* dst, const void* src, int src_bytes) {
  const unsigned addr = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(addr), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async4(void* dst, const void* src, int src_bytes) {
  const unsigned addr = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(addr), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// (re, im) -> (im, -re) / (-im, re): the B operand of the imaginary Gram part for owners carrying q / carrying k
__device__ __forceinline__ unsigned swap_neg(unsigned w) { return __byte_perm(w, 0, 0x1032) ^ 0x80000000u; }
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

// owners per CTA = 8 x warps.  4 warps (32 owners) in every pass: four CTAs per SM at 128 registers (forward, pass T),
// three at 168 (pass S); 8 warps (64 owners, 80-position chunks) stay instantiable
constexpr int TN_WARPS(int mode) { return 4; }
// positions a staged chunk advances by (a multiple of 16): 64 owners + a window of up to 17 fit one chunk of 80, 32 owners
// + 17 one of 48 (smaller buffers: four CTAs per SM).  Staged per chunk: 8 more, a step of 16 may start 8 before the end.
constexpr __host__ __device__ int tn_advance(int owners) { return owners >= 64 ? 80 : 48; }
constexpr __host__ __device__ int tn_rows(int owners) { return tn_advance(owners) + 8; }

template <int KS0, int NCF, int KSC, int TL>
struct TnLayout {
  static constexpr __host__ __device__ int align1k(int x) { return (x + 1023) / 1024 * 1024; }
  static constexpr int REAL_PITCH = 32, CX_PITCH = 32 * KSC;
  static constexpr int TN_ROWS = tn_rows(TL);
  static constexpr int REAL_BYTES = KS0 ? align1k(TN_ROWS * REAL_PITCH) : 0;
  static constexpr int CX_BYTES = align1k(TN_ROWS * CX_PITCH);
  static constexpr int FIELD_BYTES = REAL_BYTES + NCF * CX_BYTES;
  static constexpr int ENT_BYTES = (TN_ROWS + TL) * 32;
  static constexpr int BUFFER_BYTES = align1k(2 * FIELD_BYTES + ENT_BYTES + TN_ROWS * 8);  // with the (lse, Delta) pairs of pass S
  static __device__ __forceinline__ int real_chunk(int r, int cb) { return r * REAL_PITCH + 16 * (cb ^ ((r >> 2) & 1)); }
  static __device__ __forceinline__ int cx_chunk(int f, int r, int cb) {
    return REAL_BYTES + f * CX_BYTES + r * CX_PITCH + 16 * (cb ^ (KSC == 2 ? (r >> 1) & 3 : (r >> 2) & 1));
  }
  static __device__ __forceinline__ int chunk(int r, int ch) {
    if (ch < 2 * KS0) return real_chunk(r, ch);
    const int cc = ch - 2 * KS0;
    return cx_chunk(cc / (2 * KSC), r, cc % (2 * KSC));
  }
};

__device__ __forceinline__ unsigned movmatrix_trans(unsigned x) {
  unsigned y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(y) : "r"(x));
  return y;
}
__device__ __forceinline__ void mma_bf16_b2(float (&d)[4], const unsigned (&a)[4], const unsigned (&b)[2]) { mma_bf16(d, a, b[0], b[1]); }
// d = a * b (no accumulator to zero first)
__device__ __forceinline__ void mma_bf16_b2_init(float (&d)[4], const unsigned (&a)[4], const unsigned (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
               : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]), "f"(0.f));
}

__device__ __forceinline__ void ldsm_x4(unsigned (&r)[4], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(unsigned (&r)[4], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ float fast_exp2(float x) {  // ex2.approx: exp2(-inf) = 0, relative error ~2^-22
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// Per-lane byte offsets of the ldmatrix rows inside a sub-tile, for a step starting at staged row 0.  A step starts on
// a multiple of 8 rows, which leaves the swizzle term of a lane's row unchanged, so a step adds only pl * pitch.
template <int KS0, int NCF, int KSC, int TL>
struct TnLaneOffsets {
  using L = TnLayout<KS0, NCF, KSC, TL>;
  int g_real, g_cx[KSC];  // Gram A operand: matrices (rows 0-7, k 0-7), (rows 8-15, k 0-7), (rows 0-7, k 8-15), (rows 8-15, k 8-15)
  int a_real, a_cx[KSC];  // accumulation A operand = tile^T: (cols 0-7, rows 0-7), (cols 8-15, rows 0-7), (cols 0-7, rows 8-15), (cols 8-15, rows 8-15)
  __device__ __forceinline__ void init(int lane) {
    const int mi = lane >> 3, rr = lane & 7;
    g_real = L::real_chunk(8 * (mi & 1) + rr, mi >> 1);
    a_real = L::real_chunk(8 * (mi >> 1) + rr, mi & 1);
#pragma unroll
    for (int sub = 0; sub < KSC; ++sub) {
      g_cx[sub] = L::cx_chunk(0, 8 * (mi & 1) + rr, 2 * sub + (mi >> 1));
      a_cx[sub] = L::cx_chunk(0, 8 * (mi >> 1) + rr, 2 * sub + (mi & 1));
    }
  }
};

// S^T blocks of 16 staged rows (pl .. pl + 15) x 8 owners: g0 (scalar block), gr / gi per complex frequency.
// fb: the owners' fragments, fs: their pre-swapped copies for the imaginary part (complex k-steps only).
// tile: shared-memory address of the staged field.
template <int KS0, int NCF, int KSC, int TL>
__device__ __forceinline__ void gram_step(const unsigned (&fb)[KS0 + NCF * KSC][2], const unsigned (&fs)[NCF * KSC > 0 ? NCF * KSC : 1][2],
                                          unsigned tile, int pl, const TnLaneOffsets<KS0, NCF, KSC, TL>& lo, float (&g0)[4],
                                          float (&gr)[NCF > 0 ? NCF : 1][4], float (&gi)[NCF > 0 ? NCF : 1][4]) {
  using L = TnLayout<KS0, NCF, KSC, TL>;
  if constexpr (KS0 > 0) {
    unsigned af[4];
    ldsm_x4(af, tile + pl * L::REAL_PITCH + lo.g_real);
    mma_bf16_b2_init(g0, af, fb[0]);
  } else {
    g0[0] = g0[1] = g0[2] = g0[3] = 0.f;
  }
  const unsigned cx = tile + pl * L::CX_PITCH;
#pragma unroll
  for (int f = 0; f < NCF; ++f)
#pragma unroll
    for (int sub = 0; sub < KSC; ++sub) {
      unsigned af[4];
      ldsm_x4(af, cx + lo.g_cx[sub] + f * L::CX_BYTES);
      if (sub == 0) {
        mma_bf16_b2_init(gr[f], af, fb[KS0 + f * KSC + sub]);
        mma_bf16_b2_init(gi[f], af, fs[f * KSC + sub]);
      } else {
        mma_bf16_b2(gr[f], af, fb[KS0 + f * KSC + sub]);
        mma_bf16_b2(gi[f], af, fs[f * KSC + sub]);
      }
    }
}

// acc^T (padded head columns x 8 owners) += tile^T (columns x 16 staged rows pl .. pl + 15) * B, B = x0 for the scalar block,
// xr[f] into the real-phase accumulators and xi[f] into the imaginary-phase accumulators of frequency f.
template <int KS0, int NCF, int KSC, int TL>
__device__ __forceinline__ void accumulate_step(float (&acc0)[4], float (&accr)[NCF * KSC > 0 ? NCF * KSC : 1][4], float (&acci)[NCF * KSC > 0 ? NCF * KSC : 1][4],
                                                const unsigned (&x0)[2], const unsigned (&xr)[NCF > 0 ? NCF : 1][2], const unsigned (&xi)[NCF > 0 ? NCF : 1][2],
                                                unsigned tile, int pl, const TnLaneOffsets<KS0, NCF, KSC, TL>& lo) {
  using L = TnLayout<KS0, NCF, KSC, TL>;
  if constexpr (KS0 > 0) {
    unsigned af[4];
    ldsm_x4_trans(af, tile + pl * L::REAL_PITCH + lo.a_real);
    mma_bf16_b2(acc0, af, x0);
  }
  const unsigned cx = tile + pl * L::CX_PITCH;
#pragma unroll
  for (int f = 0; f < NCF; ++f)
#pragma unroll
    for (int sub = 0; sub < KSC; ++sub) {
      unsigned af[4];
      ldsm_x4_trans(af, cx + lo.a_cx[sub] + f * L::CX_BYTES);
      mma_bf16_b2(accr[f * KSC + sub], af, xr[f]);
      mma_bf16_b2(acci[f * KSC + sub], af, xi[f]);
    }
}

// Flat column of the pair of padded head-local columns (col, col + 1) of k-step / m-tile `kt` (compile-time), col even in
// 0 .. 14: first = flat column or -1 (padding), second likewise.  No division: the block is known at compile time.
template <int KS0, int NCF, int KSC, int KT>
__device__ __forceinline__ void flat_pair(const TcPlan& P, int h, int col, int& g0, int& g1) {
  if constexpr (KT < KS0) {
    const int cc = 16 * KT + col;
    g0 = cc < P.a0 ? P.real_off + h * P.a0 + cc : -1;
    g1 = cc + 1 < P.a0 ? P.real_off + h * P.a0 + cc + 1 : -1;
  } else {
    constexpr int F = (KT - KS0) / KSC, SUB = (KT - KS0) % KSC;
    const int cc = 16 * SUB + col;
    g0 = cc < 2 * P.ac ? P.cf_off[F] + 2 * h * P.ac + cc : -1;
    g1 = g0 >= 0 ? g0 + 1 : -1;  // 2 ac is even: a (re, im) pair is never split
  }
}

// First flat column of k-step / m-tile KT of head h when every block is exactly as wide as its padded slot
template <int KS0, int NCF, int KSC, int KT>
__device__ __forceinline__ int exact_block(const TcPlan& P, int h) {
  if constexpr (KT < KS0) return P.real_off + 16 * h + 16 * KT;
  else return P.cf_off[(KT - KS0) / KSC] + 16 * KSC * h + 16 * ((KT - KS0) % KSC);
}

// B-operand fragments of one owner (column n = g of the warp's 8) for every k-step of the padded head layout
template <int KS0, int NCF, int KSC, int KT = 0>
__device__ __forceinline__ void load_owner_columns(const TcPlan& P, const __nv_bfloat16* src, bool present, bool exact, bool words, int h, int c,
                                                   unsigned (&fb)[KS0 + NCF * KSC][2]) {
  if constexpr (KT < KS0 + NCF * KSC) {
    if (exact) {
      const unsigned* w = reinterpret_cast<const unsigned*>(src + exact_block<KS0, NCF, KSC, KT>(P, h)) + c;
      fb[KT][0] = present ? w[0] : 0u;
      fb[KT][1] = present ? w[4] : 0u;
    } else {
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        int g0, g1;
        flat_pair<KS0, NCF, KSC, KT>(P, h, 2 * c + 8 * r, g0, g1);
        unsigned w = 0u;
        if (present) {
          if (words && g0 >= 0 && g1 == g0 + 1 && (g0 & 1) == 0) {
            w = *reinterpret_cast<const unsigned*>(src + g0);
          } else {
            if (g0 >= 0) w = __bfloat16_as_ushort(src[g0]);
            if (g1 >= 0) w |= (unsigned)__bfloat16_as_ushort(src[g1]) << 16;
          }
        }
        fb[KT][r] = w;
      }
    }
    load_owner_columns<KS0, NCF, KSC, KT + 1>(P, src, present, exact, words, h, c, fb);
  }
}

// One m-tile (16 head columns x 8 owners, accumulator layout) of a result -> global memory: transposed in registers
// (movmatrix) so that a thread holds two adjacent columns of ONE owner (own_b): 4-byte stores.
template <int KS0, int NCF, int KSC, int KT>
__device__ __forceinline__ void store_tile(const TcPlan& P, __nv_bfloat16* dst, bool present, bool exact, bool words, int h, int c, const float (&v)[4]) {
  const unsigned w0 = movmatrix_trans(pack_bf16(v[0], v[1]));  // (owner own_b; columns 2c, 2c + 1)
  const unsigned w1 = movmatrix_trans(pack_bf16(v[2], v[3]));  // (owner own_b; columns 2c + 8, 2c + 9)
  if (exact) {
    unsigned* w = reinterpret_cast<unsigned*>(dst + exact_block<KS0, NCF, KSC, KT>(P, h)) + c;
    if (present) {
      w[0] = w0;
      w[4] = w1;
    }
    return;
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const unsigned w = r ? w1 : w0;
    int g0, g1;
    flat_pair<KS0, NCF, KSC, KT>(P, h, 2 * c + 8 * r, g0, g1);
    if (!present) continue;
    if (words && g0 >= 0 && g1 == g0 + 1 && (g0 & 1) == 0) {
      *reinterpret_cast<unsigned*>(dst + g0) = w;
    } else {
      if (g0 >= 0) dst[g0] = __ushort_as_bfloat16((unsigned short)(w & 0xffffu));
      if (g1 >= 0) dst[g1] = __ushort_as_bfloat16((unsigned short)(w >> 16));
    }
  }
}

// combine the phase accumulators of every complex m-tile and store all m-tiles of one result
template <int KS0, int NCF, int KSC, bool CONJ, int M = 0>
__device__ __forceinline__ void store_result(const TcPlan& P, __nv_bfloat16* dst, bool present, bool exact, bool words, int h, int g, int c,
                                             const float (&inv)[2],
                                             const float (&acc0)[4], const float (&accr)[NCF * KSC > 0 ? NCF * KSC : 1][4],
                                             const float (&acci)[NCF * KSC > 0 ? NCF * KSC : 1][4]) {
  if constexpr (M == 0 && KS0 > 0) {
    const float v[4] = {acc0[0] * inv[0], acc0[1] * inv[1], acc0[2] * inv[0], acc0[3] * inv[1]};
    store_tile<KS0, NCF, KSC, 0>(P, dst, present, exact, words, h, c, v);
  }
  if constexpr (M < NCF * KSC) {
    // rows of an accumulator m-tile are head columns g, g + 8: even = real part, odd = imaginary part.
    //   tau:      re = r_re - i_im,  im = r_im + i_re;      conj tau:  re = r_re + i_im,  im = r_im - i_re
    const float sgn = ((g & 1) != 0) == CONJ ? -1.f : 1.f;
    float v[4];
#pragma unroll
    for (int x = 0; x < 4; ++x) v[x] = (accr[M][x] + sgn * __shfl_xor_sync(0xffffffffu, acci[M][x], 4)) * inv[x & 1];
    store_tile<KS0, NCF, KSC, KS0 + M>(P, dst, present, exact, words, h, c, v);
    store_result<KS0, NCF, KSC, CONJ, M + 1>(P, dst, present, exact, words, h, g, c, inv, acc0, accr, acci);
  }
}

// A neighbour row of the owner row's walk, prepared once per CTA
struct TnRowPair {
  int cnt, lo, z, lon_base;  // window width, first offset, sample * rows + neighbour row, longitude of position 0 (wrapped)
  int ent_off, pad0, pad1, pad2;
};

template <int KS0, int NCF, int KSC, int MODE, int WARPS>
__global__ void __launch_bounds__(32 * WARPS, WARPS == 4 ? (MODE == TC_BWD_S ? 3 : 4) : 2) lattice_tn_kernel(const __grid_constant__ TcArgs a) {
  constexpr int TL = 8 * WARPS, THREADS = 32 * WARPS;
  constexpr int TN_ADV = tn_advance(TL), TN_ROWS = tn_rows(TL);
  using L = TnLayout<KS0, NCF, KSC, TL>;
  constexpr int KQ = KS0 + NCF * KSC, CH = 2 * KQ, NCK = NCF * KSC > 0 ? NCF * KSC : 1;
  constexpr int NF = NCF > 0 ? NCF : 1;
  constexpr bool FWD = MODE == TC_FWD, PASS_S = MODE == TC_BWD_S;
  extern __shared__ __align__(1024) unsigned char smem_dyn[];
  // swizzled sub-tiles must start on 1024-byte boundaries of the shared-memory window: align by hand (1 KB of slack is requested)
  unsigned char* const smem_raw = smem_dyn + ((1024u - ((unsigned)__cvta_generic_to_shared(smem_dyn) & 1023u)) & 1023u);
  __shared__ __align__(8) unsigned long long copy_bar[2];  // completion of the TMA copies into buffer 0 / 1
  __shared__ __align__(16) TnRowPair pairs_s[TC_MAX_WIN];
  __shared__ int n_pairs_s, failed_s;
  const TcPlan& P = a.plan;
  // two buffers, each: field 1 sub-tiles | field 2 sub-tiles | entries 2 x (TN_ROWS + TL, 4) fp32 | stats (TN_ROWS, 2) fp32 (pass S)
  constexpr int buf_bytes = L::BUFFER_BYTES;
  // a staged table entry (8 floats) is split into two arrays of 4 floats: the 16-byte reads of the phases then sit at a
  // 16-byte pitch (no bank conflicts between neighbouring offsets); the bias is float 2 NCF of the entry
  constexpr int ENT_HALF = 4 * (TN_ROWS + TL);
  constexpr int bias_at = 2 * NCF < 4 ? 2 * NCF : ENT_HALF + 2 * NCF - 4;  // the tables hold exactly the orders 1 .. NCF (host-checked)
  auto tile1 = [&](int buf) { return smem_raw + buf * buf_bytes; };
  auto tile2 = [&](int buf) { return smem_raw + buf * buf_bytes + L::FIELD_BYTES; };
  auto entry = [&](int buf) { return reinterpret_cast<float*>(smem_raw + buf * buf_bytes + 2 * L::FIELD_BYTES); };
  auto stats = [&](int buf) { return reinterpret_cast<float*>(smem_raw + buf * buf_bytes + 2 * L::FIELD_BYTES + L::ENT_BYTES); };

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, c = lane & 3;
  const int tiles = (a.nlon + TL - 1) / TL;
  const int row = a.row_order[blockIdx.x / tiles];
  const int c0 = (blockIdx.x % tiles) * TL;
  const int h = blockIdx.y;
  const int64_t b = blockIdx.z;
  const int64_t node0 = (b * a.rows + row) * (int64_t)a.nlon;
  const int own_b = 8 * warp + g;      // the owner whose column this thread holds in B fragments (and stores in the epilogue)
  const int own_c = 8 * warp + 2 * c;  // the owners (own_c, own_c + 1) of this thread's accumulator columns
  const float cscale = a.scale * TC_LOG2E;
  const bool words = (a.D & 1) == 0;   // 4-byte accesses to (even column, next column) are aligned
  const bool exact = a.exact != 0;
  TnLaneOffsets<KS0, NCF, KSC, TL> lane_off;
  lane_off.init(lane);

  // ---- the walk's row pairs, once per CTA: warp 0 compacts the non-empty ones (one lane per neighbour row)
  if (warp == 0) {
    int filled = 0;
    for (int x0 = 0; x0 < 2 * a.W + 1; x0 += 32) {
      const int x = x0 + lane, j = row + x - a.W;
      int cnt = 0;
      if (x < 2 * a.W + 1 && j >= 0 && j < a.rows) cnt = a.win_cnt[row * (2 * a.W + 1) + x];
      const unsigned have = __ballot_sync(0xffffffffu, cnt > 0);
      if (cnt > 0) {
        const int widx = row * (2 * a.W + 1) + x;
        TnRowPair rp;
        rp.cnt = cnt;
        rp.lo = a.win_lo[widx];
        rp.z = (int)(b * a.rows + j);
        rp.lon_base = tc_wrap(c0 + rp.lo, a.nlon);
        rp.ent_off = a.win_off[widx];
        rp.pad0 = rp.pad1 = rp.pad2 = 0;
        pairs_s[filled + __popc(have & ((1u << lane) - 1u))] = rp;
      }
      filled += __popc(have);
    }
    if (lane == 0) n_pairs_s = filled;
  }
  if (!a.use_tma)  // per-thread staging leaves rows beyond a window and padding columns untouched: they must be finite
    for (int x = threadIdx.x; x < 2 * buf_bytes / 16; x += THREADS) reinterpret_cast<uint4*>(smem_raw)[x] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x == 0) {
    failed_s = 0;
    mbar_init(&copy_bar[0], 1);
    mbar_init(&copy_bar[1], 1);
    fence_mbar_init();
  }

  // owners' fragments (loop-invariant B operands) and their pre-swapped copies:
  //   owners carry q: Im = sum_cols tile[col] * q'[col], q' = (-q_im, q_re);   owners carry k: k' = (k_im, -k_re)
  unsigned f1[KQ][2], s1[NCK][2], f2[FWD ? 1 : KQ][2], s2[FWD ? 1 : NCK][2];
  const bool own_b_present = c0 + own_b < a.nlon;
  const int64_t own_b_base = (node0 + c0 + own_b) * a.D;
  load_owner_columns<KS0, NCF, KSC>(P, a.own1 + own_b_base, own_b_present, exact, words, h, c, f1);
#pragma unroll
  for (int kc = 0; kc < NCF * KSC; ++kc)
#pragma unroll
    for (int r = 0; r < 2; ++r) s1[kc][r] = PASS_S ? swap_neg(f1[KS0 + kc][r]) : swap_neg_lo(f1[KS0 + kc][r]);
  if constexpr (!FWD) {
    load_owner_columns<KS0, NCF, KSC>(P, a.own2 + own_b_base, own_b_present, exact, words, h, c, f2);
#pragma unroll
    for (int kc = 0; kc < NCF * KSC; ++kc)
#pragma unroll
      for (int r = 0; r < 2; ++r) s2[kc][r] = PASS_S ? swap_neg(f2[KS0 + kc][r]) : swap_neg_lo(f2[KS0 + kc][r]);
  }
  float lse_o[2] = {0.f, 0.f}, dl_o[2] = {0.f, 0.f};  // pass T: the two accumulator-column owners' lse (base 2) and Delta
  if constexpr (MODE == TC_BWD_T) {
#pragma unroll
    for (int e = 0; e < 2; ++e)
      if (c0 + own_c + e < a.nlon) lse_o[e] = a.lse[(node0 + c0 + own_c + e) * a.H + h] * TC_LOG2E;
    if (a.delta_out != nullptr) {
      // Delta = <dO, O> over the head's columns of owner own_b: this thread holds 2 of every 8 columns of dO (f2);
      // the same columns of O, then the four lanes of the owner add up.  Written for the source-major pass, and handed
      // to the lanes that hold the owner as an accumulator column.
      unsigned of[KQ][2];
      load_owner_columns<KS0, NCF, KSC>(P, a.out_fwd + own_b_base, own_b_present, exact, words, h, c, of);
      float d = 0.f;
#pragma unroll
      for (int ks = 0; ks < KQ; ++ks)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          d = fmaf(__uint_as_float(f2[ks][r] << 16), __uint_as_float(of[ks][r] << 16), d);
          d = fmaf(__uint_as_float(f2[ks][r] & 0xffff0000u), __uint_as_float(of[ks][r] & 0xffff0000u), d);
        }
      d += __shfl_xor_sync(0xffffffffu, d, 1);
      d += __shfl_xor_sync(0xffffffffu, d, 2);
      if (c == 0 && own_b_present) a.delta_out[(node0 + c0 + own_b) * a.H + h] = d;
#pragma unroll
      for (int e = 0; e < 2; ++e) dl_o[e] = __shfl_sync(0xffffffffu, d, (2 * c + e) << 2);
    } else {
#pragma unroll
      for (int e = 0; e < 2; ++e)
        if (c0 + own_c + e < a.nlon) dl_o[e] = a.delta[(node0 + c0 + own_c + e) * a.H + h];
    }
  }
  float a1_0[4] = {0.f, 0.f, 0.f, 0.f}, a1_r[NCK][4], a1_i[NCK][4];
  float a2_0[4] = {0.f, 0.f, 0.f, 0.f}, a2_r[PASS_S ? NCK : 1][4], a2_i[PASS_S ? NCK : 1][4];
#pragma unroll
  for (int m = 0; m < NCK; ++m)
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      a1_r[m][x] = a1_i[m][x] = 0.f;
      if constexpr (PASS_S) a2_r[m][x] = a2_i[m][x] = 0.f;
    }
  float m_o[2] = {-1e30f, -1e30f}, l_o[2] = {0.f, 0.f};  // forward: reference maximum (base-2 logits), partial sums of the two owners
  __syncthreads();
  const int n_pairs = n_pairs_s;

  // ---- stages = (row pair, chunk of its window), produced in order by a cursor that runs one stage ahead of the consumer
  struct Consumed {   // what the consumer of a stage needs to know about it
    int p0, cnt;      // first position of the chunk, window width
    bool tma;         // staged by tensor copies (completion on the copy barrier)
  };
  int next_pair = 0, next_p0 = 0;  // the producer cursor
  // per-thread slot of the cp.async path: thread -> (row within a pass, 16-byte chunk of the padded head row)
  constexpr int ROWS_PER_PASS = THREADS / CH;
  const int st_row = threadIdx.x / CH, st_ch = threadIdx.x - st_row * CH;
  const bool st_active = st_row < ROWS_PER_PASS;
  auto issue_next = [&](int buf) -> Consumed {  // asynchronous copies of the cursor's stage into buffer `buf`; advances the cursor
    const int4 ra = *reinterpret_cast<const int4*>(&pairs_s[next_pair]);  // cnt, lo, z, lon_base
    const int ent_off = pairs_s[next_pair].ent_off;
    const int cnt = ra.x, z = ra.z, p0 = next_p0;
    const int n_rows = min(TN_ROWS, TL + cnt - 1 - p0);
    int lon0 = ra.w + p0;
    if (lon0 >= a.nlon) lon0 %= a.nlon;
    const bool tma = a.use_tma && lon0 + n_rows <= a.nlon;  // consecutive longitudes: no wrap at the seam
    if (p0 + TN_ADV < TL + cnt - 1) {
      next_p0 = p0 + TN_ADV;
    } else {
      ++next_pair;
      next_p0 = 0;
    }
    unsigned char* d1 = tile1(buf);
    unsigned char* d2 = tile2(buf);
    if (tma) {
      if (threadIdx.x == 0) {
        // the buffer was last touched through the generic proxy (ldmatrix, per-thread stores): order those first
        fence_proxy_async();
        mbar_expect_tx(&copy_bar[buf], 2u * TN_ROWS * (KS0 * L::REAL_PITCH + NCF * L::CX_PITCH));
        if constexpr (KS0 > 0) {
          tma_load_3d(d1, &a.maps[0][0], &copy_bar[buf], P.real_off + h * 16, lon0, z);
          tma_load_3d(d2, &a.maps[1][0], &copy_bar[buf], P.real_off + h * 16, lon0, z);
        }
#pragma unroll
        for (int f = 0; f < NCF; ++f) {
          tma_load_3d(d1 + L::REAL_BYTES + f * L::CX_BYTES, &a.maps[0][1], &copy_bar[buf], P.cf_off[f] + h * 16 * KSC, lon0, z);
          tma_load_3d(d2 + L::REAL_BYTES + f * L::CX_BYTES, &a.maps[1][1], &copy_bar[buf], P.cf_off[f] + h * 16 * KSC, lon0, z);
        }
      }
    } else if (st_active) {
      const int st_g0 = flat_column<KS0, NCF, KSC>(P, h, 8 * st_ch), st_g7 = flat_column<KS0, NCF, KSC>(P, h, 8 * st_ch + 7);
      const bool whole = st_g0 >= 0 && st_g7 == st_g0 + 7 && (a.D % 8 == 0) && (st_g0 % 8 == 0) && a.aligned16;  // one aligned 16-byte chunk of real columns
      const bool pad = st_g0 < 0 && st_g7 < 0 && flat_column<KS0, NCF, KSC>(P, h, 8 * st_ch + 3) < 0;  // all padding (stays zero)
      if (!pad) {
        // this thread's chunk of every row: block base + row * pitch + 16 (chunk ^ swizzle(row))
        const bool in_real = st_ch < 2 * KS0;
        const int cc = st_ch - 2 * KS0;
        const int blk = in_real ? 0 : L::REAL_BYTES + (cc / (2 * KSC)) * L::CX_BYTES, cb = in_real ? st_ch : cc % (2 * KSC);
        const int pitch = in_real ? L::REAL_PITCH : L::CX_PITCH;
        const bool wide = !in_real && KSC == 2;  // 64-byte rows
        const __nv_bfloat16* src1 = a.nb1 + (int64_t)z * a.nlon * a.D + st_g0;
        const __nv_bfloat16* src2 = a.nb2 + (int64_t)z * a.nlon * a.D + st_g0;
        int lon = lon0 + st_row;
        if (lon >= a.nlon) lon %= a.nlon;
        const int step = ROWS_PER_PASS % a.nlon;
        // with tensor maps in use the buffer may hold anything beyond the window: write zeros there (copies of size 0)
        const int rows_to_write = a.use_tma ? TN_ROWS : n_rows;
        for (int pl = st_row; pl < rows_to_write; pl += ROWS_PER_PASS) {
          const int off = blk + pl * pitch + 16 * (cb ^ (wide ? (pl >> 1) & 3 : (pl >> 2) & 1));
          const int64_t nb = (int64_t)lon * a.D;
          if (whole) {
            const int bytes = pl < n_rows ? 16 : 0;
            cp_async16(d1 + off, src1 + nb, bytes);
            cp_async16(d2 + off, src2 + nb, bytes);
          } else {  // a chunk that straddles padding or is misaligned: element by element (visible after the barrier)
            unsigned short u1[8], u2[8];
#pragma unroll
            for (int x = 0; x < 8; ++x) {
              const int gx = pl < n_rows ? flat_column<KS0, NCF, KSC>(P, h, 8 * st_ch + x) : -1;
              u1[x] = gx >= 0 ? __bfloat16_as_ushort(src1[nb + gx - st_g0]) : (unsigned short)0;
              u2[x] = gx >= 0 ? __bfloat16_as_ushort(src2[nb + gx - st_g0]) : (unsigned short)0;
            }
            *reinterpret_cast<uint4*>(d1 + off) =
                make_uint4(u1[0] | (u1[1] << 16), u1[2] | (u1[3] << 16), u1[4] | (u1[5] << 16), u1[6] | (u1[7] << 16));
            *reinterpret_cast<uint4*>(d2 + off) =
                make_uint4(u2[0] | (u2[1] << 16), u2[2] | (u2[3] << 16), u2[4] | (u2[5] << 16), u2[6] | (u2[7] << 16));
          }
          lon += step;
          if (lon >= a.nlon) lon -= a.nlon;
        }
      }
    }
    // table entries of the offsets x = p - owner the chunk can meet (clamped: validity is decided from x itself)
    float* de = entry(buf);
    const float* ent = a.entries + (size_t)ent_off * 8;
    static_assert(2 * (TN_ROWS + TL - 1) <= 2 * THREADS, "two guarded copies per thread cover a chunk's entries");
#pragma unroll
    for (int it = 0; it < 2; ++it) {
      const int idx = threadIdx.x + it * THREADS;
      if (idx < 2 * (n_rows + TL - 1)) {
        const int xi = idx >> 1, part = idx & 1;
        const int x = min(max(xi + p0 - (TL - 1), 0), cnt - 1);
        cp_async16(de + 4 * xi + part * ENT_HALF, ent + 8 * x + 4 * part, 16);  // the two halves of an entry go to separate arrays
      }
    }
    if constexpr (PASS_S) {
      float* ds = stats(buf);
      for (int idx = threadIdx.x; idx < 2 * n_rows; idx += THREADS) {
        const int pl = idx >> 1, which = idx & 1;
        int lon = lon0 + pl;
        if (lon >= a.nlon) lon %= a.nlon;
        const int64_t nn = ((int64_t)z * a.nlon + lon) * a.H + h;
        cp_async4(ds + 2 * pl + which, (which ? a.delta : a.lse) + nn, 4);
      }
    }
    cp_async_commit();
    return Consumed{p0, cnt, tma};
  };

  bool have = n_pairs > 0;
  int buf = 0;
  unsigned parity = 0;  // bit b: the phase of copy_bar[b] the next TMA stage into buffer b completes
  Consumed cur{0, 0, false};
  if (have) cur = issue_next(0);
  while (have) {
    const bool have_next = next_pair < n_pairs;
    Consumed nxt{0, 0, false};
    if (have_next) {
      nxt = issue_next(buf ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    if (cur.tma) {  // one warp watches the copy barrier; the others block in the CTA barrier below without issuing
      if (warp == 0 && !mbar_wait(&copy_bar[buf], (parity >> buf) & 1u)) failed_s = 1;
      parity ^= 1u << buf;
    }
    __syncthreads();
    const unsigned t1 = (unsigned)__cvta_generic_to_shared(tile1(buf));
    const unsigned t2 = (unsigned)__cvta_generic_to_shared(tile2(buf));
    const float* e_s = entry(buf);
    const float* stat_s = stats(buf);
    const int p0 = cur.p0, cnt = cur.cnt;

    // ---- this warp's steps inside the chunk: 16 positions each, on the lattice 8 warp + 16 i
    const int p_first = p0 > 8 * warp ? p0 + ((8 * warp) & 8) : 8 * warp;
    const int p_end = min(p0 + TN_ADV, 8 * warp + 7 + cnt);
    for (int p = p_first; p < p_end; p += 16) {
      const int pl = p - p0;
      // element x of a fragment: position pl + g + 8 (x >> 1), owner own_c + (x & 1)
      float lg[4], tr[NF][4], ti[NF][4];
      bool valid[4];
      const float* e_lane = e_s + 4 * (pl + g - own_c + (TL - 1));  // staged entry (first half) of the offset p - owner, element 0
      const int off0 = p0 + pl + g - own_c;
      {
        float s0[4], sr[NF][4], si[NF][4];
        gram_step<KS0, NCF, KSC, TL>(f1, s1, t1, pl, lane_off, s0, sr, si);
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const float* e = e_lane + 4 * (8 * (x >> 1) - (x & 1));
          valid[x] = (unsigned)(off0 + 8 * (x >> 1) - (x & 1)) < (unsigned)cnt;
          float sum = s0[x];
          float tau[2 * NF];
          if constexpr (NCF >= 2) {  // complex frequencies are the orders 1 .. NCF: the first two phases are the entry's first 16 bytes
            const float4 t = *reinterpret_cast<const float4*>(e);
            tau[0] = t.x; tau[1] = t.y; tau[2] = t.z; tau[3] = t.w;
            if constexpr (NCF == 3) {
              const float2 t3 = *reinterpret_cast<const float2*>(e + ENT_HALF);
              tau[4] = t3.x; tau[5] = t3.y;
            }
          } else if constexpr (NCF == 1) {
            const float2 t = *reinterpret_cast<const float2*>(e);
            tau[0] = t.x; tau[1] = t.y;
          }
#pragma unroll
          for (int f = 0; f < NCF; ++f) {
            tr[f][x] = tau[2 * f];
            ti[f][x] = tau[2 * f + 1];
            sum = fmaf(tau[2 * f], sr[f][x], sum);
            sum = fmaf(-tau[2 * f + 1], si[f][x], sum);
          }
          lg[x] = valid[x] ? fmaf(cscale, sum, TC_LOG2E * e[bias_at]) : -INFINITY;  // -inf: outside the window
        }
      }
      float w1[4], w2[4];  // the weights the two accumulations use: forward p | pass T ds | pass S ds, p
      if constexpr (FWD) {
        // online softmax over the 16 positions: column maxima over this thread's rows, then across the 8 row groups.
        // The reference maximum of an owner only moves when the new maximum exceeds it by more than 2^8 (weights stay
        // below 256: exact in the normalised result), so most steps skip the rescaling of the accumulators.
        // whether some owner's maximum has to move can be told from each thread's own four logits: most steps skip the
        // column maxima (six shuffles) as well as the rescaling
        const bool grow = fmaxf(lg[0], lg[2]) > m_o[0] + 8.f || fmaxf(lg[1], lg[3]) > m_o[1] + 8.f;
        if (__any_sync(0xffffffffu, grow)) {
          float mx[2] = {fmaxf(lg[0], lg[2]), fmaxf(lg[1], lg[3])};
#pragma unroll
          for (int d = 4; d < 32; d <<= 1) {
            mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xffffffffu, mx[0], d));
            mx[1] = fmaxf(mx[1], __shfl_xor_sync(0xffffffffu, mx[1], d));
          }
          const float nm[2] = {mx[0] > m_o[0] + 8.f ? mx[0] : m_o[0], mx[1] > m_o[1] + 8.f ? mx[1] : m_o[1]};
          const float corr[2] = {fast_exp2(m_o[0] - nm[0]), fast_exp2(m_o[1] - nm[1])};
          m_o[0] = nm[0]; m_o[1] = nm[1];
          l_o[0] *= corr[0]; l_o[1] *= corr[1];
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            a1_0[x] *= corr[x & 1];
#pragma unroll
            for (int m = 0; m < NCF * KSC; ++m) { a1_r[m][x] *= corr[x & 1]; a1_i[m][x] *= corr[x & 1]; }
          }
        }
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          w1[x] = fast_exp2(lg[x] - m_o[x & 1]);
          l_o[x & 1] += w1[x];
        }
      } else {
        // p from the logits first (the (q, k) Gram blocks die here), then d alpha from the (dO, v) Gram blocks
        float delta[4];
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          float lse;
          if (PASS_S) {
            const float2 st = *reinterpret_cast<const float2*>(stat_s + 2 * (pl + g + 8 * (x >> 1)));
            lse = st.x * TC_LOG2E; delta[x] = st.y;
          } else {
            lse = lse_o[x & 1]; delta[x] = dl_o[x & 1];
          }
          w2[x] = valid[x] ? fast_exp2(lg[x] - lse) : 0.f;
        }
        float h0[4], hr[NF][4], hi[NF][4];
        gram_step<KS0, NCF, KSC, TL>(f2, s2, t2, pl, lane_off, h0, hr, hi);
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          float dal = h0[x];
#pragma unroll
          for (int f = 0; f < NCF; ++f) {
            dal = fmaf(tr[f][x], hr[f][x], dal);
            dal = fmaf(-ti[f][x], hi[f][x], dal);
          }
          w1[x] = a.scale * w2[x] * (dal - delta[x]);
        }
      }
      // B operands: the weights (x phase parts), transposed to (owner column, position rows)
      unsigned x0[2], xr[NF][2], xim[NF][2];
      x0[0] = movmatrix_trans(pack_bf16(w1[0], w1[1]));
      x0[1] = movmatrix_trans(pack_bf16(w1[2], w1[3]));
#pragma unroll
      for (int f = 0; f < NCF; ++f) {
        xr[f][0] = movmatrix_trans(pack_bf16(w1[0] * tr[f][0], w1[1] * tr[f][1]));
        xr[f][1] = movmatrix_trans(pack_bf16(w1[2] * tr[f][2], w1[3] * tr[f][3]));
        xim[f][0] = movmatrix_trans(pack_bf16(w1[0] * ti[f][0], w1[1] * ti[f][1]));
        xim[f][1] = movmatrix_trans(pack_bf16(w1[2] * ti[f][2], w1[3] * ti[f][3]));
      }
      if constexpr (FWD) {
        accumulate_step<KS0, NCF, KSC, TL>(a1_0, a1_r, a1_i, x0, xr, xim, t2, pl, lane_off);  // out += (p tau) v
      } else {
        accumulate_step<KS0, NCF, KSC, TL>(a1_0, a1_r, a1_i, x0, xr, xim, t1, pl, lane_off);  // dq += (ds tau) k  |  dk += (ds conj tau) q
        if constexpr (PASS_S) {
          x0[0] = movmatrix_trans(pack_bf16(w2[0], w2[1]));
          x0[1] = movmatrix_trans(pack_bf16(w2[2], w2[3]));
#pragma unroll
          for (int f = 0; f < NCF; ++f) {
            xr[f][0] = movmatrix_trans(pack_bf16(w2[0] * tr[f][0], w2[1] * tr[f][1]));
            xr[f][1] = movmatrix_trans(pack_bf16(w2[2] * tr[f][2], w2[3] * tr[f][3]));
            xim[f][0] = movmatrix_trans(pack_bf16(w2[0] * ti[f][0], w2[1] * ti[f][1]));
            xim[f][1] = movmatrix_trans(pack_bf16(w2[2] * ti[f][2], w2[3] * ti[f][3]));
          }
          accumulate_step<KS0, NCF, KSC, TL>(a2_0, a2_r, a2_i, x0, xr, xim, t2, pl, lane_off);  // dv += (p conj tau) dO
        }
      }
    }
    __syncthreads();  // everyone is done with `buf` before the stage after next is copied into it
    cur = nxt;
    have = have_next;
    buf ^= 1;
  }

  // ---- epilogue: normalise, combine the two phase accumulators (multiplication by +-i = pair swap across rows g, g ^ 1),
  // transpose in registers, store
  float inv[2] = {1.f, 1.f};
  if constexpr (FWD) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
#pragma unroll
      for (int d = 4; d < 32; d <<= 1) l_o[e] += __shfl_xor_sync(0xffffffffu, l_o[e], d);
      inv[e] = l_o[e] > 0.f ? 1.f / l_o[e] : 0.f;
      if (g == 0 && c0 + own_c + e < a.nlon)
        a.lse_out[(node0 + c0 + own_c + e) * a.H + h] = l_o[e] > 0.f ? (m_o[e] + log2f(l_o[e])) * TC_LN2 : -INFINITY;
    }
  }
  // a wait that ran out anywhere in this CTA poisons its results (NaN) instead of passing half-filled tiles on as numbers
  if (*(volatile int*)&failed_s != 0) inv[0] = inv[1] = __int_as_float(0x7fc00000);
  store_result<KS0, NCF, KSC, PASS_S>(P, a.res1 + own_b_base, own_b_present, exact, words, h, g, c, inv, a1_0, a1_r, a1_i);
  if constexpr (PASS_S) store_result<KS0, NCF, KSC, true>(P, a.res2 + own_b_base, own_b_present, exact, words, h, g, c, inv, a2_0, a2_r, a2_i);
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

// Same, one warp per node with 16-byte loads: every 8-column chunk of the row belongs to one head (host-checked).
__global__ void tc_delta_vec_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ out, float* __restrict__ delta,
                                    int64_t n_nodes, int D, int H, TcPlan P) {
  const int lane = threadIdx.x & 31;
  const int64_t node = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (node >= n_nodes) return;
  float part[2] = {0.f, 0.f};
  int head[2] = {-1, -1};
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int col = 8 * (lane + 32 * r);
    if (col >= D) continue;
    if (P.a0 > 0 && col >= P.real_off && col < P.real_off + H * P.a0) head[r] = (col - P.real_off) / P.a0;
    for (int f = 0; f < P.n_cf; ++f)
      if (col >= P.cf_off[f] && col < P.cf_off[f] + 2 * H * P.ac) head[r] = (col - P.cf_off[f]) / (2 * P.ac);
    if (head[r] < 0) continue;
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(dout + node * D + col));
    const uint4 b = __ldg(reinterpret_cast<const uint4*>(out + node * D + col));
    const unsigned wa[4] = {a.x, a.y, a.z, a.w}, wb[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int x = 0; x < 4; ++x)
      part[r] += __uint_as_float(wa[x] << 16) * __uint_as_float(wb[x] << 16) + __uint_as_float(wa[x] & 0xffff0000u) * __uint_as_float(wb[x] & 0xffff0000u);
  }
  for (int h = 0; h < H; ++h) {
    const float v = warp_sum((head[0] == h ? part[0] : 0.f) + (head[1] == h ? part[1] : 0.f));
    if (lane == 0) delta[node * H + h] = v;
  }
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

// GM_LATTICE_TMA=0 stages every chunk with per-thread copies (for comparing the two staging paths)
bool tma_disabled() {
  const char* v = getenv("GM_LATTICE_TMA");
  return v && v[0] == '0';
}

// cuTensorMapEncodeTiled through the runtime's driver entry point lookup (no link against the driver library)
PFN_cuTensorMapEncodeTiled_v12000 tensor_map_encoder() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult res;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &res) != cudaSuccess || res != cudaDriverEntryPointSuccess)
      sym = nullptr;
    return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(sym);
  }();
  return fn;
}

// Tensor map over one bf16 field seen as (D columns, nlon longitudes, batch * rows): boxes of `box_cols` columns x `box_rows`
// (box_rows) longitudes of one lattice row, written to shared memory in the swizzle that spans the box's rows.
bool encode_field_map(CUtensorMap* map, const void* field, int D, int nlon, int64_t slabs, int box_cols, int box_rows) {
  auto encode = tensor_map_encoder();
  if (!encode) return false;
  const cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)nlon, (cuuint64_t)slabs};
  const cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)nlon * D * 2};
  const cuuint32_t box[3] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapSwizzle swz = box_cols == 16 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_64B;
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(field), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int KS0, int NCF, int KSC, int MODE>
int launch_tn(TcArgs& a, int n_order_rows, int64_t batch, cudaStream_t stream) {
  constexpr int WARPS = TN_WARPS(MODE), TL = 8 * WARPS, TN_ROWS = tn_rows(TL);
  using L = TnLayout<KS0, NCF, KSC, TL>;
  a.aligned16 = reinterpret_cast<uintptr_t>(a.nb1) % 16 == 0 && reinterpret_cast<uintptr_t>(a.nb2) % 16 == 0;
  bool tma = !tma_disabled() && a.D % 8 == 0 && a.nlon >= TN_ROWS && batch * a.rows < (1ll << 31) && (KS0 == 0 || (a.plan.a0 == 16 && a.plan.real_off % 8 == 0)) &&
             2 * a.plan.ac == 16 * KSC && reinterpret_cast<uintptr_t>(a.nb1) % 16 == 0 && reinterpret_cast<uintptr_t>(a.nb2) % 16 == 0;
  for (int f = 0; f < a.plan.n_cf; ++f) tma = tma && a.plan.cf_off[f] % 8 == 0;
  if (tma) {
    const void* fields[2] = {a.nb1, a.nb2};
    for (int x = 0; x < 2 && tma; ++x) {
      if (KS0 > 0) tma = tma && encode_field_map(&a.maps[x][0], fields[x], a.D, a.nlon, batch * a.rows, 16, TN_ROWS);
      tma = tma && encode_field_map(&a.maps[x][1], fields[x], a.D, a.nlon, batch * a.rows, 16 * KSC, TN_ROWS);
    }
  }
  a.use_tma = tma ? 1 : 0;
  bool exact = (KS0 == 0 || a.plan.a0 == 16) && 2 * a.plan.ac == 16 * KSC && a.D % 2 == 0 && (KS0 == 0 || a.plan.real_off % 2 == 0);
  for (int f = 0; f < a.plan.n_cf; ++f) exact = exact && a.plan.cf_off[f] % 2 == 0;
  const void* ptrs[6] = {a.own1, a.own2, a.nb1, a.nb2, a.res1, a.res2};
  for (const void* q : ptrs) exact = exact && reinterpret_cast<uintptr_t>(q) % 4 == 0;
  a.exact = exact ? 1 : 0;
  const size_t smem = 2 * (size_t)L::BUFFER_BYTES + 1024;
  auto kernel = lattice_tn_kernel<KS0, NCF, KSC, MODE, WARPS>;
  int st = allow_smem(kernel, smem, "gm_lattice_attention (tensor cores)");
  if (st != GM_OK) return st;
  const int tiles = (a.nlon + TL - 1) / TL;
  dim3 grid((unsigned)(n_order_rows * tiles), (unsigned)a.H, (unsigned)batch);
  kernel<<<grid, 32 * WARPS, smem, stream>>>(a);
  return launch_status("gm_lattice_attention (tensor cores)");
}

template <int MODE>
int dispatch_tc(TcArgs& a, int n_order_rows, int64_t batch, cudaStream_t cs) {
  const int ks0 = a.plan.a0 > 0 ? 1 : 0, ksc = a.plan.ac > 8 ? 2 : 1, ncf = a.plan.n_cf;
  for (int f = 0; f < ncf; ++f)
    GM_REQUIRE(a.plan.cf_order[f] == f + 1, GM_ERR_UNSUPPORTED, "gm_lattice_attention (tensor cores): complex frequencies must be the orders 1 .. %d", ncf);
  GM_REQUIRE(a.NORD == ncf, GM_ERR_UNSUPPORTED, "gm_lattice_attention (tensor cores): the tables must hold exactly the orders 1 .. %d (they hold %d)", ncf, a.NORD);
  if (ks0 == 1 && ncf == 2 && ksc == 2) return launch_tn<1, 2, 2, MODE>(a, n_order_rows, batch, cs);
  if (ks0 == 1 && ncf == 2 && ksc == 1) return launch_tn<1, 2, 1, MODE>(a, n_order_rows, batch, cs);
  if (ks0 == 1 && ncf == 3 && ksc == 1) return launch_tn<1, 3, 1, MODE>(a, n_order_rows, batch, cs);
  if (ks0 == 1 && ncf == 1 && ksc == 2) return launch_tn<1, 1, 2, MODE>(a, n_order_rows, batch, cs);
  if (ks0 == 1 && ncf == 1 && ksc == 1) return launch_tn<1, 1, 1, MODE>(a, n_order_rows, batch, cs);
  if (ks0 == 0 && ncf == 2 && ksc == 1) return launch_tn<0, 2, 1, MODE>(a, n_order_rows, batch, cs);
  return fail(GM_ERR_UNSUPPORTED, "gm_lattice_attention (tensor cores): no kernel for this head layout (a0=%d, %d x %d complex)",
              a.plan.a0, ncf, a.plan.ac);
}

int fill_tc_args(TcArgs& a, const int64_t* desc_host, int F, int rows, int nlon, int64_t batch, int D, int H, int W, int ES, int NORD,
                 double scale) {
  GM_REQUIRE(rows >= 1 && nlon >= 1 && batch >= 1 && D >= 1 && H >= 1 && H <= 65535 && batch <= 65535, GM_ERR_ARGUMENT,
             "gm_lattice_attention (tensor cores): bad sizes");
  GM_REQUIRE(W >= 0 && NORD >= 0, GM_ERR_ARGUMENT, "gm_lattice_attention (tensor cores): bad table sizes");
  GM_REQUIRE(2 * W + 1 <= TC_MAX_WIN, GM_ERR_UNSUPPORTED, "gm_lattice_attention (tensor cores): neighbourhoods span more than %d lattice rows", TC_MAX_WIN);
  GM_REQUIRE(ES == 8 && 2 * NORD + 1 <= 8, GM_ERR_UNSUPPORTED, "gm_lattice_attention (tensor cores): entries must be 8 floats wide (orders <= 3)");
  GM_REQUIRE(desc_host, GM_ERR_ARGUMENT, "gm_lattice_attention (tensor cores): null descriptor");
  int status = make_tc_plan(desc_host, F, H, D, a.plan);
  if (status != GM_OK) return status;
  for (int f = 0; f < a.plan.n_cf; ++f)
    GM_REQUIRE(a.plan.cf_order[f] <= NORD, GM_ERR_ARGUMENT, "gm_lattice_attention (tensor cores): tables hold %d orders", NORD);
  a.rows = rows; a.nlon = nlon; a.D = D; a.H = H; a.W = W; a.NORD = NORD; a.scale = (float)scale;
  return GM_OK;
}

}  // namespace
}  // namespace gmb

using namespace gmb;

extern "C" int gm_lattice_attention_forward_tc(const void* q, const void* k, const void* v, const int* win_cnt, const int* win_lo,
                                               const int* win_off, const float* entries, const int* row_order, int n_order_rows,
                                               const int64_t* desc_host, int F, int rows, int nlon, int64_t batch, int D, int H, int W,
                                               int ES, int NORD, double scale, void* out, float* lse, void* stream) {
  using B = __nv_bfloat16;
  TcArgs a{};
  int status = fill_tc_args(a, desc_host, F, rows, nlon, batch, D, H, W, ES, NORD, scale);
  if (status != GM_OK) return status;
  GM_REQUIRE(q && k && v && win_cnt && win_lo && win_off && entries && row_order && out && lse, GM_ERR_ARGUMENT,
             "gm_lattice_attention_forward_tc: null pointer");
  if (n_order_rows == 0) return GM_OK;
  a.own1 = (const B*)q; a.nb1 = (const B*)k; a.nb2 = (const B*)v; a.res1 = (B*)out; a.lse_out = lse;
  a.win_cnt = win_cnt; a.win_lo = win_lo; a.win_off = win_off; a.entries = entries; a.row_order = row_order;
  return dispatch_tc<TC_FWD>(a, n_order_rows, batch, (cudaStream_t)stream);
}

extern "C" int gm_lattice_attention_backward_tc_passes(const void* dout, const void* q, const void* k, const void* v, const void* out,
                                                       const float* lse, const int* win_cnt, const int* win_lo, const int* win_off,
                                                       const float* entries, const int* row_order, int n_order_rows,
                                                       const int* t_win_cnt, const int* t_win_lo, const int* t_win_off,
                                                       const float* t_entries, const int* t_row_order, int t_n_order_rows,
                                                       const int64_t* desc_host, int F, int rows, int nlon, int64_t batch, int D, int H,
                                                       int W, int ES, int NORD, double scale, void* dq, void* dk, void* dv, float* delta,
                                                       int passes, void* stream);

extern "C" int gm_lattice_attention_backward_tc(const void* dout, const void* q, const void* k, const void* v, const void* out,
                                                const float* lse, const int* win_cnt, const int* win_lo, const int* win_off,
                                                const float* entries, const int* row_order, int n_order_rows, const int* t_win_cnt,
                                                const int* t_win_lo, const int* t_win_off, const float* t_entries,
                                                const int* t_row_order, int t_n_order_rows, const int64_t* desc_host, int F, int rows,
                                                int nlon, int64_t batch, int D, int H, int W, int ES, int NORD, double scale, void* dq,
                                                void* dk, void* dv, float* delta, void* stream) {
  return gm_lattice_attention_backward_tc_passes(dout, q, k, v, out, lse, win_cnt, win_lo, win_off, entries, row_order, n_order_rows,
                                                 t_win_cnt, t_win_lo, t_win_off, t_entries, t_row_order, t_n_order_rows, desc_host, F, rows,
                                                 nlon, batch, D, H, W, ES, NORD, scale, dq, dk, dv, delta, 7, stream);
}

// passes: bit 0 = Delta, bit 1 = the target-major pass (dq), bit 2 = the source-major pass (dk, dv).  Running a
// subset is for timing the passes separately.  Bits 0 and 1 together: pass T forms Delta itself; without bit 0 the
// passes read the Delta an earlier call left in `delta`.
extern "C" int gm_lattice_attention_backward_tc_passes(const void* dout, const void* q, const void* k, const void* v, const void* out,
                                                       const float* lse, const int* win_cnt, const int* win_lo, const int* win_off,
                                                       const float* entries, const int* row_order, int n_order_rows,
                                                       const int* t_win_cnt, const int* t_win_lo, const int* t_win_off,
                                                       const float* t_entries, const int* t_row_order, int t_n_order_rows,
                                                       const int64_t* desc_host, int F, int rows, int nlon, int64_t batch, int D, int H,
                                                       int W, int ES, int NORD, double scale, void* dq, void* dk, void* dv, float* delta,
                                                       int passes, void* stream) {
  using B = __nv_bfloat16;
  cudaStream_t cs = (cudaStream_t)stream;
  TcArgs a{};
  int status = fill_tc_args(a, desc_host, F, rows, nlon, batch, D, H, W, ES, NORD, scale);
  if (status != GM_OK) return status;
  GM_REQUIRE(dout && q && k && v && out && lse && win_cnt && win_lo && win_off && entries && row_order && t_win_cnt && t_win_lo &&
                 t_win_off && t_entries && t_row_order && dq && dk && dv && delta,
             GM_ERR_ARGUMENT, "gm_lattice_attention_backward_tc: null pointer");
  const int64_t n_nodes = batch * rows * (int64_t)nlon;
  bool chunked = D % 8 == 0 && D <= 512 && a.plan.a0 % 8 == 0 && (2 * a.plan.ac) % 8 == 0 && a.plan.real_off % 8 == 0 &&
                 reinterpret_cast<uintptr_t>(dout) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0;
  for (int f = 0; f < a.plan.n_cf; ++f) chunked = chunked && a.plan.cf_off[f] % 8 == 0;
  // Delta = <dO, O>: formed inside the target-major pass when that pass runs in this call; by its own kernel otherwise
  const bool fused_delta = (passes & 2) != 0 && n_order_rows > 0;
  if (!(passes & 1) || fused_delta) {
  } else if (chunked)
    tc_delta_vec_kernel<<<(unsigned)((n_nodes + 7) / 8), 256, 0, cs>>>((const B*)dout, (const B*)out, delta, n_nodes, D, H, a.plan);
  else
    tc_delta_kernel<<<(unsigned)((n_nodes * H + 7) / 8), 256, 0, cs>>>((const B*)dout, (const B*)out, delta, n_nodes, D, H, a.plan);
  status = launch_status("gm_lattice_attention_backward_tc (delta)");
  if (status != GM_OK) return status;
  a.lse = lse; a.delta = delta;
  if (n_order_rows > 0 && (passes & 2)) {
    a.own1 = (const B*)q; a.own2 = (const B*)dout; a.nb1 = (const B*)k; a.nb2 = (const B*)v; a.res1 = (B*)dq; a.res2 = nullptr;
    a.out_fwd = (const B*)out; a.delta_out = (passes & 1) ? delta : nullptr;
    a.win_cnt = win_cnt; a.win_lo = win_lo; a.win_off = win_off; a.entries = entries; a.row_order = row_order;
    status = dispatch_tc<TC_BWD_T>(a, n_order_rows, batch, cs);
    if (status != GM_OK) return status;
  }
  if (t_n_order_rows > 0 && (passes & 4)) {
    a.own1 = (const B*)k; a.own2 = (const B*)v; a.nb1 = (const B*)q; a.nb2 = (const B*)dout; a.res1 = (B*)dk; a.res2 = (B*)dv;
    a.out_fwd = nullptr; a.delta_out = nullptr;
    a.win_cnt = t_win_cnt; a.win_lo = t_win_lo; a.win_off = t_win_off; a.entries = t_entries; a.row_order = t_row_order;
    status = dispatch_tc<TC_BWD_S>(a, t_n_order_rows, batch, cs);
  }
  return status;
}

extern "C" int gm_lattice_attention_tc_wait_expired(int* expired) {
  GM_REQUIRE(expired, GM_ERR_ARGUMENT, "gm_lattice_attention_tc_wait_expired: null pointer");
  GM_CUDA(cudaMemcpyFromSymbol(expired, g_tc_wait_expired, sizeof(int)));
  return GM_OK;
}
