// Tensor-core lattice kernels, all four heads of a tile in one CTA (bf16 node fields, head layout 16 scalar + 16 complex
// copies per frequency and head: the benchmark's 4 x 16 x (m = 0, 1, 2) and its one- and three-frequency siblings).
//
// Same arithmetic as fused_attention_lattice_tc.cu (per-frequency Gram blocks of 16 staged positions x 8 owners on
// mma.sync m16n8k16, phases / bias / window elementwise on the tile, value sums with the weights as an operand).  What
// changes is how the neighbour rows reach shared memory, because that is what bounds the per-head kernels: measured on a
// B200, a tensor copy whose rows are the 32 / 64 bytes ONE head owns of a node's 640-byte row costs the copy engine as
// much per row as a 128-byte one, and the per-head kernels spend their time waiting for those rows.  Here a CTA works on
// the same owners for all four heads, so that
//   * a neighbour row is copied as five boxes of 128-byte rows (the four heads' scalar blocks side by side; per complex
//     frequency heads 0-1 and heads 2-3), 2.4 x fewer rows per head than three boxes per head;
//   * the staged tiles use the 128-byte shared-memory swizzle, still conflict-free for ldmatrix.
// One CTA per SM, persistent: 4 G consumer warps (warp = head x group of 8 owners; G = 3: 24 owners per item) and one
// warpgroup of four producer warps that hands most of its registers to the consumers (setmaxnreg).  The producers walk
// the CTA's items (owner tile of a lattice row, sample) and their stages (neighbour row, chunk of 32 positions) without
// pause and keep a ring of three stage buffers filled; a stage's ten tensor copies and the bulk copy of its table
// entries are spread over the four producer warps (an issuing thread waits for the copy engine to take each copy; four
// wait side by side).  The owners' own rows of the next item are copied into a small tile of their own while the current
// item is still being computed, so a consumer warp crosses an item boundary with a few shared-memory loads.  No CTA-wide
// barrier runs after the first: full / empty mbarriers per stage and per owner tile, every wait bounded.
//
// Chunks that cross the longitude seam are staged by the producer lanes with cp.async (tensor copies cannot wrap).
// The entry table is the padded one of the producer / consumer design: 12 (orders <= 2) or 20 words per offset,
//   [0..3] fp32 cos, sin of orders 1, 2   [4..7] the same as bf16 pairs (entry x | entry x - 1)   [8] bias * log2(e)
//   order 3: [9..10] cos, sin   [12..13] bf16 pairs,
// with 8 entries of padding before and 24 after every row pair's run whose bias is -inf: pairs outside an owner's window
// need no test, their logit is -inf.
#include <cuda.h>
#include <cudaTypedefs.h>

#include "common.cuh"

namespace gmb {
namespace {

constexpr float T4_LOG2E = 1.4426950408889634f, T4_LN2 = 0.6931471805599453f;
constexpr unsigned T4_WAIT_LIMIT = 1u << 22;  // polls of a barrier before the kernel gives up on it
constexpr int T4_HEADS = 4, T4_PRODUCERS = 4;
constexpr __host__ __device__ int t4_stages(int ncf) { return ncf == 3 ? 2 : 3; }  // stage buffers in the ring (what fits beside the owners' tile)
constexpr int T4_ADV = 32, T4_ROWS = 40;      // positions a chunk advances by / positions it stages
constexpr int T4_PAD_BEFORE = 8, T4_PAD_AFTER = 24;
constexpr int T4_MAX_NCF = 3;
constexpr __host__ __device__ int t4_entry_words(int ncf) { return ncf == 3 ? 20 : 12; }

// set when a wait on a barrier ran out (never expected; the results of that launch are poisoned with NaN)
__device__ int g_tc4_wait_expired;

struct T4Args {
  const __nv_bfloat16 *own1, *own2;   // owners' fields:     q, -  |  q, dO  |  k, v
  const __nv_bfloat16 *nb1, *nb2;     // neighbours' fields: k, v  |  k, v   |  q, dO
  const float *lse, *delta;           // (nodes, 4), backward
  __nv_bfloat16 *res1, *res2;         // out | dq | dk, dv
  float* lse_out;                     // forward
  const int *win_cnt, *win_lo, *win_off;
  const float* entries;
  const int* row_order;
  int n_order_rows, rows, nlon, D, W, batch, tiles, n_items;
  int real_off, cf_off[T4_MAX_NCF];
  float scale;
  alignas(64) CUtensorMap nb_map[2];   // boxes of 64 columns x T4_ROWS longitudes of one lattice row, 128-byte swizzle
  alignas(64) CUtensorMap own_map[2];  // boxes of 64 columns x (8 G) longitudes
};

enum { T4_FWD = 0, T4_BWD_T = 1, T4_BWD_S = 2 };

// ---- small device helpers
__device__ __forceinline__ void t4_mma(float (&d)[4], const unsigned (&a)[4], const unsigned (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void t4_mma_init(float (&d)[4], const unsigned (&a)[4], const unsigned (&b)[2]) {  // d = a * b
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
               : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]), "f"(0.f));
}
__device__ __forceinline__ unsigned t4_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void t4_bar_init(unsigned long long* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(t4_smem(bar)), "r"(count));
}
__device__ __forceinline__ void t4_bar_expect(unsigned long long* bar, unsigned bytes) {  // one arrival + the bytes it announces
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(t4_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void t4_bar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(t4_smem(bar)) : "memory");
}
// one arrival (counted in the barrier's expected count) once every cp.async this thread issued before has completed
__device__ __forceinline__ void t4_bar_arrive_after_cp_async(unsigned long long* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(t4_smem(bar)) : "memory");
}
__device__ __forceinline__ bool t4_bar_try(unsigned long long* bar, unsigned parity) {
  unsigned done;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(done) : "r"(t4_smem(bar)), "r"(parity) : "memory");
  return done != 0;
}
// bounded wait: gives up after T4_WAIT_LIMIT polls, records it in the device-wide flag and returns false
__device__ __forceinline__ bool t4_bar_wait(unsigned long long* bar, unsigned parity) {
  for (unsigned tries = 0; tries < T4_WAIT_LIMIT; ++tries) {
    if (t4_bar_try(bar, parity)) return true;
    if (tries > 64) __nanosleep(64);
  }
  atomicOr(&g_tc4_wait_expired, 1);
  return false;
}
// tensor copy (no multicast, this GPU's own memory) and untiled bulk copy, completion on the barrier
__device__ __forceinline__ void t4_tma(void* dst, const CUtensorMap* map, unsigned long long* bar, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n"
               ::"r"(t4_smem(dst)), "l"(reinterpret_cast<unsigned long long>(map)), "r"(t4_smem(bar)), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void t4_bulk(void* dst, const void* src, unsigned bytes, unsigned long long* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
               ::"r"(t4_smem(dst)), "l"(reinterpret_cast<unsigned long long>(src)), "r"(bytes), "r"(t4_smem(bar)) : "memory");
}
__device__ __forceinline__ void t4_fence_proxy() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ void t4_cp16(void* dst, const void* src, int src_bytes) {  // src_bytes = 0 writes zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(t4_smem(dst)), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ unsigned t4_swap_neg(unsigned w) { return __byte_perm(w, 0, 0x1032) ^ 0x80000000u; }     // (re, im) -> (im, -re)
__device__ __forceinline__ unsigned t4_swap_neg_lo(unsigned w) { return __byte_perm(w, 0, 0x1032) ^ 0x00008000u; }  // (re, im) -> (-im, re)
__device__ __forceinline__ unsigned t4_pack(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const unsigned*>(&v);
}
__device__ __forceinline__ unsigned t4_mul2(unsigned x, unsigned y) {  // two bf16 products, round to nearest
  unsigned z;
  asm("mul.rn.bf16x2 %0, %1, %2;\n" : "=r"(z) : "r"(x), "r"(y));
  return z;
}
__device__ __forceinline__ unsigned t4_movm(unsigned x) {  // 8 x 8 b16 transpose across the warp
  unsigned y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(y) : "r"(x));
  return y;
}
__device__ __forceinline__ void t4_ldsm(unsigned (&r)[4], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void t4_ldsm_t(unsigned (&r)[4], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ float t4_exp2(float x) {  // ex2.approx: exp2(-inf) = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
// re-split the CTA's register pool between its warpgroups (every warp of a warpgroup executes this)
template <int REGS> __device__ __forceinline__ void t4_more_registers() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;\n" ::"n"(REGS)); }
template <int REGS> __device__ __forceinline__ void t4_fewer_registers() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;\n" ::"n"(REGS)); }
__device__ __forceinline__ int t4_wrap(int x, int n) {
  x %= n;
  return x < 0 ? x + n : x;
}

// Shared memory of a CTA.  A staged field is 2 NCF + 1 sub-tiles of 64 columns (128-byte rows, 128-byte swizzle): per
// complex frequency heads 0-1 and heads 2-3, then the four heads' scalar blocks.  Byte of (row r, 16-byte chunk c) of a
// sub-tile: r * 128 + 16 * (c ^ (r & 7)).
template <int NCF, int G>
struct T4Layout {
  static constexpr int TL = 8 * G;
  static constexpr int TILE = T4_ROWS * 128, FIELD = (2 * NCF + 1) * TILE, REAL_AT = 2 * NCF * TILE;
  static constexpr int ENT_COUNT = TL + T4_ROWS, ENT_PITCH = 4 * t4_entry_words(NCF);
  static constexpr int STATS_AT = 2 * FIELD;              // pass S: (lse x 4 heads, Delta x 4 heads) per staged position
  static constexpr int ENT_AT = STATS_AT + T4_ROWS * 32;  // entry of offset x (position - owner) at index x - (p0 - TL)
  static constexpr int STAGE = (ENT_AT + ENT_COUNT * ENT_PITCH + 1023) / 1024 * 1024;
  static constexpr int OWN_TILE = TL * 128, OWN_FIELD = (2 * NCF + 1) * OWN_TILE, OWN_REAL_AT = 2 * NCF * OWN_TILE;
  static_assert(TILE % 1024 == 0 && OWN_TILE % 1024 == 0, "sub-tiles start on swizzle periods");
};

// what a warp knows about the item it works on: the row pairs of the owner row, one per lane (lane x: neighbour row
// row + x - W), and which of them exist
struct T4Item {
  int row, c0, b;
  int cnt, lo, off;   // this lane's row pair: window width (0: none), first offset, first table entry
  unsigned present;   // lanes whose row pair has a window
};

__device__ __forceinline__ T4Item t4_item(const T4Args& a, int item, int lane, int TL) {
  T4Item it;
  const int per_row = a.tiles * a.batch;
  const int order = item / per_row, rest = item - order * per_row;
  it.row = a.row_order[order];
  it.c0 = (rest / a.batch) * TL;
  it.b = rest % a.batch;
  const int width = 2 * a.W + 1, j = it.row + lane - a.W;
  it.cnt = 0; it.lo = 0; it.off = 0;
  if (lane < width && j >= 0 && j < a.rows) {
    const int w = it.row * width + lane;
    it.cnt = a.win_cnt[w];
    it.lo = a.win_lo[w];
    it.off = a.win_off[w];
  }
  it.present = __ballot_sync(0xffffffffu, it.cnt > 0);
  return it;
}

template <int NCF, int MODE, int G>
__global__ void __launch_bounds__(32 * (T4_HEADS * G + T4_PRODUCERS), 1) lattice_tc4_kernel(const __grid_constant__ T4Args a) {
  using L = T4Layout<NCF, G>;
  constexpr int TL = L::TL, CONSUMERS = T4_HEADS * G;
  constexpr int KQ = 1 + 2 * NCF;  // k-steps of 16 columns per head: scalar block, then two per complex frequency
  constexpr int NF = NCF > 0 ? NCF : 1, NCK = 2 * NCF > 0 ? 2 * NCF : 1;
  constexpr bool FWD = MODE == T4_FWD, PASS_S = MODE == T4_BWD_S;
  constexpr int OWN_FIELDS = FWD ? 1 : 2, T4_STAGES = t4_stages(NCF);
  extern __shared__ __align__(1024) unsigned char t4_dyn[];
  unsigned char* const smem = t4_dyn + ((1024u - (t4_smem(t4_dyn) & 1023u)) & 1023u);
  unsigned char* const own_tile = smem + T4_STAGES * L::STAGE;
  __shared__ __align__(8) unsigned long long full_bar[T4_STAGES], empty_bar[T4_STAGES], own_full, own_empty;
  __shared__ int failed_s;

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    failed_s = 0;
#pragma unroll
    for (int s = 0; s < T4_STAGES; ++s) {
      t4_bar_init(&full_bar[s], 33 * T4_PRODUCERS);  // per producer warp: one arrival per lane + the one that carries its copies' bytes
      t4_bar_init(&empty_bar[s], CONSUMERS);         // one arrival per consumer warp
    }
    t4_bar_init(&own_full, T4_PRODUCERS);
    t4_bar_init(&own_empty, CONSUMERS);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();

  // =========================================================================== producer warps
  if (warp >= CONSUMERS) {
    t4_fewer_registers<G >= 3 ? 32 : 40>();
    const int pw = warp - CONSUMERS, plane = threadIdx.x - 32 * CONSUMERS;
    constexpr unsigned tile_bytes = L::TILE, own_bytes = L::OWN_TILE;
    constexpr int SUBS = 2 * NCF + 1;          // sub-tiles of a field; sub-tile u < 2 NCF: frequency u / 2, heads 2 (u % 2) .. + 1
    constexpr int N_COPIES = 1 + 2 * SUBS;     // a stage's copies: entries, then (field, sub-tile)
    int sc = 0, ic = 0;                        // stages / items issued so far by this CTA
    T4Item ahead = t4_item(a, min((int)blockIdx.x, a.n_items - 1), lane, TL);
    for (int item = blockIdx.x; item < a.n_items; item += gridDim.x, ++ic) {
      const T4Item it = ahead;
      ahead = t4_item(a, min(item + (int)gridDim.x, a.n_items - 1), lane, TL);  // the next item's tables are on their way while this one runs
      // ---- the owners' rows of this item (their previous occupants have been read into registers)
      if (ic > 0 && !t4_bar_wait(&own_empty, (unsigned)(ic - 1) & 1u)) failed_s = 1;
      if (lane == 0) {
        t4_fence_proxy();
        unsigned mine = 0;
#pragma unroll
        for (int i = 0; i < OWN_FIELDS * SUBS; ++i)
          if (i % T4_PRODUCERS == pw) mine += own_bytes;
        t4_bar_expect(&own_full, mine);
        const int z = it.b * a.rows + it.row;
#pragma unroll
        for (int i = 0; i < OWN_FIELDS * SUBS; ++i) {
          if (i % T4_PRODUCERS != pw) continue;
          const int field = i / SUBS, u = i - field * SUBS;
          const int x = u < 2 * NCF ? a.cf_off[u >> 1] + 64 * (u & 1) : a.real_off;
          t4_tma(own_tile + field * L::OWN_FIELD + u * L::OWN_TILE, &a.own_map[field], &own_full, x, it.c0, z);
        }
      }
      // ---- the item's stages: for every row pair, chunks of T4_ADV positions
      unsigned todo = it.present;
      while (todo) {
        const int src = __ffs(todo) - 1;
        todo &= todo - 1;
        const int cnt = __shfl_sync(0xffffffffu, it.cnt, src), lo = __shfl_sync(0xffffffffu, it.lo, src);
        const int ent_off = __shfl_sync(0xffffffffu, it.off, src);
        const int z = it.b * a.rows + it.row + src - a.W;
        const int lon_base = t4_wrap(it.c0 + lo, a.nlon);
        for (int p0 = 0; p0 < TL + cnt - 1; p0 += T4_ADV, ++sc) {
          const int slot = sc % T4_STAGES, use = sc / T4_STAGES;
          if (use > 0 && !t4_bar_wait(&empty_bar[slot], (unsigned)(use - 1) & 1u)) failed_s = 1;
          const int n_rows = min(T4_ROWS, TL + cnt - 1 - p0);
          int lon0 = lon_base + p0;
          if (lon0 >= a.nlon) lon0 %= a.nlon;
          const bool tma = lon0 + n_rows <= a.nlon;  // consecutive longitudes: no wrap at the seam
          unsigned char* stage = smem + slot * L::STAGE;
          if (lane == 0) {
            // the buffer was last read through the generic proxy (ldmatrix, ld.shared): order those reads before the copy engine's writes
            t4_fence_proxy();
            // the entries the stage's (position, owner) pairs can meet: offsets p0 - TL .. p0 + T4_ROWS - 1, cut to the run and its padding
            const int e_first = max(p0 - TL, -T4_PAD_BEFORE), e_last = min(p0 + T4_ROWS, cnt + T4_PAD_AFTER);
            const unsigned e_bytes = (unsigned)L::ENT_PITCH * (unsigned)(e_last - e_first);
            unsigned mine = 0;
#pragma unroll
            for (int i = 0; i < N_COPIES; ++i)
              if (i % T4_PRODUCERS == pw) mine += i == 0 ? e_bytes : (tma ? tile_bytes : 0u);
            t4_bar_expect(&full_bar[slot], mine);
#pragma unroll
            for (int i = 0; i < N_COPIES; ++i) {
              if (i % T4_PRODUCERS != pw) continue;
              if (i == 0) {
                t4_bulk(stage + L::ENT_AT + L::ENT_PITCH * (e_first - (p0 - TL)), a.entries + (L::ENT_PITCH / 4) * ((int64_t)ent_off + e_first), e_bytes,
                        &full_bar[slot]);
              } else if (tma) {
                const int field = (i - 1) / SUBS, u = (i - 1) - field * SUBS;
                const int x = u < 2 * NCF ? a.cf_off[u >> 1] + 64 * (u & 1) : a.real_off;
                t4_tma(stage + field * L::FIELD + u * L::TILE, &a.nb_map[field], &full_bar[slot], x, lon0, z);
              }
            }
          }
          if (!tma) {
            // across the seam: every producer lane copies its share of the 16-byte chunks (zeros beyond the window)
            for (int idx = plane; idx < 2 * SUBS * 8 * T4_ROWS; idx += 32 * T4_PRODUCERS) {
              const int ch = idx & 7, rest = idx >> 3;
              const int pl = rest % T4_ROWS, fu = rest / T4_ROWS;
              const int field = fu / SUBS, u = fu - field * SUBS;
              const int x = (u < 2 * NCF ? a.cf_off[u >> 1] + 64 * (u & 1) : a.real_off) + 8 * ch;
              int lon = lon0 + pl;
              if (lon >= a.nlon) lon -= a.nlon;
              const __nv_bfloat16* src_p = (field ? a.nb2 : a.nb1) + ((int64_t)z * a.nlon + lon) * a.D + x;
              t4_cp16(stage + field * L::FIELD + u * L::TILE + pl * 128 + 16 * (ch ^ (pl & 7)), src_p, pl < n_rows ? 16 : 0);
            }
          }
          if constexpr (PASS_S) {
            // (lse, Delta) of the four heads of every staged position: zeros beyond the window (size-0 copies), where the logits
            // are -inf and a stale pair could otherwise turn 0 weights into NaN
            for (int idx = plane; idx < 2 * T4_ROWS; idx += 32 * T4_PRODUCERS) {
              const int pl = idx >> 1, which = idx & 1;
              int lon = lon0 + pl;
              if (lon >= a.nlon) lon %= a.nlon;
              const int64_t nn = ((int64_t)z * a.nlon + lon) * T4_HEADS;
              t4_cp16(stage + L::STATS_AT + pl * 32 + which * 16, (which ? a.delta : a.lse) + nn, pl < n_rows ? 16 : 0);
            }
          }
          t4_bar_arrive_after_cp_async(&full_bar[slot]);  // fires once this lane's cp.async copies (if any) have landed
        }
      }
    }
    return;
  }

  // =========================================================================== consumer warps
  t4_more_registers<G >= 3 ? 160 : 224>();
  const int g = lane >> 2, c = lane & 3;
  const int hh = warp / G, gg = warp - hh * G;  // this warp's head and owner group
  const int own_b = 8 * gg + g;                 // the owner whose column this thread holds in B fragments (and stores in the epilogue)
  const int own_c = 8 * gg + 2 * c;             // the owners (own_c, own_c + 1) of this thread's accumulator columns
  const float cscale = a.scale * T4_LOG2E;
  // per-lane byte offsets of the ldmatrix rows inside a sub-tile for a step that starts at staged row 0 (a step starts on a
  // multiple of 8 rows, which leaves the swizzle term unchanged).  Gram A operand: matrices (rows 0-7, k 0-7), (rows 8-15,
  // k 0-7), (rows 0-7, k 8-15), (rows 8-15, k 8-15); accumulation A operand = tile^T: (cols 0-7, rows 0-7), (cols 8-15,
  // rows 0-7), (cols 0-7, rows 8-15), (cols 8-15, rows 8-15).
  int g_real, a_real, g_cx[2], a_cx[2];
  {
    const int mi = lane >> 3, rr = lane & 7;
    const int rg = 8 * (mi & 1) + rr, ra = 8 * (mi >> 1) + rr;
    g_real = L::REAL_AT + rg * 128 + 16 * ((2 * hh + (mi >> 1)) ^ (rg & 7));
    a_real = L::REAL_AT + ra * 128 + 16 * ((2 * hh + (mi & 1)) ^ (ra & 7));
#pragma unroll
    for (int sub = 0; sub < 2; ++sub) {
      g_cx[sub] = (hh >> 1) * L::TILE + rg * 128 + 16 * ((4 * (hh & 1) + 2 * sub + (mi >> 1)) ^ (rg & 7));
      a_cx[sub] = (hh >> 1) * L::TILE + ra * 128 + 16 * ((4 * (hh & 1) + 2 * sub + (mi & 1)) ^ (ra & 7));
    }
  }
  // Gram blocks of 16 staged rows x 8 owners: g0 (scalar block), gr / gi per complex frequency
  auto gram = [&](const unsigned (&fb)[KQ][2], const unsigned (&fs)[NCK][2], unsigned tile, int pl, float (&g0)[4], float (&gr)[NF][4], float (&gi)[NF][4]) {
    unsigned af[4];
    t4_ldsm(af, tile + pl * 128 + g_real);
    t4_mma_init(g0, af, fb[0]);
#pragma unroll
    for (int f = 0; f < NCF; ++f)
#pragma unroll
      for (int sub = 0; sub < 2; ++sub) {
        t4_ldsm(af, tile + 2 * f * L::TILE + pl * 128 + g_cx[sub]);
        if (sub == 0) {
          t4_mma_init(gr[f], af, fb[1 + 2 * f + sub]);
          t4_mma_init(gi[f], af, fs[2 * f + sub]);
        } else {
          t4_mma(gr[f], af, fb[1 + 2 * f + sub]);
          t4_mma(gi[f], af, fs[2 * f + sub]);
        }
      }
  };
  // acc^T (head columns x 8 owners) += tile^T (columns x 16 staged rows) * B
  auto accumulate = [&](float (&acc0)[4], float (&accr)[NCK][4], float (&acci)[NCK][4], const unsigned (&x0)[2], const unsigned (&xr)[NF][2],
                        const unsigned (&xi)[NF][2], unsigned tile, int pl) {
    unsigned af[4];
    t4_ldsm_t(af, tile + pl * 128 + a_real);
    t4_mma(acc0, af, x0);
#pragma unroll
    for (int f = 0; f < NCF; ++f)
#pragma unroll
      for (int sub = 0; sub < 2; ++sub) {
        t4_ldsm_t(af, tile + 2 * f * L::TILE + pl * 128 + a_cx[sub]);
        t4_mma(accr[2 * f + sub], af, xr[f]);
        t4_mma(acci[2 * f + sub], af, xi[f]);
      }
  };
  // B fragments of this thread's owner (own_b) from the owners' tile: k-step 0 = scalar block, 1 + 2 f + sub = complex
  auto owner_fragments = [&](const unsigned char* field, unsigned (&fb)[KQ][2]) {
    const int r = own_b, sw = r & 7;
    const unsigned char* row = field + r * 128 + 4 * c;
#pragma unroll
    for (int half = 0; half < 2; ++half) fb[0][half] = *reinterpret_cast<const unsigned*>(row + L::OWN_REAL_AT + 16 * ((2 * hh + half) ^ sw));
#pragma unroll
    for (int f = 0; f < NCF; ++f)
#pragma unroll
      for (int sub = 0; sub < 2; ++sub)
#pragma unroll
        for (int half = 0; half < 2; ++half)
          fb[1 + 2 * f + sub][half] =
              *reinterpret_cast<const unsigned*>(row + (2 * f + (hh >> 1)) * L::OWN_TILE + 16 * ((4 * (hh & 1) + 2 * sub + half) ^ sw));
  };
  // one result m-tile (16 head columns x 8 owners, accumulator layout) -> global memory, transposed in registers so that a
  // thread holds two adjacent columns of ONE owner (own_b): 4-byte stores
  auto store_tile = [&](__nv_bfloat16* dst, bool present, int column, const float (&v)[4]) {
    const unsigned w0 = t4_movm(t4_pack(v[0], v[1])), w1 = t4_movm(t4_pack(v[2], v[3]));
    if (present) {
      unsigned* w = reinterpret_cast<unsigned*>(dst + column) + c;
      w[0] = w0;
      w[4] = w1;
    }
  };
  auto store_result = [&](__nv_bfloat16* dst, bool present, bool conj, const float (&inv)[2], const float (&acc0)[4], const float (&accr)[NCK][4],
                          const float (&acci)[NCK][4]) {
    {
      const float v[4] = {acc0[0] * inv[0], acc0[1] * inv[1], acc0[2] * inv[0], acc0[3] * inv[1]};
      store_tile(dst, present, a.real_off + 16 * hh, v);
    }
    // rows of an accumulator m-tile are head columns g, g + 8: even = real part, odd = imaginary part.
    //   tau:      re = r_re - i_im,  im = r_im + i_re;      conj tau:  re = r_re + i_im,  im = r_im - i_re
    const float sgn = ((g & 1) != 0) == conj ? -1.f : 1.f;
#pragma unroll
    for (int m = 0; m < 2 * NCF; ++m) {
      float v[4];
#pragma unroll
      for (int x = 0; x < 4; ++x) v[x] = (accr[m][x] + sgn * __shfl_xor_sync(0xffffffffu, acci[m][x], 4)) * inv[x & 1];
      store_tile(dst, present, a.cf_off[m >> 1] + 32 * hh + 16 * (m & 1), v);
    }
  };

  int sc = 0, ic = 0;
  T4Item ahead = t4_item(a, min((int)blockIdx.x, a.n_items - 1), lane, TL);
  for (int item = blockIdx.x; item < a.n_items; item += gridDim.x, ++ic) {
    const T4Item it = ahead;
    ahead = t4_item(a, min(item + (int)gridDim.x, a.n_items - 1), lane, TL);  // the next item's tables are on their way while this one runs
    const int64_t node0 = ((int64_t)it.b * a.rows + it.row) * a.nlon;
    const bool own_b_present = it.c0 + own_b < a.nlon;
    const int64_t own_b_base = (node0 + it.c0 + own_b) * a.D;
    // ---- the owners' fragments (loop-invariant B operands) and their pre-swapped copies for the imaginary Gram part:
    //   owners carry q: q' = (-q_im, q_re);   owners carry k: k' = (k_im, -k_re)
    if (!t4_bar_wait(&own_full, (unsigned)ic & 1u)) failed_s = 1;
    __syncwarp();
    unsigned f1[KQ][2], s1[NCK][2], f2[FWD ? 1 : KQ][2], s2[FWD ? 1 : NCK][2];
    owner_fragments(own_tile, f1);
    if constexpr (!FWD) owner_fragments(own_tile + L::OWN_FIELD, f2);
    __syncwarp();
    if (lane == 0) t4_bar_arrive(&own_empty);  // this warp has its owners in registers
#pragma unroll
    for (int kc = 0; kc < 2 * NCF; ++kc)
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        s1[kc][r] = PASS_S ? t4_swap_neg(f1[1 + kc][r]) : t4_swap_neg_lo(f1[1 + kc][r]);
        if constexpr (!FWD) s2[kc][r] = PASS_S ? t4_swap_neg(f2[1 + kc][r]) : t4_swap_neg_lo(f2[1 + kc][r]);
      }
    float lse_o[2] = {0.f, 0.f}, dl_o[2] = {0.f, 0.f};  // pass T: the two accumulator-column owners' lse (base 2) and Delta
    if constexpr (MODE == T4_BWD_T) {
#pragma unroll
      for (int e = 0; e < 2; ++e)
        if (it.c0 + own_c + e < a.nlon) {
          lse_o[e] = a.lse[(node0 + it.c0 + own_c + e) * T4_HEADS + hh] * T4_LOG2E;
          dl_o[e] = a.delta[(node0 + it.c0 + own_c + e) * T4_HEADS + hh];
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

    unsigned todo = it.present;
    while (todo) {
      const int src = __ffs(todo) - 1;
      todo &= todo - 1;
      const int cnt = __shfl_sync(0xffffffffu, it.cnt, src);
      for (int p0 = 0; p0 < TL + cnt - 1; p0 += T4_ADV, ++sc) {
        const int slot = sc % T4_STAGES, use = sc / T4_STAGES;
        if (!t4_bar_wait(&full_bar[slot], (unsigned)use & 1u)) failed_s = 1;
        __syncwarp();  // lanes may leave the polling loop at different polls; the tile instructions below are warp-wide
        const unsigned char* stage = smem + slot * L::STAGE;
        const unsigned t1 = t4_smem(stage), t2 = t1 + L::FIELD;
        const unsigned char* ent_s = stage + L::ENT_AT;
        const float* stat_s = reinterpret_cast<const float*>(stage + L::STATS_AT);
        // ---- this warp's steps inside the chunk: 16 positions each, on the lattice 8 gg + 16 i
        const int p_first = p0 > 8 * gg ? p0 + ((8 * gg) & 8) : 8 * gg;
        const int p_end = min(p0 + T4_ADV, 8 * gg + 7 + cnt);
        for (int p = p_first; p < p_end; p += 16) {
          const int pl = p - p0;
          // element x of a fragment: position p + g + 8 (x >> 1), owner own_c + (x & 1); its entry: offset position - owner
          const unsigned char* e0 = ent_s + L::ENT_PITCH * (TL + pl + g - own_c);
          float lg[4], tr[NF][4], ti[NF][4];
          {
            float s0[4], sr[NF][4], si[NF][4];
            gram(f1, s1, t1, pl, s0, sr, si);
#pragma unroll
            for (int x = 0; x < 4; ++x) {
              const unsigned char* e = e0 + L::ENT_PITCH * (8 * (x >> 1) - (x & 1));
              float tau[6] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, bias2;
              {
                const float4 t = *reinterpret_cast<const float4*>(e);
                tau[0] = t.x; tau[1] = t.y; tau[2] = t.z; tau[3] = t.w;
              }
              if constexpr (NCF == 3) {
                const float4 t = *reinterpret_cast<const float4*>(e + 32);  // bias, cos, sin of order 3
                bias2 = t.x; tau[4] = t.y; tau[5] = t.z;
              } else {
                bias2 = *reinterpret_cast<const float*>(e + 32);
              }
              float sum = s0[x];
#pragma unroll
              for (int f = 0; f < NCF; ++f) {
                tr[f][x] = tau[2 * f];
                ti[f][x] = tau[2 * f + 1];
                sum = fmaf(tau[2 * f], sr[f][x], sum);
                sum = fmaf(-tau[2 * f + 1], si[f][x], sum);
              }
              lg[x] = fmaf(cscale, sum, bias2);  // -inf outside the window (the padding entries' bias)
            }
          }
          // packed bf16 phase pairs (element 0 | element 1) of row group 0 and (element 2 | element 3) of row group 1
          unsigned pk[2][2 * NF];
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const unsigned char* e = e0 + L::ENT_PITCH * 8 * r;
            const uint4 w = *reinterpret_cast<const uint4*>(e + 16);
            pk[r][0] = w.x; pk[r][1] = w.y;
            if constexpr (NCF >= 2) { pk[r][2] = w.z; pk[r][3] = w.w; }
            if constexpr (NCF == 3) {
              const uint2 w3 = *reinterpret_cast<const uint2*>(e + 48);
              pk[r][4] = w3.x; pk[r][5] = w3.y;
            }
          }
          float w1[4], w2[4];  // the weights the two accumulations use: forward p | pass T ds | pass S ds, p
          if constexpr (FWD) {
            // online softmax over the 16 positions.  The reference maximum of an owner only moves when a logit exceeds it by
            // more than 2^8 (weights stay below 256: exact in the normalised result); the test for that needs no reduction,
            // so most steps skip both the column maxima and the rescaling of the accumulators.
            const bool grow = fmaxf(lg[0], lg[2]) > m_o[0] + 8.f || fmaxf(lg[1], lg[3]) > m_o[1] + 8.f;
            if (__any_sync(0xffffffffu, grow)) {
              float mx[2] = {fmaxf(lg[0], lg[2]), fmaxf(lg[1], lg[3])};
#pragma unroll
              for (int d = 4; d < 32; d <<= 1) {
                mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xffffffffu, mx[0], d));
                mx[1] = fmaxf(mx[1], __shfl_xor_sync(0xffffffffu, mx[1], d));
              }
              const float nm[2] = {mx[0] > m_o[0] + 8.f ? mx[0] : m_o[0], mx[1] > m_o[1] + 8.f ? mx[1] : m_o[1]};
              const float corr[2] = {t4_exp2(m_o[0] - nm[0]), t4_exp2(m_o[1] - nm[1])};
              m_o[0] = nm[0]; m_o[1] = nm[1];
              l_o[0] *= corr[0]; l_o[1] *= corr[1];
#pragma unroll
              for (int x = 0; x < 4; ++x) {
                a1_0[x] *= corr[x & 1];
#pragma unroll
                for (int m = 0; m < 2 * NCF; ++m) { a1_r[m][x] *= corr[x & 1]; a1_i[m][x] *= corr[x & 1]; }
              }
            }
#pragma unroll
            for (int x = 0; x < 4; ++x) {
              w1[x] = t4_exp2(lg[x] - m_o[x & 1]);
              l_o[x & 1] += w1[x];
            }
          } else {
            // p from the logits first (the (q, k) Gram blocks die here), then d alpha from the (dO, v) Gram blocks
            float delta[4];
#pragma unroll
            for (int x = 0; x < 4; ++x) {
              float lse;
              if (PASS_S) {
                const float* st = stat_s + 8 * (pl + g + 8 * (x >> 1));
                lse = st[hh] * T4_LOG2E; delta[x] = st[4 + hh];
              } else {
                lse = lse_o[x & 1]; delta[x] = dl_o[x & 1];
              }
              w2[x] = t4_exp2(lg[x] - lse);  // 0 outside the window: exp2(-inf)
            }
            float h0[4], hr[NF][4], hi[NF][4];
            gram(f2, s2, t2, pl, h0, hr, hi);
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
          // B operands: the weights rounded to bf16, times the bf16 phase parts (packed pairs: one multiply per two
          // elements), transposed to (owner column, position rows)
          unsigned x0[2], xr[NF][2], xim[NF][2];
          {
            const unsigned wa = t4_pack(w1[0], w1[1]), wb = t4_pack(w1[2], w1[3]);
            x0[0] = t4_movm(wa);
            x0[1] = t4_movm(wb);
#pragma unroll
            for (int f = 0; f < NCF; ++f) {
              xr[f][0] = t4_movm(t4_mul2(wa, pk[0][2 * f]));
              xr[f][1] = t4_movm(t4_mul2(wb, pk[1][2 * f]));
              xim[f][0] = t4_movm(t4_mul2(wa, pk[0][2 * f + 1]));
              xim[f][1] = t4_movm(t4_mul2(wb, pk[1][2 * f + 1]));
            }
          }
          if constexpr (FWD) {
            accumulate(a1_0, a1_r, a1_i, x0, xr, xim, t2, pl);  // out += (p tau) v
          } else {
            accumulate(a1_0, a1_r, a1_i, x0, xr, xim, t1, pl);  // dq += (ds tau) k  |  dk += (ds conj tau) q
            if constexpr (PASS_S) {
              const unsigned wa = t4_pack(w2[0], w2[1]), wb = t4_pack(w2[2], w2[3]);
              x0[0] = t4_movm(wa);
              x0[1] = t4_movm(wb);
#pragma unroll
              for (int f = 0; f < NCF; ++f) {
                xr[f][0] = t4_movm(t4_mul2(wa, pk[0][2 * f]));
                xr[f][1] = t4_movm(t4_mul2(wb, pk[1][2 * f]));
                xim[f][0] = t4_movm(t4_mul2(wa, pk[0][2 * f + 1]));
                xim[f][1] = t4_movm(t4_mul2(wb, pk[1][2 * f + 1]));
              }
              accumulate(a2_0, a2_r, a2_i, x0, xr, xim, t2, pl);  // dv += (p conj tau) dO
            }
          }
        }
        __syncwarp();
        if (lane == 0) t4_bar_arrive(&empty_bar[slot]);  // this warp is done with the buffer
      }
    }

    // ---- epilogue: normalise, combine the two phase accumulators (multiplication by +-i = pair swap across rows g, g ^ 1),
    // transpose in registers, store.  A wait that ran out anywhere in this CTA poisons its results (NaN).
    float inv[2] = {1.f, 1.f};
    if constexpr (FWD) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
#pragma unroll
        for (int d = 4; d < 32; d <<= 1) l_o[e] += __shfl_xor_sync(0xffffffffu, l_o[e], d);
        inv[e] = l_o[e] > 0.f ? 1.f / l_o[e] : 0.f;
      }
    }
    const bool failed = *(volatile int*)&failed_s != 0;
    if (failed) inv[0] = inv[1] = __int_as_float(0x7fc00000);
    if constexpr (FWD) {
#pragma unroll
      for (int e = 0; e < 2; ++e)
        if (g == 0 && it.c0 + own_c + e < a.nlon)
          a.lse_out[(node0 + it.c0 + own_c + e) * T4_HEADS + hh] =
              failed ? __int_as_float(0x7fc00000) : (l_o[e] > 0.f ? (m_o[e] + log2f(l_o[e])) * T4_LN2 : -INFINITY);
    }
    store_result(a.res1 + own_b_base, own_b_present, PASS_S, inv, a1_0, a1_r, a1_i);
    if constexpr (PASS_S) store_result(a.res2 + own_b_base, own_b_present, true, inv, a2_0, a2_r, a2_i);
  }
}

PFN_cuTensorMapEncodeTiled_v12000 t4_encoder() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult res;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &res) != cudaSuccess || res != cudaDriverEntryPointSuccess)
      sym = nullptr;
    return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(sym);
  }();
  return fn;
}

// a bf16 field seen as (D columns, nlon longitudes, batch * rows): boxes of 64 columns x box_rows longitudes of one
// lattice row, written in the 128-byte shared-memory swizzle
bool t4_encode(CUtensorMap* map, const void* field, int D, int nlon, int64_t slabs, int box_rows) {
  auto encode = t4_encoder();
  if (!encode) return false;
  const cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)nlon, (cuuint64_t)slabs};
  const cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)nlon * D * 2};
  const cuuint32_t box[3] = {64u, (cuuint32_t)box_rows, 1u};
  const cuuint32_t estr[3] = {1, 1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(field), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int NCF, int MODE, int G>
int t4_launch(T4Args& a, cudaStream_t stream) {
  using L = T4Layout<NCF, G>;
  constexpr int own_fields = MODE == T4_FWD ? 1 : 2;
  a.tiles = (a.nlon + L::TL - 1) / L::TL;
  const int64_t items = (int64_t)a.n_order_rows * a.tiles * a.batch;
  GM_REQUIRE(items < (1ll << 31), GM_ERR_LIMIT, "gm_lattice_attention (four heads per CTA): too many owner tiles");
  a.n_items = (int)items;
  const void* nb[2] = {a.nb1, a.nb2};
  const void* own[2] = {a.own1, a.own2};
  for (int x = 0; x < 2; ++x) {
    GM_REQUIRE(t4_encode(&a.nb_map[x], nb[x], a.D, a.nlon, (int64_t)a.batch * a.rows, T4_ROWS), GM_ERR_CUDA,
               "gm_lattice_attention (four heads per CTA): cuTensorMapEncodeTiled failed");
    if (x < own_fields)
      GM_REQUIRE(t4_encode(&a.own_map[x], own[x], a.D, a.nlon, (int64_t)a.batch * a.rows, L::TL), GM_ERR_CUDA,
                 "gm_lattice_attention (four heads per CTA): cuTensorMapEncodeTiled failed");
  }
  const size_t smem = t4_stages(NCF) * (size_t)L::STAGE + own_fields * (size_t)L::OWN_FIELD + 1024;
  auto kernel = lattice_tc4_kernel<NCF, MODE, G>;
  int st = allow_smem(kernel, smem, "gm_lattice_attention (four heads per CTA)");
  if (st != GM_OK) return st;
  const int grid = (int)(items < sm_count() ? items : sm_count());
  kernel<<<grid, 32 * (T4_HEADS * G + T4_PRODUCERS), smem, stream>>>(a);
  return launch_status("gm_lattice_attention (four heads per CTA)");
}

template <int MODE, int G>
int t4_dispatch(T4Args& a, int ncf, cudaStream_t cs) {
  if (ncf == 1) return t4_launch<1, MODE, G>(a, cs);
  if (ncf == 2) return t4_launch<2, MODE, G>(a, cs);
  return t4_launch<3, MODE, G>(a, cs);
}

// Head layout and sizes this path serves; fills the plan.  Returns GM_ERR_UNSUPPORTED (with the reason) otherwise.
int t4_fill(T4Args& a, const int64_t* desc_host, int F, int rows, int nlon, int64_t batch, int D, int H, int W, int ES, int NORD, double scale,
            int* ncf_out) {
  GM_REQUIRE(desc_host && rows >= 1 && nlon >= 1 && batch >= 1 && batch * rows < (1ll << 31), GM_ERR_ARGUMENT,
             "gm_lattice_attention (four heads per CTA): bad sizes");
  GM_REQUIRE(H == T4_HEADS && F >= 2 && F <= T4_MAX_NCF + 1, GM_ERR_UNSUPPORTED, "gm_lattice_attention (four heads per CTA): 4 heads, 1..3 complex frequencies");
  int ncf = 0;
  bool real = false;
  for (int f = 0; f < F; ++f) {
    const int n = (int)desc_host[5 * f], a_n = (int)desc_host[5 * f + 1], off = (int)desc_host[5 * f + 2];
    GM_REQUIRE(a_n == 16 && off >= 0 && off % 8 == 0, GM_ERR_UNSUPPORTED, "gm_lattice_attention (four heads per CTA): 16 copies per head, blocks on 16-byte boundaries");
    if (n == 0) {
      GM_REQUIRE(!real && off + 64 <= D, GM_ERR_UNSUPPORTED, "gm_lattice_attention (four heads per CTA): one scalar block inside the row");
      real = true;
      a.real_off = off;
    } else {
      GM_REQUIRE(n == ncf + 1 && off + 128 <= D, GM_ERR_UNSUPPORTED, "gm_lattice_attention (four heads per CTA): complex orders 1, 2, 3 in order");
      a.cf_off[ncf++] = off;
    }
  }
  GM_REQUIRE(real && ncf >= 1 && NORD == ncf && ES == t4_entry_words(ncf), GM_ERR_UNSUPPORTED,
             "gm_lattice_attention (four heads per CTA): a scalar block, orders 1..%d, the padded %d-word entry table", ncf, t4_entry_words(ncf));
  GM_REQUIRE(D % 8 == 0 && 2 * W + 1 <= 32 && nlon >= T4_ROWS, GM_ERR_UNSUPPORTED,
             "gm_lattice_attention (four heads per CTA): D a multiple of 8, at most 32 neighbour rows, at least %d longitudes", T4_ROWS);
  a.rows = rows; a.nlon = nlon; a.D = D; a.W = W; a.batch = (int)batch; a.scale = (float)scale;
  *ncf_out = ncf;
  return GM_OK;
}

bool t4_aligned(std::initializer_list<const void*> ptrs) {
  for (const void* p : ptrs)
    if (reinterpret_cast<uintptr_t>(p) % 16 != 0) return false;
  return true;
}

// Delta[node, h] = <dO, O> over the head's columns: one warp per node, 16-byte loads
__global__ void t4_delta_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ out, float* __restrict__ delta, int64_t n_nodes,
                                int D, int real_off, int cf0, int cf1, int cf2, int ncf) {
  const int lane = threadIdx.x & 31;
  const int64_t node = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (node >= n_nodes) return;
  float part[T4_HEADS] = {0.f, 0.f, 0.f, 0.f};
  for (int col = 8 * lane; col < D; col += 256) {
    int head = -1;
    if (col >= real_off && col < real_off + 64) head = (col - real_off) >> 4;
    const int cf[3] = {cf0, cf1, cf2};
    for (int f = 0; f < ncf; ++f)
      if (col >= cf[f] && col < cf[f] + 128) head = (col - cf[f]) >> 5;
    if (head < 0) continue;
    const uint4 x = __ldg(reinterpret_cast<const uint4*>(dout + node * D + col));
    const uint4 y = __ldg(reinterpret_cast<const uint4*>(out + node * D + col));
    const unsigned wx[4] = {x.x, x.y, x.z, x.w}, wy[4] = {y.x, y.y, y.z, y.w};
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k)
      s += __uint_as_float(wx[k] << 16) * __uint_as_float(wy[k] << 16) + __uint_as_float(wx[k] & 0xffff0000u) * __uint_as_float(wy[k] & 0xffff0000u);
#pragma unroll
    for (int hd = 0; hd < T4_HEADS; ++hd) part[hd] += head == hd ? s : 0.f;
  }
#pragma unroll
  for (int hd = 0; hd < T4_HEADS; ++hd) {
    const float v = warp_sum(part[hd]);
    if (lane == 0) delta[node * T4_HEADS + hd] = v;
  }
}

}  // namespace
}  // namespace gmb

using namespace gmb;

extern "C" int gm_lattice_attention_forward_tc4(const void* q, const void* k, const void* v, const int* win_cnt, const int* win_lo,
                                                const int* win_off, const float* entries, const int* row_order, int n_order_rows,
                                                const int64_t* desc_host, int F, int rows, int nlon, int64_t batch, int D, int H, int W,
                                                int ES, int NORD, double scale, void* out, float* lse, void* stream) {
  using B = __nv_bfloat16;
  T4Args a{};
  int ncf = 0;
  int status = t4_fill(a, desc_host, F, rows, nlon, batch, D, H, W, ES, NORD, scale, &ncf);
  if (status != GM_OK) return status;
  GM_REQUIRE(q && k && v && win_cnt && win_lo && win_off && entries && row_order && out && lse, GM_ERR_ARGUMENT,
             "gm_lattice_attention_forward_tc4: null pointer");
  GM_REQUIRE(t4_aligned({q, k, v, out}), GM_ERR_UNSUPPORTED, "gm_lattice_attention_forward_tc4: fields must start on 16-byte boundaries");
  if (n_order_rows == 0) return GM_OK;
  a.own1 = (const B*)q; a.nb1 = (const B*)k; a.nb2 = (const B*)v; a.res1 = (B*)out; a.lse_out = lse;
  a.win_cnt = win_cnt; a.win_lo = win_lo; a.win_off = win_off; a.entries = entries; a.row_order = row_order; a.n_order_rows = n_order_rows;
  return t4_dispatch<T4_FWD, 3>(a, ncf, (cudaStream_t)stream);
}

// passes: bit 0 = Delta = <dO, O> (its own kernel), bit 1 = the target-major pass (dq), bit 2 = the source-major pass
// (dk, dv); passes 2 and 4 read the Delta bit 0 (of this or an earlier call) left in `delta`
extern "C" int gm_lattice_attention_backward_tc4_passes(const void* dout, const void* q, const void* k, const void* v, const void* out,
                                                        const float* lse, const int* win_cnt, const int* win_lo, const int* win_off,
                                                        const float* entries, const int* row_order, int n_order_rows,
                                                        const int* t_win_cnt, const int* t_win_lo, const int* t_win_off,
                                                        const float* t_entries, const int* t_row_order, int t_n_order_rows,
                                                        const int64_t* desc_host, int F, int rows, int nlon, int64_t batch, int D, int H,
                                                        int W, int ES, int NORD, double scale, void* dq, void* dk, void* dv, float* delta,
                                                        int passes, void* stream) {
  using B = __nv_bfloat16;
  cudaStream_t cs = (cudaStream_t)stream;
  T4Args a{};
  int ncf = 0;
  int status = t4_fill(a, desc_host, F, rows, nlon, batch, D, H, W, ES, NORD, scale, &ncf);
  if (status != GM_OK) return status;
  GM_REQUIRE(dout && q && k && v && out && lse && win_cnt && win_lo && win_off && entries && row_order && t_win_cnt && t_win_lo &&
                 t_win_off && t_entries && t_row_order && dq && dk && dv && delta,
             GM_ERR_ARGUMENT, "gm_lattice_attention_backward_tc4: null pointer");
  GM_REQUIRE(t4_aligned({dout, q, k, v, out, dq, dk, dv, lse, delta}), GM_ERR_UNSUPPORTED,
             "gm_lattice_attention_backward_tc4: fields must start on 16-byte boundaries");
  const int64_t n_nodes = batch * rows * (int64_t)nlon;
  if (passes & 1) {
    t4_delta_kernel<<<(unsigned)((n_nodes + 7) / 8), 256, 0, cs>>>((const B*)dout, (const B*)out, delta, n_nodes, D, a.real_off, a.cf_off[0], a.cf_off[1],
                                                                 a.cf_off[2], ncf);
    status = launch_status("gm_lattice_attention_backward_tc4 (delta)");
    if (status != GM_OK) return status;
  }
  a.lse = lse; a.delta = delta;
  if (n_order_rows > 0 && (passes & 2)) {
    a.own1 = (const B*)q; a.own2 = (const B*)dout; a.nb1 = (const B*)k; a.nb2 = (const B*)v; a.res1 = (B*)dq; a.res2 = nullptr;
    a.win_cnt = win_cnt; a.win_lo = win_lo; a.win_off = win_off; a.entries = entries; a.row_order = row_order; a.n_order_rows = n_order_rows;
    status = t4_dispatch<T4_BWD_T, 3>(a, ncf, cs);
    if (status != GM_OK) return status;
  }
  if (t_n_order_rows > 0 && (passes & 4)) {
    a.own1 = (const B*)k; a.own2 = (const B*)v; a.nb1 = (const B*)q; a.nb2 = (const B*)dout; a.res1 = (B*)dk; a.res2 = (B*)dv;
    a.win_cnt = t_win_cnt; a.win_lo = t_win_lo; a.win_off = t_win_off; a.entries = t_entries; a.row_order = t_row_order; a.n_order_rows = t_n_order_rows;
    status = t4_dispatch<T4_BWD_S, 3>(a, ncf, cs);
  }
  return status;
}

extern "C" int gm_lattice_attention_tc4_wait_expired(int* expired) {
  GM_REQUIRE(expired, GM_ERR_ARGUMENT, "gm_lattice_attention_tc4_wait_expired: null pointer");
  GM_CUDA(cudaMemcpyFromSymbol(expired, g_tc4_wait_expired, sizeof(int)));
  return GM_OK;
}
