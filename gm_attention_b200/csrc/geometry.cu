// On-device construction of the neighbourhood geometry: the target-major CSR
// of all directed pairs within a geodesic radius, and the per-edge tables.
//
// Membership follows the reference bit for bit
// (src/gm_attention/discretization/edge_geometry.py:371-387, 492-503): float64
// unit vectors, d = atan2(|p x q|, clamp(<p, q>, -1, 1)), pair kept iff
// d <= radius + 1e-10; sources ascending inside each target's row (:701-704).
// The reference finds candidates with a CPU KD-tree; here one warp per target
// scans a candidate index range [lo, hi) -- the whole point set, or the band of
// lattice rows that can reach the target -- 32 candidates per step, and an
// ordered ballot compaction writes the row already sorted, so no sort and no
// atomics are needed.  A cheap chord-length test in float64 prunes candidates
// before the atan2.
//
// The tables (edge_geometry.py:506-619): r, kappa = r / sin r, log map in the
// target frame, phi = atan2(y, x), Rodrigues transport R = I + K + K^2 / (1 + <p, q>)
// with K = [q x p]_x (:718-771), gamma = atan2(C10, C00) of C = E_i^T R E_j,
// tangent weight w_j kappa, and cos / sin of k phi, k gamma for k = 0..K.
// They are evaluated in float64 and rounded once to the table dtype.
#include "common.cuh"

namespace gmb {
namespace {

constexpr double EXACT_SLACK = 1e-10;

struct Vec3 { double x, y, z; };
__device__ __forceinline__ Vec3 load3(const double* p) { return {p[0], p[1], p[2]}; }
__device__ __forceinline__ double dot(Vec3 a, Vec3 b) { return a.x * b.x + a.y * b.y + a.z * b.z; }
__device__ __forceinline__ Vec3 cross(Vec3 a, Vec3 b) { return {a.y * b.z - a.z * b.y, a.z * b.x - a.x * b.z, a.x * b.y - a.y * b.x}; }

__device__ __forceinline__ double geodesic(Vec3 p, Vec3 q) {
  const Vec3 c = cross(p, q);
  const double d = fmin(1.0, fmax(-1.0, dot(p, q)));
  return atan2(sqrt(dot(c, c)), d);
}

__device__ __forceinline__ bool is_member(Vec3 p, Vec3 q, double radius, double chord2) {
  const double dx = p.x - q.x, dy = p.y - q.y, dz = p.z - q.z;
  if (dx * dx + dy * dy + dz * dz > chord2) return false;  // generous superset
  return geodesic(p, q) <= radius + EXACT_SLACK;
}

__global__ void count_kernel(const double* __restrict__ nodes, int64_t n_nodes, const int64_t* __restrict__ lo,
                             const int64_t* __restrict__ hi, double radius, double chord2, int64_t* __restrict__ degree) {
  const int lane = threadIdx.x & 31;
  const int64_t i = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= n_nodes) return;
  const Vec3 p = load3(nodes + 3 * i);
  const int64_t j0 = lo ? lo[i] : 0, j1 = hi ? hi[i] : n_nodes;
  int64_t count = 0;
  for (int64_t base = j0; base < j1; base += 32) {  // uniform trip count: every lane reaches every ballot
    const int64_t j = base + lane;
    const bool in = j < j1 && is_member(p, load3(nodes + 3 * j), radius, chord2);
    count += __popc(__ballot_sync(0xffffffffu, in));
  }
  if (lane == 0) degree[i] = count;
}

template <typename T>
struct FillArgs {
  const double *nodes, *frames, *weights;
  const int64_t *lo, *hi, *row_ptr;
  int64_t n_nodes;
  double radius, chord2;
  int orders;  // max_frequency + 1
  int64_t *target, *source;
  T *distances, *log_xy, *polar, *transport_angle, *tangent_w, *angular, *transport;
};

template <typename T>
__device__ void write_edge(const FillArgs<T>& a, int64_t e, int64_t i, int64_t j, Vec3 p, Vec3 q) {
  a.target[e] = i;
  a.source[e] = j;
  const double d = fmin(1.0, fmax(-1.0, dot(p, q)));
  const double r = geodesic(p, q);
  const double kappa = r == 0.0 ? 1.0 : r / sin(r);
  const Vec3 lg = {kappa * (q.x - d * p.x), kappa * (q.y - d * p.y), kappa * (q.z - d * p.z)};
  const double* Fi = a.frames + 6 * i;  // (3, 2): column c of row x at Fi[2 x + c]
  const double* Fj = a.frames + 6 * j;
  const Vec3 ei0 = {Fi[0], Fi[2], Fi[4]}, ei1 = {Fi[1], Fi[3], Fi[5]};
  const Vec3 ej0 = {Fj[0], Fj[2], Fj[4]};
  const double lx = dot(ei0, lg), ly = dot(ei1, lg);
  // R u = u + w x u + w x (w x u) / (1 + d),  w = q x p
  const Vec3 w = cross(q, p);
  const Vec3 wu = cross(w, ej0);
  const Vec3 wwu = cross(w, wu);
  const double s = 1.0 / (1.0 + d);
  const Vec3 ru = {ej0.x + wu.x + s * wwu.x, ej0.y + wu.y + s * wwu.y, ej0.z + wu.z + s * wwu.z};
  const double gamma = atan2(dot(ei1, ru), dot(ei0, ru));
  const double phi = atan2(ly, lx);
  a.distances[e] = (T)r;
  a.log_xy[2 * e] = (T)lx;
  a.log_xy[2 * e + 1] = (T)ly;
  a.polar[e] = (T)phi;
  a.transport_angle[e] = (T)gamma;
  a.tangent_w[e] = (T)(a.weights[j] * kappa);
  for (int k = 0; k < a.orders; ++k) {
    double sn, cs;
    sincos(k * phi, &sn, &cs);
    a.angular[(e * a.orders + k) * 2] = (T)cs;
    a.angular[(e * a.orders + k) * 2 + 1] = (T)sn;
    sincos(k * gamma, &sn, &cs);
    a.transport[(e * a.orders + k) * 2] = (T)cs;
    a.transport[(e * a.orders + k) * 2 + 1] = (T)sn;
  }
}

template <typename T>
__global__ void fill_kernel(FillArgs<T> a) {
  const int lane = threadIdx.x & 31;
  const int64_t i = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= a.n_nodes) return;
  const Vec3 p = load3(a.nodes + 3 * i);
  const int64_t j0 = a.lo ? a.lo[i] : 0, j1 = a.hi ? a.hi[i] : a.n_nodes;
  int64_t e = a.row_ptr[i];
  for (int64_t base = j0; base < j1; base += 32) {
    const int64_t j = base + lane;
    Vec3 q = {0, 0, 0};
    bool in = false;
    if (j < j1) {
      q = load3(a.nodes + 3 * j);
      in = is_member(p, q, a.radius, a.chord2);
    }
    const unsigned mask = __ballot_sync(0xffffffffu, in);
    if (in) write_edge<T>(a, e + __popc(mask & ((1u << lane) - 1u)), i, j, p, q);
    e += __popc(mask);
  }
}

double chord_bound(double radius) {
  const double h = fmin((radius + 1e-6) * 0.5, 1.5707963267948966);
  const double c = 2.0 * sin(h) + 1e-9;
  return c * c;
}

}  // namespace
}  // namespace gmb

using namespace gmb;

extern "C" int gm_geometry_count(const double* nodes, int64_t n_nodes, const int64_t* cand_lo, const int64_t* cand_hi,
                                 double radius, int64_t* degree, void* stream) {
  GM_REQUIRE(n_nodes >= 0, GM_ERR_ARGUMENT, "gm_geometry_count: negative size");
  GM_REQUIRE(radius > 0.0 && radius < 3.141592653589793, GM_ERR_ARGUMENT, "gm_geometry_count: radius must lie in (0, pi)");
  if (n_nodes == 0) return GM_OK;
  GM_REQUIRE(nodes && degree, GM_ERR_ARGUMENT, "gm_geometry_count: null pointer");
  GM_REQUIRE((cand_lo == nullptr) == (cand_hi == nullptr), GM_ERR_ARGUMENT, "gm_geometry_count: give both candidate bounds or neither");
  const int threads = 256, per_block = threads / 32;
  count_kernel<<<(unsigned)((n_nodes + per_block - 1) / per_block), threads, 0, (cudaStream_t)stream>>>(
      nodes, n_nodes, cand_lo, cand_hi, radius, chord_bound(radius), degree);
  return launch_status("gm_geometry_count");
}

extern "C" int gm_geometry_fill(const double* nodes, const double* frames, const double* weights, int64_t n_nodes,
                                const int64_t* cand_lo, const int64_t* cand_hi, double radius, const int64_t* row_ptr,
                                int max_frequency, int dtype, int64_t* target, int64_t* source, void* distances,
                                void* log_coordinates, void* polar_angles, void* transport_angles, void* tangent_weights,
                                void* angular_phases, void* transport_phases, void* stream) {
  GM_REQUIRE(n_nodes >= 0 && max_frequency >= 0, GM_ERR_ARGUMENT, "gm_geometry_fill: bad sizes");
  GM_REQUIRE(dtype == GM_F32 || dtype == GM_F64, GM_ERR_UNSUPPORTED, "gm_geometry_fill: tables are float32 or float64");
  if (n_nodes == 0) return GM_OK;
  GM_REQUIRE(nodes && frames && weights && row_ptr, GM_ERR_ARGUMENT, "gm_geometry_fill: null input");
  GM_REQUIRE(target && source && distances && log_coordinates && polar_angles && transport_angles && tangent_weights &&
                 angular_phases && transport_phases,
             GM_ERR_ARGUMENT, "gm_geometry_fill: null output");
  const int threads = 256, per_block = threads / 32;
  const unsigned blocks = (unsigned)((n_nodes + per_block - 1) / per_block);
  auto run = [&](auto tag) {
    using T = decltype(tag);
    FillArgs<T> a{nodes, frames, weights, cand_lo, cand_hi, row_ptr, n_nodes, radius, chord_bound(radius), max_frequency + 1,
                  target, source, (T*)distances, (T*)log_coordinates, (T*)polar_angles, (T*)transport_angles,
                  (T*)tangent_weights, (T*)angular_phases, (T*)transport_phases};
    fill_kernel<T><<<blocks, threads, 0, (cudaStream_t)stream>>>(a);
    return launch_status("gm_geometry_fill");
  };
  return dtype == GM_F32 ? run(float()) : run(double());
}
