// Halo exchange of the latitude-band decomposition: NCCL point-to-point groups issued from C.
//
// The reference has no distributed code; this file is new.  A rank's halo rows of a field laid out
// (batch, extended rows, nlon, D) are `batch` slabs per field.  gm_halo_move packs the slabs a neighbour needs into one
// buffer (one launch), gm_halo_exchange issues the messages -- ONE per neighbour and direction -- as one NCCL group on the
// caller's stream, and gm_halo_move unpacks (forward) or adds (backward) what arrived.  NCCL's cost per point-to-point
// operation (measured ~10 us on NVLink) is why the slabs are not sent one by one.  Nothing blocks the host; received rows
// live in this GPU's own memory; no kernel of this library reads a peer's memory.
//
// NCCL is not linked: the functions are looked up at run time in the libnccl.so.2 the process already holds (the one
// PyTorch loaded), so a machine without NCCL can still load this library for everything else.
#include <dlfcn.h>

#include <cstring>

#include "common.cuh"

namespace gmb {
namespace {

// the slice of NCCL's C API this file uses (stable since NCCL 2.7: nccl.h)
typedef struct ncclComm* NcclComm;
struct NcclUniqueId { char internal[128]; };
constexpr int NCCL_INT8 = 0;  // ncclInt8 / ncclChar: operations are counted in bytes

struct NcclApi {
  int (*GetUniqueId)(NcclUniqueId*) = nullptr;
  int (*CommInitRank)(NcclComm*, int, NcclUniqueId, int) = nullptr;
  int (*CommDestroy)(NcclComm) = nullptr;
  int (*CommGetAsyncError)(NcclComm, int*) = nullptr;
  int (*Send)(const void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
  int (*Recv)(void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  bool ok = false;
};

const NcclApi& nccl() {
  static NcclApi api = [] {
    NcclApi a;
    void* lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);  // the copy the process already uses, if any
    if (!lib) lib = dlopen("libnccl.so.2", RTLD_NOW);
    if (!lib) return a;
    auto sym = [&](const char* name) { return dlsym(lib, name); };
    a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(sym("ncclGetUniqueId"));
    a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(sym("ncclCommInitRank"));
    a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(sym("ncclCommDestroy"));
    a.CommGetAsyncError = reinterpret_cast<decltype(a.CommGetAsyncError)>(sym("ncclCommGetAsyncError"));
    a.Send = reinterpret_cast<decltype(a.Send)>(sym("ncclSend"));
    a.Recv = reinterpret_cast<decltype(a.Recv)>(sym("ncclRecv"));
    a.GroupStart = reinterpret_cast<decltype(a.GroupStart)>(sym("ncclGroupStart"));
    a.GroupEnd = reinterpret_cast<decltype(a.GroupEnd)>(sym("ncclGroupEnd"));
    a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(sym("ncclGetErrorString"));
    a.ok = a.GetUniqueId && a.CommInitRank && a.CommDestroy && a.CommGetAsyncError && a.Send && a.Recv && a.GroupStart && a.GroupEnd && a.GetErrorString;
    return a;
  }();
  return api;
}

#define GM_NCCL(call)                                                                                      \
  do {                                                                                                     \
    const int res__ = (call);                                                                              \
    if (res__ != 0) return ::gmb::fail(GM_ERR_CUDA, "%s: %s", #call, nccl().GetErrorString(res__));        \
  } while (0)

int require_nccl(const char* who) {
  GM_REQUIRE(nccl().ok, GM_ERR_UNSUPPORTED, "%s: libnccl.so.2 (NCCL >= 2.7) could not be loaded", who);
  return GM_OK;
}

// dst slab s (of `slabs`, dst_stride elements apart) += src slab s (src_stride apart), slab_elems elements each;
// 16-byte accesses where everything is aligned
template <typename T>
__global__ void accumulate_kernel(T* __restrict__ dst, const T* __restrict__ src, int64_t slab_elems, int64_t dst_stride, int64_t src_stride) {
  T* d = dst + (int64_t)blockIdx.y * dst_stride;
  const T* s = src + (int64_t)blockIdx.y * src_stride;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < slab_elems; i += (int64_t)gridDim.x * blockDim.x)
    st<T, typename Compute<T>::type>(d + i, ld<typename Compute<T>::type, T>(d + i) + ld<typename Compute<T>::type, T>(s + i));
}
__global__ void accumulate_bf16x8_kernel(__nv_bfloat16* __restrict__ dst, const __nv_bfloat16* __restrict__ src, int64_t slab_vec, int64_t dst_stride,
                                         int64_t src_stride) {
  uint4* d = reinterpret_cast<uint4*>(dst + (int64_t)blockIdx.y * dst_stride);
  const uint4* s = reinterpret_cast<const uint4*>(src + (int64_t)blockIdx.y * src_stride);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < slab_vec; i += (int64_t)gridDim.x * blockDim.x) {
    uint4 a = d[i];
    const uint4 b = __ldg(s + i);
    __nv_bfloat162* pa = reinterpret_cast<__nv_bfloat162*>(&a);
    const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 x = __bfloat1622float2(pa[k]), y = __bfloat1622float2(pb[k]);
      pa[k] = __floats2bfloat162_rn(x.x + y.x, x.y + y.y);
    }
    d[i] = a;
  }
}

// Rows r0 .. of every sample of up to 4 fields <-> one packed buffer (field, sample, rows): mode 0 packs the fields'
// slabs into the buffer, 1 unpacks the buffer into the fields, 2 adds the buffer to the fields.  16-byte units.
struct SlabFields { void* base[4]; };
template <int MODE>
__global__ void slab_move_kernel(SlabFields fields, uint4* __restrict__ packed, int64_t slab_vec, int64_t sample_vec, int bf16_add) {
  const int f = blockIdx.z, b = blockIdx.y;
  uint4* field = reinterpret_cast<uint4*>(fields.base[f]) + (int64_t)b * sample_vec;
  uint4* buf = packed + ((int64_t)f * gridDim.y + b) * slab_vec;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < slab_vec; i += (int64_t)gridDim.x * blockDim.x) {
    if (MODE == 0) {
      buf[i] = field[i];
    } else if (MODE == 1) {
      field[i] = buf[i];
    } else {
      uint4 a = field[i];
      const uint4 c = buf[i];
      if (bf16_add) {
        __nv_bfloat162* pa = reinterpret_cast<__nv_bfloat162*>(&a);
        const __nv_bfloat162* pc = reinterpret_cast<const __nv_bfloat162*>(&c);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 x = __bfloat1622float2(pa[k]), y = __bfloat1622float2(pc[k]);
          pa[k] = __floats2bfloat162_rn(x.x + y.x, x.y + y.y);
        }
      } else {
        float* pa = reinterpret_cast<float*>(&a);
        const float* pc = reinterpret_cast<const float*>(&c);
#pragma unroll
        for (int k = 0; k < 4; ++k) pa[k] += pc[k];
      }
      field[i] = a;
    }
  }
}

}  // namespace
}  // namespace gmb

using namespace gmb;

// mode 0: packed <- fields' slabs; 1: fields' slabs <- packed; 2: fields' slabs += packed.  `fields`: n_fields (<= 4) device
// pointers to the first element of sample 0's slab; sample_bytes apart per sample; slab_bytes each (multiples of 16).
extern "C" int gm_halo_move(int mode, void* const* fields, int n_fields, int64_t batch, int64_t slab_bytes, int64_t sample_bytes, void* packed,
                            int dtype, void* stream) {
  GM_REQUIRE(mode >= 0 && mode <= 2 && n_fields >= 1 && n_fields <= 4 && batch >= 1 && batch <= 65535, GM_ERR_ARGUMENT, "gm_halo_move: bad arguments");
  if (slab_bytes == 0) return GM_OK;
  GM_REQUIRE(fields && packed && slab_bytes > 0 && slab_bytes % 16 == 0 && sample_bytes % 16 == 0 && reinterpret_cast<uintptr_t>(packed) % 16 == 0,
             GM_ERR_ARGUMENT, "gm_halo_move: slabs must be whole 16-byte units on 16-byte boundaries");
  GM_REQUIRE(mode != 2 || dtype == GM_BF16 || dtype == GM_F32, GM_ERR_UNSUPPORTED, "gm_halo_move: sums in bf16 or fp32");
  SlabFields f{};
  for (int i = 0; i < n_fields; ++i) {
    GM_REQUIRE(fields[i] && reinterpret_cast<uintptr_t>(fields[i]) % 16 == 0, GM_ERR_ARGUMENT, "gm_halo_move: field %d is null or not on a 16-byte boundary", i);
    f.base[i] = fields[i];
  }
  const int64_t slab_vec = slab_bytes / 16, sample_vec = sample_bytes / 16;
  const unsigned bx = (unsigned)((slab_vec + 255) / 256 < 64 ? (slab_vec + 255) / 256 : 64);
  dim3 grid(bx, (unsigned)batch, (unsigned)n_fields);
  cudaStream_t cs = (cudaStream_t)stream;
  if (mode == 0) slab_move_kernel<0><<<grid, 256, 0, cs>>>(f, (uint4*)packed, slab_vec, sample_vec, 0);
  else if (mode == 1) slab_move_kernel<1><<<grid, 256, 0, cs>>>(f, (uint4*)packed, slab_vec, sample_vec, 0);
  else slab_move_kernel<2><<<grid, 256, 0, cs>>>(f, (uint4*)packed, slab_vec, sample_vec, dtype == GM_BF16 ? 1 : 0);
  return launch_status("gm_halo_move");
}

extern "C" int gm_halo_unique_id(void* id128) {
  GM_REQUIRE(id128, GM_ERR_ARGUMENT, "gm_halo_unique_id: null pointer");
  int status = require_nccl("gm_halo_unique_id");
  if (status != GM_OK) return status;
  NcclUniqueId id;
  GM_NCCL(nccl().GetUniqueId(&id));
  memcpy(id128, &id, sizeof(id));
  return GM_OK;
}

extern "C" int gm_halo_comm_create(const void* id128, int rank, int world, void** comm) {
  GM_REQUIRE(id128 && comm && world >= 1 && rank >= 0 && rank < world, GM_ERR_ARGUMENT, "gm_halo_comm_create: bad arguments");
  int status = require_nccl("gm_halo_comm_create");
  if (status != GM_OK) return status;
  NcclUniqueId id;
  memcpy(&id, id128, sizeof(id));
  NcclComm c = nullptr;
  GM_NCCL(nccl().CommInitRank(&c, world, id, rank));  // binds the communicator to the current device
  *comm = c;
  return GM_OK;
}

extern "C" int gm_halo_comm_destroy(void* comm) {
  if (!comm) return GM_OK;
  int status = require_nccl("gm_halo_comm_destroy");
  if (status != GM_OK) return status;
  GM_NCCL(nccl().CommDestroy(static_cast<NcclComm>(comm)));
  return GM_OK;
}

extern "C" int gm_halo_comm_error(void* comm, int* async_error) {
  GM_REQUIRE(comm && async_error, GM_ERR_ARGUMENT, "gm_halo_comm_error: null pointer");
  int status = require_nccl("gm_halo_comm_error");
  if (status != GM_OK) return status;
  GM_NCCL(nccl().CommGetAsyncError(static_cast<NcclComm>(comm), async_error));
  return GM_OK;
}

extern "C" int gm_halo_exchange(void* comm, int n_ops, const int* peers, const int* sends, void* const* pointers, const int64_t* nbytes,
                                void* stream) {
  GM_REQUIRE(comm && n_ops >= 0 && (n_ops == 0 || (peers && sends && pointers && nbytes)), GM_ERR_ARGUMENT, "gm_halo_exchange: bad arguments");
  if (n_ops == 0) return GM_OK;
  int status = require_nccl("gm_halo_exchange");
  if (status != GM_OK) return status;
  for (int i = 0; i < n_ops; ++i)
    GM_REQUIRE(pointers[i] && nbytes[i] > 0 && peers[i] >= 0, GM_ERR_ARGUMENT, "gm_halo_exchange: operation %d has a null pointer, no bytes or no peer", i);
  cudaStream_t cs = (cudaStream_t)stream;
  NcclComm c = static_cast<NcclComm>(comm);
  GM_NCCL(nccl().GroupStart());
  int first_error = 0;
  for (int i = 0; i < n_ops && first_error == 0; ++i)
    first_error = sends[i] ? nccl().Send(pointers[i], (size_t)nbytes[i], NCCL_INT8, peers[i], c, cs)
                           : nccl().Recv(pointers[i], (size_t)nbytes[i], NCCL_INT8, peers[i], c, cs);
  const int end = nccl().GroupEnd();  // always closed, also after a failed call inside it
  if (first_error != 0) return fail(GM_ERR_CUDA, "gm_halo_exchange: ncclSend / ncclRecv: %s", nccl().GetErrorString(first_error));
  if (end != 0) return fail(GM_ERR_CUDA, "gm_halo_exchange: ncclGroupEnd: %s", nccl().GetErrorString(end));
  return GM_OK;
}

extern "C" int gm_halo_accumulate(void* dst, const void* src, int64_t slabs, int64_t slab_elems, int64_t dst_stride, int64_t src_stride,
                                  int dtype, void* stream) {
  GM_REQUIRE(slabs >= 0 && slab_elems >= 0 && slabs <= 65535, GM_ERR_ARGUMENT, "gm_halo_accumulate: bad sizes");
  if (slabs == 0 || slab_elems == 0) return GM_OK;
  GM_REQUIRE(dst && src, GM_ERR_ARGUMENT, "gm_halo_accumulate: null pointer");
  cudaStream_t cs = (cudaStream_t)stream;
  const bool vec = dtype == GM_BF16 && slab_elems % 8 == 0 && dst_stride % 8 == 0 && src_stride % 8 == 0 &&
                   reinterpret_cast<uintptr_t>(dst) % 16 == 0 && reinterpret_cast<uintptr_t>(src) % 16 == 0;
  const int64_t work = vec ? slab_elems / 8 : slab_elems;
  const unsigned bx = (unsigned)((work + 255) / 256 < 1024 ? (work + 255) / 256 : 1024);
  dim3 grid(bx, (unsigned)slabs);
  if (vec) accumulate_bf16x8_kernel<<<grid, 256, 0, cs>>>((__nv_bfloat16*)dst, (const __nv_bfloat16*)src, work, dst_stride, src_stride);
  else if (dtype == GM_BF16) accumulate_kernel<<<grid, 256, 0, cs>>>((__nv_bfloat16*)dst, (const __nv_bfloat16*)src, slab_elems, dst_stride, src_stride);
  else if (dtype == GM_F32) accumulate_kernel<<<grid, 256, 0, cs>>>((float*)dst, (const float*)src, slab_elems, dst_stride, src_stride);
  else if (dtype == GM_F64) accumulate_kernel<<<grid, 256, 0, cs>>>((double*)dst, (const double*)src, slab_elems, dst_stride, src_stride);
  else return fail(GM_ERR_ARGUMENT, "gm_halo_accumulate: unknown dtype %d", dtype);
  return launch_status("gm_halo_accumulate");
}
