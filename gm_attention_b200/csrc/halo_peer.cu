// Halo exchange through peer memory: the sender's pack kernel stores the rows a neighbour needs straight into the
// neighbour's receive buffer over NVLink and then raises a flag there; the neighbour's landing kernel waits for the flag
// (with a bound) and unpacks or adds.  One launch to send to a neighbour, one to land what it sent; no library in between.
//
// The reference has no distributed code; this file is new.  It is the fast path of parallel.PeerHaloExchanger on
// machines whose GPUs can map each other's memory; the NCCL path of halo.cu serves everywhere else.
//
// Memory: every rank allocates ONE block (gm_peer_alloc: cudaMalloc, zeroed) holding its receive buffers and its flag
// words, and publishes the block's IPC handle; a neighbour maps it (gm_peer_open) and from then on only STORES into it:
// no kernel here loads from a peer's memory, no copy engine, no multicast, no collective.
//
// Protocol, per (neighbour, kind of exchange), with `step` counting that pair's exchanges from 1:
//   sender    gm_peer_send:  wait until the receiver acknowledged step - 1 (its buffer is free again; the word is in the
//             SENDER's block, stored by the receiver); copy the rows into the receiver's buffer; the last CTA to finish
//             (a ticket counter after a system-scope fence by every thread) stores `step` into the receiver's data flag.
//   receiver  gm_peer_land:  wait until its data flag reached `step`; unpack / add the buffer; the last CTA stores `step`
//             into the sender's acknowledgement word.
// Every rank sends before it lands, a send waits only for an acknowledgement of the PREVIOUS step, and a landing only for
// data of THIS step, so the waits cannot form a cycle.  Each wait is bounded (about a second of polling with nanosleep);
// a wait that runs out sets the device word behind gm_peer_error, skips the kernel's work and returns: nothing hangs,
// the host reads the word.  The waiting kernels of two ranks never share a GPU (one process per GPU).
#include <cstring>

#include "common.cuh"

namespace gmb {
namespace {

__device__ unsigned g_peer_error = 0;  // 1: a send waited too long for an acknowledgement; 2: a landing for its data

constexpr unsigned POLL_LIMIT = 4u << 20;  // x ~250 ns of nanosleep: about a second

__device__ __forceinline__ unsigned load_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void store_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// true when *flag reached `want` within the bound (thread 0 polls; the verdict is shared through shared memory)
__device__ __forceinline__ bool wait_for(const unsigned* flag, unsigned want, unsigned code) {
  __shared__ int ok;
  if (threadIdx.x == 0) {
    int reached = 0;
    for (unsigned spin = 0; spin < POLL_LIMIT; ++spin) {
      if ((int)(load_acquire_sys(flag) - want) >= 0) { reached = 1; break; }
      __nanosleep(250);
    }
    if (!reached) atomicMax(&g_peer_error, code);
    ok = reached;
  }
  __syncthreads();
  return ok != 0;
}

// the last CTA of the grid to arrive (after every thread's system-scope fence) stores `value` to *flag
__device__ __forceinline__ void signal_when_all_done(unsigned* ticket, unsigned total, unsigned* flag, unsigned value) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned mine = atomicAdd(ticket, 1u);
    if (mine == total - 1) {
      *ticket = 0;  // ready for the next launch on this stream
      __threadfence_system();
      if (flag) store_release_sys(flag, value);
    }
  }
}

// One neighbour's share of a launch: the rows of up to 4 fields, the buffer they go to / come from, and the words of the
// protocol.  A launch serves one or two neighbours (a band has at most two sides), so that their transfers overlap.
struct PeerLane {
  void* base[4];          // sample 0's slab of each field
  uint4* buffer;          // layout (field, sample, slab), 16-byte units
  int64_t slab_vec;
  const unsigned* wait_flag;
  unsigned wait_value;
  unsigned* ticket;
  unsigned* signal_flag;
  unsigned step;
};
struct PeerLanes { PeerLane lane[2]; };

// MODE 0: fields' slabs -> remote buffer, then the remote data flag.  MODE 1 / 2: local buffer -> fields' slabs
// (copy / add), then the remote acknowledgement.  blockIdx.z = lane * n_fields + field.
template <int MODE>
__global__ void peer_kernel(PeerLanes lanes, int n_fields, int64_t sample_vec, int bf16_add) {
  const PeerLane& L = lanes.lane[blockIdx.z / n_fields];
  const bool ready = wait_for(L.wait_flag, L.wait_value, MODE == 0 ? 1u : 2u);
  const int f = blockIdx.z % n_fields, b = blockIdx.y;
  const int64_t slab_vec = L.slab_vec;
  uint4* field = reinterpret_cast<uint4*>(L.base[f]) + (int64_t)b * sample_vec;
  uint4* buf = L.buffer + ((int64_t)f * gridDim.y + b) * slab_vec;
  // a wait that ran out: no data moves and nothing is signalled (the ticket is still taken, so the counter stays whole)
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; ready && i < slab_vec; i += (int64_t)gridDim.x * blockDim.x) {
    if (MODE == 0) {
      buf[i] = field[i];
    } else if (MODE == 1) {
      field[i] = __ldcg(buf + i);  // written by the neighbour: read from L2, where its stores arrive
    } else {
      uint4 a = field[i];
      const uint4 c = __ldcg(buf + i);
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
  signal_when_all_done(L.ticket, gridDim.x * gridDim.y * n_fields, ready ? L.signal_flag : nullptr, L.step);
}

// n_lanes neighbours (1 or 2) in one launch.  fields: n_lanes * n_fields pointers, lane-major.
int launch_peer(int mode, int n_lanes, void* const* fields, int n_fields, int64_t batch, const int64_t* slab_bytes, int64_t sample_bytes,
                void* const* buffers, int dtype, const uint32_t* const* wait_flags, int wait_offset, uint32_t* const* tickets,
                uint32_t* const* signal_flags, const uint32_t* steps, void* stream, const char* what) {
  GM_REQUIRE(n_lanes >= 1 && n_lanes <= 2 && n_fields >= 1 && n_fields <= 4 && batch >= 1 && batch <= 65535, GM_ERR_ARGUMENT, "%s: bad arguments", what);
  GM_REQUIRE(fields && slab_bytes && buffers && wait_flags && tickets && signal_flags && steps && sample_bytes % 16 == 0, GM_ERR_ARGUMENT,
             "%s: null pointer or a sample stride that is not a multiple of 16 bytes", what);
  GM_REQUIRE(mode != 2 || dtype == GM_BF16 || dtype == GM_F32, GM_ERR_UNSUPPORTED, "%s: sums in bf16 or fp32", what);
  PeerLanes lanes{};
  int64_t widest = 0;
  for (int l = 0; l < n_lanes; ++l) {
    GM_REQUIRE(slab_bytes[l] > 0 && slab_bytes[l] % 16 == 0 && buffers[l] && reinterpret_cast<uintptr_t>(buffers[l]) % 16 == 0, GM_ERR_ARGUMENT,
               "%s: slabs must be whole 16-byte units on 16-byte boundaries", what);
    GM_REQUIRE(wait_flags[l] && tickets[l] && signal_flags[l], GM_ERR_ARGUMENT, "%s: null flag word", what);
    PeerLane& L = lanes.lane[l];
    for (int i = 0; i < n_fields; ++i) {
      void* base = fields[l * n_fields + i];
      GM_REQUIRE(base && reinterpret_cast<uintptr_t>(base) % 16 == 0, GM_ERR_ARGUMENT, "%s: field %d is null or not on a 16-byte boundary", what, i);
      L.base[i] = base;
    }
    L.buffer = static_cast<uint4*>(buffers[l]);
    L.slab_vec = slab_bytes[l] / 16;
    L.wait_flag = wait_flags[l];
    L.wait_value = steps[l] - (unsigned)wait_offset;
    L.ticket = tickets[l];
    L.signal_flag = signal_flags[l];
    L.step = steps[l];
    widest = L.slab_vec > widest ? L.slab_vec : widest;
  }
  const unsigned bx = (unsigned)((widest + 255) / 256 < 32 ? (widest + 255) / 256 : 32);
  dim3 grid(bx, (unsigned)batch, (unsigned)(n_fields * n_lanes));
  cudaStream_t cs = (cudaStream_t)stream;
  const int64_t sample_vec = sample_bytes / 16;
  if (mode == 0) peer_kernel<0><<<grid, 256, 0, cs>>>(lanes, n_fields, sample_vec, 0);
  else if (mode == 1) peer_kernel<1><<<grid, 256, 0, cs>>>(lanes, n_fields, sample_vec, 0);
  else peer_kernel<2><<<grid, 256, 0, cs>>>(lanes, n_fields, sample_vec, dtype == GM_BF16 ? 1 : 0);
  return launch_status(what);
}

}  // namespace
}  // namespace gmb

using namespace gmb;

// A zeroed device block other processes may map, and its 64-byte IPC handle.
extern "C" int gm_peer_alloc(int64_t bytes, void** block, void* handle64) {
  GM_REQUIRE(bytes > 0 && block && handle64, GM_ERR_ARGUMENT, "gm_peer_alloc: bad arguments");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 bytes");
  void* p = nullptr;
  GM_CUDA(cudaMalloc(&p, (size_t)bytes));
  cudaError_t err = cudaMemset(p, 0, (size_t)bytes);
  cudaIpcMemHandle_t handle;
  if (err == cudaSuccess) err = cudaIpcGetMemHandle(&handle, p);
  if (err != cudaSuccess) {
    cudaFree(p);
    return fail(GM_ERR_CUDA, "gm_peer_alloc: %s", cudaGetErrorString(err));
  }
  std::memcpy(handle64, &handle, 64);
  *block = p;
  return GM_OK;
}

extern "C" int gm_peer_free(void* block) {
  if (block) GM_CUDA(cudaFree(block));
  return GM_OK;
}

// Maps another process's block into this process (peer access between the two devices is enabled on demand).
extern "C" int gm_peer_open(const void* handle64, void** mapped) {
  GM_REQUIRE(handle64 && mapped, GM_ERR_ARGUMENT, "gm_peer_open: null pointer");
  cudaIpcMemHandle_t handle;
  std::memcpy(&handle, handle64, 64);
  cudaError_t err = cudaIpcOpenMemHandle(mapped, handle, cudaIpcMemLazyEnablePeerAccess);
  if (err != cudaSuccess) {
    cudaGetLastError();
    return fail(GM_ERR_UNSUPPORTED, "gm_peer_open: %s (no peer access between these devices?)", cudaGetErrorString(err));
  }
  return GM_OK;
}

extern "C" int gm_peer_close(void* mapped) {
  if (mapped) GM_CUDA(cudaIpcCloseMemHandle(mapped));
  return GM_OK;
}

// Sender side, one neighbour: rows of up to 4 fields (fields[i]: sample 0's slab; batch slabs sample_bytes apart,
// slab_bytes each) -> remote_buffer in the neighbour's block, then remote_data_flag = step.  Waits first until
// *local_ack >= step - 1.  local_ticket: a zeroed word of this rank's own block, private to this (neighbour, kind).
extern "C" int gm_peer_send(void* const* fields, int n_fields, int64_t batch, int64_t slab_bytes, int64_t sample_bytes, void* remote_buffer,
                            const uint32_t* local_ack, uint32_t* local_ticket, uint32_t* remote_data_flag, uint32_t step, void* stream) {
  if (slab_bytes == 0) return GM_OK;
  return launch_peer(0, 1, fields, n_fields, batch, &slab_bytes, sample_bytes, &remote_buffer, GM_F32, &local_ack, 1, &local_ticket,
                     &remote_data_flag, &step, stream, "gm_peer_send");
}

// Receiver side, one neighbour: waits until *local_data_flag >= step, then fields' slabs = local_buffer (add == 0) or
// += local_buffer (add != 0; GM_BF16 or GM_F32), then remote_ack = step in the sender's block.
extern "C" int gm_peer_land(void* const* fields, int n_fields, int64_t batch, int64_t slab_bytes, int64_t sample_bytes, void* local_buffer,
                            int add, int dtype, const uint32_t* local_data_flag, uint32_t* local_ticket, uint32_t* remote_ack, uint32_t step,
                            void* stream) {
  if (slab_bytes == 0) return GM_OK;
  return launch_peer(add ? 2 : 1, 1, fields, n_fields, batch, &slab_bytes, sample_bytes, &local_buffer, dtype, &local_data_flag, 0, &local_ticket,
                     &remote_ack, &step, stream, "gm_peer_land");
}

// The same for n_lanes (1 or 2) neighbours in ONE launch, so that the transfers to / from both sides of a band overlap:
// every per-neighbour argument is an array of n_lanes; fields holds n_lanes * n_fields pointers, neighbour-major.
extern "C" int gm_peer_send_many(int n_lanes, void* const* fields, int n_fields, int64_t batch, const int64_t* slab_bytes, int64_t sample_bytes,
                                 void* const* remote_buffers, const uint32_t* const* local_acks, uint32_t* const* local_tickets,
                                 uint32_t* const* remote_data_flags, const uint32_t* steps, void* stream) {
  return launch_peer(0, n_lanes, fields, n_fields, batch, slab_bytes, sample_bytes, remote_buffers, GM_F32, local_acks, 1, local_tickets,
                     remote_data_flags, steps, stream, "gm_peer_send_many");
}

extern "C" int gm_peer_land_many(int n_lanes, void* const* fields, int n_fields, int64_t batch, const int64_t* slab_bytes, int64_t sample_bytes,
                                 void* const* local_buffers, int add, int dtype, const uint32_t* const* local_data_flags,
                                 uint32_t* const* local_tickets, uint32_t* const* remote_acks, const uint32_t* steps, void* stream) {
  return launch_peer(add ? 2 : 1, n_lanes, fields, n_fields, batch, slab_bytes, sample_bytes, local_buffers, dtype, local_data_flags, 0,
                     local_tickets, remote_acks, steps, stream, "gm_peer_land_many");
}

// 0: no wait of gm_peer_send / gm_peer_land has run out on the current device; 1: a send's; 2: a landing's.
extern "C" int gm_peer_error(int* code) {
  GM_REQUIRE(code, GM_ERR_ARGUMENT, "gm_peer_error: null pointer");
  unsigned v = 0;
  GM_CUDA(cudaMemcpyFromSymbol(&v, g_peer_error, sizeof(v)));
  *code = (int)v;
  return GM_OK;
}
