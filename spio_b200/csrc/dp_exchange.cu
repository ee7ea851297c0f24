// Data-parallel sum of the weight gradient over the GPUs of one node, by peer stores.
//
// The gw8 path shards by batch: forward and input gradient need no communication, the weight
// gradient (and the bias gradient) is a sum over the batch, so the per-rank results -- a few
// thousand floats -- are added once per step.  An NCCL all-reduce of 18 KB is pure latency, and
// issuing it from the host needs an event between the reduce and the input-gradient kernel and a
// stream wait before the next step, both of which break the chain of programmatic dependent
// launches the step is built from.  Here the exchange is one small kernel inside that chain, right
// after the weight-gradient reduce:
//
//   push  every thread owns four floats of the vector; it stores them, each paired with the tag
//         of this exchange, into slot [rank] of EVERY rank's exchange buffer (plain 16-byte
//         st.global to peer memory over NVLink; its own buffer included);
//   sum   the same thread polls the same four floats of all ranks' slots in its own buffer until
//         their tags show this exchange, adds them IN RANK ORDER and overwrites its four floats.
//         The order is fixed, so all ranks hold bit-identical sums.
//
// A word of the buffer is 8 bytes, {float, tag}, written by one store: data and tag arrive
// together, so a matching tag IS the data being there.  No flags, no memory fences, no atomics
// (system-scope fences cost several microseconds each on this machine; a first version with a
// fence and a flag per slot took 10 us where this one takes 2-3).  It is the idea of NCCL's
// low-latency protocol applied to an all-to-all of one small vector.
//
// A remote vector always lands in local memory before it is consumed; there is no remote load, no
// TMA and no multicast on peer memory.  Slots are double-buffered by the parity of the exchange
// counter `seq`: a rank can push exchange k+1 only after its own sum k, which needed every rank's
// push k, so no rank can still be reading the slots of exchange k-1 when they are rewritten.  The
// wait is bounded: after SPIO_WAIT_LIMIT_NS the kernel records SPIO_STATUS_PEER_TIMEOUT in the
// device's status word, leaves its floats untouched and returns.
//
// The reference has no multi-device support; this is the exchange its data-parallel use needs
// (one all-reduce of grad_weight per layer and step).
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>

#include "../../include/spio_b200.h"
#include "gw8_host.h"

namespace spio_b200 {

namespace {

constexpr int kMaxWorld = SPIO_DP_MAX_WORLD;
constexpr size_t kHeaderBytes = 256;  // reserved

struct PeerTable {
  unsigned char* buf[kMaxWorld];
};

// Slot of source rank `src` for exchanges of the given parity: capacity words of {float, tag},
// addressed in units of two words (16 bytes).
__device__ __forceinline__ uint4* slot_of(unsigned char* buffer, unsigned parity, int world, int src,
                                          size_t capacity) {
  return reinterpret_cast<uint4*>(buffer + kHeaderBytes) + ((size_t)parity * world + src) * (capacity / 2);
}

__device__ __forceinline__ void store_words(uint4* p, float x, float y, unsigned tag) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(__float_as_uint(x)), "r"(tag),
               "r"(__float_as_uint(y)), "r"(tag)
               : "memory");
}

__device__ __forceinline__ uint4 load_words(const uint4* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// The kernel's CTAs are small (128 threads, at most 32 registers each, no shared memory), but they do
// not share an SM with a persistent CTA of the input-gradient kernel: measured on 8 GPUs, where a CTA of
// this kernel waits longest for its peers, the input-gradient CTAs of the SMs it sat on started only when
// it had finished, and the step took 135 us instead of 115 us.  The combined backward call therefore
// launches the input-gradient kernel on as many SMs fewer as this kernel has CTAs (dp_exchange_ctas).
enum { DP_PUSH = 1, DP_SUM = 2 };
constexpr int kThreads = 128;

__global__ void __launch_bounds__(kThreads, 16)  // 16 CTAs per SM: at most 32 registers per thread
dp_exchange_kernel(PeerTable peers, float* __restrict__ a, int n_a, float* __restrict__ b, int n_b, int rank,
                   int world, unsigned seq, size_t capacity, int phases, int* __restrict__ status) {
  // the kernel after this one may start at once; this one needs the vector, which the kernel
  // before it writes
  grid_dependency_launch_dependents();
  grid_dependency_wait();
  const unsigned parity = seq & 1u;
  const unsigned tag = seq + 1u;  // never 0, the value the buffers start with
  const int na4 = n_a / 4, nb4 = n_b / 4;
  const int i = blockIdx.x * kThreads + threadIdx.x;  // this thread's four floats
  if (i >= na4 + nb4) return;
  float4* mine = i < na4 ? reinterpret_cast<float4*>(a) + i : reinterpret_cast<float4*>(b) + (i - na4);
  if (phases & DP_PUSH) {
    const float4 v = __ldcg(mine);
    for (int p = 0; p < world; ++p) {
      uint4* dst = slot_of(peers.buf[p], parity, world, rank, capacity) + 2 * i;
      store_words(dst, v.x, v.y, tag);
      store_words(dst + 1, v.z, v.w, tag);
    }
  }
  if (!(phases & DP_SUM)) return;
  float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
  u64 t0 = 0;
  for (int r = 0; r < world; ++r) {
    const uint4* src = slot_of(peers.buf[rank], parity, world, r, capacity) + 2 * i;
    uint4 lo = load_words(src), hi = load_words(src + 1);
    for (u32 it = 1; lo.y != tag || lo.w != tag || hi.y != tag || hi.w != tag; ++it) {
      if ((it & 63u) == 0u) {
        const u64 now = globaltimer_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > SPIO_WAIT_LIMIT_NS) {
          atomicExch(status, (int)GW8_PEER_TIMEOUT);
          return;
        }
      }
      // a waiting warp shares its SM with a convolution CTA: it steps aside between polls
      __nanosleep(100);
      lo = load_words(src);
      hi = load_words(src + 1);
    }
    sum.x += __uint_as_float(lo.x);
    sum.y += __uint_as_float(lo.z);
    sum.z += __uint_as_float(hi.x);
    sum.w += __uint_as_float(hi.z);
  }
  *mine = sum;
}

int launch(const void* func, int grid, void** args, cudaStream_t stream) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = gw8_pdl_enabled() ? 1 : 0;
  const cudaError_t e = cudaLaunchKernelExC(&cfg, func, args);
  if (e != cudaSuccess) return jit_fail(std::string("CUDA error: ") + cudaGetErrorString(e) + " (data-parallel exchange)");
  return 0;
}

int check(const spio_dp_exchange* dp, const float* a, size_t n_a, const float* b, size_t n_b) {
  if (dp == nullptr || dp->buffers == nullptr) return jit_fail("data-parallel exchange: NULL argument");
  if (dp->world < 1 || dp->world > kMaxWorld || dp->rank < 0 || dp->rank >= dp->world)
    return jit_fail("data-parallel exchange: rank / world out of range (world <= SPIO_DP_MAX_WORLD)");
  if (a == nullptr || n_a == 0 || n_a % 4 || n_b % 4 || (n_b != 0 && b == nullptr))
    return jit_fail("data-parallel exchange: vectors must be non-empty multiples of 4 floats");
  if ((reinterpret_cast<size_t>(a) & 15u) || (reinterpret_cast<size_t>(b) & 15u))
    return jit_fail("data-parallel exchange: vectors must be 16-byte aligned");
  if (n_a + n_b > dp->capacity || dp->capacity % 4)
    return jit_fail("data-parallel exchange: the vector exceeds the capacity the buffers were sized for");
  for (int r = 0; r < dp->world; ++r)
    if (dp->buffers[r] == nullptr) return jit_fail("data-parallel exchange: a peer buffer is NULL");
  return 0;
}

}  // namespace

// CTAs of one exchange of n floats.
int dp_exchange_ctas(size_t n_floats) { return (int)((n_floats / 4 + kThreads - 1) / kThreads); }

int dp_exchange(const spio_dp_exchange* dp, float* a, size_t n_a, float* b, size_t n_b, int phases,
                cudaStream_t stream) {
  if (check(dp, a, n_a, b, n_b)) return 1;
  int* status = nullptr;
  if (gw8_status_pointer(&status)) return 1;
  PeerTable peers{};
  for (int r = 0; r < dp->world; ++r) peers.buf[r] = static_cast<unsigned char*>(dp->buffers[r]);
  int na = (int)n_a, nb = (int)n_b, rank = dp->rank, world = dp->world;
  unsigned seq = dp->seq;
  size_t capacity = dp->capacity;
  void* args[] = {&peers, &a, &na, &b, &nb, &rank, &world, &seq, &capacity, &phases, &status};
  const int grid = (int)((n_a + n_b) / 4 + kThreads - 1) / kThreads;  // four floats per thread
  return launch(reinterpret_cast<const void*>(&dp_exchange_kernel), grid, args, stream);
}

int dp_push(const spio_dp_exchange* dp, const float* a, size_t n_a, const float* b, size_t n_b,
            cudaStream_t stream) {
  return dp_exchange(dp, const_cast<float*>(a), n_a, const_cast<float*>(b), n_b, DP_PUSH, stream);
}

int dp_sum(const spio_dp_exchange* dp, float* a, size_t n_a, float* b, size_t n_b, cudaStream_t stream) {
  return dp_exchange(dp, a, n_a, b, n_b, DP_SUM, stream);
}

int dp_allreduce(const spio_dp_exchange* dp, float* a, size_t n_a, float* b, size_t n_b, cudaStream_t stream) {
  return dp_exchange(dp, a, n_a, b, n_b, DP_PUSH | DP_SUM, stream);
}

}  // namespace spio_b200

using namespace spio_b200;

extern "C" {

size_t spio_dp_buffer_bytes(int world, size_t capacity) {
  if (world < 1 || world > kMaxWorld) return 0;
  const size_t cap4 = (capacity + 3) / 4 * 4;
  return kHeaderBytes + 2 * (size_t)world * cap4 * 8;  // a word is {float, tag}
}

int spio_dp_buffer_alloc(size_t bytes, void** buffer, void* ipc_handle) {
  if (buffer == nullptr || bytes < kHeaderBytes) return jit_fail("data-parallel exchange: bad buffer size");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e == cudaSuccess) e = cudaMemset(p, 0, bytes);  // tag 0: nothing has arrived
  if (e == cudaSuccess && ipc_handle != nullptr) {
    static_assert(sizeof(cudaIpcMemHandle_t) == SPIO_DP_IPC_HANDLE_BYTES, "IPC handle size");
    e = cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(ipc_handle), p);
  }
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    if (p) cudaFree(p);
    return jit_fail(std::string("CUDA error: ") + cudaGetErrorString(e) + " (spio_dp_buffer_alloc)");
  }
  *buffer = p;
  return 0;
}

int spio_dp_buffer_open(const void* ipc_handle, void** peer_buffer) {
  if (ipc_handle == nullptr || peer_buffer == nullptr) return jit_fail("data-parallel exchange: NULL argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, ipc_handle, sizeof h);
  void* p = nullptr;
  const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess)
    return jit_fail(std::string("CUDA error: ") + cudaGetErrorString(e) + " (cudaIpcOpenMemHandle)");
  *peer_buffer = p;
  return 0;
}

int spio_dp_buffer_close(void* peer_buffer) {
  if (peer_buffer == nullptr) return 0;
  const cudaError_t e = cudaIpcCloseMemHandle(peer_buffer);
  return e == cudaSuccess ? 0 : jit_fail(std::string("CUDA error: ") + cudaGetErrorString(e));
}

int spio_dp_buffer_free(void* buffer) {
  if (buffer == nullptr) return 0;
  const cudaError_t e = cudaFree(buffer);
  return e == cudaSuccess ? 0 : jit_fail(std::string("CUDA error: ") + cudaGetErrorString(e));
}

int spio_dp_push(const spio_dp_exchange* dp, const float* a, size_t n_a, const float* b, size_t n_b,
                 void* stream) {
  return dp_push(dp, a, n_a, b, n_b, (cudaStream_t)stream);
}

int spio_dp_sum(const spio_dp_exchange* dp, float* a, size_t n_a, float* b, size_t n_b, void* stream) {
  return dp_sum(dp, a, n_a, b, n_b, (cudaStream_t)stream);
}

int spio_dp_allreduce(const spio_dp_exchange* dp, float* a, size_t n_a, float* b, size_t n_b, void* stream) {
  return dp_allreduce(dp, a, n_a, b, n_b, (cudaStream_t)stream);
}

}  // extern "C"
