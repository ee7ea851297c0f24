// Data-parallel sum of the weight gradient over the GPUs of one node, by peer stores.
//
// The gw8 path shards by batch: forward and input gradient need no communication, the weight
// gradient (and the bias gradient) is a sum over the batch, so the per-rank results -- a few
// thousand floats -- are added once per step.  An NCCL all-reduce of 18 KB is pure latency, and
// issuing it from the host needs an event between the reduce and the input-gradient kernel and a
// stream wait before the next step, both of which break the chain of programmatic dependent
// launches the step is built from.  Here the exchange is one small kernel inside that chain, right
// after the weight-gradient reduce and before the input-gradient kernel, which does not wait for it
// and runs beside it:
//
//   push  each rank stores its vector into slot [rank] of EVERY rank's exchange buffer (plain
//         st.global to peer memory over NVLink; its own buffer included), makes the stores visible
//         system-wide and bumps a flag next to the slot;
//   sum   each rank waits until the flags of all ranks show this exchange, adds the slots IN RANK
//         ORDER and overwrites its vector.  The order is fixed, so all ranks hold bit-identical sums.
//
// A remote vector always lands in local memory before it is consumed; there is no remote load, no
// TMA and no multicast on peer memory.  Slots and flags are double-buffered by the parity of the
// exchange counter `seq`: a rank can push exchange k+1 only after its own sum k, which needed every
// rank's push k, so no rank can still be reading the slots of exchange k-1 when they are rewritten.
// The wait is bounded: after SPIO_WAIT_LIMIT_NS the kernel records SPIO_STATUS_PEER_TIMEOUT in the
// device's status word, leaves the vector untouched and returns.
//
// The reference has no multi-device support; this is the exchange its data-parallel use needs
// (one all-reduce of grad_weight per layer and step).
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <string>

#include "../../include/spio_b200.h"
#include "gw8_host.h"

namespace spio_b200 {

namespace {

constexpr int kMaxWorld = SPIO_DP_MAX_WORLD;
constexpr size_t kHeaderBytes = 256;  // flags[2][kMaxWorld] u32, two launch counters, then the slots

struct PeerTable {
  unsigned char* buf[kMaxWorld];
};

__device__ __forceinline__ unsigned* flag_of(unsigned char* buffer, unsigned parity, int src_rank) {
  return reinterpret_cast<unsigned*>(buffer) + parity * kMaxWorld + src_rank;
}

__device__ __forceinline__ float4* slot_of(unsigned char* buffer, unsigned parity, int world, int src_rank,
                                           size_t capacity) {
  return reinterpret_cast<float4*>(buffer + kHeaderBytes) +
         ((size_t)parity * world + src_rank) * (capacity / 4);
}

// One kernel does both halves of an exchange.  Its CTAs are small on purpose (128 threads, at most
// 32 registers each, a few bytes of shared memory): they fit on an SM beside a persistent CTA of
// the convolution kernels, so the exchange runs WHILE the input-gradient kernel that follows it in
// the stream computes (that kernel does not wait for it), instead of before or after it.
//
//   PUSH (CTA p): copy [a | b] (n_a + n_b floats, both multiples of 4) into slot [rank] of rank p,
//        make the stores visible system-wide, bump the flag next to the slot;
//   SUM  (CTA p): wait for the flags of all ranks in the local buffer, add slice p of the slots in
//        rank order, overwrite slice p of [a | b].
// With both phases in one launch, CTA p's push reads all of [a | b] while other CTAs' sums
// overwrite slices of it; a CTA therefore starts its sum only after ALL CTAs of the launch have
// finished their push (a counter in the local buffer's header, re-armed by the last CTA to leave).
// The sum itself never reads [a | b]: this rank's own copy is in slot [rank] like the others'.
enum { DP_PUSH = 1, DP_SUM = 2 };
constexpr int kThreads = 128;

__global__ void __launch_bounds__(kThreads, 16)  // 16 CTAs per SM: at most 32 registers per thread
dp_exchange_kernel(PeerTable peers, float* __restrict__ a, int n_a, float* __restrict__ b, int n_b, int rank,
                   int world, unsigned seq, size_t capacity, int phases, int* __restrict__ status) {
  __shared__ int ok;
  // the kernel after this one (the input-gradient kernel) may start at once; this one needs the
  // vector, which the kernel before it writes
  grid_dependency_launch_dependents();
  grid_dependency_wait();
  const int p = blockIdx.x;
  const unsigned parity = seq & 1u;
  const int na4 = n_a / 4, nb4 = n_b / 4, n4 = na4 + nb4;
  unsigned char* local = peers.buf[rank];
  unsigned* done = reinterpret_cast<unsigned*>(local) + 2 * kMaxWorld;  // CTAs of this launch that have pushed
  if (phases & DP_PUSH) {
    float4* dst = slot_of(peers.buf[p], parity, world, rank, capacity);
    const float4* a4 = reinterpret_cast<const float4*>(a);
    const float4* b4 = reinterpret_cast<const float4*>(b);
    for (int i = threadIdx.x; i < n4; i += kThreads) dst[i] = i < na4 ? a4[i] : b4[i - na4];
    __threadfence_system();  // every thread's stores are visible to the peer before the flag is
    __syncthreads();
    if (threadIdx.x == 0) {
      atomicAdd_system(flag_of(peers.buf[p], parity, rank), 1u);
      if (phases & DP_SUM) atomicAdd(done, 1u);
    }
  }
  if (!(phases & DP_SUM)) return;
  const unsigned expect = (seq >> 1) + 1u;  // flags count the exchanges of this parity so far
  if (threadIdx.x == 0) {
    int good = 1;
    u64 t0 = 0;
    auto waiting = [&](u32 it) {  // false once the limit has passed
      if ((it & 63u) != 0u) return true;
      const u64 now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      return now - t0 <= SPIO_WAIT_LIMIT_NS;
    };
    for (int r = 0; r < world && good; ++r) {
      volatile unsigned* f = flag_of(local, parity, r);
      for (u32 it = 1; (int)(*f - expect) < 0; ++it)
        if (!waiting(it)) {
          good = 0;
          break;
        }
    }
    // [a | b] may be overwritten only after every CTA of this launch has read it for its push
    if (phases & DP_PUSH) {
      volatile unsigned* d = done;
      for (u32 it = 1; good && *d < (unsigned)gridDim.x; ++it)
        if (!waiting(it)) good = 0;
    }
    __threadfence_system();  // the slots are read only after the flags were seen
    ok = good;
  }
  __syncthreads();
  if (!ok) {
    if (threadIdx.x == 0) atomicExch(status, (int)GW8_PEER_TIMEOUT);
    return;
  }
  const int i0 = (int)((long long)n4 * p / gridDim.x), i1 = (int)((long long)n4 * (p + 1) / gridDim.x);
  for (int i = i0 + threadIdx.x; i < i1; i += kThreads) {
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < world; ++r) {
      const float4 v = __ldcg(slot_of(local, parity, world, r, capacity) + i);  // L2: written by peers
      sum.x += v.x;
      sum.y += v.y;
      sum.z += v.z;
      sum.w += v.w;
    }
    if (i < na4)
      reinterpret_cast<float4*>(a)[i] = sum;
    else
      reinterpret_cast<float4*>(b)[i - na4] = sum;
  }
  // the last CTA to finish re-arms the counter for the next launch
  if (phases & DP_PUSH) {
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned* left = done + 1;
      if (atomicAdd(left, 1u) == gridDim.x - 1) {
        *done = 0;
        *left = 0;
      }
    }
  }
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
  // one CTA per rank: CTA p pushes to rank p and sums slice p
  return launch(reinterpret_cast<const void*>(&dp_exchange_kernel), world, args, stream);
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
  return kHeaderBytes + 2 * (size_t)world * cap4 * sizeof(float);
}

int spio_dp_buffer_alloc(size_t bytes, void** buffer, void* ipc_handle) {
  if (buffer == nullptr || bytes < kHeaderBytes) return jit_fail("data-parallel exchange: bad buffer size");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e == cudaSuccess) e = cudaMemset(p, 0, bytes);  // the flags start at zero
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
