// Thin inline-PTX wrappers for the sm_100a building blocks the gw8 kernels use:
// mbarrier (with time-bounded waits), TMA tiled loads/stores (never multicast),
// tcgen05 tensor-core instructions with accumulators in tensor memory,
// ldmatrix / stmatrix and warp-level mma.sync with fp32 accumulation.
//
// The file is device-only and includes no host headers, so the same text compiles
// under nvcc (ahead of time) and under NVRTC (just in time).
//
// Replaces the Ampere-era wrappers of the reference: spio/include/spio/memory.cuh:17-24
// (cp.async zfill), spio/include/spio/ldmatrix.cuh:16-109, spio/include/spio/mma.cuh:33-42.
#pragma once

namespace spio_b200 {

typedef unsigned int u32;
typedef unsigned long long u64;

// A wait gives up after this many nanoseconds of wall time and reports failure
// instead of spinning for ever.
#ifndef SPIO_WAIT_LIMIT_NS
#define SPIO_WAIT_LIMIT_NS 2000000000ull
#endif

__device__ __forceinline__ u32 smem_u32(const void* p) {
  return (u32)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ u64 globaltimer_ns() {
  u64 t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// An addition the compiler can neither hoist out of a loop nor fold with its neighbours.
// Used where precomputing every loop-invariant address would cost more registers than the
// adds it saves.
__device__ __forceinline__ u32 opaque_add(u32 a, u32 b) {
  u32 r;
  asm volatile("add.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

// ---------------------------------------------------------------- programmatic dependent launch

// When a kernel is launched with the programmatic-stream-serialization attribute its CTAs
// may become resident while the preceding kernel of the stream is still running; this wait
// returns once that kernel (and everything before it) has completed and its writes are
// visible.  Without the attribute it returns at once.
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// Allows the next kernel of the stream, if it was launched with that attribute, to start
// taking the SMs this grid's CTAs free as they exit.
__device__ __forceinline__ void grid_dependency_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---------------------------------------------------------------- mbarrier

__device__ __forceinline__ void mbar_init(u32 bar, u32 count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(u32 bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(u32 bar, u32 bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(u32 bar, u32 parity) {
  u32 ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Non-blocking poll.  Issued ahead of the point where the answer is needed, its latency
// (tens of cycles) overlaps the instructions in between.
__device__ __forceinline__ bool mbar_test_wait(u32 bar, u32 parity) {
  u32 ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Waits for the phase with the given parity to complete.  Returns false when the
// CTA-wide abort flag is (or becomes) set: either another thread gave up, or this
// wait exceeded SPIO_WAIT_LIMIT_NS.  The caller must then leave its loop.
__device__ __forceinline__ bool mbar_wait(u32 bar, u32 parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  u64 t0 = 0;
  for (u32 it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 63u) == 0u) {
      if (*abort_flag) return false;
      u64 now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > SPIO_WAIT_LIMIT_NS) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}

// ---------------------------------------------------------------- TMA (tiled, 4-D)

// Generic-proxy writes to shared memory (st.shared / stmatrix) become visible to
// the async proxy (TMA store) only after this fence.
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void prefetch_tensormap(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// Tiled load of one box.  The innermost coordinate c0 times the element size must
// be a multiple of 16 bytes; the other coordinates may be negative or out of range
// (the box is zero-filled there).
__device__ __forceinline__ void tma_load_4d(u32 dst, const void* tmap, u32 bar, int c0, int c1,
                                            int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(dst),
      "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// Asks the L2 cache for the box a later tma_load_4d with the same coordinates will read.  Nothing
// reaches the SM, so it may be issued before griddepcontrol.wait: L2 is the point of coherence, a line
// that an earlier kernel still writes after the prefetch is updated in place.
__device__ __forceinline__ void tma_prefetch_4d(const void* tmap, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];" ::"l"(tmap), "r"(c0),
               "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}

// L2 eviction-priority policies for loads: 0 = none, 1 = evict first (data that is not read
// again soon), 2 = evict last (data the next kernel reads again).
enum { L2_HINT_NONE = 0, L2_HINT_EVICT_FIRST = 1, L2_HINT_EVICT_LAST = 2 };

__device__ __forceinline__ u64 make_l2_policy(int hint) {
  u64 p = 0;
  if (hint == L2_HINT_EVICT_FIRST)
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  else if (hint == L2_HINT_EVICT_LAST)
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}

// tma_load_4d with an L2 cache policy made by make_l2_policy (hint != L2_HINT_NONE).
__device__ __forceinline__ void tma_load_4d_hint(u32 dst, const void* tmap, u32 bar, int c0, int c1,
                                                 int c2, int c3, u64 policy) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%3, %4, %5, %6}], [%2], %7;" ::"r"(dst),
      "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "l"(policy)
      : "memory");
}

// Either form, chosen by the hint the policy was made from.
__device__ __forceinline__ void tma_load_4d(u32 dst, const void* tmap, u32 bar, int c0, int c1, int c2,
                                            int c3, int hint, u64 policy) {
  if (hint == L2_HINT_NONE)
    tma_load_4d(dst, tmap, bar, c0, c1, c2, c3);
  else
    tma_load_4d_hint(dst, tmap, bar, c0, c1, c2, c3, policy);
}

// Tiled store of one box; elements outside the tensor are dropped.  All coordinates
// must be non-negative.
__device__ __forceinline__ void tma_store_4d(const void* tmap, u32 src, int c0, int c1, int c2,
                                             int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group "
      "[%0, {%2, %3, %4, %5}], [%1];" ::"l"(tmap),
      "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// Until the shared-memory source of every committed store has been read.
__device__ __forceinline__ void tma_store_wait_read0() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

// Until every committed store has completed.
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

// ---------------------------------------------------------------- tcgen05 (5th-generation tensor cores)

// Tensor memory: 128 lanes x 512 columns of 32 bits per SM.  A warp allocates a power-of-two
// number of columns (>= 32); the base address (lane in bits 31:16, column in bits 15:0) is
// written to shared memory.  The same warp must free it before the CTA exits.
__device__ __forceinline__ void tmem_alloc(u32 holder_smem, u32 columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(holder_smem),
               "r"(columns)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(u32 taddr, u32 columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tcgen05_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major operand tile whose rows are 128 bytes apart
// and stored with the 128-byte swizzle (the layout a tiled TMA load with SWIZZLE_128B writes):
// groups of 8 rows are 1024 bytes apart.  The swizzle is a function of the absolute address,
// so `addr` may point at any row (a multiple of 128 bytes) and any 32-byte k-step of a row.
__device__ __forceinline__ u64 umma_desc_k_sw128(u32 addr) {
  return (u64)((addr >> 4) & 0x3fffu)  // start address / 16
         | ((u64)1u << 16)             // leading byte offset: not used by swizzled K-major tiles
         | ((u64)(1024u >> 4) << 32)   // stride byte offset between 8-row groups / 16
         | ((u64)1u << 46)             // descriptor version of sm_100
         | ((u64)2u << 61);            // 128-byte swizzle
}

// Instruction descriptor: fp16 x fp16 -> fp32, both operands K-major, tile M x N (K = 16).
__device__ __forceinline__ constexpr u32 umma_idesc_f16_f32(int m, int n) {
  return (1u << 4) | ((u32)(n >> 3) << 17) | ((u32)(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]^T, issued by ONE thread; completion is observed through
// tcgen05_commit.
__device__ __forceinline__ void umma_f16_ss(u32 d_tmem, u64 a_desc, u64 b_desc, u32 idesc, u32 accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// The mbarrier receives one arrival once every tcgen05 operation issued so far by this thread
// has completed.
__device__ __forceinline__ void tcgen05_commit(u32 bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

// 32 lanes x 32 consecutive columns -> 32 registers per thread (thread t reads lane base + t).
__device__ __forceinline__ void tmem_ld_32x32(u32 (&v)[32], u32 taddr) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
        "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]),
        "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]),
        "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr));
}

// The same for 16 consecutive columns.
__device__ __forceinline__ void tmem_ld_32x16(u32 (&v)[16], u32 taddr) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
        "=r"(v[15])
      : "r"(taddr));
}

__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// acc += the value of lane (own lane + delta), skipped where that lane does not exist.
__device__ __forceinline__ void shfl_down_add(float& acc, float v, int delta) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .f32 t;\n\t"
      "shfl.sync.down.b32 t|p, %1, %2, 31, 0xffffffff;\n\t"
      "@p add.f32 %0, %0, t;\n\t}"
      : "+f"(acc)
      : "f"(v), "r"(delta));
}

// ---------------------------------------------------------------- ldmatrix / stmatrix

// COUNT 8x8 b16 matrices; lane L supplies the row address of matrix L/8, row L%8.
// Thread (g = L/4, t = L%4) receives elements (row g, cols 2t, 2t+1) of each matrix,
// or with TRANS elements (rows 2t, 2t+1, col g).
template <bool TRANS>
__device__ __forceinline__ void ldmatrix_x4(u32& r0, u32& r1, u32& r2, u32& r3, u32 addr) {
  if (TRANS)
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
  else
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

template <bool TRANS>
__device__ __forceinline__ void ldmatrix_x2(u32& r0, u32& r1, u32 addr) {
  if (TRANS)
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];"
                 : "=r"(r0), "=r"(r1)
                 : "r"(addr));
  else
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];"
                 : "=r"(r0), "=r"(r1)
                 : "r"(addr));
}

template <bool TRANS>
__device__ __forceinline__ void ldmatrix_x1(u32& r0, u32 addr) {
  if (TRANS)
    asm volatile("ldmatrix.sync.aligned.m8n8.x1.trans.shared.b16 {%0}, [%1];"
                 : "=r"(r0)
                 : "r"(addr));
  else
    asm volatile("ldmatrix.sync.aligned.m8n8.x1.shared.b16 {%0}, [%1];" : "=r"(r0) : "r"(addr));
}

__device__ __forceinline__ void stmatrix_x2(u32 addr, u32 r0, u32 r1) {
  asm volatile("stmatrix.sync.aligned.m8n8.x2.shared.b16 [%0], {%1,%2};" ::"r"(addr), "r"(r0),
               "r"(r1)
               : "memory");
}

// ---------------------------------------------------------------- mma.sync (fp16 x fp16 -> fp32)

// D(16x8) += A(16x16) * B(16x8).  a0:(rows 0-7,k 0-7) a1:(rows 8-15,k 0-7)
// a2:(rows 0-7,k 8-15) a3:(rows 8-15,k 8-15); b0: k 0-7, b1: k 8-15.
__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], u32 a0, u32 a1, u32 a2, u32 a3, u32 b0,
                                             u32 b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// D(16x8) += A(16x8) * B(8x8).
__device__ __forceinline__ void mma_m16n8k8(float (&d)[4], u32 a0, u32 a1, u32 b0) {
  asm(
      "mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(b0));
}

}  // namespace spio_b200
