// Typed wrappers for the sm_100a data movers: tiled TMA copies whose coordinates are typed
// indices, and a ring of shared-memory slots guarded by full / empty mbarriers.
//
//   TensorMapRef<T, Extent<D0, BOX0, 0>, Extent<D1, BOX1, 0>, ...>
//       a tiled tensor map (a kernel parameter, const __grid_constant__ TensorMap) with axes
//       D0 (innermost) .. D3 and a box of BOX0 x BOX1 x ... elements.  load() / store() take
//       typed coordinates in ANY order, a missing one is 0, a folded one is converted to the
//       axis' unit; the innermost coordinate must be a fold that is a whole number of 16-byte
//       units -- the alignment rule of cp.async.bulk.tensor, whose violation is an illegal
//       instruction at run time, becomes a compile-time error;
//   MbarrierRing<SLOTS>
//       full[i] / empty[i] barriers of a SLOTS-deep producer / consumer ring and the slot /
//       parity bookkeeping of both sides; every wait is bounded (ptx.cuh, SPIO_WAIT_LIMIT_NS)
//       and reports failure instead of spinning for ever.
//
// Device-only; compiles under nvcc and NVRTC.  The reference's typed headers predate TMA
// (its loaders are cp.async based: spio/include/spio/async_loader.cuh, memory.cuh:17-24).
#pragma once

#include <cuda_fp16.h>

#include "gw8_common.cuh"
#include "typed.h"

namespace spio_b200 {
namespace typed {

namespace detail {

// The coordinate, in units of axis dimension D, that the pack supplies for D's base dimension; 0 if none.
template <class D>
__device__ __forceinline__ constexpr int coordinate() {
  return 0;
}
template <class D, class I, class... Is>
__device__ __forceinline__ constexpr int coordinate(I i, Is... rest) {
  if constexpr (indexes<I, D>) {
    static_assert(I::stride % D::stride == 0, "a TMA coordinate must be a whole number of the axis' units");
    return i.get() * (I::stride / D::stride) + coordinate<D>(rest...);
  } else {
    return coordinate<D>(rest...);
  }
}

template <class D, class... Is>
struct inner_alignment;  // bytes the innermost coordinate is known to be a multiple of
template <class D>
struct inner_alignment<D> {
  static constexpr int units = 0;  // no coordinate given: zero, aligned to anything
};
template <class D, class I, class... Is>
struct inner_alignment<D, I, Is...> {
  static constexpr int rest = inner_alignment<D, Is...>::units;
  static constexpr int here = indexes<I, D> ? I::stride / D::stride : 0;
  // gcd-like: both contributions must be aligned, so the guarantee is the smaller non-zero one
  static constexpr int units = here == 0 ? rest : (rest == 0 ? here : (here < rest ? here : rest));
};

template <class... Es>
struct box_elems;
template <>
struct box_elems<> {
  static constexpr int value = 1;
};
template <class E, class... Es>
struct box_elems<E, Es...> {
  static constexpr int value = E::size * box_elems<Es...>::value;
};

}  // namespace detail

template <class T, class E0, class E1, class E2, class E3>
struct TensorMapRef {
  const TensorMap* map;
  __device__ __forceinline__ explicit TensorMapRef(const TensorMap& m) : map(&m) {}
  static constexpr u32 box_bytes = sizeof(T) * detail::box_elems<E0, E1, E2, E3>::value;

  template <class... Is>
  static constexpr void check_alignment() {
    constexpr int units = detail::inner_alignment<typename E0::dim, Is...>::units;
    static_assert(units == 0 || (units * E0::dim::stride * (int)sizeof(T)) % 16 == 0,
                  "the innermost TMA coordinate must be a fold whose stride is a multiple of 16 bytes");
  }

  __device__ __forceinline__ void prefetch() const { prefetch_tensormap(map); }

  // One box into shared memory at `dst` (1 KiB aligned for the 128-byte swizzle); completion is
  // signalled on the mbarrier `bar` as box_bytes transaction bytes.
  template <class... Is>
  __device__ __forceinline__ void load(u32 dst, u32 bar, Is... idx) const {
    check_alignment<Is...>();
    tma_load_4d(dst, map, bar, detail::coordinate<typename E0::dim>(idx...),
                detail::coordinate<typename E1::dim>(idx...), detail::coordinate<typename E2::dim>(idx...),
                detail::coordinate<typename E3::dim>(idx...));
  }

  // One box from shared memory; coordinates must be non-negative, elements outside the tensor
  // are dropped.  Follow with tma_store_commit() and a bulk-group wait.
  template <class... Is>
  __device__ __forceinline__ void store(u32 src, Is... idx) const {
    check_alignment<Is...>();
    tma_store_4d(map, src, detail::coordinate<typename E0::dim>(idx...),
                 detail::coordinate<typename E1::dim>(idx...), detail::coordinate<typename E2::dim>(idx...),
                 detail::coordinate<typename E3::dim>(idx...));
  }
};

// A SLOTS-deep ring between `producers` arriving threads on the full side (1 for a TMA issuing
// lane, which arrives with expect_tx) and `consumers` arriving threads on the empty side.
template <int SLOTS>
struct MbarrierRing {
  static_assert(SLOTS >= 1 && SLOTS <= 32, "ring depth");
  u64 full_bar[SLOTS];
  u64 empty_bar[SLOTS];

  // one thread, before the CTA-wide barrier that publishes the ring
  __device__ __forceinline__ void init(int producers, int consumers) {
    for (int i = 0; i < SLOTS; ++i) {
      mbar_init(smem_u32(&full_bar[i]), (u32)producers);
      mbar_init(smem_u32(&empty_bar[i]), (u32)consumers);
    }
    mbar_fence_init();
  }
  __device__ __forceinline__ u32 full(int i) const { return smem_u32(&full_bar[i]); }
  __device__ __forceinline__ u32 empty(int i) const { return smem_u32(&empty_bar[i]); }

  // Position of one side in the ring.
  struct Cursor {
    int slot = 0;
    u32 parity = 0;
    __device__ __forceinline__ void advance() {
      if (++slot == SLOTS) {
        slot = 0;
        parity ^= 1u;
      }
    }
  };

  // producer: wait until the slot is free, then announce `bytes` of TMA traffic on its full barrier
  __device__ __forceinline__ bool acquire(const Cursor& c, u32 bytes, volatile int* abort_flag) {
    if (!mbar_wait(empty(c.slot), c.parity ^ 1u, abort_flag)) return false;
    mbar_arrive_expect_tx(full(c.slot), bytes);
    return true;
  }
  // consumer: wait until the slot is full / hand it back
  __device__ __forceinline__ bool wait_full(const Cursor& c, volatile int* abort_flag) {
    return mbar_wait(full(c.slot), c.parity, abort_flag);
  }
  __device__ __forceinline__ void release(const Cursor& c) { mbar_arrive(empty(c.slot)); }
};

}  // namespace typed
}  // namespace spio_b200
