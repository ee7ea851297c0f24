// Typed dimensions for CUDA kernels: index arithmetic that the compiler checks.
//
//   Dim<Tag>            an integer that counts positions along ONE named dimension; dimensions
//                       of different names do not mix (no implicit conversion, no comparison)
//   Fold<D, STRIDE>     the same dimension counted in blocks of STRIDE (C8 = channels / 8)
//   Extent<D, N, S>     "dimension D has N positions, S elements apart" -- a tensor axis
//   Tensor<T, Extent..> a pointer with compile-time sizes and strides; subscripting by a typed
//                       index moves along that index's axis whatever the order of subscripts
//                       (position-free), a folded index moves by its stride
//   CompoundIndex<Extent..> decodes a linear offset (threadIdx.x, blockIdx.x) into typed indices
//
// The header is plain C++17 and compiles for the host (g++) as well as under nvcc and NVRTC.
// Same job as the reference's typed-dimension headers (spio/include/spio/dim.h:79-227,
// tensor.h:426-903, compound_index.h:20-157, coordinates.h), written anew and smaller: all
// sizes are template arguments, there is no run-time stride.
#pragma once

#if defined(__CUDACC__) || defined(__CUDACC_RTC__)
#define SPIO_HD __host__ __device__ __forceinline__
#else
#define SPIO_HD inline
#endif

namespace spio_b200 {
namespace typed {

// ---------------------------------------------------------------- dimensions

template <class Tag>
struct Dim {
  using tag = Tag;
  using base = Dim;                       // the unfolded dimension
  static constexpr int stride = 1;        // base positions per count
  int v;
  SPIO_HD constexpr Dim() : v(0) {}
  SPIO_HD constexpr explicit Dim(int value) : v(value) {}
  SPIO_HD constexpr int get() const { return v; }
  SPIO_HD constexpr Dim operator+(Dim o) const { return Dim(v + o.v); }
  SPIO_HD constexpr Dim operator-(Dim o) const { return Dim(v - o.v); }
  SPIO_HD constexpr Dim operator*(int k) const { return Dim(v * k); }
  SPIO_HD constexpr Dim operator/(int k) const { return Dim(v / k); }
  SPIO_HD constexpr Dim operator%(Dim o) const { return Dim(v % o.v); }
  SPIO_HD constexpr Dim& operator+=(Dim o) { v += o.v; return *this; }
  SPIO_HD constexpr Dim& operator++() { ++v; return *this; }
  SPIO_HD constexpr bool operator==(Dim o) const { return v == o.v; }
  SPIO_HD constexpr bool operator!=(Dim o) const { return v != o.v; }
  SPIO_HD constexpr bool operator<(Dim o) const { return v < o.v; }
  SPIO_HD constexpr bool operator<=(Dim o) const { return v <= o.v; }
  SPIO_HD constexpr bool operator>(Dim o) const { return v > o.v; }
  SPIO_HD constexpr bool operator>=(Dim o) const { return v >= o.v; }
  // the position counted in blocks of S (rounding down), and the remainder inside the block
  template <int S> SPIO_HD constexpr auto fold() const;
  template <int S> SPIO_HD constexpr Dim rem() const { return Dim(v % S); }
  SPIO_HD constexpr Dim unfold() const { return *this; }
};

template <class D, int STRIDE>
struct Fold {
  static_assert(STRIDE > 0, "fold stride must be positive");
  using tag = typename D::tag;
  using base = typename D::base;
  static constexpr int stride = STRIDE * D::stride;
  int v;
  SPIO_HD constexpr Fold() : v(0) {}
  SPIO_HD constexpr explicit Fold(int value) : v(value) {}
  SPIO_HD constexpr int get() const { return v; }
  SPIO_HD constexpr Fold operator+(Fold o) const { return Fold(v + o.v); }
  SPIO_HD constexpr Fold operator-(Fold o) const { return Fold(v - o.v); }
  SPIO_HD constexpr Fold& operator+=(Fold o) { v += o.v; return *this; }
  SPIO_HD constexpr Fold& operator++() { ++v; return *this; }
  SPIO_HD constexpr bool operator==(Fold o) const { return v == o.v; }
  SPIO_HD constexpr bool operator!=(Fold o) const { return v != o.v; }
  SPIO_HD constexpr bool operator<(Fold o) const { return v < o.v; }
  SPIO_HD constexpr bool operator>=(Fold o) const { return v >= o.v; }
  // the same position in units of the unfolded dimension
  SPIO_HD constexpr base unfold() const { return base(v * stride); }
};

template <class Tag>
template <int S>
SPIO_HD constexpr auto Dim<Tag>::fold() const {
  return Fold<Dim<Tag>, S>(v / S);
}

// A folded and an unfolded index of the same dimension add in base units.
template <class D, int S>
SPIO_HD constexpr typename D::base operator+(Fold<D, S> a, typename D::base b) {
  return a.unfold() + b;
}
template <class D, int S>
SPIO_HD constexpr typename D::base operator+(typename D::base a, Fold<D, S> b) {
  return a + b.unfold();
}

template <class A, class B>
struct same_dim {
  static constexpr bool value = false;
};
template <class T>
struct same_dim<Dim<T>, Dim<T>> {
  static constexpr bool value = true;
};
// true when I (a Dim or a Fold) counts along the base dimension of D
template <class I, class D>
constexpr bool indexes = same_dim<typename I::base, typename D::base>::value;

// ---------------------------------------------------------------- tensor axes

// Dimension D (a Dim or a Fold: the unit the axis is counted in), SIZE positions, STRIDE elements apart.
template <class D, int SIZE, int STRIDE>
struct Extent {
  using dim = D;
  static constexpr int size = SIZE;
  static constexpr int stride = STRIDE;
};

namespace detail {

constexpr int imax(int a, int b) { return a > b ? a : b; }

// Index arithmetic of a typed index I on the axes Es.  The index stands at base position
// v * I::stride of its dimension; every axis of that dimension contributes
//   (base position / axis unit) [modulo the axis size, except on the coarsest axis] * axis stride,
// so a folded index moves along the folded axis, an unfolded index is split over the folded and
// the unfolded axis, and axes of other dimensions contribute nothing.
template <class I, class... Es>
struct axis_math {
  template <class E>
  static constexpr int unit_of() {
    return indexes<I, typename E::dim> ? E::dim::stride : 0;
  }
  static constexpr int max_unit = [] {
    int m = 0;
    ((m = imax(m, unit_of<Es>())), ...);
    return m;
  }();
  static constexpr bool found = max_unit > 0;
  template <class E>
  SPIO_HD static constexpr int term(int base_pos) {
    if constexpr (indexes<I, typename E::dim>) {
      int pos = base_pos / E::dim::stride;
      if (E::dim::stride != max_unit) pos %= E::size;
      return pos * E::stride;
    } else {
      return 0;
    }
  }
  SPIO_HD static constexpr int offset(int v) {
    const int base_pos = v * I::stride;
    int off = 0;
    ((off += term<Es>(base_pos)), ...);
    return off;
  }
};

template <class... Es>
struct storage;
template <>
struct storage<> {
  static constexpr int value = 1;
};
template <class E, class... Es>
struct storage<E, Es...> {
  static constexpr int value = (E::size - 1) * E::stride + storage<Es...>::value;
};

template <class D, class... Es>
struct axis_size;
template <class D>
struct axis_size<D> {
  static constexpr int value = 0;
};
template <class D, class E, class... Es>
struct axis_size<D, E, Es...> {
  static constexpr bool here = indexes<D, typename E::dim> && D::stride == E::dim::stride;
  static constexpr int value = here ? E::size : axis_size<D, Es...>::value;
};

// Positions, in base units, that the axes of I's dimension cover: the size of the coarsest axis times its unit.
template <class I, class... Es>
struct dim_span {
  static constexpr int value = [] {
    int unit = 0, size = 0;
    (((indexes<I, typename Es::dim> && Es::dim::stride > unit) ? (unit = Es::dim::stride, size = Es::size) : 0), ...);
    return unit * size;
  }();
};

}  // namespace detail

// ---------------------------------------------------------------- tensor and cursor

template <class T, class... Es>
struct Tensor {
  using data_type = T;
  T* p;
  SPIO_HD constexpr explicit Tensor(T* ptr) : p(ptr) {}
  // elements from the first to one past the last addressable one
  static constexpr int storage_size() { return detail::storage<Es...>::value; }
  // positions along the axis counted in units of D (0 if the tensor has no such axis)
  template <class D>
  static constexpr D size() {
    return D(detail::axis_size<D, Es...>::value);
  }
  // Moves along the axes of the index's dimension (see detail::axis_math); an index of a
  // dimension the tensor does not have is a compile-time error.  Offsets of several subscripts
  // of one dimension simply add: split a sum into fold and remainder before subscripting a
  // tensor whose folded axis is not contiguous with the unfolded one.
  template <class I>
  SPIO_HD constexpr Tensor operator[](I i) const {
    using math = detail::axis_math<I, Es...>;
    static_assert(math::found, "the tensor has no axis of this index's dimension");
    return Tensor(p + math::offset(i.get()));
  }
  // element offset of an index, for address arithmetic done by hand (shared-memory byte offsets)
  template <class I>
  SPIO_HD static constexpr int offset_of(I i) {
    using math = detail::axis_math<I, Es...>;
    static_assert(math::found, "the tensor has no axis of this index's dimension");
    return math::offset(i.get());
  }
  // Whether an index lies inside the tensor along its dimension (counted in the index's own unit: a
  // folded index is compared with the number of whole folds).  For masks at ragged edges, as the
  // reference's Tensor::inbounds (spio/include/spio/tensor.h:580-609): `if (X::in_range(h) && X::in_range(w))`.
  template <class I>
  SPIO_HD static constexpr bool in_range(I i) {
    using math = detail::axis_math<I, Es...>;
    static_assert(math::found, "the tensor has no axis of this index's dimension");
    return i.get() >= 0 && i.get() * I::stride < detail::dim_span<I, Es...>::value;
  }
  template <class I, class... Is>
  SPIO_HD static constexpr bool inbounds(I i, Is... rest) {
    if constexpr (sizeof...(Is) == 0)
      return in_range(i);
    else
      return in_range(i) && inbounds(rest...);
  }
  SPIO_HD constexpr T* get() const { return p; }
  SPIO_HD constexpr T& operator*() const { return *p; }
};

// ---------------------------------------------------------------- carving tensors out of a buffer

// Hands out typed tensors one after the other from a byte buffer, typically the dynamic shared memory of
// a kernel: `StackAllocator a(smem); auto x = a.allocate<XTile>(); auto w = a.allocate<WTile, 128>();`.
// Each tensor starts on an ALIGN-byte boundary (16 by default, what vector loads, ldmatrix rows and bulk
// copies need; 128 or 1024 for swizzled TMA boxes).  The reference's spio/include/spio/allocator.h does
// the same with a deallocate that this one leaves out: kernels here carve once.
struct StackAllocator {
  unsigned char* next;
  SPIO_HD explicit StackAllocator(void* base) : next(static_cast<unsigned char*>(base)) {}
  template <class TensorT, int ALIGN = 16>
  SPIO_HD TensorT allocate() {
    static_assert(ALIGN > 0 && (ALIGN & (ALIGN - 1)) == 0, "alignment must be a power of two");
    using T = typename TensorT::data_type;
    const unsigned long long at = (reinterpret_cast<unsigned long long>(next) + ALIGN - 1) & ~(unsigned long long)(ALIGN - 1);
    next = reinterpret_cast<unsigned char*>(at) + sizeof(T) * TensorT::storage_size();
    return TensorT(reinterpret_cast<T*>(at));
  }
  // bytes handed out so far, counted from `base`
  SPIO_HD long long used(const void* base) const { return next - static_cast<const unsigned char*>(base); }
};

// ---------------------------------------------------------------- compound index

// Splits a linear offset into typed indices, the first extent varying slowest.  The stride of an
// extent is ignored; its size is what counts.  get<D>() returns the index of the axis counted in D.
template <class... Es>
struct CompoundIndex;

template <>
struct CompoundIndex<> {
  int rest;
  SPIO_HD constexpr explicit CompoundIndex(int offset) : rest(offset) {}
  static constexpr int total = 1;
};

template <class E, class... Es>
struct CompoundIndex<E, Es...> {
  using tail = CompoundIndex<Es...>;
  static constexpr int total = E::size * tail::total;
  int offset;
  SPIO_HD constexpr explicit CompoundIndex(int linear) : offset(linear) {}
  static constexpr int size() { return total; }
  template <class D>
  SPIO_HD constexpr D get() const {
    if constexpr (same_dim<typename D::base, typename E::dim::base>::value && D::stride == E::dim::stride) {
      return D((offset / tail::total) % E::size);
    } else {
      static_assert(sizeof...(Es) > 0, "the compound index has no such dimension");
      return tail(offset % tail::total).template get<D>();
    }
  }
};

}  // namespace typed
}  // namespace spio_b200
