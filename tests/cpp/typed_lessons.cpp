// Host-side checks of the typed-dimension header (spio_b200/csrc/typed.h) against types generated
// from the @spio blocks below; compiled with g++ by tests/test_generators.py.  In the spirit of the
// reference's tutorial lessons (spio/src_tests/tutorial/01_commutativity.cpp ... 05_compound_index.cpp):
// type safety, position-free subscripting, folding, compound indices, and the lane maps of the typed MMA
// fragments (spio_b200/csrc/typed_mma.cuh; the reference's spio/include/spio/fragment_index.h).
/*@spio
I = Dim()
J = Dim()
K = Dim()
K8 = Fold(K, 8)
A = Tensor(dtype.float, Dims(I(16), K(32)))
B = Tensor(dtype.float, Dims(K(32), J(64)))
Folded = Tensor(dtype.float, Dims(I(4), K8(4), K(8)), Strides(K8=9))
Threads = CompoundIndex(Dims(I(4), K8(2), J(16)))
Acc = Fragment(FragmentType.M16_N8_F32_C, I, J)
AFrag = Fragment(FragmentType.M16_K16_F16_A, I, K)
BFrag = Fragment(FragmentType.N8_K16_F16_B, J, K)
Tile = ParamsSpec(dict(rows=16, cols=8, scale=0.5, transposed=False))
Names = Macro(dict(LESSON_COUNT=6))
@spio*/
#include <cstdio>
#include <type_traits>

#include "types.h"

#define CHECK(cond)                                                   \
  do {                                                                \
    if (!(cond)) {                                                    \
      std::printf("FAILED line %d: %s\n", __LINE__, #cond);          \
      return 1;                                                       \
    }                                                                 \
  } while (0)

template <class X, class Y, class = void>
struct comparable : std::false_type {};
template <class X, class Y>
struct comparable<X, Y, std::void_t<decltype(std::declval<X>() == std::declval<Y>())>> : std::true_type {};

template <class T, class Idx, class = void>
struct subscriptable : std::false_type {};
template <class T, class Idx>
struct subscriptable<T, Idx, std::void_t<decltype(T::offset_of(std::declval<Idx>()))>> : std::true_type {};

int main() {
  // dimensions behave like integers, each is a type of its own, and they do not mix
  static_assert(I(2) + I(4) == I(6));
  static_assert(I(8) < I(10));
  static_assert(!std::is_same_v<I, J>);
  static_assert(comparable<I, I>::value && !comparable<I, J>::value);

  // tensors know their sizes
  static_assert(A::size<I>() == I(16) && A::size<K>() == K(32) && B::size<J>() == J(64));
  static_assert(A::storage_size() == 16 * 32 && B::storage_size() == 32 * 64);
  float a_data[A::storage_size()], b_data[B::storage_size()];
  const A a(a_data);
  const B b(b_data);

  // position-free subscripting: the order of subscripts does not change the element
  CHECK(a[I(2)][K(4)].get() == a[K(4)][I(2)].get());
  CHECK(b[K(4)][J(3)].get() == b[J(3)][K(4)].get());
  CHECK(a[I(2)][K(4)].get() == a_data + 2 * 32 + 4);
  // offset_of() on a dimension the tensor lacks does not compile (checked through SFINAE here)
  static_assert(subscriptable<A, I>::value && subscriptable<A, K>::value);

  // folding: K8 counts K in blocks of 8
  static_assert(K(19).fold<8>() == K8(2));
  static_assert(K(19).rem<8>() == K(3));
  static_assert(K8(2).unfold() == K(16));
  static_assert(K8(2) + K(3) == K(19));
  // a tensor with a folded axis whose rows are padded to 9 floats: a folded index moves along the
  // folded axis, an unfolded one is split into fold and remainder
  static_assert(Folded::storage_size() == 3 * 36 + 3 * 9 + 7 + 1);
  float f_data[Folded::storage_size()];
  const Folded f(f_data);
  CHECK(f[I(1)][K8(2)][K(3)].get() == f_data + 36 + 2 * 9 + 3);
  CHECK(f[I(1)][K(19)].get() == f[I(1)][K8(2)][K(3)].get());

  // compound index: a linear thread index split into typed coordinates
  static_assert(Threads::size() == 4 * 2 * 16);
  const Threads t(1 * 32 + 1 * 16 + 5);
  CHECK(t.get<I>() == I(1));
  CHECK(t.get<K8>() == K8(1));
  CHECK(t.get<J>() == J(5));
  // fragments: every element of the 16 x 8 accumulator belongs to exactly one (lane, register), and the
  // coordinates are typed (a row is an I, a column a J)
  static_assert(std::is_same_v<decltype(Acc::row(0, 0)), I> && std::is_same_v<decltype(Acc::col(0, 0)), J>);
  int seen_c[16][8] = {};
  for (int lane = 0; lane < 32; ++lane)
    for (int i = 0; i < Acc::size; ++i) ++seen_c[Acc::row(lane, i).get()][Acc::col(lane, i).get()];
  for (int r = 0; r < 16; ++r)
    for (int c = 0; c < 8; ++c) CHECK(seen_c[r][c] == 1);
  // the A operand: 16 x 16 halves, register j of a lane holds two consecutive k
  int seen_a[16][16] = {};
  for (int lane = 0; lane < 32; ++lane)
    for (int j = 0; j < AFrag::size; ++j)
      for (int h = 0; h < 2; ++h) ++seen_a[AFrag::row(lane, j).get()][AFrag::k(lane, j).get() + h];
  for (int r = 0; r < 16; ++r)
    for (int k = 0; k < 16; ++k) CHECK(seen_a[r][k] == 1);
  // the row addresses the lanes hand to ldmatrix.x4 cover the four 8 x 8 matrices in register order
  for (int lane = 0; lane < 32; ++lane) {
    const int m = lane / 8;  // matrix = destination register
    CHECK(AFrag::load_row(lane).get() == lane % 8 + 8 * (m % 2));
    CHECK(AFrag::load_k(lane).get() == 8 * (m / 2));
    CHECK(AFrag::row(4 * (lane % 8), m).get() == AFrag::load_row(lane).get());
    CHECK(AFrag::k(0, m).get() == AFrag::load_k(lane).get());
  }
  int seen_b[8][16] = {};
  for (int lane = 0; lane < 32; ++lane)
    for (int j = 0; j < BFrag::size; ++j)
      for (int h = 0; h < 2; ++h) ++seen_b[BFrag::col(lane, j).get()][BFrag::k(lane, j).get() + h];
  for (int c = 0; c < 8; ++c)
    for (int k = 0; k < 16; ++k) CHECK(seen_b[c][k] == 1);
  // masks at ragged edges: is an index inside the tensor along its dimension?
  static_assert(A::in_range(I(15)) && !A::in_range(I(16)) && !A::in_range(I(-1)));
  static_assert(A::inbounds(I(3), K(31)) && !A::inbounds(I(3), K(32)));
  static_assert(Folded::in_range(K(31)) && !Folded::in_range(K(32)));    // 4 folds of 8
  static_assert(Folded::in_range(K8(3)) && !Folded::in_range(K8(4)));
  // carving typed tensors out of one buffer, each on its alignment
  alignas(128) unsigned char buffer[4096];
  spio_b200::typed::StackAllocator alloc(buffer);
  const A first = alloc.allocate<A>();
  const Folded second = alloc.allocate<Folded, 128>();
  CHECK(reinterpret_cast<unsigned char*>(first.get()) == buffer);
  CHECK(reinterpret_cast<unsigned char*>(second.get()) == buffer + 16 * 32 * 4);  // already a multiple of 128
  const Folded third = alloc.allocate<Folded, 128>();
  CHECK((reinterpret_cast<unsigned long long>(third.get()) & 127u) == 0);
  CHECK(third.get() >= second.get() + Folded::storage_size());
  CHECK(alloc.used(buffer) <= (long long)sizeof buffer);
  // named constants and macros
  static_assert(Tile::rows == 16 && Tile::cols == 8 && !Tile::transposed && Tile::scale == 0.5f);
  static_assert(LESSON_COUNT == 6);
  std::puts("typed lessons ok");
  return 0;
}
