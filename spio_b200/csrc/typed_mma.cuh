// Typed matrix fragments of the warp-level fp16 x fp16 -> fp32 MMA (m16n8k16 and m16n8k8).
//
// A fragment knows the dimensions of its rows and columns, so the multiply-accumulate below only
// compiles when the operands fit together (A is ROW x K, B is COL x K, C is ROW x COL), and a lane's
// registers are addressed by typed coordinates: `Acc::row(lane, i)` is a ROW, `Acc::col(lane, i)` a COL,
// ready to subscript a typed tensor.  The reference provides the same through its fragment classes and
// index maps (spio/include/spio/fragment.cuh, fragment_index.h, fragment_load_index.h); the lane maps
// are those of the PTX ISA's description of mma.sync.m16n8k16 / m16n8k8 for .f16 operands.
//
// The lane maps are plain constexpr functions and compile on the host; loading (ldmatrix) and the MMA
// itself need nvcc / NVRTC.
#pragma once

#include "typed.h"

#ifdef __CUDACC__
#include "ptx.cuh"
#endif

namespace spio_b200 {
namespace typed {

// Accumulator / result: 16 rows x 8 columns of fp32, four values per lane.
//   value i of lane l: row = l / 4 + 8 * (i / 2), column = 2 * (l % 4) + i % 2
template <class ROW, class COL>
struct MmaM16N8F32C {
  using row_dim = ROW;
  using col_dim = COL;
  static constexpr int rows = 16, cols = 8, size = 4;
  float v[4];
  SPIO_HD static constexpr ROW row(int lane, int i) { return ROW(lane / 4 + 8 * (i / 2)); }
  SPIO_HD static constexpr COL col(int lane, int i) { return COL(2 * (lane % 4) + i % 2); }
  SPIO_HD void zero() {
    for (int i = 0; i < 4; ++i) v[i] = 0.f;
  }
  // Adds nothing, stores every value where its typed coordinates point: dst[row][col] = value.
  template <class TensorT>
  SPIO_HD void store(const TensorT& dst, int lane) const {
    for (int i = 0; i < 4; ++i) *dst[row(lane, i)][col(lane, i)] = v[i];
  }
};

// A operand of m16n8k16: 16 rows x 16 k of fp16, eight values per lane in four registers.
//   register j of lane l holds k = 2 * (l % 4) + 8 * (j / 2) + {0, 1} of row l / 4 + 8 * (j % 2)
template <class ROW, class KD>
struct MmaM16K16F16A {
  using row_dim = ROW;
  using k_dim = KD;
  static constexpr int rows = 16, ks = 16, size = 4;
  unsigned r[4];
  SPIO_HD static constexpr ROW row(int lane, int j) { return ROW(lane / 4 + 8 * (j % 2)); }
  SPIO_HD static constexpr KD k(int lane, int j) { return KD(2 * (lane % 4) + 8 * (j / 2)); }  // and k + 1
  // ldmatrix.x4 takes one row address per 8 x 8 matrix from every lane: lane l names row
  // l % 8 + 8 * ((l / 8) % 2) of the tile at k = 8 * (l / 16).
  SPIO_HD static constexpr ROW load_row(int lane) { return ROW(lane % 8 + 8 * ((lane / 8) % 2)); }
  SPIO_HD static constexpr KD load_k(int lane) { return KD(8 * (lane / 16)); }
#ifdef __CUDACC__
  // tile: a shared-memory tensor of __half with a ROW axis and a contiguous K axis, whose rows start on
  // 16-byte boundaries
  template <class TensorT>
  __device__ void load(const TensorT& tile, int lane) {
    ldmatrix_x4<false>(r[0], r[1], r[2], r[3], smem_u32(tile[load_row(lane)][load_k(lane)].get()));
  }
#endif
};

// B operand of m16n8k16: 8 columns x 16 k of fp16 (k contiguous in memory), four values per lane in two
// registers.  register j of lane l holds k = 2 * (l % 4) + 8 * j + {0, 1} of column l / 4.
template <class COL, class KD>
struct MmaN8K16F16B {
  using col_dim = COL;
  using k_dim = KD;
  static constexpr int cols = 8, ks = 16, size = 2;
  unsigned r[2];
  SPIO_HD static constexpr COL col(int lane, int) { return COL(lane / 4); }
  SPIO_HD static constexpr KD k(int lane, int j) { return KD(2 * (lane % 4) + 8 * j); }
  SPIO_HD static constexpr COL load_col(int lane) { return COL(lane % 8); }
  SPIO_HD static constexpr KD load_k(int lane) { return KD(8 * ((lane / 8) % 2)); }
#ifdef __CUDACC__
  template <class TensorT>
  __device__ void load(const TensorT& tile, int lane) {
    ldmatrix_x2<false>(r[0], r[1], smem_u32(tile[load_col(lane)][load_k(lane)].get()));
  }
#endif
};

// The k8 forms: half of the above along k.
template <class ROW, class KD>
struct MmaM16K8F16A {
  using row_dim = ROW;
  using k_dim = KD;
  static constexpr int rows = 16, ks = 8, size = 2;
  unsigned r[2];
  SPIO_HD static constexpr ROW row(int lane, int j) { return ROW(lane / 4 + 8 * j); }
  SPIO_HD static constexpr KD k(int lane, int) { return KD(2 * (lane % 4)); }
  SPIO_HD static constexpr ROW load_row(int lane) { return ROW(lane % 8 + 8 * ((lane / 8) % 2)); }
#ifdef __CUDACC__
  template <class TensorT>
  __device__ void load(const TensorT& tile, int lane) {
    ldmatrix_x2<false>(r[0], r[1], smem_u32(tile[load_row(lane)].get()));
  }
#endif
};

template <class COL, class KD>
struct MmaN8K8F16B {
  using col_dim = COL;
  using k_dim = KD;
  static constexpr int cols = 8, ks = 8, size = 1;
  unsigned r[1];
  SPIO_HD static constexpr COL col(int lane, int) { return COL(lane / 4); }
  SPIO_HD static constexpr KD k(int lane, int) { return KD(2 * (lane % 4)); }
};

#ifdef __CUDACC__
// d = a * b + c.  The dimensions must fit: rows of A are rows of C, columns of B are columns of C, and
// A and B are multiplied along the same dimension.
template <class ROW, class COL, class KD>
__device__ __forceinline__ void mma(MmaM16N8F32C<ROW, COL>& d, const MmaM16K16F16A<ROW, KD>& a,
                                    const MmaN8K16F16B<COL, KD>& b, const MmaM16N8F32C<ROW, COL>& c) {
  if (&d != &c) {
    for (int i = 0; i < 4; ++i) d.v[i] = c.v[i];
  }
  mma_m16n8k16(d.v, a.r[0], a.r[1], a.r[2], a.r[3], b.r[0], b.r[1]);
}
#endif

}  // namespace typed
}  // namespace spio_b200
