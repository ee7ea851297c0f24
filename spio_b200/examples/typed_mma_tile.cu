// A small matrix product written against generated typed fragments: C[I][J] = sum over K of A[I][K] * B[J][K]
// (fp16 operands with k contiguous, fp32 result), one warp per 16 x 8 tile of C.
//
// The `@spio` blocks are Python; spio_b200.generators.generate_from_source turns them into "types.h".
// The fragments carry the dimensions of their rows, columns and k: `mma(acc, a, b, acc)` compiles only
// because A is I x K, B is J x K and the accumulator I x J, and the lanes find their elements through typed
// coordinates (`Acc::row(lane, i)` is an I, `Acc::col(lane, i)` a J), never through a hand-written offset.
/*@spio
I = Dim()
J = Dim()
K = Dim()
Shape = ParamsSpec(dict(m=64, n=48, k=96))
A = Tensor(dtype.half, Dims(I(64), K(96)), constant=True)
B = Tensor(dtype.half, Dims(J(48), K(96)), constant=True)
C = Tensor(dtype.float, Dims(I(64), J(48)))
ATile = Tensor(dtype.half, Dims(I(16), K(16)), Strides(i=24))
BTile = Tensor(dtype.half, Dims(J(8), K(16)), Strides(j=24))
Tiles = CompoundIndex(Dims(I(4), J(6)))
AFrag = Fragment(FragmentType.M16_K16_F16_A, I, K)
BFrag = Fragment(FragmentType.N8_K16_F16_B, J, K)
Acc = Fragment(FragmentType.M16_N8_F32_C, I, J)
Limits = Macro(dict(TILE_K=16))
@spio*/
#include <cuda_fp16.h>

#include "types.h"

using namespace spio_b200;
using namespace spio_b200::typed;

extern "C" __global__ void typed_mma_tile(const __half* __restrict__ a_ptr, const __half* __restrict__ b_ptr,
                                          float* __restrict__ c_ptr) {
  // rows of the tiles are 24 halves apart: 48 bytes, so the eight row addresses of an ldmatrix fall into
  // different banks and every row starts on a 16-byte boundary
  __shared__ __align__(16) __half a_smem[ATile::storage_size() + 8];
  __shared__ __align__(16) __half b_smem[BTile::storage_size() + 8];
  const int lane = threadIdx.x;
  const Tiles tile(blockIdx.x);
  const I i0 = I(tile.get<I>().get() * 16);
  const J j0 = J(tile.get<J>().get() * 8);
  const A a(a_ptr);
  const B b(b_ptr);
  const ATile at(a_smem);
  const BTile bt(b_smem);

  Acc acc;
  acc.zero();
  for (int k0 = 0; k0 < Shape::k; k0 += TILE_K) {
    // 16 x 16 halves of A and 8 x 16 of B into shared memory, one element per lane and step
    for (int e = lane; e < 16 * TILE_K; e += 32) {
      const I i(e / TILE_K);
      const K k(e % TILE_K);
      *at[i][k] = *a[i0 + i][K(k0) + k];
    }
    for (int e = lane; e < 8 * TILE_K; e += 32) {
      const J j(e / TILE_K);
      const K k(e % TILE_K);
      *bt[j][k] = *b[j0 + j][K(k0) + k];
    }
    __syncwarp();
    AFrag af;
    BFrag bf;
    af.load(at, lane);
    bf.load(bt, lane);
    mma(acc, af, bf, acc);
    __syncwarp();
  }
  const C c(c_ptr);
  acc.store(c[i0][j0], lane);
}
