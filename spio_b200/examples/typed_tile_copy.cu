// A kernel written against generated typed-dimension types: it copies an NHWC fp16 tensor tile by
// tile through shared memory, loading each tile with one tiled TMA copy.
//
// The `@spio` blocks below are Python; spio_b200.generators.generate_from_source turns them into the
// header "types.h" this file includes (names on the left become C++ types).  Nothing here computes
// an offset by hand: coordinates are typed indices, the tensor map takes them in any order, and the
// compiler rejects a coordinate of the wrong dimension or an innermost TMA coordinate that is not a
// whole number of 16 bytes.
/*@spio
N = Dim()
H = Dim()
W = Dim()
C = Dim()
C8 = Fold(C, 8)
XMap = TensorMapSpec(dtype.half, Dims(C(64), W(16), H(4), N(1)), swizzle=0)
Tile = Tensor(dtype.uint4, Dims(H(4), W(16), C8(8)))
Y = Tensor(dtype.uint4, Dims(N(3), H(8), W(16), C8(8)))
Block = CompoundIndex(Dims(N(3), H(2)))
Piece = CompoundIndex(Dims(H(4), W(16), C8(8)))
Ring = MbarrierRing(1)
@spio*/
#include "types.h"

using namespace spio_b200;

extern "C" __global__ void typed_tile_copy(const __grid_constant__ TensorMap x_map, uint4* __restrict__ y,
                                           int* __restrict__ status) {
  __shared__ __align__(128) uint4 tile[Tile::storage_size()];
  __shared__ Ring ring;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    ring.init(1, 1);
    abort_flag = 0;
  }
  __syncthreads();
  volatile int* abortp = &abort_flag;

  // blockIdx.x -> (image, block of four rows)
  const Block block(blockIdx.x);
  const N n = block.get<N>();
  const H h0 = H(block.get<H>().get() * 4);

  Ring::Cursor cur;
  if (threadIdx.x == 0) {
    const XMap map(x_map);
    // coordinates in any order; W is left out and therefore 0; the channel coordinate is a fold of
    // 8 halves = 16 bytes, which is what the copy engine requires of the innermost coordinate
    if (ring.acquire(cur, XMap::box_bytes, abortp)) map.load(smem_u32(tile), ring.full(cur.slot), n, h0, C8(0));
  }
  const bool ok = ring.wait_full(cur, abortp);
  if (ok) {
    const Tile src(tile);
    const Y dst(y);
    for (int i = threadIdx.x; i < Piece::size(); i += blockDim.x) {
      const Piece piece(i);
      const H h = piece.get<H>();
      const W w = piece.get<W>();
      const C8 c8 = piece.get<C8>();
      *dst[n][h0 + h][w][c8] = *src[c8][w][h];  // subscript order does not matter
    }
  }
  __syncthreads();
  if (!ok && threadIdx.x == 0) atomicExch(status, (int)GW8_WAIT_TIMEOUT);
}
