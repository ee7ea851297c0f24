// Ahead-of-time instantiations of the tcgen05 forward kernel for filters up to 3 x 3.
#include "conv2d_gw8_fwd_tc.cuh"
#include "gw8_host.h"

namespace spio_b200 {

namespace {

template <int R, int S>
const void* tc_kernel() {
  return (const void*)&conv2d_gw8_fwd_tc_kernel<Gw8TcConfig<R, S>>;
}

}  // namespace

const void* gw8_tc_kernel(int r, int s) {
  static const void* const table[3][3] = {
      {tc_kernel<1, 1>(), tc_kernel<1, 2>(), tc_kernel<1, 3>()},
      {tc_kernel<2, 1>(), tc_kernel<2, 2>(), tc_kernel<2, 3>()},
      {tc_kernel<3, 1>(), tc_kernel<3, 2>(), tc_kernel<3, 3>()},
  };
  if (r < 1 || r > 3 || s < 1 || s > 3) return nullptr;
  return table[r - 1][s - 1];
}

}  // namespace spio_b200

