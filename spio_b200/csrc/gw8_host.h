// Host-side plumbing shared by the translation units of libspio_b200: the launcher
// table filled by the per-filter-height instantiation files, and the planning of a
// launch (tile geometry, shared-memory budget, tensor maps).
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <string>

#include "../../include/spio_b200.h"

#include "gw8_common.cuh"

namespace spio_b200 {

// Tile configuration requested by the caller; zero fields are chosen by the planner.
struct Gw8Tune {
  int wpg;  // warps per group (compiled variants only)
  int tpw;  // tiles per warp  (compiled variants only)
  int ns;   // ring slots
  int nob;  // output staging buffers
  int ncb;  // column blocks per column tile
  int nb;   // images per slot
  int grid; // CTAs (0: one per SM)
  int pps;  // row pairs per ring slot (compiled variants only)
  int engine;  // 0 auto, 1 warp-level mma.sync kernels, 2 tcgen05 forward kernel
};

struct Gw8Variant {
  int r, s, wpg, tpw, pps;
  int fwd_threads, wgrad_threads;
  const void* fwd_kernel;    // conv2d_gw8_fwd_kernel<Cfg>
  const void* wgrad_kernel;       // conv2d_gw8_wgrad_kernel<Cfg, false>
  const void* wgrad_bias_kernel;  // conv2d_gw8_wgrad_kernel<Cfg, true>: also sums dy for the bias gradient
};

// Each gw8_inst.cu build (one per filter height R) exports its variants.
int gw8_variants_r1(const Gw8Variant** out);
int gw8_variants_r2(const Gw8Variant** out);
int gw8_variants_r3(const Gw8Variant** out);
int gw8_variants_r4(const Gw8Variant** out);
int gw8_variants_r5(const Gw8Variant** out);

// Shared by the translation units of the library (gw8_capi.cu).
int jit_fail(const std::string& msg);  // sets the calling thread's last-error string, returns 1
bool gw8_pdl_enabled();                // programmatic dependent launch (SPIO_PDL=0 turns it off)
int gw8_status_pointer(int** status);  // device address of the current device's status word

// The data-parallel exchange of the weight gradient (dp_exchange.cu).
int dp_exchange_ctas(size_t n_floats);  // CTAs of one exchange of n floats
int dp_push(const spio_dp_exchange* dp, const float* a, size_t n_a, const float* b, size_t n_b,
            cudaStream_t stream);
int dp_sum(const spio_dp_exchange* dp, float* a, size_t n_a, float* b, size_t n_b, cudaStream_t stream);
int dp_allreduce(const spio_dp_exchange* dp, float* a, size_t n_a, float* b, size_t n_b, cudaStream_t stream);

// Driver-API launch of a just-in-time compiled function (jit_driver.cpp).
int jit_launch(void* function, int grid, int block, int smem_bytes, cudaStream_t stream, void** args,
               bool programmatic);

// conv2d_gw8_fwd_tc_kernel<Gw8TcConfig<r, s>> for 1 <= r, s <= 3, else NULL.
const void* gw8_tc_kernel(int r, int s);

}  // namespace spio_b200
