// Ahead-of-time instantiations of the gw8 kernels for one filter height.
// Compiled once per GW8_R in 1..5 so the five builds run in parallel.
#include "conv2d_gw8_fwd.cuh"
#include "conv2d_gw8_wgrad.cuh"
#include "gw8_host.h"

#ifndef GW8_R
#error "compile with -DGW8_R=<filter height 1..5>"
#endif

namespace spio_b200 {

namespace {

template <int S, int WPG, int TPW, int PPS = 1>
Gw8Variant make_variant() {
  using Cfg = Gw8Config<GW8_R, S, WPG, TPW, PPS>;                // weight gradient: 8 x 2 tiles
  using FwdCfg = Gw8Config<GW8_R, S, WPG, (TPW + 1) / 2, PPS>;  // forward: 16 x 1 block tiles
  return Gw8Variant{GW8_R,
                    S,
                    WPG,
                    TPW,
                    PPS,
                    Cfg::THREADS,
                    Cfg::WGRAD_THREADS,
                    (const void*)&conv2d_gw8_fwd_kernel<FwdCfg>,
                    (const void*)&conv2d_gw8_wgrad_kernel<Cfg, false>,
                    (const void*)&conv2d_gw8_wgrad_kernel<Cfg, true>};
}

// The register window costs WIN * S * TPW registers per thread, so wide or tall
// filters get fewer tiles per warp.
// The first variant listed for a filter size is the planner's default.
const Gw8Variant kVariants[] = {
#if GW8_R <= 3
    make_variant<1, 2, 4, 2>(), make_variant<2, 2, 4, 2>(), make_variant<3, 2, 4, 2>(),
    make_variant<4, 2, 2, 2>(), make_variant<5, 2, 2, 2>(),
    make_variant<1, 2, 4, 1>(), make_variant<2, 2, 4, 1>(), make_variant<3, 2, 4, 1>(),
    make_variant<4, 2, 2, 1>(), make_variant<5, 2, 2, 1>(),
#if GW8_R == 3
    // extra 3x3 variants for tuning
    make_variant<3, 1, 4, 1>(), make_variant<3, 1, 8, 1>(), make_variant<3, 1, 8, 2>(),
    make_variant<3, 2, 2, 1>(), make_variant<3, 3, 2, 1>(), make_variant<3, 3, 3, 2>(),
#endif
#else
    make_variant<1, 2, 4, 2>(), make_variant<2, 2, 2, 2>(), make_variant<3, 2, 2, 2>(),
    make_variant<4, 2, 2, 2>(), make_variant<5, 2, 1, 2>(),
    make_variant<1, 2, 4, 1>(), make_variant<2, 2, 2, 1>(), make_variant<3, 2, 2, 1>(),
    make_variant<4, 2, 2, 1>(), make_variant<5, 2, 1, 1>(),
#endif
};

}  // namespace

#define GW8_CAT_(a, b) a##b
#define GW8_CAT(a, b) GW8_CAT_(a, b)

int GW8_CAT(gw8_variants_r, GW8_R)(const Gw8Variant** out) {
  *out = kVariants;
  return (int)(sizeof(kVariants) / sizeof(kVariants[0]));
}

}  // namespace spio_b200
