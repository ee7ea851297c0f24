// Group-width-8 convolution, forward and input-gradient, for sm_100a.
//
//   fprop:  y[n,p,q,k]  = bias[k] + sum_{r,s,c in group(k)} x[n,p+r-pad_h,q+s-pad_w,c] * w[k,r,s,c]
//   dgrad:  dx[n,h,w,c] = sum_{r,s,k in group(c)} dy[n,h+r-pad_h',w+s-pad_w',k] * w[k,R-1-r,S-1-s,c]
//           with pad' = (R-1-pad_h, S-1-pad_w); the host passes pad' as the padding.
//
// Tensors are NHWC fp16; weights are [K][R][S][8] fp16; accumulation is fp32 and the
// result is rounded to fp16 once.  Same arithmetic contract as the reference kernel
// spio/src/conv2d_gw8.cu:10-224 (dgrad = its Mode::igrad, :99-105), but a different
// machine mapping:
//
//   * one persistent CTA per SM streams its share of output row pairs top to bottom;
//   * a load warp feeds a ring of shared-memory slots with TMA (128-byte swizzle, halo
//     and zero padding come from the out-of-range fill of the tiled copy);
//   * 8*WPG compute warps (one group of 8 channels each) read every slot exactly once
//     with ldmatrix, keep a window of WIN input rows x S column shifts in registers and
//     issue mma.sync m16n8k16 with the two k-halves fed by two different filter taps;
//   * results are staged with stmatrix in swizzled shared memory and written by a
//     store warp with TMA, so every global access is a full 128-byte line.
#pragma once

#include <cuda_fp16.h>

#include "gw8_common.cuh"

namespace spio_b200 {

template <int V>
struct IntC {
  static constexpr int value = V;
};

template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, 1)
conv2d_gw8_fwd_kernel(const __grid_constant__ TensorMap in_map,
                      const __grid_constant__ TensorMap out_map, const Gw8Geom g,
                      const __half* __restrict__ wgt, const float* __restrict__ bias,
                      int ns, int nob, int* __restrict__ status) {
  constexpr int R = Cfg::R, S = Cfg::S, WPG = Cfg::WPG, TPW = Cfg::TPW;
  constexpr int E = Cfg::E, WIN = Cfg::WIN, NT = Cfg::NT, NCW = Cfg::NCW;
  constexpr int NPH = WIN / 2;  // the window rotates by one slot (2 rows) per stage
  constexpr int MAX_NS = 16, MAX_NOB = 4;

  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) u64 bars[2 * MAX_NS + 2 * MAX_NOB];
  __shared__ int abort_flag;

  const u32 base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const u32 slot_bytes = (u32)(g.nb * 2 * g.bw) * 128u;
  const u32 obuf_bytes = (u32)(g.nb * 2 * g.wt) * 128u;
  const u32 ring = base;
  const u32 obufs = base + (u32)ns * slot_bytes;
  const u32 bar0 = smem_u32(bars);
  auto full = [&](int i) { return bar0 + 8u * (u32)i; };
  auto empty = [&](int i) { return bar0 + 8u * (u32)(MAX_NS + i); };
  auto ofull = [&](int i) { return bar0 + 8u * (u32)(2 * MAX_NS + i); };
  auto oempty = [&](int i) { return bar0 + 8u * (u32)(2 * MAX_NS + MAX_NOB + i); };

  if (threadIdx.x == 0) {
    for (int i = 0; i < ns; ++i) {
      mbar_init(full(i), 1);
      mbar_init(empty(i), NCW);
    }
    for (int i = 0; i < nob; ++i) {
      mbar_init(ofull(i), NCW);
      mbar_init(oempty(i), 1);
    }
    abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();

  const int total = g.n_chunks * g.n_ig * g.n_ct * g.n_pairs;
  const int u0 = gw8_span_begin(total, blockIdx.x, gridDim.x);
  const int u1 = gw8_span_begin(total, blockIdx.x + 1, gridDim.x);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* abortp = &abort_flag;

  if (warp == NCW) {
    // ------------------------------------------------------------ load warp
    if (lane == 0) {
      prefetch_tensormap(&in_map);
      Gw8Walk walk(u0, u1, g);
      Gw8Segment seg;
      int slot = 0;
      u32 par = 0;
      bool ok = true;
      while (ok && walk.next(seg)) {
        const int nst = seg.m1 - seg.m0 + E;
        const int c0 = seg.ck * 64;
        const int w0 = seg.ct * g.wt - g.pad_w;
        const int n0 = seg.ig * g.nb;
        for (int j = 0; j < nst; ++j) {
          if (!mbar_wait(empty(slot), par ^ 1u, abortp)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(full(slot), slot_bytes);
          tma_load_4d(ring + (u32)slot * slot_bytes, &in_map, full(slot), c0, w0,
                      2 * (seg.m0 + j) - g.pad_h, n0);
          if (++slot == ns) {
            slot = 0;
            par ^= 1u;
          }
        }
      }
    }
  } else if (warp == NCW + 1) {
    // ------------------------------------------------------------ store warp
    // Lane i owns staging buffer i: it waits until the compute warps have filled it,
    // issues the TMA store and releases the buffer once the store has read it.  Bulk
    // groups are tracked per thread, so the buffers drain independently.
    if (lane < nob) {
      prefetch_tensormap(&out_map);
      Gw8Walk walk(u0, u1, g);
      Gw8Segment seg;
      int turn = 0;   // which buffer the next pair goes to
      u32 opar = 0;   // parity of this lane's next use of its buffer
      bool ok = true;
      while (ok && walk.next(seg)) {
        const int c0 = seg.ck * 64;
        const int w0 = seg.ct * g.wt;
        const int n0 = seg.ig * g.nb;
        for (int m = seg.m0; m < seg.m1; ++m) {
          if (turn == lane) {
            if (!mbar_wait(ofull(lane), opar, abortp)) {
              ok = false;
              break;
            }
            tma_store_4d(&out_map, obufs + (u32)lane * obuf_bytes, c0, w0, 2 * m, n0);
            tma_store_commit();
            tma_store_wait_read0();
            mbar_arrive(oempty(lane));
            opar ^= 1u;
          }
          if (++turn == nob) turn = 0;
        }
      }
      tma_store_wait_all();
    }
  } else {
    // ------------------------------------------------------------ compute warps
    const int grp = warp & 7;
    const int wsub = warp >> 3;
    const u32 l7 = lane & 7;
    const int gq = lane >> 2;  // fragment row / column index "g"
    const int t4 = lane & 3;   // fragment pair index "t"

    // ldmatrix row addresses of this lane inside a slot, one per instruction.
    constexpr int NMAT = 2 * S;          // matrices per tile per stage: 2 rows x S shifts
    constexpr int NLD4 = NMAT / 4;       // x4 instructions
    constexpr bool LD2 = (NMAT % 4) != 0;  // plus one x2
    constexpr int NLD = NLD4 + (LD2 ? 1 : 0);
    u32 ld_off[NLD];
#pragma unroll
    for (int q = 0; q < NLD; ++q) {
      int f = 4 * q + (lane >> 3);
      if (LD2 && q == NLD4) f = 4 * q + ((lane >> 3) & 1);
      const u32 rowsel = (u32)(f / S), s = (u32)(f % S);
      ld_off[q] = (rowsel * (u32)g.bw + s + l7) * 128u + (((u32)grp ^ ((s + l7) & 7u)) << 4);
    }
    const u32 st_off = ((u32)((lane >> 3) & 1) * (u32)g.wt + l7) * 128u + (((u32)grp ^ l7) << 4);

    u32 in_off[TPW], out_off[TPW];
    bool tile_on[TPW];
#pragma unroll
    for (int t = 0; t < TPW; ++t) {
      const int tidx = wsub + WPG * t;
      tile_on[t] = tidx < g.ntiles;
      const int img = tidx / g.ncb, cb = tidx % g.ncb;
      in_off[t] = (u32)(img * 2 * g.bw + cb * 8) * 128u;
      out_off[t] = (u32)(img * 2 * g.wt + cb * 8) * 128u;
    }

    u32 wreg[NT];            // B fragments, one per tap
    float bias0 = 0.f, bias1 = 0.f;
    bool grp_on = false;
    int cur_ck = -1;
    u32 X[TPW][WIN][S];      // register window: [tile][physical row][column shift]

    Gw8Walk walk(u0, u1, g);
    Gw8Segment seg;
    int slot = 0, ob = 0;
    u32 par = 0, opar = 0;
    bool ok = true;

    while (ok && walk.next(seg)) {
      if (seg.ck != cur_ck) {
        cur_ck = seg.ck;
        const int ch0 = seg.ck * 64 + grp * 8;  // first channel of this warp's group
        grp_on = ch0 < g.c;
        bias0 = bias1 = 0.f;
#pragma unroll
        for (int f = 0; f < NT; ++f) wreg[f] = 0u;
        if (grp_on) {
          if (!g.dgrad) {
            // B[k = in-channel 2t,2t+1][n = out-channel g] of tap f = w[ch0+g][f][2t..2t+1]
            const __half* wp = wgt + ((size_t)(ch0 + gq) * NT) * 8 + 2 * t4;
#pragma unroll
            for (int f = 0; f < NT; ++f) wreg[f] = *reinterpret_cast<const u32*>(wp + f * 8);
            if (bias != nullptr) {
              bias0 = bias[ch0 + 2 * t4];
              bias1 = bias[ch0 + 2 * t4 + 1];
            }
          } else {
            // B[k = out-channel 2t,2t+1][n = in-channel g] of tap f = w[ch0+2t(+1)][NT-1-f][g]
            const __half* wp0 = wgt + ((size_t)(ch0 + 2 * t4) * NT) * 8 + gq;
            const __half* wp1 = wp0 + (size_t)NT * 8;
#pragma unroll
            for (int f = 0; f < NT; ++f) {
              const __half2 h = __halves2half2(wp0[(NT - 1 - f) * 8], wp1[(NT - 1 - f) * 8]);
              wreg[f] = *reinterpret_cast<const u32*>(&h);
            }
          }
        }
      }
      const int nst = seg.m1 - seg.m0 + E;

      // One stage: take slot j of the segment into the window, then (from stage E on)
      // produce pair j - E.  PH = j mod NPH fixes which physical window rows are which.
      auto stage = [&](auto phc, int j) -> bool {
        constexpr int PH = decltype(phc)::value;
        if (!mbar_wait(full(slot), par, abortp)) return false;
        const u32 sbase = ring + (u32)slot * slot_bytes;
        if (grp_on) {
#pragma unroll
          for (int t = 0; t < TPW; ++t) {
            if (tile_on[t]) {
              const u32 a = sbase + in_off[t];
#pragma unroll
              for (int q = 0; q < NLD4; ++q) {
                const int f0 = 4 * q;
                ldmatrix_x4<false>(X[t][2 * PH + (f0 + 0) / S][(f0 + 0) % S],
                                   X[t][2 * PH + (f0 + 1) / S][(f0 + 1) % S],
                                   X[t][2 * PH + (f0 + 2) / S][(f0 + 2) % S],
                                   X[t][2 * PH + (f0 + 3) / S][(f0 + 3) % S], a + ld_off[q]);
              }
              if (LD2) {
                const int f0 = 4 * NLD4;
                ldmatrix_x2<false>(X[t][2 * PH + (f0 + 0) / S][(f0 + 0) % S],
                                   X[t][2 * PH + (f0 + 1) / S][(f0 + 1) % S],
                                   a + ld_off[NLD - 1]);
              }
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty(slot));
        if (++slot == ns) {
          slot = 0;
          par ^= 1u;
        }
        if (j >= E) {
          if (!mbar_wait(oempty(ob), opar ^ 1u, abortp)) return false;
          const u32 obase = obufs + (u32)ob * obuf_bytes;
          if (grp_on) {
#pragma unroll
            for (int t = 0; t < TPW; ++t) {
              if (tile_on[t]) {
                float acc0[4] = {bias0, bias1, bias0, bias1};
                float acc1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int i = 0; i < NT / 2; ++i) {
                  // logical window row l (padded input row 2m + l) sits in physical row
                  // 2*((PH + 1 + l/2) % NPH) + (l & 1)
                  const int fa = 2 * i, fb = 2 * i + 1;
                  const int ra = fa / S, sa = fa % S, rb = fb / S, sb = fb % S;
                  const int pa0 = 2 * ((PH + 1 + ra / 2) % NPH) + (ra & 1);
                  const int pa1 = 2 * ((PH + 1 + (ra + 1) / 2) % NPH) + ((ra + 1) & 1);
                  const int pb0 = 2 * ((PH + 1 + rb / 2) % NPH) + (rb & 1);
                  const int pb1 = 2 * ((PH + 1 + (rb + 1) / 2) % NPH) + ((rb + 1) & 1);
                  if (i & 1)
                    mma_m16n8k16(acc1, X[t][pa0][sa], X[t][pa1][sa], X[t][pb0][sb], X[t][pb1][sb],
                                 wreg[fa], wreg[fb]);
                  else
                    mma_m16n8k16(acc0, X[t][pa0][sa], X[t][pa1][sa], X[t][pb0][sb], X[t][pb1][sb],
                                 wreg[fa], wreg[fb]);
                }
                if (NT & 1) {
                  const int fa = NT - 1;
                  const int ra = fa / S, sa = fa % S;
                  const int pa0 = 2 * ((PH + 1 + ra / 2) % NPH) + (ra & 1);
                  const int pa1 = 2 * ((PH + 1 + (ra + 1) / 2) % NPH) + ((ra + 1) & 1);
                  mma_m16n8k8(acc1, X[t][pa0][sa], X[t][pa1][sa], wreg[fa]);
                }
                const __half2 top = __floats2half2_rn(acc0[0] + acc1[0], acc0[1] + acc1[1]);
                const __half2 bot = __floats2half2_rn(acc0[2] + acc1[2], acc0[3] + acc1[3]);
                stmatrix_x2(obase + out_off[t] + st_off, *reinterpret_cast<const u32*>(&top),
                            *reinterpret_cast<const u32*>(&bot));
              }
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(ofull(ob));
          if (++ob == nob) {
            ob = 0;
            opar ^= 1u;
          }
        }
        return true;
      };

      for (int j = 0; ok && j < nst; j += NPH) {
        ok = stage(IntC<0>{}, j);
        if (NPH > 1 && ok && j + 1 < nst) ok = stage(IntC<(NPH > 1 ? 1 : 0)>{}, j + 1);
        if (NPH > 2 && ok && j + 2 < nst) ok = stage(IntC<(NPH > 2 ? 2 : 0)>{}, j + 2);
      }
    }
  }

  __syncthreads();
  if (abort_flag) {
    // Let copies that may still be in flight land before the CTA gives up its
    // shared memory, then report.
    for (int i = 0; i < 64; ++i) __nanosleep(20000);
    if (threadIdx.x == 0) atomicExch(status, (int)GW8_WAIT_TIMEOUT);
  }
}

}  // namespace spio_b200
