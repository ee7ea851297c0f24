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
//     and zero padding come from the out-of-range fill of the tiled copy); a slot holds
//     PPS row pairs, so one barrier hand-off is amortised over 2*PPS image rows;
//   * 8*WPG compute warps (one group of 8 channels each) read every slot exactly once
//     with ldmatrix, keep a window of WIN input rows x S column shifts in registers and
//     issue mma.sync m16n8k16 (M = 16 pixels of one row) with the two k-halves fed by two
//     horizontally adjacent filter taps;
//   * results are staged with stmatrix in swizzled shared memory and written by the
//     lanes of a store warp with TMA, so every global access is a full 128-byte line;
//   * barrier polls are issued ahead of the work that hides their latency.
#pragma once

#include <cuda_fp16.h>

#include "gw8_common.cuh"

namespace spio_b200 {

// The kernel body is a device function so that both the ahead-of-time instantiations and
// the just-in-time wrappers (one extern "C" kernel per layer shape) can share it.
template <class Cfg>
__device__ __forceinline__ void
conv2d_gw8_fwd_body(const TensorMap& in_map, const TensorMap& out_map, const Gw8Geom& g,
                    const __half* __restrict__ wgt, const float* __restrict__ bias, int ns, int nob,
                    int* __restrict__ status) {
  constexpr int S = Cfg::S, WPG = Cfg::WPG, TPW = Cfg::TPW, PPS = Cfg::PPS;
  constexpr int E = Cfg::E, WIN = Cfg::WIN, NT = Cfg::NT, NCW = Cfg::NCW;
  constexpr int NPH = WIN / 2;  // the window rotates by one row pair per sub-step
  constexpr int MAX_NS = 16, MAX_NOB = 4;

  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) u64 bars[2 * MAX_NS + 2 * MAX_NOB];
  __shared__ Gw8StageDesc desc[MAX_NS];
  __shared__ int abort_flag;
  constexpr int DYNQ = 32;         // claims in flight between the load lane and the store lanes
  __shared__ int dynq[DYNQ];       // first unit of every piece the load lane claimed from the pool
  __shared__ int dynlen[DYNQ];     // and its length in pairs
  __shared__ int dyn_count;        // how many it has claimed so far
  volatile int* const dyn_n = &dyn_count;

  // ring slots: [nb][2*PPS rows][bw][64 ch]; staging buffers: PPS x [nb][2 rows][wt][64 ch]
  const u32 ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const u32 obufs = ring + (u32)ns * g.slot_bytes;
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
    dyn_count = 0;
    mbar_fence_init();
  }
  __syncthreads();
  // The tensor maps are kernel parameters: fetching them does not depend on earlier kernels.
  if (threadIdx.x == 32 * NCW) prefetch_tensormap(&in_map);
  if (threadIdx.x == 32 * (NCW + 1)) prefetch_tensormap(&out_map);
  // Everything above touches only shared memory and may overlap the tail of the preceding
  // kernel.  Dependents are released only after the wait, so a chain of such launches never
  // runs ahead of the work that precedes its first kernel.
  // A segment of L pairs is streamed in ceil((L + E) / PPS) stages.  Stage i brings the
  // input row pairs PPS*i .. PPS*i+PPS-1 (relative to the segment) and completes the
  // output pairs PPS*i+u-E, u < PPS, that lie in [0, L).  The load warp and the store
  // lanes walk the CTA's span; the compute warps are told what a slot holds by the
  // descriptor the load warp writes next to it.
  auto stages_of = [&](const Gw8Segment& sg) { return (sg.m1 - sg.m0 + E + PPS - 1) / PPS; };
  const int total = g.n_chunks * g.n_ig * g.n_ct * g.n_pairs;
  const int n_static = g.dyn_chunk > 0 ? g.dyn_begin : total;
  if (threadIdx.x == 32 * NCW && g.warm > 0 && !g.independent) {
    // The load lane asks L2 for the boxes of its first stages while the preceding kernel drains.
    Gw8Walk walk(gw8_span_begin(n_static, blockIdx.x, gridDim.x), gw8_span_begin(n_static, blockIdx.x + 1, gridDim.x), g);
    Gw8Segment seg;
    int left = g.warm;
    while (left > 0 && walk.next(seg)) {
      const int nst = stages_of(seg);
      for (int i = 0; i < nst && left > 0; ++i, --left)
        tma_prefetch_4d(&in_map, seg.ck * 64, seg.ct * g.wt - g.pad_w, 2 * (seg.m0 + PPS * i) - g.pad_h,
                        seg.ig * g.nb);
    }
  }
  if (!g.independent) grid_dependency_wait();
  grid_dependency_launch_dependents();

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* abortp = &abort_flag;

  auto out_mask = [&](int i, int len) {
    int m = 0;
#pragma unroll
    for (int u = 0; u < PPS; ++u) {
      const int q = PPS * i + u - E;
      if (q >= 0 && q < len) m |= 1 << u;
    }
    return m;
  };

  if (warp >= NCW) {
    // the producer warpgroup keeps 24 registers per thread and frees the rest for the consumers
    if (Cfg::FWD_SETMAXNREG) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(Cfg::FWD_REGS_PRODUCER));
    // The first g.dyn_begin units of the flattened work are cut into equal static spans, one
    // per CTA; the rest (none unless the launch asks for it) is a pool that the load warps
    // claim from in pieces of g.dyn_chunk pairs, so that CTAs whose HBM traffic was served
    // faster take more of the tail.  The load lane publishes every piece it claims in `dynq`
    // for the store lanes, which walk the same sequence.
    const int u0 = gw8_span_begin(n_static, blockIdx.x, gridDim.x);
    const int u1 = gw8_span_begin(n_static, blockIdx.x + 1, gridDim.x);
    if (warp == NCW) {
      // ---------------------------------------------------------- load warp
      if (lane == 0) {
        prefetch_tensormap(&in_map);
        const u64 in_policy = make_l2_policy(g.hint_in);
        int slot = 0;
        u32 par = 0;
        bool ok = true;
        int issued = 0;  // stages issued so far, counted only until the start-up window has been passed
        auto load_span = [&](int ua, int ub) {
          Gw8Walk walk(ua, ub, g);
          Gw8Segment seg;
          while (ok && walk.next(seg)) {
            const int nst = stages_of(seg);
            const int len = seg.m1 - seg.m0;
            const int c0 = seg.ck * 64;
            const int w0 = seg.ct * g.wt - g.pad_w;
            const int n0 = seg.ig * g.nb;
            for (int i = 0; i < nst; ++i) {
              if (issued >= 0 && g.prefill > 0 && issued++ == g.prefill) {
                // start-up window: let the first slot land before the rest of the ring is requested
                issued = -1;
                if (!mbar_wait(full(0), 0u, abortp)) {
                  ok = false;
                  break;
                }
              }
              if (!mbar_wait(empty(slot), par ^ 1u, abortp)) {
                ok = false;
                break;
              }
              desc[slot].ck = seg.ck;
              desc[slot].mask = out_mask(i, len);
              desc[slot].ph0 = (PPS * i) % NPH;
              desc[slot].flags = 0;
              mbar_arrive_expect_tx(full(slot), g.slot_bytes);
              tma_load_4d(ring + (u32)slot * g.slot_bytes, &in_map, full(slot), c0, w0,
                          2 * (seg.m0 + PPS * i) - g.pad_h, n0, g.hint_in, in_policy);
              if (++slot == ns) {
                slot = 0;
                par ^= 1u;
              }
            }
          }
        };
        load_span(u0, u1);
        if (g.dyn_chunk > 0) {
          // Pieces shrink as the pool drains (about what is left divided by twice the number of
          // CTAs, at most g.dyn_chunk pairs), so that the CTAs finish within one small piece of
          // each other.  A piece of c pairs is streamed in ceil((c + E) / PPS) stages; sizes with
          // (c + E) a multiple of PPS waste no part of a stage.  What is left is estimated from
          // the counter value the previous claim returned: a stale value only makes a piece a
          // little larger than intended, the pieces themselves never overlap.
          constexpr int CMIN = PPS - (E % PPS);
          int k = 0, seen = 0;
          while (ok) {
            int c = (total - g.dyn_begin - seen) / (2 * (int)gridDim.x);
            if (c > g.dyn_chunk) c = g.dyn_chunk;
            c = (c + E) / PPS * PPS - E;
            if (c < CMIN) c = CMIN;
            const int taken = atomicAdd(status + 1 + g.dyn_slot, c);
            seen = taken + c;
            const int u = g.dyn_begin + taken;
            dynq[k & (DYNQ - 1)] = u < total ? u : -1;  // -1: the pool is empty
            dynlen[k & (DYNQ - 1)] = c;
            __threadfence_block();
            *dyn_n = ++k;
            if (u >= total) break;
            load_span(u, u + c < total ? u + c : total);
          }
        }
        if (ok && mbar_wait(empty(slot), par ^ 1u, abortp)) {
          desc[slot].flags = GW8_STAGE_END;
          mbar_arrive(full(slot));
        }
      }
    } else if (warp == NCW + 1) {
      // ---------------------------------------------------------- store warp
      // Lane i owns staging buffer i: it waits until the compute warps have filled it,
      // issues the TMA stores of the stage and releases the buffer once they have read
      // it.  Bulk groups are tracked per thread, so the buffers drain independently.
      if (lane < nob) {
        prefetch_tensormap(&out_map);
        int turn = 0;  // which buffer the next stage goes to
        u32 opar = 0;  // parity of this lane's next use of its buffer
        bool ok = true;
        auto store_span = [&](int ua, int ub) {
          Gw8Walk walk(ua, ub, g);
          Gw8Segment seg;
          while (ok && walk.next(seg)) {
            const int nst = stages_of(seg);
            const int len = seg.m1 - seg.m0;
            const int c0 = seg.ck * 64;
            const int w0 = seg.ct * g.wt;
            const int n0 = seg.ig * g.nb;
            for (int i = 0; i < nst; ++i) {
              const int mask = out_mask(i, len);
              if (mask == 0) continue;
              if (turn == lane) {
                if (!mbar_wait(ofull(lane), opar, abortp)) {
                  ok = false;
                  break;
                }
#pragma unroll
                for (int u = 0; u < PPS; ++u) {
                  if (mask & (1 << u))
                    tma_store_4d(&out_map,
                                 obufs + (u32)lane * g.obuf_bytes + (u32)u * g.out_pair_bytes, c0, w0,
                                 2 * (seg.m0 + PPS * i + u - E), n0);
                }
                tma_store_commit();
                tma_store_wait_read0();
                mbar_arrive(oempty(lane));
                opar ^= 1u;
              }
              if (++turn == nob) turn = 0;
            }
          }
        };
        store_span(u0, u1);
        if (g.dyn_chunk > 0) {
          for (int k = 0; ok; ++k) {
            // wait (bounded) until the load lane has published its k-th claim
            u64 t0 = 0;
            for (u32 it = 1; *dyn_n <= k; ++it) {
              if ((it & 63u) == 0u) {
                if (*abortp) ok = false;
                const u64 now = globaltimer_ns();
                if (t0 == 0) t0 = now;
                else if (now - t0 > SPIO_WAIT_LIMIT_NS) {
                  *abortp = 1;
                  ok = false;
                }
                if (!ok) break;
              }
            }
            if (!ok) break;
            __threadfence_block();
            const int u = dynq[k & (DYNQ - 1)];
            const int c = dynlen[k & (DYNQ - 1)];
            if (u < 0) break;
            store_span(u, u + c < total ? u + c : total);
          }
        }
        tma_store_wait_all();
      }
    }
  } else {
    if (Cfg::FWD_SETMAXNREG) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(Cfg::FWD_REGS_CONSUMER));
    // ------------------------------------------------------------ compute warps
    // A warp owns one channel group and TPW "block tiles": 16 consecutive pixels of the
    // rows of one image.  For each input row and each pair of column shifts (s, s+1) ONE
    // ldmatrix.x4 delivers {shift s: px 0-7, px 8-15; shift s+1: px 0-7, px 8-15}, which is
    // exactly the A operand of an m16n8k16 whose k-halves are the taps (r,s) and (r,s+1);
    // an odd last shift comes from an .x2 and feeds an m16n8k8.  Operands therefore sit in
    // consecutive registers as the hardware wants them: no register moves.
    const int grp = warp & 7;
    const int wsub = warp >> 3;
    const u32 l7 = lane & 7;
    constexpr int NQ = S / 2;         // shift pairs per row  -> x4 loads, k16 MMAs
    constexpr bool ODD = (S & 1) != 0;  // last shift alone     -> x2 load,  k8 MMA
    constexpr int NLD = NQ + (ODD ? 1 : 0);

    // per-lane byte offset of each load instruction: the NQ shift-pair loads address one row,
    // the load of the odd last shift addresses both rows of a row pair
    // {row 0: px 0-7, px 8-15; row 1: px 0-7, px 8-15}
    // The second 8-pixel half of a block tile lies 8 pixels further along the row, or, for
    // images at most 8 pixels wide (g.pair_images), at the same place in the next image of the
    // slot: ldmatrix and stmatrix take one row address per 8x8 matrix, so only these per-lane
    // offsets differ between the two layouts.  Both distances are multiples of 1 KiB, which
    // leaves the swizzle phase (pixel & 7) of an address unchanged.
    const u32 half_in = g.pair_images ? g.img_in_bytes : 8u * 128u;
    const u32 half_out = g.pair_images ? g.img_out_bytes : 8u * 128u;
    u32 ld_off[NLD];
#pragma unroll
    for (int q = 0; q < NLD; ++q) {
      const u32 mi = (u32)lane >> 3;  // matrix this lane addresses
      const bool odd_col = ODD && q == NQ;
      const u32 sh = odd_col ? (u32)(S - 1) : (u32)(2 * q) + (mi >> 1);  // column shift
      const u32 px = sh + l7;                                            // pixel within its half
      const u32 row = odd_col ? (mi >> 1) : 0u;
      ld_off[q] = (mi & 1u) * half_in + (row * (u32)g.bw + px) * 128u + (((u32)grp ^ (px & 7u)) << 4);
    }
    const u32 st_off = (((u32)lane >> 3) & 1u) * half_out + l7 * 128u + (((u32)grp ^ l7) << 4);
    const u32 in_row_bytes = g.in_pair_bytes >> 1;        // bw * 128
    const u32 out_row_bytes = g.img_out_bytes >> 1;       // wt * 128

    // Block tile t of this warp: image img of the slot, first pixel px0 of the block.
    u32 tile_code[TPW];  // (img << 16) | (px0 * 128)
    // Tiles wsub + WPG * t below `tiles_live` are computed: the slot's tile count, or none while
    // the warp's channel group lies beyond the last channel.
    int tiles_live = 0;
    auto tile_on = [&](int t) { return wsub + WPG * t < tiles_live; };
#pragma unroll
    for (int t = 0; t < TPW; ++t) {
      const int tidx = wsub + WPG * t;
      const int blk = tidx % g.nblk;
      int px0 = 16 * blk;
      if (px0 > g.wt - 16) px0 = g.wt - 16;  // the last block is shifted left, never past the tile
      if (g.pair_images)
        tile_code[t] = (u32)(2 * tidx) << 16;  // images 2 * tidx and 2 * tidx + 1, pixels 0-7 of each
      else
        tile_code[t] = ((u32)(tidx / g.nblk) << 16) | ((u32)px0 * 128u);
    }
    auto in_off = [&](int t) { return (tile_code[t] & 0xffffu) + (tile_code[t] >> 16) * g.img_in_bytes; };
    auto out_off = [&](int t) { return (tile_code[t] & 0xffffu) + (tile_code[t] >> 16) * g.img_out_bytes; };

    u32 wreg[NT];  // B fragments, one per tap
    float bias0 = 0.f, bias1 = 0.f;
    bool grp_on = false;
    int cur_ck = -1;
    // register window: [tile][physical row][shift pair][4] and, for odd S, the last shift of
    // both rows of a row pair: [tile][phase][4]
    u32 XQ[TPW][WIN][NQ > 0 ? NQ : 1][4];
    u32 XP[TPW][NPH][4];

    int slot = 0, ob = 0;
    u32 par = 0, opar = 0;
    bool full_seen = mbar_test_wait(full(0), 0u);  // poll issued ahead of its use

    // One stage.  PH0 fixes which physical window rows the PPS sub-steps overwrite.
    // ALL: every tile of the warp is live (the usual case), no per-tile tests.
    // FULL: every sub-step completes an output pair (the interior of an image), no mask tests.
    auto stage = [&](auto ph0c, auto allc, auto fullc, const int mask) -> bool {
      constexpr int PH0 = decltype(ph0c)::value;
      constexpr bool ALL = decltype(allc)::value != 0;
      constexpr bool FULL = decltype(fullc)::value != 0;
      const u32 sbase = ring + (u32)slot * g.slot_bytes;
      bool obuf_seen = (FULL || mask) ? mbar_test_wait(oempty(ob), opar ^ 1u) : true;
      const u32 obase = obufs + (u32)ob * g.obuf_bytes;
#pragma unroll
      for (int u = 0; u < PPS; ++u) {
        const int PH = (PH0 + u) % NPH;
        {
#pragma unroll
          for (int t = 0; t < TPW; ++t) {
            if (ALL || tile_on(t)) {
              const u32 a = opaque_add(sbase, in_off(t)) + (u32)u * g.in_pair_bytes;
#pragma unroll
              for (int row = 0; row < 2; ++row) {
#pragma unroll
                for (int q = 0; q < NQ; ++q)
                  ldmatrix_x4<false>(XQ[t][2 * PH + row][q][0], XQ[t][2 * PH + row][q][1],
                                     XQ[t][2 * PH + row][q][2], XQ[t][2 * PH + row][q][3],
                                     a + (u32)row * in_row_bytes + ld_off[q]);
              }
              if (ODD)
                ldmatrix_x4<false>(XP[t][PH][0], XP[t][PH][1], XP[t][PH][2], XP[t][PH][3],
                                   a + ld_off[NLD - 1]);
            }
          }
        }
        if (u == PPS - 1) {
          // every row of the slot is in registers: hand it back and look ahead
          __syncwarp();
          if (lane == 0) mbar_arrive(empty(slot));
          if (++slot == ns) {
            slot = 0;
            par ^= 1u;
          }
          full_seen = mbar_test_wait(full(slot), par);
        }
        if (FULL || (mask & (1 << u))) {  // this sub-step completes an output pair
          if (!obuf_seen) {
            if (!mbar_wait(oempty(ob), opar ^ 1u, abortp)) return false;
            obuf_seen = true;
          }
          {
#pragma unroll
            for (int t = 0; t < TPW; ++t) {
              if (ALL || tile_on(t)) {
                const u32 o = opaque_add(obase, out_off(t)) + (u32)u * g.out_pair_bytes + st_off;
#pragma unroll
                for (int y = 0; y < 2; ++y) {  // the two output rows of the pair
                  float acc[4] = {bias0, bias1, bias0, bias1};
#pragma unroll
                  for (int r = 0; r < Cfg::R; ++r) {
                    // logical window row l = y + r (padded input row 2m + l) sits in
                    // physical row 2*((PH + 1 + l/2) % NPH) + (l & 1)
                    const int l = y + r;
                    const int pp = (PH + 1 + l / 2) % NPH;  // phase slot holding row l
                    const int pr = 2 * pp + (l & 1);
#pragma unroll
                    for (int q = 0; q < NQ; ++q)
                      mma_m16n8k16(acc, XQ[t][pr][q][0], XQ[t][pr][q][1], XQ[t][pr][q][2],
                                   XQ[t][pr][q][3], wreg[r * S + 2 * q], wreg[r * S + 2 * q + 1]);
                    if (ODD) {
                      // Last column of taps: two vertically adjacent taps share one k16 MMA when
                      // their input rows are the two rows of one slot, else a k8 MMA.
                      const bool starts_pair = (l & 1) == 0 && r + 1 < Cfg::R;
                      const bool in_prev_pair = (l & 1) == 1 && r >= 1;
                      if (starts_pair)
                        mma_m16n8k16(acc, XP[t][pp][0], XP[t][pp][1], XP[t][pp][2], XP[t][pp][3],
                                     wreg[r * S + S - 1], wreg[(r + 1) * S + S - 1]);
                      else if (!in_prev_pair)
                        mma_m16n8k8(acc, XP[t][pp][2 * (l & 1)], XP[t][pp][2 * (l & 1) + 1],
                                    wreg[r * S + S - 1]);
                    }
                  }
                  const __half2 lo = __floats2half2_rn(acc[0], acc[1]);  // pixels 0-7 of the block
                  const __half2 hi = __floats2half2_rn(acc[2], acc[3]);  // pixels 8-15
                  stmatrix_x2(o + (u32)y * out_row_bytes, *reinterpret_cast<const u32*>(&lo),
                              *reinterpret_cast<const u32*>(&hi));
                }
              }
            }
          }
        }
      }
      if (FULL || mask) {
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

    for (;;) {
      if (!full_seen && !mbar_wait(full(slot), par, abortp)) break;
      const int4 d = *reinterpret_cast<const int4*>(&desc[slot]);  // ck, mask, ph0, flags
      if (d.w & GW8_STAGE_END) break;
      if (d.x != cur_ck) {
        cur_ck = d.x;
        const int gq = lane >> 2;  // fragment row / column index "g"
        const int t4 = lane & 3;   // fragment pair index "t"
        const int ch0 = d.x * 64 + grp * 8;  // first channel of this warp's group
        grp_on = ch0 < g.c;
        tiles_live = grp_on ? g.ntiles : 0;
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
      auto run = [&](auto allc, auto fullc) -> bool {
        if (d.z == 0) return stage(IntC<0>{}, allc, fullc, d.y);
        if (d.z == 1) return stage(IntC<(NPH > 1 ? 1 : 0)>{}, allc, fullc, d.y);
        return stage(IntC<(NPH > 2 ? 2 : 0)>{}, allc, fullc, d.y);
      };
      bool ok;
      if (tiles_live >= WPG * TPW) {
        if (d.y == (1 << PPS) - 1)
          ok = run(IntC<1>{}, IntC<1>{});
        else
          ok = run(IntC<1>{}, IntC<0>{});
      } else {
        ok = run(IntC<0>{}, IntC<0>{});
      }
      if (!ok) break;
    }
  }

  __syncthreads();
  // A kernel that did not wait for its predecessors at the start must not COMPLETE before
  // them either: a later kernel that waits for this one relies on that to be ordered after
  // the whole chain.  By now they have long finished, so this returns at once.
  if (g.independent) grid_dependency_wait();
  if (g.dyn_chunk > 0 && threadIdx.x == 0) {
    // every load warp has seen the pool empty by now; the last CTA to leave clears the counters
    if (atomicAdd(status + 1 + GW8_DYN_SLOTS + g.dyn_slot, 1) == (int)gridDim.x - 1) {
      status[1 + g.dyn_slot] = 0;
      status[1 + GW8_DYN_SLOTS + g.dyn_slot] = 0;
    }
  }
  if (abort_flag) {
    // Let copies that may still be in flight land before the CTA gives up its
    // shared memory, then report.
    for (int i = 0; i < 64; ++i) __nanosleep(20000);
    if (threadIdx.x == 0) atomicExch(status, (int)GW8_WAIT_TIMEOUT);
  }
}

template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, 1)
conv2d_gw8_fwd_kernel(const __grid_constant__ TensorMap in_map,
                      const __grid_constant__ TensorMap out_map, const Gw8Geom g,
                      const __half* __restrict__ wgt, const float* __restrict__ bias,
                      int ns, int nob, int* __restrict__ status) {
  conv2d_gw8_fwd_body<Cfg>(in_map, out_map, g, wgt, bias, ns, nob, status);
}

}  // namespace spio_b200
