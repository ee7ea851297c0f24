// Group-width-8 convolution, weight gradient, for sm_100a.
//
//   dw[k,r,s,c] = sum_{n,p,q} x[n,p+r-pad_h,q+s-pad_w,c] * dy[n,p,q,k]     (c in group(k))
//
// x and dy are NHWC fp16, dw is [K][R][S][8] fp32.  Same arithmetic contract as the
// reference kernel spio/src/conv2d_gw8_wgrad.cu:10-226, which sums CTA partials with
// fp32 atomicAdd into a pre-zeroed buffer (:207-224).  Here the sum is two-level and
// has a fixed order: every compute warp keeps its taps x 8 x 8 partial in registers for
// its whole share of the pixels and writes it once to a scratch buffer; a second small
// kernel adds the partials of a chunk in a fixed order and overwrites dw, so dw needs no
// zero fill and the result does not vary from run to run.
//
// Mapping: per group the contraction is M = two taps x 8 in-channels, N = 8 out-channels,
// K = 16 pixels (8 columns of two output rows), mma.sync m16n8k16; both operands come
// from shared memory with ldmatrix.trans.  x rows are read once and kept in a register
// window exactly as in the forward kernel; pixels outside the image contribute nothing
// because the tiled copy of dy zero-fills them.
#pragma once

#include <cuda_fp16.h>

#include "conv2d_gw8_fwd.cuh"

namespace spio_b200 {

// Scratch layout: [chunk][part]{[64 local out-channels][taps][8 in-channels], [64 bias sums]} fp32
// with part = split index of the CTA, n_parts = n_split: the WPG warps of a group are summed
// inside the CTA through shared memory before the partial is written.  CTAs that walk
// several chunks (more chunks than CTAs) keep one part per warp instead, n_parts = n_split * WPG.
//
// Bias gradient almost for free: two filter taps share one m16n8k16 (tap 2i in rows 0-7 of A,
// tap 2i+1 in rows 8-15).  With an odd number of taps the last MMA has rows 8-15 to spare; with
// WITH_BIAS they are fed ones, so rows 8-15 of its accumulator hold sum over pixels of
// dy[pixel][k], which is the gradient of the bias.  It is written behind the weight partial of
// each part.  Feeding a register instead of a literal zero costs about 5 % of the kernel's
// time (measured), so the kernel without it is a separate instantiation.
#define GW8_PART_FLOATS(taps) (64 * (taps) * 8 + 64)
// The kernel body is a device function so that both the ahead-of-time instantiations and
// the just-in-time wrappers (one extern "C" kernel per layer shape) can share it.
template <class Cfg, bool WITH_BIAS = false>
__device__ __forceinline__ void
conv2d_gw8_wgrad_body(const TensorMap& x_map, const TensorMap& dy_map, const Gw8Geom& g,
                      float* __restrict__ scratch, int ns, int* __restrict__ status) {
  constexpr int S = Cfg::S, WPG = Cfg::WPG, TPW = Cfg::TPW, PPS = Cfg::PPS;
  constexpr int E = Cfg::E, WIN = Cfg::WIN, NT = Cfg::NT, NCW = Cfg::NCW;
  constexpr int NPH = WIN / 2;
  constexpr int NACC = (NT + 1) / 2;
  constexpr bool BIAS = WITH_BIAS && (NT & 1) != 0;  // the spare half of the last MMA sums dy
  constexpr u32 ONES = 0x3C003C00u;       // half2(1, 1)
  constexpr int MAX_NS = 16;

  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) u64 bars[2 * MAX_NS];
  __shared__ int abort_flag;

  const u32 base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const u32 x_pair_bytes = (u32)(2 * g.bw) * 128u;   // one row pair of one image of x
  const u32 d_pair_bytes = (u32)(2 * g.wt) * 128u;   // one row pair of one image of dy
  const u32 xslot_bytes = (u32)(g.nb * PPS) * x_pair_bytes;  // [nb][2*PPS rows][bw][64]
  const u32 dslot_bytes = (u32)(g.nb * PPS) * d_pair_bytes;  // [nb][2*PPS rows][wt][64]
  const u32 stage_bytes = xslot_bytes + dslot_bytes;
  const u32 bar0 = smem_u32(bars);
  auto full = [&](int i) { return bar0 + 8u * (u32)i; };
  auto empty = [&](int i) { return bar0 + 8u * (u32)(MAX_NS + i); };

  if (threadIdx.x == 0) {
    for (int i = 0; i < ns; ++i) {
      mbar_init(full(i), 1);
      mbar_init(empty(i), NCW);
    }
    abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  // The tensor maps are kernel parameters: fetching them does not depend on earlier kernels.
  if (threadIdx.x == 32 * NCW) {
    prefetch_tensormap(&x_map);
    prefetch_tensormap(&dy_map);
  }
  // Everything above touches only shared memory and may overlap the tail of the preceding
  // kernel.  Dependents are released only after the wait, so a chain of such launches never
  // runs ahead of the work that precedes its first kernel.
  // CTA b works on split `si` of chunks cl, cl + chunk_step, ...
  const int si = blockIdx.x % g.n_split;
  const int cl = blockIdx.x / g.n_split;
  const int chunk_step = gridDim.x / g.n_split;
  const int per_chunk = g.n_ig * g.n_ct * g.n_pairs;
  const int s0 = gw8_span_begin(per_chunk, si, g.n_split);
  const int s1 = gw8_span_begin(per_chunk, si + 1, g.n_split);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* abortp = &abort_flag;

  // Stage i of a segment brings the x row pairs PPS*i .. PPS*i+PPS-1 and the dy row pairs
  // PPS*i-E .. PPS*i+PPS-1-E (relative to the segment); pair q = PPS*i+u-E is accumulated
  // in sub-step u if it lies in [0, L).
  auto stages_of = [&](const Gw8Segment& sg) { return (sg.m1 - sg.m0 + E + PPS - 1) / PPS; };
  auto stage_has_pairs = [&](int i) { return PPS * i + PPS - 1 >= E; };

  if (threadIdx.x == 32 * NCW && g.warm > 0 && !g.independent && cl < g.n_chunks) {
    // The load lane asks L2 for the boxes of its first stages while the preceding kernel drains.
    Gw8Walk walk(cl * per_chunk + s0, cl * per_chunk + s1, g);
    Gw8Segment seg;
    int left = g.warm;
    while (left > 0 && walk.next(seg)) {
      const int nst = stages_of(seg);
      for (int i = 0; i < nst && left > 0; ++i, --left) {
        tma_prefetch_4d(&x_map, seg.ck * 64, seg.ct * g.wt - g.pad_w, 2 * (seg.m0 + PPS * i) - g.pad_h,
                        seg.ig * g.nb);
        if (stage_has_pairs(i))
          tma_prefetch_4d(&dy_map, seg.ck * 64, seg.ct * g.wt, 2 * (seg.m0 + PPS * i - E), seg.ig * g.nb);
      }
    }
  }
  if (!g.independent) grid_dependency_wait();
  grid_dependency_launch_dependents();

  if (warp == NCW) {
    // ------------------------------------------------------------ load warp
    if (lane == 0) {
      prefetch_tensormap(&x_map);
      prefetch_tensormap(&dy_map);
      const u64 x_policy = make_l2_policy(g.hint_in);
      const u64 dy_policy = make_l2_policy(g.hint_tiled);
      int slot = 0;
      u32 par = 0;
      bool ok = true;
      for (int ck = cl; ok && ck < g.n_chunks; ck += chunk_step) {
        Gw8Walk walk(ck * per_chunk + s0, ck * per_chunk + s1, g);
        Gw8Segment seg;
        while (ok && walk.next(seg)) {
          const int nst = stages_of(seg);
          const int c0 = seg.ck * 64;
          const int n0 = seg.ig * g.nb;
          for (int i = 0; i < nst; ++i) {
            if (!mbar_wait(empty(slot), par ^ 1u, abortp)) {
              ok = false;
              break;
            }
            const u32 dst = base + (u32)slot * stage_bytes;
            const bool with_dy = stage_has_pairs(i);
            mbar_arrive_expect_tx(full(slot), with_dy ? stage_bytes : xslot_bytes);
            tma_load_4d(dst, &x_map, full(slot), c0, seg.ct * g.wt - g.pad_w,
                        2 * (seg.m0 + PPS * i) - g.pad_h, n0, g.hint_in, x_policy);
            if (with_dy)
              tma_load_4d(dst + xslot_bytes, &dy_map, full(slot), c0, seg.ct * g.wt,
                          2 * (seg.m0 + PPS * i - E), n0, g.hint_tiled, dy_policy);
            if (++slot == ns) {
              slot = 0;
              par ^= 1u;
            }
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------ compute warps
    const int grp = warp & 7;
    const int wsub = warp >> 3;
    const u32 l7 = lane & 7;
    const int gq = lane >> 2;
    const int t4 = lane & 3;

    constexpr int NMAT = 2 * S;
    constexpr int NLD4 = NMAT / 4;
    constexpr bool LD2 = (NMAT % 4) != 0;
    constexpr int NLD = NLD4 + (LD2 ? 1 : 0);
    u32 ld_off[NLD];
#pragma unroll
    for (int q = 0; q < NLD; ++q) {
      int f = 4 * q + (lane >> 3);
      if (LD2 && q == NLD4) f = 4 * q + ((lane >> 3) & 1);
      const u32 rowsel = (u32)(f / S), s = (u32)(f % S);
      ld_off[q] = (rowsel * (u32)g.bw + s + l7) * 128u + (((u32)grp ^ ((s + l7) & 7u)) << 4);
    }
    // dy: matrix 0 = the 8 pixels of the top row, matrix 1 = bottom row
    const u32 dy_off = ((u32)((lane >> 3) & 1) * (u32)g.wt + l7) * 128u + (((u32)grp ^ l7) << 4);

    // Tile t of this warp is tile wsub + WPG * t of the slot.  With one image per slot (NB1,
    // every image wide enough to fill the warps) its offset inside the x rows and the dy rows
    // is the same compile-time multiple of 8 pixels past the warp's first tile, so it costs no
    // registers; with several images per slot the offsets are kept per tile.
    auto compute = [&](auto nb1c) {
    constexpr bool NB1 = decltype(nb1c)::value != 0;
    u32 x_off[TPW], d_off[TPW];
    const u32 t_off0 = (u32)wsub * 1024u;
    int tiles_live = 0;  // tiles of the slot this warp computes; none beyond the last channel
    auto tile_on = [&](int t) { return wsub + WPG * t < tiles_live; };
#pragma unroll
    for (int t = 0; t < TPW; ++t) {
      const int tidx = wsub + WPG * t;
      if (!NB1) {
        const int img = tidx / g.ncb, cb = tidx % g.ncb;
        x_off[t] = (u32)(img * 2 * PPS * g.bw + cb * 8) * 128u;
        d_off[t] = (u32)(img * 2 * PPS * g.wt + cb * 8) * 128u;
      }
    }

    u32 X[TPW][WIN][S];
    float acc[NACC][4];
    int slot = 0;
    u32 par = 0;
    bool ok = true;
    bool full_seen = mbar_test_wait(full(0), 0u);
    // Running addresses of this lane's ldmatrix rows in the current slot (x: A, dy: Dp); they
    // advance by one stage per hand-off and wrap with the ring, which keeps the slot base, the
    // lane offsets and the x / dy split out of the registers that live across the loop.
    u32 A[NLD];
#pragma unroll
    for (int q = 0; q < NLD; ++q) A[q] = base + (NB1 ? t_off0 : 0u) + ld_off[q];
    u32 Dp = base + (NB1 ? t_off0 : 0u) + xslot_bytes + dy_off;

    for (int ck = cl; ok && ck < g.n_chunks; ck += chunk_step) {
      tiles_live = (ck * 64 + grp * 8) < g.c ? g.ntiles : 0;
#pragma unroll
      for (int i = 0; i < NACC; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;

      Gw8Walk walk(ck * per_chunk + s0, ck * per_chunk + s1, g);
      Gw8Segment seg;
      while (ok && walk.next(seg)) {
        const int nst = stages_of(seg);
        const int len = seg.m1 - seg.m0;

        // ALL: every tile of the warp is live; FULL: every sub-step has its dy pair (the interior
        // of an image): the usual case runs without per-tile and per-pair tests.
        auto stage = [&](auto ph0c, auto allc, auto fullc, int i) -> bool {
          constexpr int PH0 = decltype(ph0c)::value;
          constexpr bool ALL = decltype(allc)::value != 0;
          constexpr bool FULL = decltype(fullc)::value != 0;
          if (!full_seen && !mbar_wait(full(slot), par, abortp)) return false;
          {
#pragma unroll
            for (int u = 0; u < PPS; ++u) {
              const int PH = (PH0 + u) % NPH;
              const int q = PPS * i + u - E;
              const bool pair_on = FULL || (q >= 0 && q < len);
#pragma unroll
              for (int t = 0; t < TPW; ++t) {
                if (ALL || tile_on(t)) {
                  // row pair u of tile t: (2 * bw) pixels of 128 bytes per pair
                  const u32 xu = (u32)u * ((u32)g.bw << 8);
                  const u32 ao = NB1 ? (u32)(t * WPG) * 1024u + xu : opaque_add(x_off[t], xu);
#pragma unroll
                  for (int v = 0; v < NLD4; ++v) {
                    const int f0 = 4 * v;
                    ldmatrix_x4<true>(X[t][2 * PH + (f0 + 0) / S][(f0 + 0) % S],
                                      X[t][2 * PH + (f0 + 1) / S][(f0 + 1) % S],
                                      X[t][2 * PH + (f0 + 2) / S][(f0 + 2) % S],
                                      X[t][2 * PH + (f0 + 3) / S][(f0 + 3) % S], A[v] + ao);
                  }
                  if (LD2) {
                    const int f0 = 4 * NLD4;
                    ldmatrix_x2<true>(X[t][2 * PH + (f0 + 0) / S][(f0 + 0) % S],
                                      X[t][2 * PH + (f0 + 1) / S][(f0 + 1) % S],
                                      A[NLD - 1] + ao);
                  }
                  if (pair_on) {
                    u32 d0, d1;
                    const u32 du = (u32)u * ((u32)g.wt << 8);
                    ldmatrix_x2<true>(d0, d1, Dp + (NB1 ? (u32)(t * WPG) * 1024u + du : opaque_add(d_off[t], du)));
#pragma unroll
                    for (int k = 0; k < NACC; ++k) {
                      const int fa = 2 * k, fb = 2 * k + 1;
                      const int ra = fa / S, sa = fa % S;
                      const int pa0 = 2 * ((PH + 1 + ra / 2) % NPH) + (ra & 1);
                      const int pa1 = 2 * ((PH + 1 + (ra + 1) / 2) % NPH) + ((ra + 1) & 1);
                      if (fb < NT) {
                        const int rb = fb / S, sb = fb % S;
                        const int pb0 = 2 * ((PH + 1 + rb / 2) % NPH) + (rb & 1);
                        const int pb1 = 2 * ((PH + 1 + (rb + 1) / 2) % NPH) + ((rb + 1) & 1);
                        mma_m16n8k16(acc[k], X[t][pa0][sa], X[t][pb0][sb], X[t][pa1][sa],
                                     X[t][pb1][sb], d0, d1);
                      } else {
                        mma_m16n8k16(acc[k], X[t][pa0][sa], BIAS ? ONES : 0u, X[t][pa1][sa], BIAS ? ONES : 0u, d0, d1);
                      }
                    }
                  }
                }
              }
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(empty(slot));
#pragma unroll
          for (int q = 0; q < NLD; ++q) A[q] += stage_bytes;
          Dp += stage_bytes;
          if (++slot == ns) {
            slot = 0;
            par ^= 1u;
            const u32 ring = (u32)ns * stage_bytes;
#pragma unroll
            for (int q = 0; q < NLD; ++q) A[q] -= ring;
            Dp -= ring;
          }
          full_seen = mbar_test_wait(full(slot), par);
          return true;
        };

        const bool all_live = wsub + WPG * (TPW - 1) < tiles_live;
        for (int i = 0; ok && i < nst; ++i) {
          const int ph0 = (PPS * i) % NPH;
          auto run = [&](auto allc, auto fullc) -> bool {
            if (ph0 == 0) return stage(IntC<0>{}, allc, fullc, i);
            if (ph0 == 1) return stage(IntC<(NPH > 1 ? 1 : 0)>{}, allc, fullc, i);
            return stage(IntC<(NPH > 2 ? 2 : 0)>{}, allc, fullc, i);
          };
          if (all_live) {
            if (PPS * i >= E && PPS * i + PPS - 1 - E < len)
              ok = run(IntC<1>{}, IntC<1>{});
            else
              ok = run(IntC<1>{}, IntC<0>{});
          } else {
            ok = run(IntC<0>{}, IntC<0>{});
          }
        }
      }

      // Sum the WPG warps of each group inside the CTA, then flush one partial per CTA:
      // acc[i] = {(tap 2i, c=g, k=2t), (.., k=2t+1), (tap 2i+1, c=g, k=2t), (.., k=2t+1)}.
      // The staging for that sum reuses the ring: a CTA that sums in shared memory works on one
      // chunk only, so when it flushes every slot has been consumed and the load warp has
      // nothing left to issue.
      const bool cta_sum = WPG > 1 && !g.warp_parts;
      const int n_parts = cta_sum ? g.n_split : g.n_split * WPG;
      float* red = reinterpret_cast<float*>(smem_raw + (base - smem_u32(smem_raw)));
      if (cta_sum) {
        // every compute warp must have finished reading the ring before it is overwritten
        asm volatile("bar.sync 1, %0;" ::"r"(NCW * 32) : "memory");
        if (wsub > 0) {
          float* dst = red + (size_t)((wsub - 1) * 8 + grp) * (NACC * 4 * 32) + lane;
#pragma unroll
          for (int i = 0; i < NACC; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) dst[(i * 4 + e) * 32] = acc[i][e];
        }
        asm volatile("bar.sync 1, %0;" ::"r"(NCW * 32) : "memory");
        if (wsub == 0) {
#pragma unroll
          for (int w = 1; w < WPG; ++w) {
            const float* src = red + (size_t)((w - 1) * 8 + grp) * (NACC * 4 * 32) + lane;
#pragma unroll
            for (int i = 0; i < NACC; ++i)
#pragma unroll
              for (int e = 0; e < 4; ++e) acc[i][e] += src[(i * 4 + e) * 32];
          }
        }
        asm volatile("bar.sync 1, %0;" ::"r"(NCW * 32) : "memory");  // red may be reused
      }
      if (wsub == 0 || !cta_sum) {
        float* part = scratch + ((size_t)ck * n_parts + (size_t)(cta_sum ? si : si * WPG + wsub)) *
                                    GW8_PART_FLOATS(NT);
        const int kl = grp * 8 + 2 * t4;
#pragma unroll
        for (int i = 0; i < NACC; ++i) {
          const int fa = 2 * i, fb = 2 * i + 1;
          part[((kl + 0) * NT + fa) * 8 + gq] = acc[i][0];
          part[((kl + 1) * NT + fa) * 8 + gq] = acc[i][1];
          if (fb < NT) {
            part[((kl + 0) * NT + fb) * 8 + gq] = acc[i][2];
            part[((kl + 1) * NT + fb) * 8 + gq] = acc[i][3];
          }
        }
        if (BIAS && gq == 0) {  // rows 8-15 of the last accumulator are eight copies of the sum
          part[64 * NT * 8 + kl + 0] = acc[NACC - 1][2];
          part[64 * NT * 8 + kl + 1] = acc[NACC - 1][3];
        }
      }
    }
    };  // compute
    if (g.nb == 1)
      compute(IntC<1>{});
    else
      compute(IntC<0>{});
  }

  __syncthreads();
  // A kernel that did not wait for its predecessors at the start must not COMPLETE before
  // them either: a later kernel that waits for this one relies on that to be ordered after
  // the whole chain.  By now they have long finished, so this returns at once.
  if (g.independent) grid_dependency_wait();
  if (abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(20000);
    if (threadIdx.x == 0) atomicExch(status, (int)GW8_WAIT_TIMEOUT);
  }
}

template <class Cfg, bool WITH_BIAS = false>
__global__ void __launch_bounds__(Cfg::WGRAD_THREADS, 1)
conv2d_gw8_wgrad_kernel(const __grid_constant__ TensorMap x_map,
                        const __grid_constant__ TensorMap dy_map, const Gw8Geom g,
                        float* __restrict__ scratch, int ns, int* __restrict__ status) {
  conv2d_gw8_wgrad_body<Cfg, WITH_BIAS>(x_map, dy_map, g, scratch, ns, status);
}

// dw[k][tap][c] = sum over parts of scratch[chunk(k)][part][k % 64][tap][c] (fp32, or rounded once
// to fp16 when dw_f16 is set: the parameter's own type, which saves autograd's cast), and, when dbias
// is not NULL, dbias[k] = sum over parts of the bias sums behind it, added in a fixed order.
// A block owns 8 float4 columns of a part at a time (n_groups = ceil(n_chunks * GW8_PART_FLOATS(taps)
// / 4 / 8) such groups, walked with a grid stride); thread (cx, q) adds the parts q, q + 4 * WARPS, ...
// of column cx, then the partial sums of a column are combined by two shuffle steps and a pass over
// shared memory.
//
// Launch with 256 threads and one block per group: the fastest reduction, for a weight gradient computed on
// its own (conv2d_gw8_wgrad_reduce_light_kernel is the form the combined backward call uses).
template <int THREADS>
__global__ void __launch_bounds__(THREADS)
conv2d_gw8_wgrad_reduce_kernel(void* __restrict__ dw, float* __restrict__ dbias,
                               const float* __restrict__ scratch, int c, int taps, int n_parts, int dw_f16,
                               int n_groups) {
  constexpr int WARPS = THREADS / 32;
  constexpr int QN = 4 * WARPS;  // threads that share a column
  __shared__ float4 red[WARPS][8];
  // Let an independent successor take SMs as they become free, then wait for the partials.
  grid_dependency_launch_dependents();
  grid_dependency_wait();
  const int cx = threadIdx.x & 7;
  const int pl = (threadIdx.x >> 3) & 3;
  const int wy = threadIdx.x >> 5;
  const int q = wy * 4 + pl;
  const int dw_f4 = 64 * taps * 2;                 // float4 of weight gradient per chunk
  const int chunk_f4 = GW8_PART_FLOATS(taps) / 4;  // float4 per part
  const int n_chunks = (c + 63) / 64;
  for (int grp = blockIdx.x; grp < n_groups; grp += gridDim.x) {
    const int col = grp * 8 + cx;
    const int ck = col / chunk_f4;
    const int e = col - ck * chunk_f4;
    // where the column goes: a float4 of dw, a float4 of dbias, or nowhere (channels >= c)
    // With dw_f16 the weight gradient is stored as fp16 (four values = 8 bytes per column); the
    // bias gradient stays fp32.
    float4* out = nullptr;
    uint2* out_h = nullptr;
    if (ck < n_chunks) {
      if (e < dw_f4) {
        if (ck * 64 + e / (taps * 2) < c) {
          out = reinterpret_cast<float4*>(dw) + (size_t)ck * dw_f4 + e;
          if (dw_f16) out_h = reinterpret_cast<uint2*>(dw) + (size_t)ck * dw_f4 + e;
        }
      } else if (dbias != nullptr && ck * 64 + 4 * (e - dw_f4) < c) {
        out = reinterpret_cast<float4*>(dbias) + ck * 16 + (e - dw_f4);
      }
    }
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
    if (out != nullptr) {
      const float4* src =
          reinterpret_cast<const float4*>(scratch) + (size_t)ck * n_parts * chunk_f4 + e;
#pragma unroll 4
      for (int p = q; p < n_parts; p += QN) {
        const float4 v = __ldcg(src + (size_t)p * chunk_f4);
        sum.x += v.x;
        sum.y += v.y;
        sum.z += v.z;
        sum.w += v.w;
      }
    }
#pragma unroll
    for (int d = 8; d <= 16; d <<= 1) {
      sum.x += __shfl_xor_sync(0xffffffffu, sum.x, d);
      sum.y += __shfl_xor_sync(0xffffffffu, sum.y, d);
      sum.z += __shfl_xor_sync(0xffffffffu, sum.z, d);
      sum.w += __shfl_xor_sync(0xffffffffu, sum.w, d);
    }
    if (pl == 0) red[wy][cx] = sum;
    __syncthreads();
    if (wy == 0 && pl == 0 && out != nullptr) {
#pragma unroll
      for (int w = 1; w < WARPS; ++w) {
        const float4 v = red[w][cx];
        sum.x += v.x;
        sum.y += v.y;
        sum.z += v.z;
        sum.w += v.w;
      }
      if (out_h != nullptr) {
        const __half2 lo = __floats2half2_rn(sum.x, sum.y), hi = __floats2half2_rn(sum.z, sum.w);
        *out_h = make_uint2(*reinterpret_cast<const u32*>(&lo), *reinterpret_cast<const u32*>(&hi));
      } else {
        *out = sum;
      }
    }
    __syncthreads();  // red is reused by the next group
  }
}

// The same reduction in the shape the combined backward call needs.  The blocks of a reduce kernel sit on
// the SMs, waiting, while the weight-gradient kernel runs, and the input-gradient kernel launched behind
// them (which does not wait for the reduction) needs 640 x 96 of an SM's 65,536 registers: a waiting block
// of 256 threads keeps it off that SM until the reduction has finished, one of 128 x 32 registers fits
// beside it.  So: 128 threads, at most 32 registers, at most one block per SM (grid-stride over the groups
// of 8 columns).  Thread (cx, q), q < 16, keeps the two sums that threads q and q + 16 of the wide kernel
// keep, and the 32 sums of a column are added in the wide kernel's order (pairs, pairs of pairs, then the
// eight groups of four one after the other), so both kernels give the same bits.
template <int THREADS = 128>  // a template only so that the header can be included in several translation units
__global__ void __launch_bounds__(THREADS, 2048 / THREADS)
conv2d_gw8_wgrad_reduce_light_kernel(void* __restrict__ dw, float* __restrict__ dbias,
                                     const float* __restrict__ scratch, int c, int taps, int n_parts, int dw_f16,
                                     int n_groups) {
  static_assert(THREADS == 128, "the column / thread split below assumes 128 threads");
  __shared__ float4 red[32][8];
  grid_dependency_launch_dependents();
  grid_dependency_wait();
  const int cx = threadIdx.x & 7;
  const int q = threadIdx.x >> 3;
  const int dw_f4 = 64 * taps * 2;
  const int chunk_f4 = GW8_PART_FLOATS(taps) / 4;
  const int n_chunks = (c + 63) / 64;
  for (int grp = blockIdx.x; grp < n_groups; grp += gridDim.x) {
    const int col = grp * 8 + cx;
    const int ck = col / chunk_f4;
    const int e = col - ck * chunk_f4;
    float4* out = nullptr;
    bool half_out = false;
    if (ck < n_chunks) {
      if (e < dw_f4) {
        if (ck * 64 + e / (taps * 2) < c) {
          out = reinterpret_cast<float4*>(dw) + (size_t)ck * dw_f4 + e;
          half_out = dw_f16 != 0;
        }
      } else if (dbias != nullptr && ck * 64 + 4 * (e - dw_f4) < c) {
        out = reinterpret_cast<float4*>(dbias) + ck * 16 + (e - dw_f4);
      }
    }
    float4 lo = make_float4(0.f, 0.f, 0.f, 0.f), hi = lo;
    if (out != nullptr) {
      const float4* src = reinterpret_cast<const float4*>(scratch) + (size_t)ck * n_parts * chunk_f4 + e;
      for (int p = q; p < n_parts; p += 32) {
        const float4 v = __ldcg(src + (size_t)p * chunk_f4);
        lo.x += v.x, lo.y += v.y, lo.z += v.z, lo.w += v.w;
        if (p + 16 < n_parts) {
          const float4 u = __ldcg(src + (size_t)(p + 16) * chunk_f4);
          hi.x += u.x, hi.y += u.y, hi.z += u.z, hi.w += u.w;
        }
      }
    }
    red[q][cx] = lo;
    red[q + 16][cx] = hi;
    __syncthreads();
    if (q == 0 && out != nullptr) {
      float4 sum;
      for (int w = 0; w < 8; ++w) {
        const float4 a = red[4 * w][cx], b = red[4 * w + 1][cx], cc = red[4 * w + 2][cx], d = red[4 * w + 3][cx];
        const float4 t = make_float4((a.x + b.x) + (cc.x + d.x), (a.y + b.y) + (cc.y + d.y),
                                     (a.z + b.z) + (cc.z + d.z), (a.w + b.w) + (cc.w + d.w));
        if (w == 0)
          sum = t;
        else
          sum.x += t.x, sum.y += t.y, sum.z += t.z, sum.w += t.w;
      }
      if (half_out) {
        const __half2 l2 = __floats2half2_rn(sum.x, sum.y), h2 = __floats2half2_rn(sum.z, sum.w);
        reinterpret_cast<uint2*>(dw)[(size_t)ck * dw_f4 + e] =
            make_uint2(*reinterpret_cast<const u32*>(&l2), *reinterpret_cast<const u32*>(&h2));
      } else {
        *out = sum;
      }
    }
    __syncthreads();  // red is reused by the next group
  }
}

}  // namespace spio_b200
