// Forward / input-gradient kernel of the group-width-8 convolution on the 5th-generation
// tensor cores: tcgen05.mma with both operands in shared memory and the accumulators in
// tensor memory.
//
//   y[n][p][q][k] = bias[k] + sum_{r,s,c} x[n][p+r-pad][q+s-pad][8*(k/8)+c] * w[k][r][s][c]
//
// Same streaming skeleton as conv2d_gw8_fwd.cuh (persistent CTA per SM, TMA ring with
// out-of-range zero fill as padding, staged TMA stores), but no input byte passes through
// a register:
//
//  * a ring slot is one row pair of one image: 2 rows x 64 pixels x 64 channels, each pixel
//    one 128-byte row of a K-major, 128-byte-swizzled operand tile;
//  * an output row pair is ONE accumulator tile of 128 pixels (fp32, in tensor memory).  A
//    tcgen05.mma of this shape takes about 75 cycles whatever its N (measured for N = 16..128),
//    and K is fixed at 16, so the instruction count decides: shifting the A operand for each
//    of the R*S taps would cost R*S*4 instructions per tile, twice the time the HBM stream
//    leaves.  Only the VERTICAL taps shift A (a shared-memory descriptor that points into the
//    ring at input row r of the window; nothing is copied).  The S horizontal taps of a row
//    are computed side by side in N from the same unshifted A,
//        D[p][s][k] = sum_r sum_c x[row + r][p][c] * w[k][r][s][c],
//    and the shift moves to the output side, y[p][k] = sum_s D[p + s][s][k], which the
//    epilogue does with warp shuffles: R*4 instructions of shape M128 N(16*S) K16 per tile;
//  * the group structure is block-diagonal weights: channels 16j..16j+15 (two groups) multiply
//    B_{r,j}[S*16 (s, out)][16 in], two 8x8 blocks on the diagonal per s, into columns
//    j*16*S .. of D; the instructions are issued by one thread;
//  * the window of R+1 input rows spans two ring slots; where the ring wraps, the first row
//    of slot 0 is loaded a second time behind the last slot so that the 128 rows of every
//    tap stay contiguous;
//  * sixteen epilogue warps read the accumulator (one pixel and 16 channels per thread), add the S shifted
//    partial sums (the two pixels past a warp's 32 lanes come from the next warp through
//    shared memory), add the bias, round to fp16 and write swizzled 128-byte pixel rows
//    into a staging buffer for the TMA store.
//
// Restrictions (the launch planner falls back to the mma.sync kernel otherwise): R, S <= 3,
// column tile + S - 1 <= 64 pixels, one image per slot.
//
// Replaces the reference's spio/src/conv2d_gw8.cu:10-224 (fprop, and dgrad = Mode::igrad).
#pragma once

#include <cuda_fp16.h>

#include "gw8_common.cuh"

namespace spio_b200 {


enum { TC_END = 1, TC_HAS_OUT = 2, TC_SEG_LAST = 4 };

// What the load warp tells the MMA warp about a slot, and what travels on with the
// accumulator and the staging buffer.
struct alignas(16) Gw8TcDesc {
  int ck;     // chunk
  int flags;  // TC_*
  int row;    // first output row of the pair this stage completes
  int n0;     // image
  int w0;     // first output column of the column tile
  int pad0, pad1, pad2;
};

template <int R_, int S_>
struct Gw8TcConfig {
  static constexpr int R = R_, S = S_, NT = R_ * S_;
  static constexpr int E = R_ / 2;          // stages of lead-in per segment
  static constexpr int THREADS = 640;       // load, mma, weights, store, 16 x epilogue
  static constexpr int ACC_COLS = 64 * S_;                 // columns of one accumulator tile
  static constexpr int NACC = S_ == 3 ? 2 : 4;             // accumulator tiles in tensor memory
  static constexpr int TMEM_COLS = S_ == 1 ? 256 : 512;    // power of two >= NACC * ACC_COLS
  static constexpr int SLOT_BYTES = 2 * 64 * 128;
  static constexpr int ROW_BYTES = 64 * 128;
  static constexpr int B_BYTES = NT * 2048;  // per chunk: NT taps x 16 rows x 128 bytes
  static_assert(R_ >= 1 && R_ <= 3 && S_ >= 1 && S_ <= 3, "filter size");
};

template <class Cfg>
__device__ __forceinline__ void
conv2d_gw8_fwd_tc_body(const TensorMap& in_map, const TensorMap& row_map, const TensorMap& out_map,
                       const Gw8Geom& g, const __half* __restrict__ wgt, const float* __restrict__ bias,
                       int ns, int nob, int* __restrict__ status) {
  constexpr int R = Cfg::R, S = Cfg::S, NT = Cfg::NT, E = Cfg::E, NACC = Cfg::NACC;
  constexpr u32 SLOT = Cfg::SLOT_BYTES, ROW = Cfg::ROW_BYTES, BB = Cfg::B_BYTES;
  constexpr int MAX_NS = 12, MAX_NOB = 4;

  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) u64 bars[2 * MAX_NS + 2 * NACC + 4 + 2 * MAX_NOB + 32];
  // what lanes 30 and 31 of an even quarter need from the odd quarter after it:
  // [warp pair][tile parity][0: X30, 1: X31][channel]
  __shared__ float xch[2][2][2][64];
  __shared__ Gw8TcDesc desc[MAX_NS];
  __shared__ Gw8TcDesc tdesc[NACC];
  __shared__ Gw8TcDesc odesc[MAX_NOB];
  __shared__ int abort_flag;
  __shared__ u32 tmem_holder;

  const u32 ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* const smem = smem_raw + (ring - smem_u32(smem_raw));  // generic pointer to `ring`
  const u32 mirror = ring + (u32)ns * SLOT;
  const u32 bbuf = mirror + ROW;
  const u32 obufs = bbuf + 2u * BB;
  const u32 bar0 = smem_u32(bars);
  auto full = [&](int i) { return bar0 + 8u * (u32)i; };
  auto empty = [&](int i) { return bar0 + 8u * (u32)(MAX_NS + i); };
  auto acc_full = [&](int i) { return bar0 + 8u * (u32)(2 * MAX_NS + i); };
  auto acc_empty = [&](int i) { return bar0 + 8u * (u32)(2 * MAX_NS + NACC + i); };
  auto b_full = [&](int i) { return bar0 + 8u * (u32)(2 * MAX_NS + 2 * NACC + i); };
  auto b_empty = [&](int i) { return bar0 + 8u * (u32)(2 * MAX_NS + 2 * NACC + 2 + i); };
  auto ofull = [&](int i) { return bar0 + 8u * (u32)(2 * MAX_NS + 2 * NACC + 4 + i); };
  auto oempty = [&](int i) { return bar0 + 8u * (u32)(2 * MAX_NS + 2 * NACC + 4 + MAX_NOB + i); };
  auto xfull = [&](int pair, int cq, int par) {
    return bar0 + 8u * (u32)(2 * MAX_NS + 2 * NACC + 4 + 2 * MAX_NOB + 8 * pair + 2 * cq + par);
  };
  auto xempty = [&](int pair, int cq, int par) {
    return bar0 + 8u * (u32)(2 * MAX_NS + 2 * NACC + 20 + 2 * MAX_NOB + 8 * pair + 2 * cq + par);
  };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < ns; ++i) {
      mbar_init(full(i), 1);
      mbar_init(empty(i), 1);  // one tcgen05.commit
    }
    for (int i = 0; i < NACC; ++i) {
      mbar_init(acc_full(i), 2);   // the issuing thread (descriptor written) + tcgen05.commit
      mbar_init(acc_empty(i), 16);  // the sixteen epilogue warps
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(b_full(i), 1);
      mbar_init(b_empty(i), 1);
    }
    for (int i = 0; i < nob; ++i) {
      mbar_init(ofull(i), 16);
      mbar_init(oempty(i), 1);
    }
    for (int i = 0; i < 16; ++i) {
      mbar_init(xfull(i >> 3, (i >> 1) & 3, i & 1), 1);
      mbar_init(xempty(i >> 3, (i >> 1) & 3, i & 1), 1);
    }
    abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(smem_u32(&tmem_holder), Cfg::TMEM_COLS);
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const u32 tmem = tmem_holder;
  // Everything above touches only shared and tensor memory and may overlap the tail of the
  // preceding kernel; dependents are released only after the wait.
  if (!g.independent) grid_dependency_wait();
  grid_dependency_launch_dependents();

  volatile int* abortp = &abort_flag;
  const int total = g.n_chunks * g.n_ig * g.n_ct * g.n_pairs;
  const int u0 = gw8_span_begin(total, blockIdx.x, gridDim.x);
  const int u1 = gw8_span_begin(total, blockIdx.x + 1, gridDim.x);

  if (warp == 0) {
    // ------------------------------------------------------------ load warp
    if (lane == 0) {
      prefetch_tensormap(&in_map);
      prefetch_tensormap(&row_map);
      const u64 policy = make_l2_policy(g.hint_in);
      Gw8Walk walk(u0, u1, g);
      Gw8Segment seg;
      int slot = 0;
      u32 par = 0;
      bool ok = true;
      while (ok && walk.next(seg)) {
        const int len = seg.m1 - seg.m0;
        const int nst = len + E;
        const int c0 = seg.ck * 64;
        const int w0 = seg.ct * g.wt;
        for (int i = 0; i < nst; ++i) {
          if (!mbar_wait(empty(slot), par ^ 1u, abortp)) {
            ok = false;
            break;
          }
          Gw8TcDesc d;
          d.ck = seg.ck;
          d.flags = ((i >= E) ? TC_HAS_OUT : 0) | ((i == nst - 1) ? TC_SEG_LAST : 0);
          d.row = 2 * (seg.m0 + i - E);
          d.n0 = seg.ig;
          d.w0 = w0;
          d.pad0 = d.pad1 = d.pad2 = 0;
          desc[slot] = d;
          // the row pair that follows the last slot of the ring is slot 0: its first row is
          // loaded twice, the copy continues the last slot
          const bool wrap = E > 0 && slot == 0 && i > 0;
          const int row0 = 2 * (seg.m0 + i) - g.pad_h;
          mbar_arrive_expect_tx(full(slot), wrap ? SLOT + ROW : SLOT);
          tma_load_4d(ring + (u32)slot * SLOT, &in_map, full(slot), c0, w0 - g.pad_w, row0, seg.ig,
                      g.hint_in, policy);
          if (wrap) tma_load_4d(mirror, &row_map, full(slot), c0, w0 - g.pad_w, row0, seg.ig, g.hint_in, policy);
          if (++slot == ns) {
            slot = 0;
            par ^= 1u;
          }
        }
      }
      if (ok && mbar_wait(empty(slot), par ^ 1u, abortp)) {
        desc[slot].flags = TC_END;
        mbar_arrive(full(slot));
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA warp (one thread issues)
    if (lane == 0) {
      constexpr u32 IDESC = umma_idesc_f16_f32(128, 16 * S);
      int slot = 0, prev = 0, ab = 0, bq = -1, cur_ck = -1;
      u32 par = 0, apar = 0;
      for (;;) {
        if (!mbar_wait(full(slot), par, abortp)) break;
        const Gw8TcDesc d = desc[slot];
        if (d.flags & TC_END) {
          // pass the end mark to the epilogue warps through the next accumulator slot
          if (mbar_wait(acc_empty(ab), apar ^ 1u, abortp)) {
            tdesc[ab].flags = TC_END;
            mbar_arrive(acc_full(ab));
            mbar_arrive(acc_full(ab));
          }
          break;
        }
        if (d.ck != cur_ck) {
          if (cur_ck >= 0) tcgen05_commit(b_empty(bq & 1));  // the old weights are free once their MMAs are done
          ++bq;
          if (!mbar_wait(b_full(bq & 1), (u32)(bq >> 1) & 1u, abortp)) break;
          cur_ck = d.ck;
        }
        if (d.flags & TC_HAS_OUT) {
          if (!mbar_wait(acc_empty(ab), apar ^ 1u, abortp)) break;
          tcgen05_fence_after_sync();
          const u32 d_tmem = tmem + (u32)ab * (u32)Cfg::ACC_COLS;
          const u32 bb = bbuf + (u32)(bq & 1) * BB;
          const u32 a_prev = ring + (u32)prev * SLOT, a_cur = ring + (u32)slot * SLOT;
#pragma unroll
          for (int r = 0; r < R; ++r) {
            // window row r: rows 0, 1 are the previous slot, rows 2, 3 this slot (E = 1);
            // without lead-in (R = 1) the window is this slot
            const u32 a_row = E == 0 ? a_cur : (r < 2 ? a_prev + (u32)r * ROW : a_cur + (u32)(r - 2) * ROW);
#pragma unroll
            for (int j = 0; j < 4; ++j)  // channels 16j..16j+15 -> columns j*16*S.. (all S horizontal taps)
              umma_f16_ss(d_tmem + (u32)(16 * S * j), umma_desc_k_sw128(a_row + 32u * (u32)j),
                          umma_desc_k_sw128(bb + (u32)(r * S) * 2048u + 32u * (u32)j), IDESC, r != 0 ? 1u : 0u);
          }
          tdesc[ab] = d;
          mbar_arrive(acc_full(ab));     // orders the descriptor before the epilogue's read
          tcgen05_commit(acc_full(ab));  // arrives when the MMAs above have completed
          if (E > 0) tcgen05_commit(empty(prev));
          if (E == 0 || (d.flags & TC_SEG_LAST)) tcgen05_commit(empty(slot));
          if (++ab == NACC) {
            ab = 0;
            apar ^= 1u;
          }
        }
        prev = slot;
        if (++slot == ns) {
          slot = 0;
          par ^= 1u;
        }
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------ weights warp
    // Builds the block-diagonal B tiles of each chunk this CTA visits, double-buffered.
    // Tile of tap t: 16 rows (n = output channel within a 16-channel block) x 128 bytes; the
    // 32 bytes of k-step j hold the block of channels 16j..16j+15: the 16-byte half that
    // matches the row's group carries the 8 weights, the other half is zero.
    Gw8Walk walk(u0, u1, g);
    Gw8Segment seg;
    int bq = -1, cur_ck = -1;
    bool ok = true;
    while (ok && walk.next(seg)) {
      if (seg.ck == cur_ck) continue;
      cur_ck = seg.ck;
      ++bq;
      if (!mbar_wait(b_empty(bq & 1), ((u32)(bq >> 1) & 1u) ^ 1u, abortp)) break;
      unsigned char* const bdst = smem + (bbuf - ring) + (u32)(bq & 1) * BB;
      for (int e = lane; e < NT * 16 * 4; e += 32) {
        const int j = e & 3, n = (e >> 2) & 15, t = e >> 6;
        const int grp_half = n >> 3;                  // which of the two groups of the block
        const int ch = cur_ck * 64 + 16 * j + n;      // fprop: output channel; dgrad: input channel
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (ch < g.c) {
          if (!g.dgrad) {
            v = *reinterpret_cast<const uint4*>(wgt + ((size_t)ch * NT + t) * 8);
          } else {
            // B[n = in-channel][k = out-channel of the same group] = w[out][flipped tap][in % 8]
            const int out0 = cur_ck * 64 + 16 * j + 8 * grp_half;
            __half h[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) h[k] = wgt[((size_t)(out0 + k) * NT + (NT - 1 - t)) * 8 + (n & 7)];
            v = *reinterpret_cast<const uint4*>(h);
          }
        }
        unsigned char* const row = bdst + t * 2048 + n * 128;
        const u32 c_on = (u32)(2 * j + grp_half), c_off = (u32)(2 * j + 1 - grp_half);
        *reinterpret_cast<uint4*>(row + ((c_on ^ (u32)(n & 7)) << 4)) = v;
        *reinterpret_cast<uint4*>(row + ((c_off ^ (u32)(n & 7)) << 4)) = make_uint4(0u, 0u, 0u, 0u);
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(b_full(bq & 1));
    }
  } else if (warp == 3) {
    // ------------------------------------------------------------ store warp
    if (lane < nob) {
      prefetch_tensormap(&out_map);
      u32 opar = 0;
      for (;;) {
        if (!mbar_wait(ofull(lane), opar, abortp)) break;
        const Gw8TcDesc d = odesc[lane];
        if (d.flags & TC_END) break;
        tma_store_4d(&out_map, obufs + (u32)lane * g.obuf_bytes, d.ck * 64, d.w0, d.row, d.n0);
        tma_store_commit();
        tma_store_wait_read0();
        mbar_arrive(oempty(lane));
        opar ^= 1u;
      }
      tma_store_wait_all();
    }
  } else {
    // ------------------------------------------------------------ epilogue warps
    // Sixteen warps: warp (quarter q = warp % 4, channel block cq) owns pixels 32q..32q+31 of
    // the tile (thread = pixel p = 32q + lane: row p / 64, column p % 64) and channels
    // 16cq..16cq+15.  y[p] = sum_s D[p + s][s]: the partial sums of the next one or two pixels
    // come from the neighbouring lanes by shuffle.  Lanes 30, 31 of an even quarter lack
    // pixels 32, 33, which belong to the odd quarter that follows; that warp leaves
    // X30 = D[32][2] and X31 = D[32][1] + D[33][2] in shared memory for them.  (The last lanes
    // of an odd quarter are columns 62, 63 of the 64-pixel row, which are never stored.)
    const int quarter = warp & 3, pair = quarter >> 1, cq = (warp - 4) >> 2;
    const bool odd = (quarter & 1) != 0;
    const int p = 32 * quarter + lane;
    const int row = p >> 6, col = p & 63;
    int ab = 0, ob = 0, tile = 0;
    u32 apar = 0, opar = 0;
    for (;;) {
      if (!mbar_wait(acc_full(ab), apar, abortp)) break;
      const Gw8TcDesc d = tdesc[ab];
      if (d.flags & TC_END) {
        // pass the end mark to every store lane
        for (int i = 0; i < nob; ++i) {
          if (!mbar_wait(oempty(ob), opar ^ 1u, abortp)) break;
          if (warp == 4 && lane == 0) odesc[ob].flags = TC_END;
          __syncwarp();
          if (lane == 0) mbar_arrive(ofull(ob));
          if (++ob == nob) {
            ob = 0;
            opar ^= 1u;
          }
        }
        break;
      }
      tcgen05_fence_after_sync();
      const u32 t_base = tmem + ((u32)(32 * quarter) << 16) + (u32)ab * (u32)Cfg::ACC_COLS + (u32)(16 * S * cq);
      const int xp = tile & 1;                     // exchange buffer of this tile
      const u32 xpar = (u32)(tile >> 1) & 1u;      // parity of this use of the buffer
      u32 v[S][16];  // partial sums of this thread's pixel: v[s][k], channel 16cq + k
#pragma unroll
      for (int s = 0; s < S; ++s) tmem_ld_32x16(v[s], t_base + (u32)(16 * s));
      tmem_ld_wait();
      tcgen05_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty(ab));  // the accumulator tile is free again
      if (S > 1 && odd) {
        if (!mbar_wait(xempty(pair, cq, xp), xpar ^ 1u, abortp)) break;
#pragma unroll
        for (int k = 0; k < 16; ++k) {
          float x31 = __uint_as_float(v[1][k]);
          if (S > 2) x31 += __shfl_down_sync(0xffffffffu, __uint_as_float(v[S > 2 ? 2 : 0][k]), 1);
          if (lane == 0) {
            xch[pair][xp][1][16 * cq + k] = x31;
            if (S > 2) xch[pair][xp][0][16 * cq + k] = __uint_as_float(v[S > 2 ? 2 : 0][k]);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(xfull(pair, cq, xp));
      }
      float f[16];
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        f[k] = __uint_as_float(v[0][k]);
        if (S > 1) shfl_down_add(f[k], __uint_as_float(v[S > 1 ? 1 : 0][k]), 1);
        if (S > 2) shfl_down_add(f[k], __uint_as_float(v[S > 2 ? 2 : 0][k]), 2);
      }
      if (S > 1 && !odd) {
        if (!mbar_wait(xfull(pair, cq, xp), xpar, abortp)) break;
        if (lane >= (S > 2 ? 30 : 31)) {
#pragma unroll
          for (int k = 0; k < 16; ++k) f[k] += xch[pair][xp][lane - 30][16 * cq + k];
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(xempty(pair, cq, xp));
      }
      if (!mbar_wait(oempty(ob), opar ^ 1u, abortp)) break;
      if (col < g.wt) {
        unsigned char* const dst = smem + (obufs - ring) + (u32)ob * g.obuf_bytes + (u32)(row * g.wt + col) * 128u;
        const float* const bp = bias != nullptr ? bias + d.ck * 64 : nullptr;
#pragma unroll
        for (int h = 0; h < 2; ++h) {  // 16-byte piece c = 2cq + h: channels 8c..8c+7 of the chunk
          const int c = 2 * cq + h;
          float* const e = f + 8 * h;
          if (bp != nullptr && d.ck * 64 + 8 * c < g.c) {
            const float4 b0 = __ldg(reinterpret_cast<const float4*>(bp + 8 * c));
            const float4 b1 = __ldg(reinterpret_cast<const float4*>(bp + 8 * c + 4));
            e[0] += b0.x, e[1] += b0.y, e[2] += b0.z, e[3] += b0.w;
            e[4] += b1.x, e[5] += b1.y, e[6] += b1.z, e[7] += b1.w;
          }
          const __half2 h0 = __floats2half2_rn(e[0], e[1]), h1 = __floats2half2_rn(e[2], e[3]);
          const __half2 h2 = __floats2half2_rn(e[4], e[5]), h3 = __floats2half2_rn(e[6], e[7]);
          uint4 o;
          o.x = *reinterpret_cast<const u32*>(&h0);
          o.y = *reinterpret_cast<const u32*>(&h1);
          o.z = *reinterpret_cast<const u32*>(&h2);
          o.w = *reinterpret_cast<const u32*>(&h3);
          *reinterpret_cast<uint4*>(dst + (((u32)c ^ (u32)(col & 7)) << 4)) = o;
        }
      }
      fence_proxy_async_smem();
      if (warp == 4 && lane == 0) odesc[ob] = d;
      __syncwarp();
      if (lane == 0) mbar_arrive(ofull(ob));
      if (++ob == nob) {
        ob = 0;
        opar ^= 1u;
      }
      if (++ab == NACC) {
        ab = 0;
        apar ^= 1u;
      }
      ++tile;
    }
  }

  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, Cfg::TMEM_COLS);
  if (g.independent) grid_dependency_wait();
  if (abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(20000);
    if (threadIdx.x == 0) atomicExch(status, (int)GW8_WAIT_TIMEOUT);
  }
}

template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, 1)
conv2d_gw8_fwd_tc_kernel(const __grid_constant__ TensorMap in_map, const __grid_constant__ TensorMap row_map,
                         const __grid_constant__ TensorMap out_map, const Gw8Geom g,
                         const __half* __restrict__ wgt, const float* __restrict__ bias, int ns, int nob,
                         int* __restrict__ status) {
  conv2d_gw8_fwd_tc_body<Cfg>(in_map, row_map, out_map, g, wgt, bias, ns, nob, status);
}

}  // namespace spio_b200
