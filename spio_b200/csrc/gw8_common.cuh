// Shared definitions of the group-width-8 convolution kernels: the launch-time
// geometry, the compile-time tile configuration and the walk of a CTA over its
// share of the work.
//
// Vocabulary (all sizes in output coordinates unless noted):
//   chunk      64 consecutive channels = 8 groups of width 8; one TMA box is 64
//              channels (128 bytes) wide and is stored with the 128-byte swizzle.
//   pair       two consecutive output rows (2m, 2m+1).
//   col tile   Wt = 8*ncb output columns, ncb "column blocks" of 8 pixels.
//   image group NB consecutive images that share one box.
//   slot       one TMA box of the streamed tensor: NB images x 2*PPS rows x BW columns
//              x 64 channels, BW = round_up(Wt + S - 1, 8).  Slot j of a segment
//              holds padded rows 2*PPS*j .. 2*PPS*(j+1)-1 (padded row = input row + pad_h).
//   segment    a run of pairs of one (chunk, image group, col tile) that one CTA
//              streams top to bottom, carrying its register window of input rows.
//
// The tiling arithmetic replaces the reference's per-shape generated index types
// (spio/kernels/conv2d_gw8_kernel.py:62-238, conv2d_gw8_wgrad_kernel.py:92-285).
#pragma once

#include "ptx.cuh"

namespace spio_b200 {

// Opaque 128-byte tensor map; <cuda.h> is not includable under NVRTC.
struct alignas(64) TensorMap {
  unsigned long long opaque[16];
};

// The status word is followed by GW8_DYN_SLOTS claim counters and as many exit counters, all
// zero between launches (the last CTA of a launch clears the pair it used).
enum { GW8_DYN_SLOTS = 64 };

enum Gw8Status {
  GW8_OK = 0,
  GW8_WAIT_TIMEOUT = 1,  // a bounded mbarrier wait gave up
  GW8_PEER_TIMEOUT = 2,  // the data-parallel exchange waited in vain for a peer's contribution
};

// Launch-time geometry.  "in" is the streamed operand with a halo (x for fprop and
// wgrad, dy for dgrad); "out" is the tensor tiled without halo (y, dx; dy for wgrad).
struct Gw8Geom {
  int n, c;            // batch, channels (multiple of 8)
  int in_h, in_w;      // streamed-operand height / width
  int out_h, out_w;    // tiled-operand height / width
  int pad_h, pad_w;    // zero padding of the streamed operand (may be negative)
  int n_chunks;        // ceil(c / 64)
  int n_ig;            // ceil(n / nb)
  int n_ct;            // column tiles
  int n_pairs;         // ceil(out_h / 2)
  int ncb;             // column blocks (of 8 pixels) per column tile
  int nb;              // images per slot
  int wt;              // 8 * ncb
  int bw;              // slot width in pixels, multiple of 8
  int nblk;            // fprop/dgrad: 16-pixel blocks per column tile, ceil(wt / 16)
  int ntiles;          // tiles per slot: nb * nblk (fprop/dgrad) or nb * ncb (wgrad); <= WPG * TPW
  int dgrad;           // 1: weights are used transposed and flipped
  int n_split;         // wgrad: CTAs that share one chunk
  int warp_parts;      // wgrad: 1 = every compute warp writes its own partial (CTAs that walk
                       // several chunks), 0 = the warps of a group are summed inside the CTA
  int independent;     // 1: the caller guarantees that this launch neither reads nor overwrites
                       // anything the preceding kernels of its programmatic-launch chain write or
                       // read, so the kernel does not wait for them
  int dyn_begin;       // forward kernel: first unit of the dynamically claimed pool
  int dyn_chunk;       // pairs per claim; 0 = everything is split statically
  int dyn_slot;        // which pair of counters behind the status word this launch uses
  int hint_in;         // L2 eviction hint (L2_HINT_*) for loads of the streamed operand
  int hint_tiled;      // wgrad: the same for loads of dy
  int prefill;         // stages the load lane issues at kernel start before it waits for the first one to
                       // land (0 = no limit).  With the whole ring requested at once, every CTA's first
                       // slot competes with its later slots (and all other CTAs') for the memory system
                       // and lands after about 3 us; requested with one companion it lands in about half
                       // that, and the compute warps start that much earlier.
  int warm;            // stages whose boxes the load lane asks L2 for BEFORE the kernel waits for its
                       // predecessors (0 = none): the requests overlap the predecessor's tail, warm the
                       // TLB, and the first loads after the wait hit L2.  Measured without it: the first
                       // stage lands 3-4 us after the wait has passed, of which about 1 us is the transfer.
  int chunk_inner;     // fprop/dgrad: order of the flattened work.  0: chunk, image group, column
                       // tile, pair (a CTA stays in one 64-channel chunk); 1: image group, column
                       // tile, chunk, pair (a CTA does all chunks of an image one after the other,
                       // so the 128-byte pieces of a pixel's channels are read and written within a
                       // short time of each other)
  int pair_images;     // fprop/dgrad, images at most 8 pixels wide: the two 8-pixel halves of a
                       // 16-pixel block tile are pixels 0-7 of two consecutive images of the slot
                       // (wt = 8, nb even, ntiles = nb / 2)
  // byte sizes derived from the above (kept here so that the kernels read them from the
  // constant bank instead of holding them in registers); pps = row pairs per slot
  unsigned in_pair_bytes;    // 2 rows of one image of the streamed operand: 2*bw*128
  unsigned out_pair_bytes;   // 2 rows of nb images of the tiled operand:   nb*2*wt*128
  unsigned slot_bytes;       // nb * pps * in_pair_bytes
  unsigned obuf_bytes;       // pps * out_pair_bytes (fwd staging buffer / dy part of a wgrad slot)
  unsigned img_in_bytes;     // one image inside a slot:        2*pps*bw*128
  unsigned img_out_bytes;    // one image inside a staging pair: 2*wt*128
};

// What the load warp tells the compute warps about the slot it has just filled.
struct alignas(16) Gw8StageDesc {
  int ck;     // chunk the slot belongs to
  int mask;   // bit u set: sub-step u completes an output pair
  int ph0;    // window phase of sub-step 0: (PPS * stage index) mod (WIN / 2)
  int flags;  // GW8_STAGE_END: no more work, the slot holds no data
};
enum { GW8_STAGE_END = 1 };

// Compile-time tile configuration.
//   R, S   filter size;  WPG warps per group;  TPW tiles (8 px x 2 rows) per warp;
//   PPS    row pairs per ring slot (one barrier hand-off per 2*PPS rows).
// The number of ring slots and of output staging buffers is a launch argument.
template <int R_, int S_, int WPG_, int TPW_, int PPS_ = 1>
struct Gw8Config {
  static constexpr int R = R_, S = S_, WPG = WPG_, TPW = TPW_, PPS = PPS_;
  static constexpr int E = R / 2;          // extra slots a pair needs below its own
  static constexpr int WIN = 2 * E + 2;    // rows of the register window
  static constexpr int NT = R * S;         // taps
  static constexpr int NCW = 8 * WPG;      // consumer warps
  // Forward kernel: the consumer warps plus one warpgroup (4 warps) of producers: load warp,
  // store warp and two idle warps.  The padding makes the producers a warpgroup of their own,
  // so they can hand most of their registers to the consumers (setmaxnreg): the CTA is launched
  // with FWD_REGS_LAUNCH registers per thread (what ptxas allocates under the launch bound when
  // the kernel contains setmaxnreg), the producers drop to FWD_REGS_PRODUCER and the consumers
  // rise to FWD_REGS_CONSUMER.  The rise must fit what the drop frees,
  //   NCW*32 * (CONSUMER - LAUNCH) <= 128 * (LAUNCH - PRODUCER),
  // or the consumers would wait for registers for ever; the library checks the allocated count
  // of every loaded kernel against this before it launches it.
  static constexpr int THREADS = (NCW + 4) * 32;
  static constexpr bool FWD_SETMAXNREG = WPG >= 2;  // one warp per group has registers to spare
  static constexpr int FWD_REGS_LAUNCH = WPG == 2 ? 96 : 72;
  static constexpr int FWD_REGS_PRODUCER = 24;
  static constexpr int FWD_REGS_CONSUMER = WPG == 2 ? 112 : 80;
  static_assert(!FWD_SETMAXNREG ||
                    NCW * 32 * (FWD_REGS_CONSUMER - FWD_REGS_LAUNCH) <= 128 * (FWD_REGS_LAUNCH - FWD_REGS_PRODUCER),
                "the consumers' extra registers must fit what the producers give up");
  static constexpr int MAX_TILES = WPG * TPW;
  static constexpr int WGRAD_THREADS = (NCW + 1) * 32;  // no store warp
};

// Carries a compile-time integer into a generic lambda.
template <int V>
struct IntC {
  static constexpr int value = V;
};

// One segment of a CTA's span.
struct Gw8Segment {
  int ck, ig, ct;  // chunk, image group, column tile
  int m0, m1;      // pairs [m0, m1)
};

// Walks the span [u0, u1) of the flattened (chunk, image group, col tile, pair)
// sequence and cuts it into segments.  Every role of a CTA (load, compute, store)
// runs the same walk, so they agree on the order of slots without communicating.
struct Gw8Walk {
  int u, u1, n_pairs, n_ct, n_ig, n_chunks_inner;

  __device__ __forceinline__ Gw8Walk(int u0_, int u1_, const Gw8Geom& g)
      : u(u0_), u1(u1_), n_pairs(g.n_pairs), n_ct(g.n_ct), n_ig(g.n_ig),
        n_chunks_inner(g.chunk_inner ? g.n_chunks : 0) {}

  __device__ __forceinline__ bool next(Gw8Segment& s) {
    if (u >= u1) return false;
    int m = u % n_pairs;
    int rest = u / n_pairs;
    if (n_chunks_inner > 0) {
      s.ck = rest % n_chunks_inner;
      rest /= n_chunks_inner;
      s.ct = rest % n_ct;
      s.ig = rest / n_ct;
    } else {
      s.ct = rest % n_ct;
      rest /= n_ct;
      s.ig = rest % n_ig;
      s.ck = rest / n_ig;
    }
    s.m0 = m;
    int len = n_pairs - m;
    if (len > u1 - u) len = u1 - u;
    s.m1 = m + len;
    u += len;
    return true;
  }
};

// Span of CTA `b` out of `nb` over `total` units, balanced to within one unit.
__device__ __forceinline__ int gw8_span_begin(int total, int b, int nb) {
  return (int)(((long long)total * b) / nb);
}

// Byte offset inside a swizzled slot of the 16-byte piece holding channels
// [8*grp, 8*grp+8) of pixel `pix`; the slot base must be 1024-byte aligned.
__device__ __forceinline__ u32 gw8_swizzle(u32 pix, u32 grp) {
  return pix * 128u + ((grp ^ (pix & 7u)) << 4);
}

}  // namespace spio_b200
