// C ABI of libspio_b200 (declared in include/spio_b200.h): planning and launch of the
// gw8 forward / input-gradient / weight-gradient kernels.
//
// Host-side counterpart of the reference's launch path
//   spio/kernels/kernel.py:135-154 (Kernel.launch) -> spio/cuda/driver.pyx:171-208
// with the per-shape kernel specification (spio/kernels/conv2d_gw8_kernel.py:62-238,
// conv2d_gw8_wgrad_kernel.py:92-285) replaced by a launch-time plan.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <atomic>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/spio_b200.h"
#include "conv2d_gw8_wgrad.cuh"
#include "gw8_host.h"

namespace spio_b200 {

namespace {

thread_local std::string g_last_error;

int fail(const std::string& msg) {
  g_last_error = msg;
  return 1;
}

}  // namespace
int jit_fail(const std::string& msg) { return fail(msg); }  // used by jit_driver.cpp
namespace {

}  // namespace
bool gw8_pdl_enabled();
namespace {

int fail_cuda(const char* what, cudaError_t e) {
  return fail(std::string("CUDA error: ") + cudaGetErrorString(e) + " (" + what + ")");
}

#define GW8_CUDA(call)                                   \
  do {                                                   \
    cudaError_t e_ = (call);                             \
    if (e_ != cudaSuccess) return fail_cuda(#call, e_);  \
  } while (0)

// Status word the kernels write when a bounded wait gives up; one per device because
// the symbol is instantiated in every context that loads the library.
__device__ int g_status_word[1 + 2 * GW8_DYN_SLOTS];  // status, claim counters, exit counters

constexpr int kMaxDevices = 64;

// Scratch of the entry point that allocates nothing.  It is part of the library image, so
// every GPU that loads the library sets this much memory aside until the process exits.
constexpr size_t kStaticScratchBytes = 4u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
unsigned char* g_static_scratch_addr[kMaxDevices] = {};  // device address, per device
constexpr int kFwdStaticSmem = 1024;   // >= static shared memory of the kernels
constexpr int kTcStaticSmem = 6144;    // >= static shared memory of the tcgen05 kernel
constexpr int kAlignSlack = 1024;      // dynamic shared memory is re-aligned to 1 KiB

struct DeviceInfo {
  bool ready = false;
  int dev = 0;
  int sms = 0;
  int smem_optin = 0;
  int* status = nullptr;
};

std::mutex g_mutex;
DeviceInfo g_devices[kMaxDevices];
std::vector<Gw8Variant> g_variants;

// Counter pairs of the forward kernel's dynamic tail are owned per stream.  Kernels of one
// stream that use the counters never overlap in their use of them: a launch touches them only
// after it has waited for its predecessors (or, for the input-gradient kernel of the combined
// backward call, after kernels that do not use them), and the last CTA clears them before the
// grid completes.  Kernels of different streams may run at the same time, so they get different
// pairs; a device that has used all pairs launches statically on further streams.
struct SlotTable {
  cudaStream_t streams[GW8_DYN_SLOTS];
  int used = 0;
};
SlotTable g_slots[kMaxDevices];

int slot_of_stream(int dev, cudaStream_t stream) {
  std::lock_guard<std::mutex> lock(g_mutex);
  SlotTable& t = g_slots[dev];
  for (int i = 0; i < t.used; ++i)
    if (t.streams[i] == stream) return i;
  if (t.used == GW8_DYN_SLOTS) return -1;
  t.streams[t.used] = stream;
  return t.used++;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

void load_variants_locked() {
  if (!g_variants.empty()) return;
  const Gw8Variant* v = nullptr;
  int n;
  n = gw8_variants_r1(&v);
  g_variants.insert(g_variants.end(), v, v + n);
  n = gw8_variants_r2(&v);
  g_variants.insert(g_variants.end(), v, v + n);
  n = gw8_variants_r3(&v);
  g_variants.insert(g_variants.end(), v, v + n);
  n = gw8_variants_r4(&v);
  g_variants.insert(g_variants.end(), v, v + n);
  n = gw8_variants_r5(&v);
  g_variants.insert(g_variants.end(), v, v + n);
}

// Per-device set-up: limits, the status word's device address, the driver entry point
// for tensor-map encoding and the opt-in shared-memory size of every kernel.
int device_info(const DeviceInfo** out) {
  int dev = 0;
  GW8_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail("device ordinal out of range");
  // Tensor maps are encoded through the driver API, which needs the device's primary
  // context current on the calling thread; a thread that has only inherited the runtime's
  // device choice (an autograd worker, say) may not have it bound yet.
  GW8_CUDA(cudaSetDevice(dev));
  std::lock_guard<std::mutex> lock(g_mutex);
  load_variants_locked();
  DeviceInfo& d = g_devices[dev];
  if (!d.ready) {
    GW8_CUDA(cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev));
    GW8_CUDA(cudaDeviceGetAttribute(&d.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    int major = 0;
    GW8_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    if (major != 10)
      return fail("unsupported device: libspio_b200 is built for sm_100a only");
    GW8_CUDA(cudaGetSymbolAddress((void**)&d.status, g_status_word));
    GW8_CUDA(cudaMemset(d.status, 0, sizeof(g_status_word)));
    if (g_encode == nullptr) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult qres;
      GW8_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
      if (fn == nullptr || qres != cudaDriverEntryPointSuccess)
        return fail("cuTensorMapEncodeTiled is not available from this driver");
      g_encode = (EncodeTiledFn)fn;
    }
    for (int r = 1; r <= 3; ++r)
      for (int sft = 1; sft <= 3; ++sft)
        GW8_CUDA(cudaFuncSetAttribute(gw8_tc_kernel(r, sft), cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      d.smem_optin - kTcStaticSmem));
    for (const Gw8Variant& v : g_variants) {
      // Forward kernels that move registers from the producer warpgroup to the consumers
      // (setmaxnreg) must have been allocated the count the move was sized for; otherwise the
      // consumers could wait for registers that never become free.
      if (v.wpg >= 2) {
        cudaFuncAttributes fa;
        GW8_CUDA(cudaFuncGetAttributes(&fa, v.fwd_kernel));
        const int launch = fa.numRegs, consumer = v.wpg == 2 ? 112 : 80;
        if (launch > consumer || 8 * v.wpg * 32 * (consumer - launch) > 128 * (launch - 24)) {
          char buf[160];
          snprintf(buf, sizeof buf,
                   "forward kernel r%d s%d wpg%d tpw%d pps%d was allocated %d registers per thread; "
                   "its register hand-over does not fit", v.r, v.s, v.wpg, v.tpw, v.pps, launch);
          return fail(buf);
        }
      }
      GW8_CUDA(cudaFuncSetAttribute(v.fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    d.smem_optin - kFwdStaticSmem));
      GW8_CUDA(cudaFuncSetAttribute(v.wgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    d.smem_optin - kFwdStaticSmem));
      GW8_CUDA(cudaFuncSetAttribute(v.wgrad_bias_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    d.smem_optin - kFwdStaticSmem));
    }
    d.dev = dev;
    d.ready = true;
  }
  *out = &d;
  return 0;
}

}  // namespace
int gw8_status_pointer(int** status) {
  const DeviceInfo* d = nullptr;
  if (device_info(&d)) return 1;
  *status = d->status;
  return 0;
}
namespace {

inline int cdiv(int a, int b) { return (a + b - 1) / b; }
inline int round_up(int a, int b) { return cdiv(a, b) * b; }

struct Plan {
  int kind = 0;
  const Gw8Variant* v = nullptr;
  Gw8Geom g{};
  int ns = 0, nob = 0, grid = 0, threads = 0;
  int smem = 0;
  size_t scratch_bytes = 0;
  int n_parts = 1;  // wgrad partials per chunk
  int engine = 1;   // 1: warp-level mma.sync kernels (v), 2: tcgen05 forward kernel (tc_kernel)
  const void* tc_kernel = nullptr;
};

int check_shape(const spio_gw8_shape* sh) {
  if (sh == nullptr) return fail("shape is NULL");
  if (sh->n <= 0 || sh->c <= 0 || sh->h <= 0 || sh->w <= 0) return fail("n, c, h, w must be positive");
  if (sh->c % 8 != 0) return fail("Number of channels must be divisible by group width.");
  if (sh->r < 1 || sh->r > 5) return fail("Kernel height must be between 1 and 5.");
  if (sh->s < 1 || sh->s > 5) return fail("Kernel width must be between 1 and 5.");
  if (sh->pad_h < 0 || sh->pad_w < 0) return fail("padding must be non-negative");
  const int p = sh->h + 2 * sh->pad_h - sh->r + 1;
  const int q = sh->w + 2 * sh->pad_w - sh->s + 1;
  if (p <= 0 || q <= 0) return fail("output height / width must be positive");
  return 0;
}

// The plan needs only the SM count and the shared-memory limit, so it can be computed
// (and unit-tested) without a device.
// SPIO_ENGINE=1 / 2 sets the engine used when the caller leaves spio_gw8_tune.engine at 0.
int default_engine() {
  static const int e = [] {
    const char* s = getenv("SPIO_ENGINE");
    return (s != nullptr && (s[0] == '1' || s[0] == '2')) ? s[0] - '0' : 0;
  }();
  return e;
}

// Launch plan of the tcgen05 forward kernel: one image and one row pair per 16 KB slot of
// 2 rows x 64 pixels, column tiles of at most 64 - (s - 1) pixels.
int make_plan_tc(int kind, const spio_gw8_shape* sh, const spio_gw8_tune& t, int sms, int smem_optin, int p,
                 int q, Plan* plan) {
  if (kind == SPIO_GW8_WGRAD) return fail("engine 2 (tcgen05) computes fprop and dgrad only");
  if (sh->r > 3 || sh->s > 3) return fail("engine 2 (tcgen05) supports filters up to 3 x 3");
  if (t.nb > 1) return fail("engine 2 (tcgen05) streams one image per slot (nb = 1)");
  Plan pl;
  pl.kind = kind;
  pl.engine = 2;
  pl.tc_kernel = gw8_tc_kernel(sh->r, sh->s);
  Gw8Geom& g = pl.g;
  g.n = sh->n;
  g.c = sh->c;
  g.dgrad = kind == SPIO_GW8_DGRAD;
  if (kind == SPIO_GW8_DGRAD) {
    g.in_h = p, g.in_w = q, g.out_h = sh->h, g.out_w = sh->w;
    g.pad_h = sh->r - 1 - sh->pad_h, g.pad_w = sh->s - 1 - sh->pad_w;
  } else {
    g.in_h = sh->h, g.in_w = sh->w, g.out_h = p, g.out_w = q;
    g.pad_h = sh->pad_h, g.pad_w = sh->pad_w;
  }
  const int qb = cdiv(g.out_w, 8);
  const int max_ncb = (64 - (sh->s - 1)) / 8;
  int ncb = t.ncb;
  if (ncb <= 0) ncb = cdiv(qb, cdiv(qb, max_ncb));
  if (ncb > max_ncb) return fail("engine 2 (tcgen05): the column tile plus s - 1 must fit 64 pixels");
  const int taps = sh->r * sh->s;
  const int slot = 2 * 64 * 128, row = 64 * 128, bbytes = taps * 2048;
  const int obuf = 2 * ncb * 8 * 128;
  const int nob = t.nob ? t.nob : 2;
  if (nob > 4) return fail("nob must be at most 4");
  const int avail = smem_optin - kTcStaticSmem - kAlignSlack - row - 2 * bbytes - nob * obuf;
  int ns = avail / slot;
  if (ns > 12) ns = 12;
  if (!t.ns && ns > 8) ns = 8;
  if (t.ns) {
    if (t.ns > ns) return fail("requested ring does not fit in shared memory");
    ns = t.ns;
  }
  if (ns < 3) return fail("engine 2 (tcgen05) needs at least 3 ring slots");
  pl.ns = ns;
  pl.nob = nob;
  pl.smem = kAlignSlack + ns * slot + row + 2 * bbytes + nob * obuf;
  pl.threads = 640;
  g.ncb = ncb;
  g.nb = 1;
  g.wt = 8 * ncb;
  g.bw = 64;
  g.in_pair_bytes = (unsigned)slot;
  g.slot_bytes = (unsigned)slot;
  g.out_pair_bytes = (unsigned)obuf;
  g.obuf_bytes = (unsigned)obuf;
  g.img_in_bytes = (unsigned)slot;
  g.img_out_bytes = (unsigned)obuf;
  g.n_chunks = cdiv(g.c, 64);
  g.n_ig = g.n;
  g.n_ct = cdiv(qb, ncb);
  g.n_pairs = cdiv(g.out_h, 2);
  g.n_split = 1;
  const long long total = (long long)g.n_ig * g.n_ct * g.n_pairs * g.n_chunks;
  if (total > 0x7fffffffLL / 2) return fail("problem too large for 32-bit work indices");
  const int ctas = t.grid > 0 ? t.grid : sms;
  pl.grid = (int)(total < ctas ? total : ctas);
  *plan = pl;
  return 0;
}

// Soft cap on shared memory: stay inside the SM's 196 KiB shared-memory configuration (dynamic +
// static + 1 KiB reserved per CTA) instead of the 228 KiB one, which leaves only 28 KiB of L1.
// The kernels with the largest tiles keep a small stack frame (16-64 bytes per thread of spilled
// loop invariants); for the 544 threads of the weight-gradient kernel that is more than the 28 KiB
// L1 holds, and every reload then goes to L2.  Measured: wgrad on 256 x 256 x 28 x 28 takes 67.5 us
// with a 3-slot ring of 217 KiB and 49.9 us with 2 slots of 145 KiB.  The configuration is
// sticky across dependent launches: after a forward kernel with 217 KiB the following wgrad ran
// in the 228 KiB configuration although it needs 181 KiB (fprop + backward at N = 256 on
// 64 x 56 x 56: 141.0 us per step, 134.0 us with the forward ring capped); kernels separated by
// an idle SM get the configuration they need.  The planner's own choice of ring depth therefore
// stops at this size while 3 (forward) or 2 (wgrad) slots remain; an explicit ns is taken as given.
constexpr int kSmemSoftCap = 194 * 1024;

// SPIO_PAIR_IMAGES=0 keeps the unpaired layout for images at most 8 pixels wide.
bool pair_images_enabled() {
  static const bool on = [] {
    const char* e = getenv("SPIO_PAIR_IMAGES");
    return !(e != nullptr && e[0] == '0');
  }();
  return on;
}

// SPIO_CHUNK_INNER=0 / 1: order of the forward kernel's work when there are several 64-channel
// chunks (see Gw8Geom::chunk_inner).
bool chunk_inner_enabled() {
  static const bool on = [] {
    const char* e = getenv("SPIO_CHUNK_INNER");
    return e != nullptr && e[0] == '1';
  }();
  return on;
}

// Largest piece (in pairs) a CTA claims from the pool of the forward kernel's dynamic tail (pieces
// shrink as the pool drains); SPIO_DYN=<n> changes it, SPIO_DYN=0 turns the dynamic tail off.
int dyn_chunk_setting() {
  static const int v = [] {
    const char* e = getenv("SPIO_DYN");
    const int n = e ? atoi(e) : 7;
    return n > 0 && n <= 64 ? n : 0;
  }();
  return v;
}

// Stages requested at kernel start before the load lane waits for the first to land
// (Gw8Geom::prefill); SPIO_PREFILL=<n> changes it, 0 requests the whole ring at once.
int prefill_setting() {
  static const int v = [] {
    const char* e = getenv("SPIO_PREFILL");
    const int n = e ? atoi(e) : 2;
    return n >= 0 && n <= 16 ? n : 2;
  }();
  return v;
}

// Stages whose boxes a kernel asks L2 for before it waits for its predecessors (Gw8Geom::warm);
// SPIO_WARM=<n> changes it, 0 switches the requests off.
int warm_setting() {
  static const int v = [] {
    const char* e = getenv("SPIO_WARM");
    const int n = e ? atoi(e) : 2;
    return n >= 0 && n <= 16 ? n : 2;
  }();
  return v;
}

// SPIO_LIGHT_REDUCE=0: the combined backward call reduces with the wide kernel, as a bare wgrad call does.
bool light_reduce_enabled() {
  static const bool v = [] {
    const char* e = getenv("SPIO_LIGHT_REDUCE");
    return !(e && e[0] == '0');
  }();
  return v;
}

// Pairs per CTA from which the dynamic tail is used.
int dyn_min_pairs() {
  static const int v = [] {
    const char* e = getenv("SPIO_DYN_MIN_PAIRS");
    const int n = e ? atoi(e) : 72;
    return n >= 4 ? n : 72;
  }();
  return v;
}

// Largest share of the work (per cent) the dynamic pool may take; SPIO_DYN_POOL changes it.
int dyn_pool_percent() {
  static const int v = [] {
    const char* e = getenv("SPIO_DYN_POOL");
    const int n = e ? atoi(e) : 25;
    return n >= 1 && n <= 100 ? n : 25;
  }();
  return v;
}

int make_plan_once(int kind, const spio_gw8_shape* sh, const spio_gw8_tune* tune, int sms, int smem_optin,
                   const std::vector<Gw8Variant>& variants, Plan* plan, const Gw8Variant* forced);

// The planner's own choice of row pairs per slot for the weight-gradient kernel: two, unless that
// leaves a ring of only two slots (a stage holds an x box and a dy box; several images of a small
// picture per slot make it 70-80 KiB) -- then one, which halves the stage and doubles the ring
// (measured: 256 x 256 x 28 x 28 48.9 -> 45.5 us, 256 x 512 x 14 x 14 32.1 -> 29.6 us).
int make_plan(int kind, const spio_gw8_shape* sh, const spio_gw8_tune* tune, int sms, int smem_optin,
              const std::vector<Gw8Variant>& variants, Plan* plan, const Gw8Variant* forced = nullptr) {
  if (make_plan_once(kind, sh, tune, sms, smem_optin, variants, plan, forced)) return 1;
  const bool open_pps = forced == nullptr && (tune == nullptr || (!tune->pps && !tune->ns && !tune->wpg && !tune->tpw));
  if (kind == SPIO_GW8_WGRAD && open_pps && plan->ns <= 2 && plan->v != nullptr && plan->v->pps == 2) {
    spio_gw8_tune t = tune ? *tune : spio_gw8_tune{0, 0, 0, 0, 0, 0, 0, 0, 0};
    t.pps = 1;
    Plan alt;
    const std::string keep = g_last_error;
    if (make_plan_once(kind, sh, &t, sms, smem_optin, variants, &alt, nullptr) == 0 && alt.ns >= 3)
      *plan = alt;
    else
      g_last_error = keep;
  }
  return 0;
}

int make_plan_once(int kind, const spio_gw8_shape* sh, const spio_gw8_tune* tune, int sms, int smem_optin,
                   const std::vector<Gw8Variant>& variants, Plan* plan, const Gw8Variant* forced) {
  if (check_shape(sh)) return 1;
  static const spio_gw8_tune kAuto = {0, 0, 0, 0, 0, 0, 0, 0, 0};
  const spio_gw8_tune& t = tune ? *tune : kAuto;
  const int p = sh->h + 2 * sh->pad_h - sh->r + 1;
  const int q = sh->w + 2 * sh->pad_w - sh->s + 1;
  if (t.engine < 0 || t.engine > 2) return fail("engine must be 0, 1 or 2");
  int engine = t.engine;
  if (engine == 0 && forced == nullptr && !t.wpg && !t.tpw && !t.pps && t.nb <= 1 && kind != SPIO_GW8_WGRAD &&
      sh->r <= 3 && sh->s <= 3)
    engine = default_engine();
  if (engine == 2) {
    if (forced != nullptr) return fail("engine 2 (tcgen05) has no just-in-time variants");
    return make_plan_tc(kind, sh, t, sms, smem_optin, p, q, plan);
  }

  // Unless the caller asks otherwise, both kernels stream two row pairs per slot: half the
  // barrier hand-offs per byte (the forward kernel fits that without spills since its compute
  // warps take over registers of the producer warpgroup).
  // Images of at most 8 output rows are streamed one row pair per slot: with two, a third of the
  // sub-steps of a 7-row image carry no output row, and the slots are twice as large for the same
  // images per slot (measured on 256 x 768 x 7 x 7: fprop 20.5 -> 15.7 us, wgrad 23.4 -> 19.0 us).
  const int out_rows = kind == SPIO_GW8_DGRAD ? sh->h : p;
  const int default_pps = out_rows <= 8 ? 1 : 2;
  const Gw8Variant* v = forced;
  for (int pass = 0; pass < 2 && v == nullptr; ++pass) {
    for (const Gw8Variant& cand : variants) {
      if (cand.r != sh->r || cand.s != sh->s) continue;
      if (t.wpg && cand.wpg != t.wpg) continue;
      if (t.tpw && cand.tpw != t.tpw) continue;
      if (t.pps && cand.pps != t.pps) continue;
      if (pass == 0 && !t.pps && cand.pps != default_pps) continue;
      v = &cand;
      break;
    }
  }
  if (v == nullptr) return fail("no compiled kernel variant matches r, s, wpg, tpw, pps");

  Plan pl;
  pl.kind = kind;
  pl.v = v;
  Gw8Geom& g = pl.g;
  g.n = sh->n;
  g.c = sh->c;
  g.dgrad = kind == SPIO_GW8_DGRAD;
  if (kind == SPIO_GW8_DGRAD) {
    g.in_h = p, g.in_w = q, g.out_h = sh->h, g.out_w = sh->w;
    g.pad_h = sh->r - 1 - sh->pad_h, g.pad_w = sh->s - 1 - sh->pad_w;
  } else {
    g.in_h = sh->h, g.in_w = sh->w, g.out_h = p, g.out_w = q;
    g.pad_h = sh->pad_h, g.pad_w = sh->pad_w;
  }
  // Tile capacity of the compute warps.  The weight-gradient kernel works on tiles of 8
  // pixels x 2 rows (TPW per warp); the forward kernel on blocks of 16 pixels x 1 row, of
  // which a warp keeps (TPW + 1) / 2, so both hold the same number of window registers.
  const bool fwd = kind != SPIO_GW8_WGRAD;
  const int max_tiles = fwd ? v->wpg * ((v->tpw + 1) / 2) : v->wpg * v->tpw;
  const int min_ncb = fwd ? 2 : 1;  // a forward column tile is at least one 16-pixel block
  auto tiles_needed = [&](int ncb8) { return fwd ? cdiv(ncb8 < 2 ? 2 : ncb8, 2) : ncb8; };
  const int pps = v->pps;
  const int avail = smem_optin - kFwdStaticSmem - kAlignSlack;
  const int qb = cdiv(g.out_w, 8);

  // Forward kernel on images at most 8 pixels wide: a 16-pixel block tile would be half empty, so
  // its two halves are given to two consecutive images of the slot (ncb = 1, nb even).  ncb = 2
  // asks for the unpaired layout.
  const bool pair = fwd && qb == 1 && sh->n >= 2 && t.ncb <= 1 && pair_images_enabled();
  int ncb = t.ncb ? t.ncb : 0;
  int nb = t.nb ? t.nb : 0;
  if (pair) {
    ncb = 1;
    if (nb <= 0) {
      nb = 2 * max_tiles;
      if (nb > sh->n) nb = sh->n & ~1;
    }
    if (nb < 2 || (nb & 1) || nb > 2 * max_tiles)
      return fail("paired images (ncb = 1) need an even nb of at most 2 * wpg * ceil(tpw / 2)");
  } else {
    if (ncb <= 0) {
      const int n_ct0 = cdiv(tiles_needed(qb), max_tiles);
      ncb = cdiv(qb, n_ct0);
    }
    if (ncb < min_ncb) ncb = min_ncb;
    if (tiles_needed(ncb) > max_tiles) return fail("ncb exceeds the tile capacity of wpg * tpw");
    if (nb <= 0) {
      nb = 1;
      if (ncb >= qb) {  // the whole width fits one column tile: batch images into a slot
        nb = max_tiles / tiles_needed(ncb);
        if (nb > sh->n) nb = sh->n;
        if (nb < 1) nb = 1;
      }
    }
    if (nb * tiles_needed(ncb) > max_tiles) return fail("nb * ncb exceeds the tile capacity of wpg * tpw");
  }

  const int min_slots = 2;
  for (;;) {
    g.ncb = ncb;
    g.nb = nb;
    g.wt = 8 * ncb;
    g.bw = round_up(g.wt + sh->s - 1, 8);
    const int slot = nb * 2 * pps * g.bw * 128;   // one ring slot of the streamed operand
    const int oslot = nb * 2 * pps * g.wt * 128;  // staging buffer (fwd) / dy part of a slot (wgrad)
    int ns, nob = 0;
    if (kind == SPIO_GW8_WGRAD) {
      ns = avail / (slot + oslot);
    } else {
      nob = t.nob ? t.nob : 2;  // measured: more staging buffers do not help the forward kernel
      if (nob > 4) return fail("nob must be at most 4");
      ns = (avail - nob * oslot) / slot;
    }
    if (ns > 16) ns = 16;
    if (!t.ns && ns > 8) ns = 8;  // a deeper ring buys nothing and shrinks the L1 cache
    if (!t.ns) {
      const int stage = kind == SPIO_GW8_WGRAD ? slot + oslot : slot;
      const int ns_floor = kind == SPIO_GW8_WGRAD ? 2 : 3;
      while (ns > ns_floor && kAlignSlack + ns * stage + nob * oslot > kSmemSoftCap) --ns;
    }
    if (t.ns) {
      if (t.ns > ns) return fail("requested ring does not fit in shared memory");
      ns = t.ns;
    }
    const bool box_ok = g.bw <= 256 && nb <= 256;
    if (ns >= min_slots && box_ok &&
        (t.nb || t.ncb || slot <= 48 * 1024 || (nb == (pair ? 2 : 1) && ncb == (pair ? 1 : min_ncb)))) {
      pl.ns = ns;
      pl.nob = nob;
      pl.smem = kAlignSlack + ns * (kind == SPIO_GW8_WGRAD ? slot + oslot : slot) + nob * oslot;
      break;
    }
    if (t.nb || t.ncb) return fail("requested tile does not fit in shared memory");
    if (pair && nb > 2)
      nb = (nb / 2 + 1) & ~1;
    else if (pair)
      return fail("tile does not fit in shared memory");
    else if (nb > 1)
      nb = nb / 2;
    else if (ncb > min_ncb)
      ncb = cdiv(ncb, 2) < min_ncb ? min_ncb : cdiv(ncb, 2);
    else
      return fail("tile does not fit in shared memory");
  }
  // the start-up window pays on the forward kernel's ordinary layout only: measured, it gains about
  // 0.7 us per launch there, loses as much on paired 7x7 images and does nothing for the weight gradient
  g.prefill = fwd && !pair && prefill_setting() < pl.ns ? prefill_setting() : 0;
  g.warm = gw8_pdl_enabled() ? warm_setting() : 0;
  g.nblk = cdiv(g.wt, 16);
  g.ntiles = pair ? g.nb / 2 : g.nb * tiles_needed(g.ncb);
  g.pair_images = pair ? 1 : 0;
  g.in_pair_bytes = (unsigned)(2 * g.bw * 128);
  g.out_pair_bytes = (unsigned)(g.nb * 2 * g.wt * 128);
  g.slot_bytes = (unsigned)(g.nb * pps) * g.in_pair_bytes;
  g.obuf_bytes = (unsigned)pps * g.out_pair_bytes;
  g.img_in_bytes = (unsigned)(2 * pps * g.bw * 128);
  g.img_out_bytes = (unsigned)(2 * g.wt * 128);
  g.n_chunks = cdiv(g.c, 64);
  g.n_ig = cdiv(g.n, g.nb);
  g.n_ct = cdiv(qb, g.ncb);
  g.n_pairs = cdiv(g.out_h, 2);
  const long long per_chunk = (long long)g.n_ig * g.n_ct * g.n_pairs;
  const long long total = per_chunk * g.n_chunks;
  if (total > 0x7fffffffLL / 2) return fail("problem too large for 32-bit work indices");
  const int ctas = t.grid > 0 ? t.grid : sms;
  g.n_split = 1;
  if (kind == SPIO_GW8_WGRAD) {
    pl.threads = v->wgrad_threads;
    if (g.n_chunks <= ctas) {
      long long split = ctas / g.n_chunks;
      if (split > per_chunk) split = per_chunk;
      g.n_split = (int)split;
      pl.grid = g.n_split * g.n_chunks;
    } else {
      pl.grid = ctas;
    }
    // CTAs that walk several chunks cannot reuse the ring for the in-CTA sum
    g.warp_parts = (pl.grid / g.n_split < g.n_chunks) ? 1 : 0;
    const int red_need = (v->wpg - 1) * 8 * ((sh->r * sh->s + 1) / 2) * 4 * 32 * (int)sizeof(float);
    if (red_need > pl.smem - kAlignSlack) g.warp_parts = 1;  // staging would not fit in the ring
    pl.n_parts = g.n_split * (g.warp_parts ? v->wpg : 1);
    pl.scratch_bytes = (size_t)g.n_chunks * pl.n_parts * GW8_PART_FLOATS(sh->r * sh->s) * sizeof(float);
  } else {
    pl.threads = v->fwd_threads;
    pl.grid = (int)(total < ctas ? total : ctas);
    g.chunk_inner = (g.n_chunks > 1 && chunk_inner_enabled()) ? 1 : 0;
    // Dynamic tail: the last quarter of the work (at most 2 * chunk pairs per CTA on average) is not
    // assigned statically but claimed from a pool, when a CTA has enough work for it.  Every piece
    // re-reads a halo and every claim is a round trip to a global counter, which costs more than the
    // better balance gains while a CTA has few pairs: measured on the 64-channel 56 x 56 layer,
    // 97 pairs per CTA (512 images) 73.8 -> 70.6 us with the pool, 48 pairs (256 images) 39.1 -> 40.1 us,
    // 24 pairs (128 images) 22.3 -> 25.9 us.  SPIO_DYN_MIN_PAIRS moves the threshold.
    const int chunk = dyn_chunk_setting();
    if (chunk > 0 && total >= (long long)dyn_min_pairs() * pl.grid) {
      long long pool = 2LL * chunk * pl.grid;
      const long long cap = total * dyn_pool_percent() / 100;
      if (pool > cap) pool = cap;
      g.dyn_chunk = chunk;
      g.dyn_begin = (int)(total - pool);
    }
  }
  *plan = pl;
  return 0;
}

int encode_map(CUtensorMap* m, const void* ptr, int c, int w, int h, int n, int box_w, int box_h,
               int box_n) {
  if ((reinterpret_cast<size_t>(ptr) & 15u) != 0) return fail("tensor pointers must be 16-byte aligned");
  const cuuint64_t dims[4] = {(cuuint64_t)c, (cuuint64_t)w, (cuuint64_t)h, (cuuint64_t)n};
  const cuuint64_t strides[3] = {(cuuint64_t)c * 2, (cuuint64_t)w * c * 2, (cuuint64_t)h * w * c * 2};
  const cuuint32_t box[4] = {64u, (cuuint32_t)box_w, (cuuint32_t)box_h, (cuuint32_t)box_n};
  const cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  // L2 promotion: a box row is 128 bytes of each pixel.  With 64 channels the pixels are contiguous and
  // fetching 256 bytes per request is free; with more channels a 256-byte fetch also brings the
  // neighbouring 64-channel chunk of the pixel, which another CTA reads at another time -- measured on
  // 256 x 128 x 56 x 56 fprop under ncu: 309 MB of DRAM reads for 205.5 MB of input, L2 hit rate 5 %.
  // With a channel count that is not a multiple of 64 a pixel (2 c bytes) does not start on a 128-byte line
  // and its last chunk is shorter than a line, so a 128-byte fetch brings bytes of the neighbouring chunk or
  // pixel: 64 bytes then.  Measured, 128 -> 64 -> none (32-byte sectors): 256 x 96 x 56 x 56 fprop 79.1 -> 67.8
  // -> 77.8 us, 256 x 72 x 56 x 56 89.6 -> 86.2 -> 89.7 us, 256 x 160 x 28 x 28 32.3 -> 30.9 -> 32.1 us; the
  // weight-gradient kernel does not care.
  // SPIO_L2_PROMOTION=32 / 64 / 128 / 256 overrides the choice.
  static const int forced = [] {
    const char* e = getenv("SPIO_L2_PROMOTION");
    return e ? atoi(e) : 0;
  }();
  const int bytes = forced ? forced : c <= 64 ? 256 : c % 64 == 0 ? 128 : 64;
  const CUtensorMapL2promotion promotion = bytes >= 256  ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B
                                           : bytes >= 128 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B
                                           : bytes >= 64  ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B
                                                          : CU_TENSOR_MAP_L2_PROMOTION_NONE;
  const CUresult r = g_encode(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(ptr), dims,
                              strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, promotion,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[160];
    snprintf(buf, sizeof buf,
             "CUDA error: cuTensorMapEncodeTiled failed with code %d (dims %d,%d,%d,%d box 64,%d,%d,%d)",
             (int)r, c, w, h, n, box_w, box_h, box_n);
    return fail(buf);
  }
  return 0;
}

static_assert(sizeof(TensorMap) == sizeof(CUtensorMap), "tensor map size");

// SPIO_PDL=0 turns programmatic dependent launch off (every kernel then starts only after
// the preceding one has drained).
bool pdl_enabled() {
  static const bool on = [] {
    const char* e = getenv("SPIO_PDL");
    return !(e != nullptr && e[0] == '0');
  }();
  return on;
}
}  // namespace
bool gw8_pdl_enabled() { return pdl_enabled(); }
namespace {

// SPIO_L2_HINTS=0 turns the L2 eviction hints of the combined backward call off.
bool l2_hints_enabled() {
  static const bool on = [] {
    const char* e = getenv("SPIO_L2_HINTS");
    return !(e != nullptr && e[0] == '0');
  }();
  return on;
}

// Launches with the programmatic-stream-serialization attribute: the kernel's CTAs may take
// SMs while the preceding kernel of the stream drains, and the kernel itself waits
// (griddepcontrol.wait) before it touches global memory.
int launch_kernel(const void* func, int grid, int threads, size_t smem, cudaStream_t stream, void** args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  GW8_CUDA(cudaLaunchKernelExC(&cfg, func, args));
  return 0;
}

// The variant record of a kernel that is compiled just in time for (r, s, wpg, tpw, pps).
int jit_variant(int kind, const spio_gw8_shape* shape, const spio_gw8_tune* tune, Gw8Variant* v) {
  if (tune == nullptr) return fail("a just-in-time kernel needs a tile configuration");
  if (kind < SPIO_GW8_FPROP || kind > SPIO_GW8_WGRAD) return fail("unknown kind");
  if (tune->wpg < 1 || tune->wpg > 3 || tune->tpw < 1 || tune->tpw > 8 || tune->pps < 1 || tune->pps > 4)
    return fail("a just-in-time kernel needs explicit wpg (1..3), tpw (1..8) and pps (1..4)");
  if (check_shape(shape)) return 1;
  *v = Gw8Variant{};
  v->r = shape->r, v->s = shape->s, v->wpg = tune->wpg, v->tpw = tune->tpw, v->pps = tune->pps;
  v->fwd_threads = (8 * tune->wpg + 4) * 32;
  v->wgrad_threads = (8 * tune->wpg + 1) * 32;
  return 0;
}

// A launch that repeats (same kind, shape, tuning, operand addresses, variant) reuses the plan
// and the encoded tensor maps of the first time: both are pure functions of those values and of
// the device's limits.  The cache is per host thread, direct-mapped; a collision just re-plans.
struct LaunchKey {
  int dev, kind, jit;
  spio_gw8_shape sh;
  spio_gw8_tune t;
  const void* a;
  const void* b;
};
struct LaunchEntry {
  bool valid = false;
  LaunchKey key;
  Plan pl;
  CUtensorMap m0, m1, m2;
};
constexpr int kLaunchCacheSize = 64;
thread_local LaunchEntry g_launch_cache[kLaunchCacheSize];

bool launch_cache_enabled() {
  static const bool on = [] {
    const char* e = getenv("SPIO_PLAN_CACHE");
    return !(e != nullptr && e[0] == '0');
  }();
  return on;
}

LaunchEntry* launch_cache_slot(const LaunchKey& key, bool* hit) {
  const unsigned char* bytes = reinterpret_cast<const unsigned char*>(&key);
  unsigned long long h = 1469598103934665603ull;
  for (size_t i = 0; i < sizeof(LaunchKey); ++i) h = (h ^ bytes[i]) * 1099511628211ull;
  LaunchEntry* e = &g_launch_cache[h % kLaunchCacheSize];
  *hit = launch_cache_enabled() && e->valid && memcmp(&e->key, &key, sizeof(LaunchKey)) == 0;
  return e;
}

void make_key(LaunchKey* key, int dev, int kind, bool jit, const spio_gw8_shape* sh, const spio_gw8_tune* tune,
              const void* a, const void* b) {
  memset(key, 0, sizeof *key);  // padding bytes take part in the comparison
  key->dev = dev;
  key->kind = kind;
  key->jit = jit ? 1 : 0;
  key->sh = *sh;
  if (tune != nullptr) key->t = *tune;
  key->a = a;
  key->b = b;
}

// Plan and tensor maps of a forward / input-gradient launch (cached).
int prepare_fwd(const DeviceInfo* d, int kind, void* out, const void* in, const spio_gw8_shape* sh,
                const spio_gw8_tune* tune, bool jit, LaunchEntry** entry) {
  if (sh == nullptr) return fail("shape is NULL");
  LaunchKey key;
  make_key(&key, d->dev, kind, jit, sh, tune, in, out);
  bool hit = false;
  LaunchEntry* e = launch_cache_slot(key, &hit);
  *entry = e;
  if (hit) return 0;
  e->valid = false;
  Gw8Variant v;
  if (jit && jit_variant(kind, sh, tune, &v)) return 1;
  if (make_plan(kind, sh, tune, d->sms, d->smem_optin, g_variants, &e->pl, jit ? &v : nullptr)) return 1;
  const Gw8Geom& g = e->pl.g;
  if (e->pl.engine == 2) {
    if (encode_map(&e->m0, in, g.c, g.in_w, g.in_h, g.n, 64, 2, 1)) return 1;
    if (encode_map(&e->m2, in, g.c, g.in_w, g.in_h, g.n, 64, 1, 1)) return 1;
    if (encode_map(&e->m1, out, g.c, g.out_w, g.out_h, g.n, g.wt, 2, 1)) return 1;
  } else {
    const int pps = jit ? v.pps : e->pl.v->pps;
    if (encode_map(&e->m0, in, g.c, g.in_w, g.in_h, g.n, g.bw, 2 * pps, g.nb)) return 1;
    if (encode_map(&e->m1, out, g.c, g.out_w, g.out_h, g.n, g.wt, 2, g.nb)) return 1;
  }
  if (jit) e->pl.v = nullptr;  // the variant record lived on this stack frame
  e->key = key;
  e->valid = true;
  return 0;
}

// jit_fn: a CUfunction compiled just in time for tune's (wpg, tpw, pps), or NULL for the variant
// built into the library.
int launch_fwd(int kind, void* out, const void* in, const void* w, const float* bias,
               const spio_gw8_shape* sh, const spio_gw8_tune* tune, cudaStream_t stream,
               bool independent = false, int hint_in = L2_HINT_NONE, void* jit_fn = nullptr) {
  if (out == nullptr || in == nullptr || w == nullptr) return fail("NULL tensor pointer");
  const DeviceInfo* d = nullptr;
  if (device_info(&d)) return 1;
  const bool jit = jit_fn != nullptr && !(tune != nullptr && tune->engine == 2);
  LaunchEntry* e = nullptr;
  if (prepare_fwd(d, kind, out, in, sh, tune, jit, &e)) return 1;
  if ((reinterpret_cast<size_t>(w) & 15u) != 0) return fail("weight pointer must be 16-byte aligned");
  const Plan& pl = e->pl;
  Gw8Geom g = pl.g;
  g.independent = (independent && pdl_enabled()) ? 1 : 0;
  g.hint_in = hint_in;
  if (g.dyn_chunk > 0) {
    // A launch recorded into a CUDA graph may be replayed on any stream, beside anything: recorded
    // launches stay static.  So do launches on streams beyond the number of counter pairs.
    cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
    GW8_CUDA(cudaStreamIsCapturing(stream, &capture));
    const int slot = capture != cudaStreamCaptureStatusNone ? -1 : slot_of_stream(d->dev, stream);
    if (slot < 0)
      g.dyn_chunk = 0;
    else
      g.dyn_slot = slot;
  }
  const __half* wp = static_cast<const __half*>(w);
  int ns = pl.ns, nob = pl.nob;
  int* status = d->status;
  if (pl.engine == 2) {
    void* args[] = {&e->m0, &e->m2, &e->m1, (void*)&g, &wp, &bias, &ns, &nob, &status};
    if (jit_fn != nullptr) return jit_launch(jit_fn, pl.grid, pl.threads, pl.smem, stream, args, pdl_enabled());
    return launch_kernel(pl.tc_kernel, pl.grid, pl.threads, pl.smem, stream, args);
  }
  void* args[] = {&e->m0, &e->m1, (void*)&g, &wp, &bias, &ns, &nob, &status};
  if (jit) return jit_launch(jit_fn, pl.grid, pl.threads, pl.smem, stream, args, pdl_enabled());
  return launch_kernel(pl.v->fwd_kernel, pl.grid, pl.threads, pl.smem, stream, args);
}

// light: the reduction is followed by a kernel that does not wait for it (the input-gradient kernel of the
// combined backward call); its blocks must then be small enough to sit beside that kernel's CTAs.
int launch_reduce(void* dw, float* dbias, const float* scratch, int c, int taps, int n_parts,
                  cudaStream_t stream, int dw_f16 = 0, bool light = false, int sms = 0) {
  if (dbias != nullptr && taps % 2 == 0)
    return fail("the fused bias gradient needs an odd number of filter taps (r * s)");
  if ((reinterpret_cast<size_t>(dbias) & 15u) != 0) return fail("dbias must be 16-byte aligned");
  const int total_f4 = cdiv(c, 64) * (GW8_PART_FLOATS(taps) / 4);
  int n_groups = cdiv(total_f4, 8);
  void* args[] = {&dw, &dbias, &scratch, &c, &taps, &n_parts, &dw_f16, &n_groups};
  // The light form walks the groups with at most one block per SM; beyond four passes (more than 256
  // channels) it is slower than the wide form, and such layers have few parts per column anyway.
  if (light && sms > 0 && n_groups <= 4 * sms)
    return launch_kernel(reinterpret_cast<const void*>(&conv2d_gw8_wgrad_reduce_light_kernel<128>),
                         n_groups < sms ? n_groups : sms, 128, 0, stream, args);
  return launch_kernel(reinterpret_cast<const void*>(&conv2d_gw8_wgrad_reduce_kernel<256>), n_groups, 256,
                       0, stream, args);
}

// jit_fn: as for launch_fwd; with dbias it must be the instantiation that also sums dy.
// dw_f16: dw points to fp16 and receives the fp32 sums rounded once.
int launch_wgrad(void* dw, const void* x, const void* dy, const spio_gw8_shape* sh,
                 const spio_gw8_tune* tune, void* scratch, size_t scratch_bytes,
                 cudaStream_t stream, int hint_x = L2_HINT_NONE, int hint_dy = L2_HINT_NONE,
                 float* dbias = nullptr, void* jit_fn = nullptr, int dw_f16 = 0, bool light_reduce = false) {
  if (dw == nullptr || x == nullptr || dy == nullptr) return fail("NULL tensor pointer");
  if (sh == nullptr) return fail("shape is NULL");
  const DeviceInfo* d = nullptr;
  if (device_info(&d)) return 1;
  const bool jit = jit_fn != nullptr;
  LaunchKey key;
  make_key(&key, d->dev, SPIO_GW8_WGRAD, jit, sh, tune, x, dy);
  bool hit = false;
  LaunchEntry* e = launch_cache_slot(key, &hit);
  if (!hit) {
    e->valid = false;
    Gw8Variant v;
    if (jit && jit_variant(SPIO_GW8_WGRAD, sh, tune, &v)) return 1;
    if (make_plan(SPIO_GW8_WGRAD, sh, tune, d->sms, d->smem_optin, g_variants, &e->pl, jit ? &v : nullptr)) return 1;
    const Gw8Geom& g = e->pl.g;
    const int pps = jit ? v.pps : e->pl.v->pps;
    if (encode_map(&e->m0, x, g.c, g.in_w, g.in_h, g.n, g.bw, 2 * pps, g.nb)) return 1;
    if (encode_map(&e->m1, dy, g.c, g.out_w, g.out_h, g.n, g.wt, 2 * pps, g.nb)) return 1;
    if (jit) e->pl.v = nullptr;
    e->key = key;
    e->valid = true;
  }
  const Plan& pl = e->pl;
  if (scratch == nullptr || scratch_bytes < pl.scratch_bytes) return fail("wgrad scratch buffer is too small");
  if ((reinterpret_cast<size_t>(scratch) & 15u) != 0 || (reinterpret_cast<size_t>(dw) & 15u) != 0)
    return fail("dw and scratch must be 16-byte aligned");
  Gw8Geom g = pl.g;
  g.hint_in = hint_x;
  g.hint_tiled = hint_dy;
  float* sc = static_cast<float*>(scratch);
  int ns = pl.ns;
  int* status = d->status;
  void* args[] = {&e->m0, &e->m1, (void*)&g, &sc, &ns, &status};
  if (jit) {
    if (jit_launch(jit_fn, pl.grid, pl.threads, pl.smem, stream, args, pdl_enabled())) return 1;
  } else {
    const void* kernel = dbias != nullptr ? pl.v->wgrad_bias_kernel : pl.v->wgrad_kernel;
    if (launch_kernel(kernel, pl.grid, pl.threads, pl.smem, stream, args)) return 1;
  }
  return launch_reduce(dw, dbias, sc, g.c, sh->r * sh->s, pl.n_parts, stream, dw_f16, light_reduce, d->sms);
}

// ---------------------------------------------------------------- host-buffer variants

constexpr int kStageBuffers = 9;
constexpr int kStepChunks = 32;  // pieces of the batch the pipelined step call works in

struct HostStage {
  cudaStream_t stream = nullptr;
  // the pipelined step call: upload, compute and download streams, one event pair per piece
  cudaStream_t up = nullptr, down = nullptr;
  cudaEvent_t uploaded[kStepChunks] = {}, computed[kStepChunks + 1] = {};
  bool step_ready = false;
  void* buf[kStageBuffers] = {};
  size_t cap[kStageBuffers] = {};
};
HostStage g_stage[kMaxDevices];
std::mutex g_stage_mutex;

int stage_reserve(HostStage& st, int i, size_t bytes) {
  if (bytes <= st.cap[i]) return 0;
  if (st.buf[i]) GW8_CUDA(cudaFree(st.buf[i]));
  st.buf[i] = nullptr;
  st.cap[i] = 0;
  GW8_CUDA(cudaMalloc(&st.buf[i], bytes));
  st.cap[i] = bytes;
  return 0;
}

int get_stage(HostStage** out) {
  int dev = 0;
  GW8_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail("device ordinal out of range");
  HostStage& st = g_stage[dev];
  if (st.stream == nullptr) GW8_CUDA(cudaStreamCreateWithFlags(&st.stream, cudaStreamNonBlocking));
  *out = &st;
  return 0;
}

size_t act_bytes(const spio_gw8_shape* sh, bool output) {
  const int p = sh->h + 2 * sh->pad_h - sh->r + 1;
  const int q = sh->w + 2 * sh->pad_w - sh->s + 1;
  return (size_t)sh->n * sh->c * (output ? (size_t)p * q : (size_t)sh->h * sh->w) * 2;
}

size_t weight_elems(const spio_gw8_shape* sh) { return (size_t)sh->c * sh->r * sh->s * 8; }

void fill_info(const Plan& pl, spio_gw8_plan_info* info) {
  info->engine = pl.engine;
  info->wpg = pl.v ? pl.v->wpg : 0;
  info->tpw = pl.v ? pl.v->tpw : 0;
  info->pps = pl.v ? pl.v->pps : 1;
  info->ns = pl.ns;
  info->nob = pl.nob;
  info->ncb = pl.g.ncb;
  info->nb = pl.g.nb;
  info->grid = pl.grid;
  info->threads = pl.threads;
  info->smem_bytes = pl.smem;
  info->n_chunks = pl.g.n_chunks;
  info->n_image_groups = pl.g.n_ig;
  info->n_col_tiles = pl.g.n_ct;
  info->n_pairs = pl.g.n_pairs;
  info->n_split = pl.g.n_split;
  info->scratch_bytes = pl.scratch_bytes;
}

}  // namespace

}  // namespace spio_b200

using namespace spio_b200;

extern "C" {

int spio_conv2d_gw8_fprop(void* y, const void* x, const void* w, const float* bias,
                          const spio_gw8_shape* shape, const spio_gw8_tune* tune, void* stream) {
  return launch_fwd(SPIO_GW8_FPROP, y, x, w, bias, shape, tune, (cudaStream_t)stream);
}

int spio_conv2d_gw8_dgrad(void* dx, const void* dy, const void* w, const spio_gw8_shape* shape,
                          const spio_gw8_tune* tune, void* stream) {
  return launch_fwd(SPIO_GW8_DGRAD, dx, dy, w, nullptr, shape, tune, (cudaStream_t)stream);
}

size_t spio_conv2d_gw8_wgrad_scratch_bytes(const spio_gw8_shape* shape, const spio_gw8_tune* tune) {
  const DeviceInfo* d = nullptr;
  if (device_info(&d)) return 0;
  Plan pl;
  if (make_plan(SPIO_GW8_WGRAD, shape, tune, d->sms, d->smem_optin, g_variants, &pl)) return 0;
  return pl.scratch_bytes;
}

int spio_conv2d_gw8_wgrad(float* dw, const void* x, const void* dy, const spio_gw8_shape* shape,
                          const spio_gw8_tune* tune, void* scratch, size_t scratch_bytes,
                          void* stream) {
  return launch_wgrad(dw, x, dy, shape, tune, scratch, scratch_bytes, (cudaStream_t)stream);
}

int spio_conv2d_gw8_backward_ex(void* dx, void* dw, float* dbias, const void* x, const void* dy, const void* w,
                                const spio_gw8_shape* shape, const spio_gw8_tune* dgrad_tune,
                                const spio_gw8_tune* wgrad_tune, void* scratch, size_t scratch_bytes, void* stream,
                                void* dw_ready, const spio_gw8_backward_opts* opts) {
  if (dx == nullptr && dw == nullptr) return fail("neither gradient was asked for");
  if (dbias != nullptr && dw == nullptr) return fail("the bias gradient is computed together with dw");
  if (dbias != nullptr && (shape == nullptr || (shape->r * shape->s) % 2 == 0))
    return fail("the fused bias gradient needs an odd number of filter taps (r * s)");
  static const spio_gw8_backward_opts kNone = {0, nullptr, nullptr, nullptr, nullptr};
  const spio_gw8_backward_opts& o = opts ? *opts : kNone;
  if (o.dp != nullptr && (dw == nullptr || o.dw_f16))
    return fail("the data-parallel exchange sums an fp32 dw");
  const size_t dw_floats = shape ? (size_t)shape->c * 8 * shape->r * shape->s : 0;
  const size_t db_floats = (shape && dbias != nullptr) ? (size_t)shape->c : 0;
  if (o.dp != nullptr && db_floats % 4 != 0)
    return fail("the data-parallel exchange of dbias needs a channel count that is a multiple of 4");
  void* wgrad_fn = dbias != nullptr ? o.wgrad_dbias_function : o.wgrad_function;
  if (dw != nullptr && dbias != nullptr && o.wgrad_function != nullptr && wgrad_fn == nullptr)
    return fail("a just-in-time weight-gradient kernel needs its bias-summing instantiation for dbias");
  cudaStream_t st = (cudaStream_t)stream;
  // Both kernels read dy.  The weight-gradient kernel asks the L2 to keep dy and to let x go
  // first, so that the input-gradient kernel finds as much of dy in the cache as fits; that
  // kernel in turn marks dy as done with.
  // With the exchange in the chain the input-gradient kernel leaves one SM to each of its CTAs: a waiting
  // exchange CTA keeps the input-gradient CTA of its SM from starting (measured on 8 GPUs: 135 us per step
  // with 148 input-gradient CTAs, 115 us with 139).
  spio_gw8_tune dgrad_dp_tune;
  if (o.dp != nullptr && dx != nullptr && (dgrad_tune == nullptr || dgrad_tune->grid == 0)) {
    const DeviceInfo* d = nullptr;
    if (device_info(&d)) return 1;
    const int ctas = dp_exchange_ctas(dw_floats + db_floats);
    if (ctas > 0 && ctas < d->sms / 2) {
      memset(&dgrad_dp_tune, 0, sizeof dgrad_dp_tune);
      if (dgrad_tune != nullptr) dgrad_dp_tune = *dgrad_tune;
      dgrad_dp_tune.grid = d->sms - ctas;
      dgrad_tune = &dgrad_dp_tune;
    }
  }
  const bool both = dx != nullptr && dw != nullptr && l2_hints_enabled();
  if (dw != nullptr && launch_wgrad(dw, x, dy, shape, wgrad_tune, scratch, scratch_bytes, st,
                                    both ? L2_HINT_EVICT_FIRST : L2_HINT_NONE,
                                    both ? L2_HINT_EVICT_LAST : L2_HINT_NONE, dbias, wgrad_fn, o.dw_f16,
                                    dx != nullptr && light_reduce_enabled()))
    return 1;
  // Data-parallel: one small kernel stores this rank's dw (and dbias) into every rank's exchange
  // buffer, waits for the others' and overwrites dw with the sum in rank order (2-3 us).  No event,
  // no second stream: the chain of dependent launches stays intact.
  if (o.dp != nullptr && dp_allreduce(o.dp, static_cast<float*>(dw), dw_floats, dbias, db_floats, st)) return 1;
  if (dw != nullptr && dw_ready != nullptr && o.dp == nullptr) GW8_CUDA(cudaEventRecord((cudaEvent_t)dw_ready, st));
  // dgrad reads dy and w and writes dx; the weight-gradient kernels read x and dy and write
  // scratch and dw (the exchange reads dw and writes the exchange buffers).  Neither touches what
  // the other writes, so dgrad need not wait for them.
  if (dx != nullptr && launch_fwd(SPIO_GW8_DGRAD, dx, dy, w, nullptr, shape, dgrad_tune, st, dw != nullptr,
                                  both ? L2_HINT_EVICT_FIRST : L2_HINT_NONE, o.dgrad_function))
    return 1;
  // the input-gradient kernel completes only after everything before it (it waits at its end), so
  // an event recorded here also covers the sum over the ranks
  if (o.dp != nullptr && dw_ready != nullptr) GW8_CUDA(cudaEventRecord((cudaEvent_t)dw_ready, st));
  return 0;
}

int spio_conv2d_gw8_backward(void* dx, float* dw, float* dbias, const void* x, const void* dy, const void* w,
                             const spio_gw8_shape* shape, const spio_gw8_tune* dgrad_tune,
                             const spio_gw8_tune* wgrad_tune, void* scratch, size_t scratch_bytes, void* stream,
                             void* dw_ready) {
  return spio_conv2d_gw8_backward_ex(dx, dw, dbias, x, dy, w, shape, dgrad_tune, wgrad_tune, scratch, scratch_bytes,
                                     stream, dw_ready, nullptr);
}

int spio_conv2d_gw8_fprop_jit(void* function, void* y, const void* x, const void* w, const float* bias,
                              const spio_gw8_shape* shape, const spio_gw8_tune* tune, void* stream) {
  if (function == nullptr) return fail("NULL function");
  return launch_fwd(SPIO_GW8_FPROP, y, x, w, bias, shape, tune, (cudaStream_t)stream, false, L2_HINT_NONE, function);
}

int spio_conv2d_gw8_dgrad_jit(void* function, void* dx, const void* dy, const void* w, const spio_gw8_shape* shape,
                              const spio_gw8_tune* tune, void* stream) {
  if (function == nullptr) return fail("NULL function");
  return launch_fwd(SPIO_GW8_DGRAD, dx, dy, w, nullptr, shape, tune, (cudaStream_t)stream, false, L2_HINT_NONE,
                    function);
}

int spio_conv2d_gw8_wgrad_jit(void* function, float* dw, const void* x, const void* dy, const spio_gw8_shape* shape,
                              const spio_gw8_tune* tune, void* scratch, size_t scratch_bytes, void* stream) {
  if (function == nullptr) return fail("NULL function");
  return launch_wgrad(dw, x, dy, shape, tune, scratch, scratch_bytes, (cudaStream_t)stream, L2_HINT_NONE,
                      L2_HINT_NONE, nullptr, function);
}

size_t spio_conv2d_gw8_wgrad_scratch_bytes_jit(const spio_gw8_shape* shape, const spio_gw8_tune* tune) {
  const DeviceInfo* d = nullptr;
  if (device_info(&d)) return 0;
  Gw8Variant v;
  if (jit_variant(SPIO_GW8_WGRAD, shape, tune, &v)) return 0;
  Plan pl;
  if (make_plan(SPIO_GW8_WGRAD, shape, tune, d->sms, d->smem_optin, g_variants, &pl, &v)) return 0;
  return pl.scratch_bytes;
}

int spio_conv2d_gw8_wgrad_static(float* dw, const void* x, const void* dy,
                                 const spio_gw8_shape* shape, const spio_gw8_tune* tune,
                                 void* stream) {
  int dev = 0;
  GW8_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail("device ordinal out of range");
  const DeviceInfo* d = nullptr;
  if (device_info(&d)) return 1;  // first call on a device: limits, kernel attributes (no allocation)
  Plan pl;
  if (make_plan(SPIO_GW8_WGRAD, shape, tune, d->sms, d->smem_optin, g_variants, &pl)) return 1;
  if (pl.scratch_bytes > kStaticScratchBytes) {
    char buf[200];
    snprintf(buf, sizeof buf,
             "spio_conv2d_gw8_wgrad_static: this shape needs %zu bytes of scratch, the built-in "
             "buffer holds %zu; use spio_conv2d_gw8_wgrad with caller-provided scratch",
             pl.scratch_bytes, kStaticScratchBytes);
    return fail(buf);
  }
  unsigned char* scratch = nullptr;
  {
    // In host code `g_static_scratch` is only a handle for the symbol; the address a kernel
    // can use has to be asked for, once per device, with that device current.
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_static_scratch_addr[dev] == nullptr) {
      void* p = nullptr;
      GW8_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
      g_static_scratch_addr[dev] = static_cast<unsigned char*>(p);
    }
    scratch = g_static_scratch_addr[dev];
  }
  return launch_wgrad(dw, x, dy, shape, tune, scratch, kStaticScratchBytes, (cudaStream_t)stream);
}

int spio_conv2d_gw8_fprop_host(void* y, const void* x, const void* w, const float* bias,
                               const spio_gw8_shape* shape, const spio_gw8_tune* tune) {
  if (check_shape(shape)) return 1;
  std::lock_guard<std::mutex> lock(g_stage_mutex);
  HostStage* st = nullptr;
  if (get_stage(&st)) return 1;
  const size_t xb = act_bytes(shape, false), yb = act_bytes(shape, true);
  const size_t wb = weight_elems(shape) * 2, bb = (size_t)shape->c * 4;
  if (stage_reserve(*st, 0, xb) || stage_reserve(*st, 1, yb) || stage_reserve(*st, 2, wb)) return 1;
  if (bias && stage_reserve(*st, 3, bb)) return 1;
  GW8_CUDA(cudaMemcpyAsync(st->buf[0], x, xb, cudaMemcpyHostToDevice, st->stream));
  GW8_CUDA(cudaMemcpyAsync(st->buf[2], w, wb, cudaMemcpyHostToDevice, st->stream));
  if (bias) GW8_CUDA(cudaMemcpyAsync(st->buf[3], bias, bb, cudaMemcpyHostToDevice, st->stream));
  if (launch_fwd(SPIO_GW8_FPROP, st->buf[1], st->buf[0], st->buf[2],
                 bias ? (const float*)st->buf[3] : nullptr, shape, tune, st->stream))
    return 1;
  GW8_CUDA(cudaMemcpyAsync(y, st->buf[1], yb, cudaMemcpyDeviceToHost, st->stream));
  GW8_CUDA(cudaStreamSynchronize(st->stream));
  return 0;
}

int spio_conv2d_gw8_step_host(void* y, void* dx, float* dw, float* dbias, const void* x, const void* dy,
                              const void* w, const float* bias, const spio_gw8_shape* shape) {
  return spio_conv2d_gw8_step_host_dp(y, dx, dw, dbias, x, dy, w, bias, shape, nullptr);
}

int spio_conv2d_gw8_step_host_dp(void* y, void* dx, float* dw, float* dbias, const void* x, const void* dy,
                                 const void* w, const float* bias, const spio_gw8_shape* shape,
                                 const spio_dp_exchange* dp) {
  if (check_shape(shape)) return 1;
  if (y == nullptr || dx == nullptr || dw == nullptr || x == nullptr || dy == nullptr || w == nullptr)
    return fail("NULL host pointer");
  if (dbias != nullptr && (shape->r * shape->s) % 2 == 0)
    return fail("the fused bias gradient needs an odd number of filter taps (r * s)");
  std::lock_guard<std::mutex> lock(g_stage_mutex);
  HostStage* st = nullptr;
  if (get_stage(&st)) return 1;
  if (!st->step_ready) {
    GW8_CUDA(cudaStreamCreateWithFlags(&st->up, cudaStreamNonBlocking));
    GW8_CUDA(cudaStreamCreateWithFlags(&st->down, cudaStreamNonBlocking));
    for (int i = 0; i < kStepChunks; ++i) GW8_CUDA(cudaEventCreateWithFlags(&st->uploaded[i], cudaEventDisableTiming));
    for (int i = 0; i <= kStepChunks; ++i) GW8_CUDA(cudaEventCreateWithFlags(&st->computed[i], cudaEventDisableTiming));
    st->step_ready = true;
  }
  const size_t xb = act_bytes(shape, false), yb = act_bytes(shape, true);
  const size_t wb = weight_elems(shape) * 2, dwb = weight_elems(shape) * 4, bb = (size_t)shape->c * 4;
  const size_t scratch = spio_conv2d_gw8_wgrad_scratch_bytes(shape, nullptr);
  if (scratch == 0) return 1;
  // device copies of x, dy (whole batch: the weight gradient needs all of it), y, dx, w, bias, dw, dbias, scratch
  if (stage_reserve(*st, 0, xb) || stage_reserve(*st, 1, yb) || stage_reserve(*st, 2, wb) ||
      stage_reserve(*st, 3, bb) || stage_reserve(*st, 4, scratch) || stage_reserve(*st, 5, yb) ||
      stage_reserve(*st, 6, xb) || stage_reserve(*st, 7, dwb) || stage_reserve(*st, 8, bb))
    return 1;
  char* d_x = static_cast<char*>(st->buf[0]);
  char* d_dy = static_cast<char*>(st->buf[1]);
  char* d_y = static_cast<char*>(st->buf[5]);
  char* d_dx = static_cast<char*>(st->buf[6]);
  const float* d_bias = bias ? static_cast<const float*>(st->buf[3]) : nullptr;
  GW8_CUDA(cudaMemcpyAsync(st->buf[2], w, wb, cudaMemcpyHostToDevice, st->up));
  if (bias) GW8_CUDA(cudaMemcpyAsync(st->buf[3], bias, bb, cudaMemcpyHostToDevice, st->up));
  // Pieces of at least 16 MB of x (a copy much smaller than that does not reach the link rate),
  // at least 4 so that uploads, kernels and downloads overlap, at most kStepChunks.
  const int n = shape->n;
  int pieces = (int)(xb >> 24);
  if (pieces < 4) pieces = 4;
  if (pieces > kStepChunks) pieces = kStepChunks;
  if (pieces > n) pieces = n;
  const size_t x_img = xb / (size_t)n, y_img = yb / (size_t)n;
  // Piece i: upload its images of x and dy; as soon as they are there, fprop and dgrad run on
  // them; as soon as those are done, y and dx of the piece go back.  The three streams overlap,
  // so the step costs about one upload of x and dy.
  for (int i = 0; i < pieces; ++i) {
    const int n0 = (int)((long long)n * i / pieces), n1 = (int)((long long)n * (i + 1) / pieces);
    const size_t xo = x_img * (size_t)n0, yo = y_img * (size_t)n0;
    const size_t xs = x_img * (size_t)(n1 - n0), ys = y_img * (size_t)(n1 - n0);
    GW8_CUDA(cudaMemcpyAsync(d_x + xo, static_cast<const char*>(x) + xo, xs, cudaMemcpyHostToDevice, st->up));
    GW8_CUDA(cudaMemcpyAsync(d_dy + yo, static_cast<const char*>(dy) + yo, ys, cudaMemcpyHostToDevice, st->up));
    GW8_CUDA(cudaEventRecord(st->uploaded[i], st->up));
    GW8_CUDA(cudaStreamWaitEvent(st->stream, st->uploaded[i], 0));
    spio_gw8_shape part = *shape;
    part.n = n1 - n0;
    if (launch_fwd(SPIO_GW8_FPROP, d_y + yo, d_x + xo, st->buf[2], d_bias, &part, nullptr, st->stream)) return 1;
    if (launch_fwd(SPIO_GW8_DGRAD, d_dx + xo, d_dy + yo, st->buf[2], nullptr, &part, nullptr, st->stream)) return 1;
    GW8_CUDA(cudaEventRecord(st->computed[i], st->stream));
    GW8_CUDA(cudaStreamWaitEvent(st->down, st->computed[i], 0));
    GW8_CUDA(cudaMemcpyAsync(static_cast<char*>(y) + yo, d_y + yo, ys, cudaMemcpyDeviceToHost, st->down));
    GW8_CUDA(cudaMemcpyAsync(static_cast<char*>(dx) + xo, d_dx + xo, xs, cudaMemcpyDeviceToHost, st->down));
  }
  // the weight (and bias) gradient over the whole batch, now resident on the device
  if (launch_wgrad(static_cast<float*>(st->buf[7]), d_x, d_dy, shape, nullptr, st->buf[4], scratch, st->stream,
                   L2_HINT_NONE, L2_HINT_NONE, dbias ? static_cast<float*>(st->buf[8]) : nullptr))
    return 1;
  // data-parallel: the sum over the ranks happens on the device, before dw goes back
  if (dp != nullptr) {
    float* d_dw = static_cast<float*>(st->buf[7]);
    float* d_db = dbias ? static_cast<float*>(st->buf[8]) : nullptr;
    const size_t n_dw = weight_elems(shape), n_db = dbias ? (size_t)shape->c : 0;
    if (dp_allreduce(dp, d_dw, n_dw, d_db, n_db, st->stream)) return 1;
  }
  GW8_CUDA(cudaEventRecord(st->computed[kStepChunks], st->stream));
  GW8_CUDA(cudaStreamWaitEvent(st->down, st->computed[kStepChunks], 0));
  GW8_CUDA(cudaMemcpyAsync(dw, st->buf[7], dwb, cudaMemcpyDeviceToHost, st->down));
  if (dbias) GW8_CUDA(cudaMemcpyAsync(dbias, st->buf[8], bb, cudaMemcpyDeviceToHost, st->down));
  GW8_CUDA(cudaStreamSynchronize(st->down));
  GW8_CUDA(cudaStreamSynchronize(st->stream));
  return 0;
}

int spio_conv2d_gw8_dgrad_host(void* dx, const void* dy, const void* w, const spio_gw8_shape* shape,
                               const spio_gw8_tune* tune) {
  if (check_shape(shape)) return 1;
  std::lock_guard<std::mutex> lock(g_stage_mutex);
  HostStage* st = nullptr;
  if (get_stage(&st)) return 1;
  const size_t xb = act_bytes(shape, false), yb = act_bytes(shape, true);
  const size_t wb = weight_elems(shape) * 2;
  if (stage_reserve(*st, 0, xb) || stage_reserve(*st, 1, yb) || stage_reserve(*st, 2, wb)) return 1;
  GW8_CUDA(cudaMemcpyAsync(st->buf[1], dy, yb, cudaMemcpyHostToDevice, st->stream));
  GW8_CUDA(cudaMemcpyAsync(st->buf[2], w, wb, cudaMemcpyHostToDevice, st->stream));
  if (launch_fwd(SPIO_GW8_DGRAD, st->buf[0], st->buf[1], st->buf[2], nullptr, shape, tune, st->stream))
    return 1;
  GW8_CUDA(cudaMemcpyAsync(dx, st->buf[0], xb, cudaMemcpyDeviceToHost, st->stream));
  GW8_CUDA(cudaStreamSynchronize(st->stream));
  return 0;
}

int spio_conv2d_gw8_wgrad_host(float* dw, const void* x, const void* dy, const spio_gw8_shape* shape,
                               const spio_gw8_tune* tune) {
  if (check_shape(shape)) return 1;
  const size_t scratch = spio_conv2d_gw8_wgrad_scratch_bytes(shape, tune);
  if (scratch == 0) return 1;
  std::lock_guard<std::mutex> lock(g_stage_mutex);
  HostStage* st = nullptr;
  if (get_stage(&st)) return 1;
  const size_t xb = act_bytes(shape, false), yb = act_bytes(shape, true);
  const size_t wb = weight_elems(shape) * 4;
  if (stage_reserve(*st, 0, xb) || stage_reserve(*st, 1, yb) || stage_reserve(*st, 2, wb) ||
      stage_reserve(*st, 4, scratch))
    return 1;
  GW8_CUDA(cudaMemcpyAsync(st->buf[0], x, xb, cudaMemcpyHostToDevice, st->stream));
  GW8_CUDA(cudaMemcpyAsync(st->buf[1], dy, yb, cudaMemcpyHostToDevice, st->stream));
  if (launch_wgrad((float*)st->buf[2], st->buf[0], st->buf[1], shape, tune, st->buf[4], scratch,
                   st->stream))
    return 1;
  GW8_CUDA(cudaMemcpyAsync(dw, st->buf[2], wb, cudaMemcpyDeviceToHost, st->stream));
  GW8_CUDA(cudaStreamSynchronize(st->stream));
  return 0;
}

int spio_conv2d_gw8_plan_jit(int kind, const spio_gw8_shape* shape, const spio_gw8_tune* tune, int sm_count,
                             int smem_optin_bytes, spio_gw8_plan_info* info) {
  if (info == nullptr) return fail("info is NULL");
  if (sm_count <= 0 || smem_optin_bytes <= 0) return fail("sm_count and smem_optin_bytes must be positive");
  Plan pl;
  if (tune != nullptr && tune->engine == 2) {  // the tcgen05 kernel has one configuration per filter size
    if (make_plan(kind, shape, tune, sm_count, smem_optin_bytes, g_variants, &pl)) return 1;
  } else {
    Gw8Variant v;
    if (jit_variant(kind, shape, tune, &v)) return 1;
    if (make_plan(kind, shape, tune, sm_count, smem_optin_bytes, g_variants, &pl, &v)) return 1;
  }
  fill_info(pl, info);
  return 0;
}

int spio_conv2d_gw8_prepare_launch(int kind, const spio_gw8_shape* shape, const spio_gw8_tune* tune,
                                   const void* streamed, const void* tiled, spio_gw8_launch* out) {
  static_assert(sizeof(Gw8Geom) <= sizeof(out->geom), "geometry blob too small");
  static_assert(sizeof(CUtensorMap) == sizeof(out->in_map), "tensor map size");
  if (out == nullptr) return fail("NULL argument");
  if (streamed == nullptr || tiled == nullptr) return fail("NULL tensor pointer");
  const DeviceInfo* d = nullptr;
  if (device_info(&d)) return 1;
  Plan pl;
  CUtensorMap a, b, row;
  memset(out, 0, sizeof *out);
  if (tune != nullptr && tune->engine == 2) {
    if (make_plan(kind, shape, tune, d->sms, d->smem_optin, g_variants, &pl)) return 1;
    if (encode_map(&a, streamed, pl.g.c, pl.g.in_w, pl.g.in_h, pl.g.n, 64, 2, 1)) return 1;
    if (encode_map(&row, streamed, pl.g.c, pl.g.in_w, pl.g.in_h, pl.g.n, 64, 1, 1)) return 1;
    if (encode_map(&b, tiled, pl.g.c, pl.g.out_w, pl.g.out_h, pl.g.n, pl.g.wt, 2, 1)) return 1;
    memcpy(out->row_map, &row, sizeof row);
  } else {
    Gw8Variant v;
    if (jit_variant(kind, shape, tune, &v)) return 1;
    if (make_plan(kind, shape, tune, d->sms, d->smem_optin, g_variants, &pl, &v)) return 1;
    if (encode_map(&a, streamed, pl.g.c, pl.g.in_w, pl.g.in_h, pl.g.n, pl.g.bw, 2 * v.pps, pl.g.nb)) return 1;
    if (encode_map(&b, tiled, pl.g.c, pl.g.out_w, pl.g.out_h, pl.g.n, pl.g.wt,
                   kind == SPIO_GW8_WGRAD ? 2 * v.pps : 2, pl.g.nb))
      return 1;
  }
  // A launch assembled by the caller has no counter pair of its own: its work is split statically.
  pl.g.dyn_chunk = 0;
  pl.g.dyn_begin = 0;
  const Gw8Geom& g = pl.g;
  memcpy(out->in_map, &a, sizeof a);
  memcpy(out->out_map, &b, sizeof b);
  memcpy(out->geom, &g, sizeof g);
  out->ns = pl.ns;
  out->nob = pl.nob;
  out->grid = pl.grid;
  out->threads = pl.threads;
  out->smem_bytes = pl.smem;
  out->n_parts = pl.n_parts;
  out->scratch_bytes = pl.scratch_bytes;
  out->status = d->status;
  return 0;
}

int spio_conv2d_gw8_wgrad_reduce(float* dw, float* dbias, const float* scratch, int c, int taps, int n_parts,
                                 void* stream) {
  if (dw == nullptr || scratch == nullptr || c <= 0 || c % 8 || taps <= 0 || n_parts <= 0)
    return fail("bad argument");
  return launch_reduce(dw, dbias, scratch, c, taps, n_parts, (cudaStream_t)stream);
}

int spio_tensor_map_encode(void* map_out, const void* base, int elem_bytes, int rank,
                           const unsigned long long* sizes, const unsigned long long* strides_bytes,
                           const unsigned* box, int swizzle) {
  if (map_out == nullptr || base == nullptr || sizes == nullptr || box == nullptr) return fail("NULL argument");
  if (rank < 1 || rank > 5) return fail("a tiled tensor map has 1 to 5 axes");
  if (rank > 1 && strides_bytes == nullptr) return fail("strides_bytes is NULL");
  CUtensorMapDataType type;
  switch (elem_bytes) {
    case 1: type = CU_TENSOR_MAP_DATA_TYPE_UINT8; break;
    case 2: type = CU_TENSOR_MAP_DATA_TYPE_UINT16; break;
    case 4: type = CU_TENSOR_MAP_DATA_TYPE_UINT32; break;
    case 8: type = CU_TENSOR_MAP_DATA_TYPE_UINT64; break;
    default: return fail("element size must be 1, 2, 4 or 8 bytes");
  }
  static const CUtensorMapSwizzle kSwizzle[4] = {CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_SWIZZLE_32B,
                                                 CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_SWIZZLE_128B};
  if (swizzle < 0 || swizzle > 3) return fail("swizzle must be 0 (none), 1 (32 B), 2 (64 B) or 3 (128 B)");
  if ((reinterpret_cast<size_t>(base) & 15u) != 0) return fail("tensor pointers must be 16-byte aligned");
  if (((size_t)box[0] * elem_bytes) % 16 != 0) return fail("the innermost box extent must be a multiple of 16 bytes");
  const DeviceInfo* d = nullptr;
  if (device_info(&d)) return 1;  // loads the driver entry point
  cuuint64_t dims[5], strides[4];
  cuuint32_t bx[5], estr[5];
  for (int i = 0; i < rank; ++i) {
    if (sizes[i] == 0 || box[i] == 0 || box[i] > 256) return fail("sizes must be positive and box extents 1..256");
    dims[i] = sizes[i];
    bx[i] = box[i];
    estr[i] = 1;
    if (i > 0) {
      if (strides_bytes[i - 1] % 16 != 0) return fail("tensor strides must be multiples of 16 bytes");
      strides[i - 1] = strides_bytes[i - 1];
    }
  }
  CUtensorMap m;
  const CUresult r = g_encode(&m, type, (cuuint32_t)rank, const_cast<void*>(base), dims, strides, bx, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, kSwizzle[swizzle], CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[96];
    snprintf(buf, sizeof buf, "CUDA error: cuTensorMapEncodeTiled failed with code %d", (int)r);
    return fail(buf);
  }
  memcpy(map_out, &m, sizeof m);
  return 0;
}

int spio_b200_status_address(void** address) {
  if (address == nullptr) return fail("address is NULL");
  const DeviceInfo* d = nullptr;
  if (device_info(&d)) return 1;
  *address = d->status;
  return 0;
}

int spio_conv2d_gw8_plan(int kind, const spio_gw8_shape* shape, const spio_gw8_tune* tune,
                         spio_gw8_plan_info* info) {
  if (info == nullptr) return fail("info is NULL");
  if (kind < SPIO_GW8_FPROP || kind > SPIO_GW8_WGRAD) return fail("unknown kind");
  const DeviceInfo* d = nullptr;
  if (device_info(&d)) return 1;
  Plan pl;
  if (make_plan(kind, shape, tune, d->sms, d->smem_optin, g_variants, &pl)) return 1;
  fill_info(pl, info);
  return 0;
}

int spio_conv2d_gw8_plan_for(int kind, const spio_gw8_shape* shape, const spio_gw8_tune* tune,
                             int sm_count, int smem_optin_bytes, spio_gw8_plan_info* info) {
  if (info == nullptr) return fail("info is NULL");
  if (kind < SPIO_GW8_FPROP || kind > SPIO_GW8_WGRAD) return fail("unknown kind");
  if (sm_count <= 0 || smem_optin_bytes <= 0) return fail("sm_count and smem_optin_bytes must be positive");
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    load_variants_locked();
  }
  Plan pl;
  if (make_plan(kind, shape, tune, sm_count, smem_optin_bytes, g_variants, &pl)) return 1;
  fill_info(pl, info);
  return 0;
}

int spio_conv2d_gw8_num_variants(void) {
  std::lock_guard<std::mutex> lock(g_mutex);
  load_variants_locked();
  return (int)g_variants.size();
}

int spio_conv2d_gw8_variant(int i, int* r, int* s, int* wpg, int* tpw, int* pps) {
  std::lock_guard<std::mutex> lock(g_mutex);
  load_variants_locked();
  if (i < 0 || i >= (int)g_variants.size()) return fail("variant index out of range");
  if (r) *r = g_variants[i].r;
  if (s) *s = g_variants[i].s;
  if (wpg) *wpg = g_variants[i].wpg;
  if (tpw) *tpw = g_variants[i].tpw;
  if (pps) *pps = g_variants[i].pps;
  return 0;
}

int spio_b200_device_status(int* status) {
  if (status == nullptr) return fail("status is NULL");
  const DeviceInfo* d = nullptr;
  if (device_info(&d)) return 1;
  GW8_CUDA(cudaDeviceSynchronize());
  GW8_CUDA(cudaMemcpy(status, d->status, sizeof(int), cudaMemcpyDeviceToHost));
  if (*status != 0) GW8_CUDA(cudaMemset(d->status, 0, sizeof(int)));
  return 0;
}

const char* spio_b200_last_error(void) { return g_last_error.c_str(); }

const char* spio_b200_version(void) { return "spio_b200 0.2 (sm_100a)"; }

}  // extern "C"
