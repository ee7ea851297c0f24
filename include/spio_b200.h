/* libspio_b200 -- C ABI of the B200 (sm_100a) group-width-8 convolution path.
 *
 * Every entry point takes plain pointers and sizes.  Device-pointer entry points
 * enqueue work on the given CUDA stream (a cudaStream_t passed as void*, NULL = the
 * legacy default stream) and return without synchronising.  All return 0 on success
 * and a non-zero code on failure; spio_b200_last_error() gives the message of the last
 * failure on the calling thread.
 *
 * Tensor layouts (the ones the reference's kernels take):
 *   activations and gradients  NHWC fp16            (torch channels_last of (N,C,H,W))
 *   weight                     [K][R][S][8] fp16    (torch channels_last of (K,8,R,S)), K == C
 *   bias                       [K] fp32 or NULL
 *   weight gradient            [K][R][S][8] fp32
 * Stride 1, dilation 1, 1 <= R,S <= 5, C a multiple of 8, P = H + 2*pad_h - R + 1,
 * Q = W + 2*pad_w - S + 1.  Device pointers must be 16-byte aligned.
 */
#ifndef SPIO_B200_H_
#define SPIO_B200_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Problem shape; mirrors spio.kernels.Conv2dGw8Params
 * (reference: spio/kernels/conv2d_gw8_params.py:10-44). */
typedef struct spio_gw8_shape {
  int n, c, h, w;     /* input batch, channels, height, width */
  int r, s;           /* filter height, width */
  int pad_h, pad_w;   /* zero padding */
} spio_gw8_shape;

/* Tile configuration; every zero field is chosen by the library.  Plays the role of
 * the reference's Conv2dGw8Config / Conv2dGw8WgradConfig
 * (spio/kernels/conv2d_gw8_kernel.py:30-36, conv2d_gw8_wgrad_kernel.py:27-35). */
typedef struct spio_gw8_tune {
  int wpg;   /* compute warps per channel group: 1, 2 or 3 */
  int tpw;   /* 8-pixel x 2-row tiles per warp */
  int ns;    /* shared-memory ring slots */
  int nob;   /* output staging buffers (fprop / dgrad) */
  int ncb;   /* 8-pixel column blocks per column tile */
  int nb;    /* images per ring slot */
  int grid;  /* CTAs; 0 = one per SM */
  int pps;   /* row pairs per ring slot: 1 or 2 (built-in variants), up to 4 just in time */
  int engine; /* 0 = the planner chooses; 1 = warp-level mma.sync kernels; 2 = tcgen05 kernel with the
                 accumulators in tensor memory (fprop and dgrad, filters up to 3 x 3; it ignores
                 wpg, tpw, nb and pps) */
} spio_gw8_tune;

/* What a launch will look like; filled by spio_conv2d_gw8_plan. */
typedef struct spio_gw8_plan_info {
  int wpg, tpw, ns, nob, ncb, nb, grid, threads;
  int pps, smem_bytes;
  int n_chunks, n_image_groups, n_col_tiles, n_pairs, n_split;
  int engine;           /* 1 or 2, see spio_gw8_tune */
  size_t scratch_bytes; /* wgrad only */
} spio_gw8_plan_info;

enum {
  SPIO_GW8_FPROP = 0,
  SPIO_GW8_DGRAD = 1,
  SPIO_GW8_WGRAD = 2
};

/* Forward: y = conv2d(x, w, groups = C/8) + bias.
 * Replaces the launch of the reference kernel spio_conv2d_gw8_fprop__<params>
 * (spio/src/conv2d_gw8.cu:10-12; launched by spio/kernels/kernel.py:135-154 from
 * spio/functional/conv2d_gw8_function.py:59-62). */
int spio_conv2d_gw8_fprop(void* y, const void* x, const void* w, const float* bias,
                          const spio_gw8_shape* shape, const spio_gw8_tune* tune, void* stream);

/* Input gradient: dx = conv2d_transpose(dy, w).  dy is (N,P,Q,K), dx is (N,H,W,C).
 * Replaces spio_conv2d_gw8_dgrad__<params> (spio/src/conv2d_gw8.cu:10-12 with
 * Mode::igrad, :99-105; called at spio/functional/conv2d_gw8_function.py:140-144). */
int spio_conv2d_gw8_dgrad(void* dx, const void* dy, const void* w,
                          const spio_gw8_shape* shape, const spio_gw8_tune* tune, void* stream);

/* Bytes of device scratch spio_conv2d_gw8_wgrad needs for this shape and tuning. */
size_t spio_conv2d_gw8_wgrad_scratch_bytes(const spio_gw8_shape* shape,
                                           const spio_gw8_tune* tune);

/* Weight gradient: dw = sum over pixels of x (shifted) * dy, fp32.  dw is overwritten
 * (it need not be zeroed first) and the summation order is fixed.  `scratch` is device
 * memory of at least spio_conv2d_gw8_wgrad_scratch_bytes(); its contents on entry do
 * not matter.  Replaces spio_conv2d_gw8_wgrad__<params>
 * (spio/src/conv2d_gw8_wgrad.cu:10-12) together with the zero fill that precedes it
 * (spio/functional/conv2d_gw8_function.py:125-130). */
int spio_conv2d_gw8_wgrad(float* dw, const void* x, const void* dy,
                          const spio_gw8_shape* shape, const spio_gw8_tune* tune,
                          void* scratch, size_t scratch_bytes, void* stream);

/* All gradients of one layer in one call (dx or dw may be NULL to skip it).  dbias, if not
 * NULL, receives the gradient of the bias, sum over n, h, w of dy (fp32, c values, 16-byte
 * aligned): for filters with an odd number of taps the weight-gradient kernel computes it in
 * the unused half of its last MMA, which replaces the separate reduction over dy of the
 * reference (spio/functional/conv2d_gw8_function.py:136); for an even number of taps dbias
 * must be NULL.  Launches the
 * weight-gradient kernel, its reduce kernel and the input-gradient kernel back to back with
 * programmatic dependent launch: the input-gradient kernel shares no output with the other
 * two, so its CTAs take over SMs as theirs finish instead of waiting for the whole grid to
 * drain; dw is complete first, and `dw_ready` (a cudaEvent_t, or NULL) is recorded at that
 * point, so a data-parallel caller can make its communication stream wait for the event and
 * all-reduce dw while the input gradient is still being computed.  Replaces the two launches of the reference's
 * backward operator (spio/functional/conv2d_gw8_function.py:93-147). */
int spio_conv2d_gw8_backward(void* dx, float* dw, float* dbias, const void* x, const void* dy, const void* w,
                             const spio_gw8_shape* shape, const spio_gw8_tune* dgrad_tune,
                             const spio_gw8_tune* wgrad_tune, void* scratch, size_t scratch_bytes,
                             void* stream, void* dw_ready);

/* spio_conv2d_gw8_backward with options (NULL = none).
 *   dw_f16: dw points to fp16 [K][R][S][8] and receives the fp32 sums rounded once -- the
 *     parameter's own type, which saves the cast autograd would otherwise launch after the
 *     reference's fp32 grad_weight (spio/functional/conv2d_gw8_function.py:127).
 *   *_function: CUfunction handles of kernels compiled just in time for the given tunes
 *     (see the just-in-time section below); NULL = the variant built into the library.  They are
 *     launched with cuLaunchKernelEx and the same programmatic-dependent-launch attribute, so a
 *     just-in-time kernel takes part in the chain like a built-in one.  With dbias the
 *     weight-gradient kernel must be the instantiation that also sums dy
 *     (wgrad_dbias_function).
 *   dp: after the reduce step one small kernel (spio_dp_allreduce) stores this rank's dw (and
 *     dbias) into every rank's exchange buffer and overwrites them with the sum over the ranks,
 *     added in rank order (bit-identical on all ranks), while the input-gradient kernel runs
 *     beside it.  dw must be fp32.  `dw_ready`, if given, is then recorded after the
 *     input-gradient kernel, whose completion implies that of the sum.  The input-gradient kernel
 *     is launched on as many SMs fewer as the exchange has CTAs (one per 512 floats), unless
 *     dgrad_tune names a grid: its CTAs cannot start on an SM where an exchange CTA is waiting. */
struct spio_dp_exchange;
typedef struct spio_gw8_backward_opts {
  int dw_f16;
  void* wgrad_function;
  void* wgrad_dbias_function;
  void* dgrad_function;
  const struct spio_dp_exchange* dp; /* data-parallel sum of dw (and dbias) over the GPUs of the
                                        node, see below; NULL = single GPU */
} spio_gw8_backward_opts;
int spio_conv2d_gw8_backward_ex(void* dx, void* dw, float* dbias, const void* x, const void* dy, const void* w,
                                const spio_gw8_shape* shape, const spio_gw8_tune* dgrad_tune,
                                const spio_gw8_tune* wgrad_tune, void* scratch, size_t scratch_bytes,
                                void* stream, void* dw_ready, const spio_gw8_backward_opts* opts);

/* ---- data-parallel sum of the weight gradient ----------------------------------------
 * The path shards by batch (one process per GPU); its only exchange is the sum of the per-rank
 * weight (and bias) gradients, a few thousand floats.  Instead of a host-issued all-reduce the
 * sum runs inside the step's chain of dependent launches: every thread of spio_dp_allreduce owns
 * four floats of the vector [a | b]; it stores them, each paired with a tag that names the
 * exchange, into slot [rank] of EVERY rank's exchange buffer (plain 16-byte peer stores over
 * NVLink), then polls the same four floats of all ranks' slots in its own buffer until the tags
 * match (bounded: SPIO_STATUS_PEER_TIMEOUT), adds them in rank order and overwrites its floats.
 * Data and tag travel in one 8-byte word, so there are no flags, fences or atomics, and all ranks
 * get bit-identical sums.  Remote data always lands in local memory before it is used; nothing
 * loads from a peer, and no TMA or multicast touches peer memory.  The reference has no
 * multi-device support (its kernel cache is merely keyed by device ordinal,
 * spio/kernels/kernel_key.py:13-18); a trainer would otherwise call torch.distributed.all_reduce
 * on grad_weight after spio/functional/conv2d_gw8_function.py:147.  spio_dp_push and spio_dp_sum
 * are the two halves as separate launches (for tests that emulate several ranks on one GPU).
 *
 * Set-up, once: every rank allocates a buffer of spio_dp_buffer_bytes(world, capacity) with
 * spio_dp_buffer_alloc (zero-filled; returns a 64-byte CUDA IPC handle), the ranks exchange the
 * handles by any means (torch.distributed.all_gather_object, say) and open each other's with
 * spio_dp_buffer_open.  `buffers[r]` is rank r's buffer as mapped in THIS process
 * (buffers[rank] = the local one).  `seq` counts exchanges, starts at 0, is the same on all
 * ranks and is incremented by the caller after every push + sum pair; every rank must take part
 * in every exchange.  n_a and n_b are multiples of 4 floats, n_a + n_b <= capacity. */
enum { SPIO_DP_MAX_WORLD = 16, SPIO_DP_IPC_HANDLE_BYTES = 64 };
typedef struct spio_dp_exchange {
  void* const* buffers;
  int rank, world;
  unsigned seq;
  size_t capacity; /* floats per slot */
} spio_dp_exchange;
size_t spio_dp_buffer_bytes(int world, size_t capacity);
int spio_dp_buffer_alloc(size_t bytes, void** buffer, void* ipc_handle /* 64 bytes out, or NULL */);
int spio_dp_buffer_open(const void* ipc_handle, void** peer_buffer);
int spio_dp_buffer_close(void* peer_buffer);
int spio_dp_buffer_free(void* buffer);
int spio_dp_push(const spio_dp_exchange* dp, const float* a, size_t n_a, const float* b, size_t n_b, void* stream);
int spio_dp_sum(const spio_dp_exchange* dp, float* a, size_t n_a, float* b, size_t n_b, void* stream);
/* Both halves in ONE kernel, which is what the combined backward call launches. */
int spio_dp_allreduce(const spio_dp_exchange* dp, float* a, size_t n_a, float* b, size_t n_b, void* stream);

/* Weight gradient for callers that must not allocate device memory.  It has no counterpart
 * in the reference.  Some callers cannot call cudaMalloc at the point where they need the
 * gradient: code running inside another framework's memory pool with a fixed budget, a
 * real-time loop that may not block on the allocator, a plugin that is handed tensors but no
 * allocator.  This variant does the same computation as spio_conv2d_gw8_wgrad but takes its
 * scratch from a 4 MiB buffer built into the library image (each GPU that loads the library
 * holds those 4 MiB until the process exits), so the caller passes only inputs and output.
 *  - It calls no cudaMalloc / cudaFree and no allocating library routine.
 *  - Shapes whose plan needs more than 4 MiB of scratch (3x3 filters on a 148-SM part need
 *    2.6 MiB; 5x5 filters spread over all SMs need more) are rejected with an error; use
 *    spio_conv2d_gw8_wgrad with your own scratch for those, or a smaller `tune->grid`.
 *  - The first call on a device looks up the buffer's device address and sets kernel
 *    attributes; make that first call before starting any stream capture.
 *  - All calls share the one buffer.  Nothing in it has to be cleared (every part the reduce
 *    step reads is overwritten first), but two calls that overlap on the GPU -- different
 *    streams, or different host threads -- race on it; run them in stream order. */
int spio_conv2d_gw8_wgrad_static(float* dw, const void* x, const void* dy,
                                 const spio_gw8_shape* shape, const spio_gw8_tune* tune,
                                 void* stream);

/* Host-buffer variants: copy the operands to the device, run, copy the result back and
 * wait for it.  Device staging buffers are owned by the library and grow on demand.
 * Pinned host memory makes the copies asynchronous; pageable memory also works. */
int spio_conv2d_gw8_fprop_host(void* y, const void* x, const void* w, const float* bias,
                               const spio_gw8_shape* shape, const spio_gw8_tune* tune);
int spio_conv2d_gw8_dgrad_host(void* dx, const void* dy, const void* w,
                               const spio_gw8_shape* shape, const spio_gw8_tune* tune);
int spio_conv2d_gw8_wgrad_host(float* dw, const void* x, const void* dy,
                               const spio_gw8_shape* shape, const spio_gw8_tune* tune);

/* One training step of a layer on host buffers: y = fprop(x, w, bias), dx = dgrad(dy, w),
 * dw = wgrad(x, dy) and, if dbias is not NULL (odd number of taps only), dbias.  x and dy are
 * uploaded once, in 4 to 32 pieces of the batch (16 MB of x or more each); fprop and dgrad of a piece run while the next piece
 * uploads and the previous one's y and dx download, so the call costs about one upload of x and
 * dy instead of the four uploads and two downloads of the three separate calls.  Pinned host
 * memory is needed for the copies to overlap.  Returns after all results are in host memory. */
int spio_conv2d_gw8_step_host(void* y, void* dx, float* dw, float* dbias, const void* x, const void* dy,
                              const void* w, const float* bias, const spio_gw8_shape* shape);
/* The same step of a data-parallel rank: after the weight gradient over the rank's images, dw
 * (and dbias) are summed over the ranks on the device (spio_dp_push / spio_dp_sum, declared
 * below) before they are copied back, so every rank returns the gradient of the global batch.
 * dp = NULL is spio_conv2d_gw8_step_host. */
struct spio_dp_exchange;
int spio_conv2d_gw8_step_host_dp(void* y, void* dx, float* dw, float* dbias, const void* x, const void* dy,
                                 const void* w, const float* bias, const spio_gw8_shape* shape,
                                 const struct spio_dp_exchange* dp);

/* Reports the launch the library would make; kind is SPIO_GW8_FPROP/DGRAD/WGRAD.
 * Needs a CUDA device (it reads the SM count and the shared-memory limit). */
int spio_conv2d_gw8_plan(int kind, const spio_gw8_shape* shape, const spio_gw8_tune* tune,
                         spio_gw8_plan_info* info);

/* The same plan for a device with the given SM count and opt-in shared-memory limit;
 * touches no device, so it also works on a machine without a GPU. */
int spio_conv2d_gw8_plan_for(int kind, const spio_gw8_shape* shape, const spio_gw8_tune* tune,
                             int sm_count, int smem_optin_bytes, spio_gw8_plan_info* info);

/* ---- just-in-time path --------------------------------------------------------------
 * NVRTC compilation and driver-API module load / launch, for kernels specialised per layer
 * shape and for tile configurations that are not compiled into the library.  Replaces the
 * reference's spio/cuda/nvrtc_ctypes.py:152-217 and spio/compiler/compile.py:22-77 (compile)
 * and spio/cuda/driver.pyx:126-273 (Module, Function.launch). */
int spio_jit_set_nvrtc_path(const char* path);           /* where libnvrtc.so.12 lives */
int spio_jit_nvrtc_version(int* major, int* minor);
/* Compiles `source` (options as for nvrtcCompileProgram, e.g. "-arch=sm_100a"; headers are
 * given in memory).  On success *cubin / *cubin_size hold the image; *log (if not NULL)
 * receives the compiler log, which contains the register / spill report when
 * "--ptxas-options=-v" is among the options.  Free both with spio_jit_free. */
int spio_jit_compile(const char* source, const char* file_name, const char* const* options, int n_options,
                     const char* const* header_names, const char* const* header_sources, int n_headers,
                     void** cubin, size_t* cubin_size, char** log);
void spio_jit_free(void* p);
int spio_module_load(const void* cubin, void** module);
int spio_module_unload(void* module);
int spio_module_get_function(void* module, const char* name, void** function);
int spio_function_set_max_dynamic_smem(void* function, int bytes);
/* which: 0 registers per thread, 1 local (spill) bytes, 2 static shared bytes, 3 max threads */
int spio_function_get_attribute(void* function, int which, int* value);
/* args: one pointer per kernel parameter, as for cuLaunchKernel */
int spio_function_launch(void* function, int grid, int block, int smem_bytes, void* stream, void** args);
/* The same through cuLaunchKernelEx.  SPIO_LAUNCH_PROGRAMMATIC adds the programmatic-stream-
 * serialization attribute: the kernel may become resident while its predecessor in the stream
 * drains, so it MUST execute griddepcontrol.wait before it touches memory that predecessor
 * writes (every gw8 kernel of this library does). */
enum { SPIO_LAUNCH_PROGRAMMATIC = 1 };
int spio_function_launch_ex(void* function, int grid, int block, int smem_bytes, void* stream, void** args,
                            int flags);

/* Launch of a gw8 kernel compiled just in time (`function`, a CUfunction from
 * spio_module_get_function) for tune->wpg, tpw, pps (or tune->engine = 2): planning, tensor maps,
 * the dynamic-tail counters and programmatic dependent launch are handled exactly as for the
 * built-in variants, and the weight-gradient call is followed by the library's reduce kernel.
 * These replace Kernel.launch -> Function.launch of the reference for its NVRTC-compiled kernels
 * (spio/kernels/kernel.py:135-154, spio/cuda/driver.pyx:171-208). */
int spio_conv2d_gw8_fprop_jit(void* function, void* y, const void* x, const void* w, const float* bias,
                              const spio_gw8_shape* shape, const spio_gw8_tune* tune, void* stream);
int spio_conv2d_gw8_dgrad_jit(void* function, void* dx, const void* dy, const void* w,
                              const spio_gw8_shape* shape, const spio_gw8_tune* tune, void* stream);
int spio_conv2d_gw8_wgrad_jit(void* function, float* dw, const void* x, const void* dy,
                              const spio_gw8_shape* shape, const spio_gw8_tune* tune, void* scratch,
                              size_t scratch_bytes, void* stream);
size_t spio_conv2d_gw8_wgrad_scratch_bytes_jit(const spio_gw8_shape* shape, const spio_gw8_tune* tune);

/* Encodes a tiled TMA tensor map (128 bytes, passed to a kernel by value as a
 * `const __grid_constant__` parameter) for kernels written against the package's typed headers
 * (spio_b200/csrc/typed_tma.cuh, generated by spio_b200.generators.TensorMapSpec).  Axes are given
 * innermost first; strides_bytes has rank - 1 entries (axis 0 is contiguous); swizzle is 0 (none),
 * 1 (32 B), 2 (64 B) or 3 (128 B).  Needs a CUDA device.  The reference's kernels take plain
 * pointers (spio/cuda/driver.pyx:182-188); tensor maps are what the typed-dimension layer gains for
 * sm_100a. */
int spio_tensor_map_encode(void* map_out, const void* base, int elem_bytes, int rank,
                           const unsigned long long* sizes, const unsigned long long* strides_bytes,
                           const unsigned* box, int swizzle);

/* Everything a just-in-time compiled gw8 kernel needs for one launch: the two tensor maps
 * and the geometry it takes by value, the launch dimensions and the status word.  Kernel
 * parameter lists:
 *   fprop / dgrad: (in_map, out_map, geom, const half* w, const float* bias, int ns, int nob, int* status)
 *   fprop / dgrad, engine 2 (tcgen05 kernel, conv2d_gw8_fwd_tc_body<Gw8TcConfig<R, S>>):
 *                  (in_map, row_map, out_map, geom, const half* w, const float* bias, int ns, int nob, int* status)
 *   wgrad:         (in_map, out_map, geom, float* scratch, int ns, int* status), followed by
 *                  spio_conv2d_gw8_wgrad_reduce(dw, dbias or NULL, scratch, c, r*s, n_parts, stream). */
typedef struct spio_gw8_launch {
  unsigned long long in_map[16];   /* CUtensorMap of the streamed operand (x; dy for dgrad) */
  unsigned long long out_map[16];  /* CUtensorMap of the tiled operand (y; dx; dy for wgrad) */
  unsigned long long row_map[16];  /* engine 2 only: the streamed operand with a box of one row */
  int geom[40];                    /* kernel-side geometry struct, opaque */
  int ns, nob, grid, threads, smem_bytes, n_parts;
  size_t scratch_bytes;
  int* status;
} spio_gw8_launch;
/* tune->wpg, tpw, pps must be given (or tune->engine = 2); they need not be a compiled variant.  plan_jit is the
 * host-only planner for such a configuration (cf. spio_conv2d_gw8_plan_for).  prepare_launch serves callers that
 * launch the function themselves (spio_function_launch); such a launch splits its work statically (no dynamic
 * tail), because the counters of the dynamic tail are handed out per stream by the library's own launches. */
int spio_conv2d_gw8_plan_jit(int kind, const spio_gw8_shape* shape, const spio_gw8_tune* tune, int sm_count,
                             int smem_optin_bytes, spio_gw8_plan_info* info);
int spio_conv2d_gw8_prepare_launch(int kind, const spio_gw8_shape* shape, const spio_gw8_tune* tune,
                                   const void* streamed, const void* tiled, spio_gw8_launch* out);
int spio_conv2d_gw8_wgrad_reduce(float* dw, float* dbias, const float* scratch, int c, int taps, int n_parts,
                                 void* stream);

/* ---- LayerNorm2d ---------------------------------------------------------------------
 * LayerNorm over the channels of an NHWC fp16 tensor, the op that follows the gw8 convolution
 * in a ConvNeXt block.  rows = n * h * w pixels of c channels (c a multiple of 8, at most 1024);
 * weight / bias are fp32 [c] or NULL; statistics are fp32.  The forward pass covers the
 * reference's kernel spio/src/layernorm_2d.cu:82-221 (which the reference ships but wires to no
 * operator); the backward pass has no counterpart there.
 *   fwd: y = (x - mean) * rstd * weight + bias; stats[row] = {mean, rstd} if stats != NULL.
 *   bwd: dx from dy, x, stats and weight; dweight / dbias (fp32 [c], may be NULL) are summed
 *        over all pixels through `scratch` (spio_layernorm_2d_bwd_scratch_bytes) in a fixed order. */
int spio_layernorm_2d_fwd(void* y, float* stats, const void* x, const float* weight, const float* bias,
                          long long rows, int c, float eps, void* stream);
size_t spio_layernorm_2d_bwd_scratch_bytes(long long rows, int c);
int spio_layernorm_2d_bwd(void* dx, float* dweight, float* dbias, const void* dy, const void* x,
                          const float* stats, const float* weight, long long rows, int c, void* scratch,
                          size_t scratch_bytes, void* stream);

/* Number of compiled (r, s, wpg, tpw, pps) variants, and the i-th one. */
int spio_conv2d_gw8_num_variants(void);
int spio_conv2d_gw8_variant(int i, int* r, int* s, int* wpg, int* tpw, int* pps);

/* Kernels record a bounded wait that gave up in a per-device status word
 * (SPIO_STATUS_WAIT_TIMEOUT: an mbarrier wait inside a convolution kernel;
 * SPIO_STATUS_PEER_TIMEOUT: the data-parallel exchange waited in vain for a peer).  This call
 * synchronises the current device, returns the word through *status (0 = ok) and clears
 * it.  Corresponds to the reference's error path in spio/cuda/driver.pyx:118-123. */
enum { SPIO_STATUS_OK = 0, SPIO_STATUS_WAIT_TIMEOUT = 1, SPIO_STATUS_PEER_TIMEOUT = 2 };
int spio_b200_device_status(int* status);
/* Device address of that word on the current device (an int), for kernels written against
 * the package's headers, whose last parameter it is. */
int spio_b200_status_address(void** address);

/* Message of the last failure on this thread ("" if none). */
const char* spio_b200_last_error(void);

/* Library version string. */
const char* spio_b200_version(void);

#ifdef __cplusplus
}
#endif

#endif /* SPIO_B200_H_ */
