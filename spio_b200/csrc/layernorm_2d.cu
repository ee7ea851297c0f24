// LayerNorm over the channel dimension of an NHWC fp16 tensor ("LayerNorm2d"), forward and
// backward.  The op that follows every gw8 convolution in a ConvNeXt block.
//
//   y[p][c]  = (x[p][c] - mean_p) * rstd_p * weight[c] + bias[c]          p = (n, h, w)
//   dx[p][c] = rstd_p * (g[p][c] - mean_c(g[p]) - xhat[p][c] * mean_c(g[p] * xhat[p])),  g = dy * weight
//   dweight[c] = sum_p dy[p][c] * xhat[p][c],  dbias[c] = sum_p dy[p][c]
//
// HBM-bound: one pass over x (and dy) with 16-byte accesses.  A pixel is handled by a group
// of T lanes (T = 4, 8, 16 or 32, chosen so that each lane owns at most 4 pieces of 8
// channels); all statistics are fp32 and reduced by xor shuffles inside the group; weight and
// bias live in shared memory.  The backward kernel keeps
// the per-channel sums of a thread in registers, combines the groups of a warp by shuffles and
// the warps of a CTA through shared memory, and writes one partial per CTA; a second kernel
// adds the partials in a fixed order (no atomics, bit-reproducible).
//
// The forward pass covers what the reference's spio/src/layernorm_2d.cu:82-221 computes (a
// kernel the reference ships but does not wire to an operator); the backward pass has no
// counterpart there.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <string>

#include "ptx.cuh"
#include "../../include/spio_b200.h"

namespace spio_b200 {

int jit_fail(const std::string& msg);  // sets the thread's last-error text, returns 1

namespace {

constexpr int kLnThreads = 256;
constexpr int kMaxPieces = 4;  // 16-byte pieces of a pixel per lane
constexpr int kMaxChannels = 32 * kMaxPieces * 8;

__device__ __forceinline__ float group_sum(float v, int t) {
  for (int d = t >> 1; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
  return v;
}

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __half22float2(h[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}

__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  __half2* h = reinterpret_cast<__half2*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
  return u;
}

// The 16-byte pieces of one pixel row that this lane owns (zeros where the pixel or the piece is out of range).
template <int K>
__device__ __forceinline__ void fetch_pieces(uint4 (&u)[K], const uint4* __restrict__ p, long long row,
                                             long long rows, int lane_in_group, int t, int pieces) {
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int piece = lane_in_group + k * t;
    u[k] = make_uint4(0u, 0u, 0u, 0u);
    if (row < rows && piece < pieces) u[k] = __ldcs(p + row * pieces + piece);
  }
}

// dst[0 .. c) = src, or `fill` when src is NULL (all threads of the CTA; the caller synchronises).
__device__ __forceinline__ void stage_vector(float* __restrict__ dst, const float* __restrict__ src, int c, float fill) {
  for (int i = threadIdx.x; i < c; i += kLnThreads) dst[i] = src != nullptr ? __ldg(src + i) : fill;
}

__device__ __forceinline__ void read8(float (&f)[8], const float* __restrict__ sm, int piece) {
  const float4 a = reinterpret_cast<const float4*>(sm)[2 * piece];
  const float4 b = reinterpret_cast<const float4*>(sm)[2 * piece + 1];
  f[0] = a.x, f[1] = a.y, f[2] = a.z, f[3] = a.w, f[4] = b.x, f[5] = b.y, f[6] = b.z, f[7] = b.w;
}

// K = pieces per lane, t = lanes per pixel (power of two), pieces = c / 8.
//
// The kernel is a stream: what limits it is the number of bytes each SM keeps in flight.  Weight and bias
// therefore sit in shared memory, not in 16 * K registers per thread (three CTAs per SM instead of two),
// and the pieces of a warp's NEXT pixels are requested before the current ones are worked on.
template <int K>
__global__ void __launch_bounds__(kLnThreads, 3)
layernorm_2d_fwd_kernel(uint4* __restrict__ y, float2* __restrict__ stats, const uint4* __restrict__ x,
                        const float* __restrict__ weight, const float* __restrict__ bias, long long rows,
                        int pieces, int t, float inv_c, float eps) {
  __shared__ __align__(16) float sw[kMaxChannels], sb[kMaxChannels];
  grid_dependency_wait();
  grid_dependency_launch_dependents();
  stage_vector(sw, weight, pieces * 8, 1.f);
  stage_vector(sb, bias, pieces * 8, 0.f);
  __syncthreads();
  const int lane_in_group = threadIdx.x & (t - 1);
  // All lanes of a warp run the same number of iterations (the shuffles below name every
  // lane); a group whose pixel lies past the end works on zeros and stores nothing.
  const int groups_per_warp = 32 / t;
  const long long warp_first = (((long long)blockIdx.x * kLnThreads + threadIdx.x) >> 5) * groups_per_warp;
  const long long warp_step = (long long)gridDim.x * (kLnThreads / 32) * groups_per_warp;
  const int group_in_warp = (threadIdx.x & 31) / t;

  uint4 nxt[K];
  fetch_pieces<K>(nxt, x, warp_first + group_in_warp, rows, lane_in_group, t, pieces);
  for (long long base = warp_first; base < rows; base += warp_step) {
    const long long row = base + group_in_warp;
    const bool valid = row < rows;
    float v[K][8];
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      unpack8(nxt[k], v[k]);
#pragma unroll
      for (int i = 0; i < 8; ++i) sum += v[k][i];
    }
    fetch_pieces<K>(nxt, x, row + warp_step, rows, lane_in_group, t, pieces);
    const float mean = group_sum(sum, t) * inv_c;
    float sq = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      if (lane_in_group + k * t < pieces) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float d = v[k][i] - mean;
          sq += d * d;
        }
      }
    }
    const float rstd = rsqrtf(group_sum(sq, t) * inv_c + eps);
    if (stats != nullptr && valid && lane_in_group == 0) stats[row] = make_float2(mean, rstd);
    uint4* yr = y + row * pieces;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int piece = lane_in_group + k * t;
      if (valid && piece < pieces) {
        float o[8], w[8], b[8];
        read8(w, sw, piece);
        read8(b, sb, piece);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = (v[k][i] - mean) * rstd * w[i] + b[i];
        yr[piece] = pack8(o);
      }
    }
  }
}

// Partials: part[cta][0][c] = sum of dy * xhat, part[cta][1][c] = sum of dy over the CTA's pixels.
// The weight sits in shared memory, as in the forward kernel; the per-channel sums stay in registers.
template <int K>
__global__ void __launch_bounds__(kLnThreads, 2)
layernorm_2d_bwd_kernel(uint4* __restrict__ dx, float* __restrict__ part, const uint4* __restrict__ dy,
                        const uint4* __restrict__ x, const float2* __restrict__ stats,
                        const float* __restrict__ weight, long long rows, int pieces, int t, float inv_c) {
  extern __shared__ float red[];  // [warps][2][c]
  __shared__ __align__(16) float sw[kMaxChannels];
  grid_dependency_wait();
  grid_dependency_launch_dependents();
  const int c = pieces * 8;
  stage_vector(sw, weight, c, 1.f);
  __syncthreads();
  const int lane_in_group = threadIdx.x & (t - 1);
  // as in the forward kernel: uniform trip count per warp, out-of-range groups work on zeros
  const int groups_per_warp = 32 / t;
  const long long warp_first = (((long long)blockIdx.x * kLnThreads + threadIdx.x) >> 5) * groups_per_warp;
  const long long warp_step = (long long)gridDim.x * (kLnThreads / 32) * groups_per_warp;
  const int group_in_warp = (threadIdx.x & 31) / t;

  float gw[K][8], gb[K][8];
#pragma unroll
  for (int k = 0; k < K; ++k)
#pragma unroll
    for (int i = 0; i < 8; ++i) gw[k][i] = gb[k][i] = 0.f;

  // the operands stay packed (fp16) between the two passes to keep the register count low
  uint4 nx[K], nd[K];
  float2 nst = make_float2(0.f, 0.f);
  {
    const long long row = warp_first + group_in_warp;
    fetch_pieces<K>(nx, x, row, rows, lane_in_group, t, pieces);
    fetch_pieces<K>(nd, dy, row, rows, lane_in_group, t, pieces);
    if (row < rows) nst = stats[row];
  }
  for (long long base = warp_first; base < rows; base += warp_step) {
    const long long row = base + group_in_warp;
    const bool valid = row < rows;
    const float2 st = nst;
    uint4 ux[K], ud[K];
#pragma unroll
    for (int k = 0; k < K; ++k) ux[k] = nx[k], ud[k] = nd[k];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int piece = lane_in_group + k * t;
      const bool on = valid && piece < pieces;
      float xv[8], dv[8], w[8];
      unpack8(ux[k], xv);
      unpack8(ud[k], dv);
      read8(w, sw, on ? piece : 0);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float xh = on ? (xv[i] - st.x) * st.y : 0.f;
        const float g = dv[i] * w[i];
        s1 += g;
        s2 += g * xh;
        gw[k][i] += dv[i] * xh;
        gb[k][i] += dv[i];
      }
    }
    s1 = group_sum(s1, t) * inv_c;
    s2 = group_sum(s2, t) * inv_c;
    uint4* or_ = dx + row * pieces;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int piece = lane_in_group + k * t;
      if (valid && piece < pieces) {
        float xv[8], dv[8], w[8], o[8];
        unpack8(ux[k], xv);
        unpack8(ud[k], dv);
        read8(w, sw, piece);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float xh = (xv[i] - st.x) * st.y;
          o[i] = st.y * (dv[i] * w[i] - s1 - xh * s2);
        }
        or_[piece] = pack8(o);
      }
    }
    // (requesting the next pixels before working on these ones, as the forward kernel does, made this
    // kernel spill and cost 15 % at 96 channels: the per-channel sums already fill the registers)
    fetch_pieces<K>(nx, x, row + warp_step, rows, lane_in_group, t, pieces);
    fetch_pieces<K>(nd, dy, row + warp_step, rows, lane_in_group, t, pieces);
    nst = row + warp_step < rows ? stats[row + warp_step] : make_float2(0.f, 0.f);
  }

  // groups of a warp own the same channels: add them (lane bits t .. 16), then the warps
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int k = 0; k < K; ++k)
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      for (int d = t; d < 32; d <<= 1) {
        gw[k][i] += __shfl_xor_sync(0xffffffffu, gw[k][i], d);
        gb[k][i] += __shfl_xor_sync(0xffffffffu, gb[k][i], d);
      }
    }
  if (lane < t) {
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int piece = lane + k * t;
      if (piece < pieces) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          red[(warp * 2 + 0) * c + piece * 8 + i] = gw[k][i];
          red[(warp * 2 + 1) * c + piece * 8 + i] = gb[k][i];
        }
      }
    }
  }
  __syncthreads();
  constexpr int kWarps = kLnThreads / 32;
  for (int e = threadIdx.x; e < 2 * c; e += kLnThreads) {
    float s = 0.f;
#pragma unroll
    for (int wv = 0; wv < kWarps; ++wv) s += red[wv * 2 * c + e];
    part[(size_t)blockIdx.x * 2 * c + e] = s;
  }
}

// dweight[c] / dbias[c] = sum over CTAs of the partials, in a fixed order: one warp per output
// value, lane l adds the partials l, l + 32, ... and the 32 lane sums are combined by a shuffle tree.
// (One thread per value walking all ~600 partials one after the other took 45 us, a third of the
// backward pass of a 96-channel layer.)
__global__ void __launch_bounds__(256)
layernorm_2d_bwd_reduce_kernel(float* __restrict__ dweight, float* __restrict__ dbias,
                               const float* __restrict__ part, int c, int n_parts) {
  grid_dependency_launch_dependents();
  grid_dependency_wait();
  const int e = (blockIdx.x * 256 + threadIdx.x) >> 5;  // the same for all lanes of a warp
  const int lane = threadIdx.x & 31;
  if (e >= 2 * c) return;
  float s = 0.f;
#pragma unroll 4
  for (int p = lane; p < n_parts; p += 32) s += __ldcg(part + (size_t)p * 2 * c + e);
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
  if (lane != 0) return;
  if (e < c) {
    if (dweight != nullptr) dweight[e] = s;
  } else if (dbias != nullptr) {
    dbias[e - c] = s;
  }
}

struct LnPlan {
  int pieces, t, k, grid;
};

int ln_plan(long long rows, int c, int ctas_per_sm, LnPlan* p) {
  if (rows <= 0) return jit_fail("rows must be positive");
  if (c <= 0 || c % 8 != 0) return jit_fail("Number of channels must be a multiple of 8.");
  p->pieces = c / 8;
  int t = 4;
  while (t < 32 && (p->pieces + t - 1) / t > kMaxPieces) t <<= 1;
  p->t = t;
  p->k = (p->pieces + t - 1) / t;
  if (p->k > kMaxPieces) return jit_fail("LayerNorm2d supports at most 1024 channels");
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return jit_fail("CUDA error: no device");
  const long long groups_per_cta = kLnThreads / t;
  long long want = (rows + groups_per_cta - 1) / groups_per_cta;
  const long long cap = (long long)sms * ctas_per_sm;  // one wave of resident CTAs, each a grid-stride loop
  p->grid = (int)(want < cap ? want : cap);
  return 0;
}

int ln_launch(const void* func, int grid, size_t smem, cudaStream_t stream, void** args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kLnThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelExC(&cfg, func, args);
  if (e != cudaSuccess) return jit_fail(std::string("CUDA error: ") + cudaGetErrorString(e));
  return 0;
}

}  // namespace

}  // namespace spio_b200

using namespace spio_b200;

extern "C" {

int spio_layernorm_2d_fwd(void* y, float* stats, const void* x, const float* weight, const float* bias,
                          long long rows, int c, float eps, void* stream) {
  if (y == nullptr || x == nullptr) return jit_fail("NULL tensor pointer");
  if (((reinterpret_cast<size_t>(y) | reinterpret_cast<size_t>(x)) & 15u) != 0)
    return jit_fail("tensor pointers must be 16-byte aligned");
  if ((reinterpret_cast<size_t>(stats) & 7u) != 0) return jit_fail("stats must be 8-byte aligned");
  LnPlan p;
  if (ln_plan(rows, c, 3, &p)) return 1;
  const void* fn[4] = {(const void*)&layernorm_2d_fwd_kernel<1>, (const void*)&layernorm_2d_fwd_kernel<2>,
                       (const void*)&layernorm_2d_fwd_kernel<3>, (const void*)&layernorm_2d_fwd_kernel<4>};
  float inv_c = 1.f / (float)c;
  void* args[] = {&y, &stats, (void*)&x, (void*)&weight, (void*)&bias, &rows, &p.pieces, &p.t, &inv_c, &eps};
  return ln_launch(fn[p.k - 1], p.grid, 0, (cudaStream_t)stream, args);
}

size_t spio_layernorm_2d_bwd_scratch_bytes(long long rows, int c) {
  LnPlan p;
  if (ln_plan(rows, c, 2, &p)) return 0;
  return (size_t)p.grid * 2 * c * sizeof(float);
}

int spio_layernorm_2d_bwd(void* dx, float* dweight, float* dbias, const void* dy, const void* x,
                          const float* stats, const float* weight, long long rows, int c, void* scratch,
                          size_t scratch_bytes, void* stream) {
  if (dx == nullptr || dy == nullptr || x == nullptr || stats == nullptr) return jit_fail("NULL tensor pointer");
  if (((reinterpret_cast<size_t>(dx) | reinterpret_cast<size_t>(dy) | reinterpret_cast<size_t>(x)) & 15u) != 0)
    return jit_fail("tensor pointers must be 16-byte aligned");
  LnPlan p;
  if (ln_plan(rows, c, 2, &p)) return 1;
  const size_t need = (size_t)p.grid * 2 * c * sizeof(float);
  if (scratch == nullptr || scratch_bytes < need) return jit_fail("LayerNorm2d scratch buffer is too small");
  const void* fn[4] = {(const void*)&layernorm_2d_bwd_kernel<1>, (const void*)&layernorm_2d_bwd_kernel<2>,
                       (const void*)&layernorm_2d_bwd_kernel<3>, (const void*)&layernorm_2d_bwd_kernel<4>};
  float* part = static_cast<float*>(scratch);
  float inv_c = 1.f / (float)c;
  void* args[] = {&dx, &part, (void*)&dy, (void*)&x, (void*)&stats, (void*)&weight, &rows, &p.pieces, &p.t, &inv_c};
  const size_t smem = (size_t)(kLnThreads / 32) * 2 * c * sizeof(float);
  if (smem + sizeof(float) * kMaxChannels > 48 * 1024) {
    const cudaError_t ea = cudaFuncSetAttribute(fn[p.k - 1], cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (ea != cudaSuccess) return jit_fail(std::string("CUDA error: ") + cudaGetErrorString(ea));
  }
  if (ln_launch(fn[p.k - 1], p.grid, smem, (cudaStream_t)stream, args)) return 1;
  if (dweight == nullptr && dbias == nullptr) return 0;
  int n_parts = p.grid;
  void* rargs[] = {&dweight, &dbias, &part, &c, &n_parts};
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((2 * c + 7) / 8);  // eight warps per CTA, one warp per output value
  cfg.blockDim = dim3(256);
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelExC(&cfg, (const void*)&layernorm_2d_bwd_reduce_kernel, rargs);
  if (e != cudaSuccess) return jit_fail(std::string("CUDA error: ") + cudaGetErrorString(e));
  return 0;
}

}  // extern "C"
