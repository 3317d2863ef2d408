// Bandwidth-bound row kernels: RMSNorm (eps, optional gain) and stable row softmax.
//
// A row is spread over kThreads lanes (32..256), each keeping at most four 16-byte vectors in
// registers, so every element is read from HBM once and written once while the register
// footprint stays small enough for dozens of resident warps per SM: algorithmic traffic is
// rows*cols*2 B in + rows*cols*2 B out (+ cols*2 B gain).  Loads and stores are 128-bit,
// coalesced (a warp covers 512 contiguous bytes per access) and carry streaming cache hints;
// all loads of a thread are issued before the first use.  Reductions are FP32 warp shuffles,
// joined through shared memory when a row spans several warps.
#include "host_common.h"
#include "sm100_ptx.cuh"

namespace trinity_sm100 {
namespace {

constexpr int kRowBlock = 128;  // minimum CTA size; narrower rows share a CTA

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ uint4 load_stream(const uint4* p) { return __ldcs(p); }
__device__ __forceinline__ void store_stream(uint4* p, uint4 v) { __stcs(p, v); }

// Reduction over the kThreads lanes that share a row.  `scratch` holds one float per warp of
// the CTA; every thread of the CTA must call this (it contains a CTA barrier when a row spans
// more than one warp).
template <int kThreads, bool kMax>
__device__ __forceinline__ float row_reduce(float v, float* scratch) {
  v = kMax ? warp_max(v) : warp_sum(v);
  if (kThreads > 32) {
    constexpr int kWarpsPerRow = kThreads / 32;
    const int warp = threadIdx.x >> 5;
    __syncthreads();  // scratch may still be read by the previous reduction
    if ((threadIdx.x & 31) == 0) scratch[warp] = v;
    __syncthreads();
    const int first = (warp / kWarpsPerRow) * kWarpsPerRow;
    v = scratch[first];
#pragma unroll
    for (int w = 1; w < kWarpsPerRow; ++w) v = kMax ? fmaxf(v, scratch[first + w]) : v + scratch[first + w];
  }
  return v;
}

// kThreads lanes per row, kVec 16-byte vectors per lane (kThreads * kVec * 8 >= cols).
template <int kThreads, int kVec, bool kHasGain>
__global__ void __launch_bounds__(kThreads > kRowBlock ? kThreads : kRowBlock)
rmsnorm_rows_kernel(const uint4* __restrict__ x, const uint4* __restrict__ gain,
                    uint4* __restrict__ y, long long rows, int cols, float eps) {
  constexpr int kBlock = kThreads > kRowBlock ? kThreads : kRowBlock;
  constexpr int kRowsPerCta = kBlock / kThreads;
  __shared__ float scratch[kBlock / 32];
  grid_dependents_may_launch();
  grid_dependency_wait();   // the previous kernel of the stream may have produced x
  const int lane = threadIdx.x % kThreads;
  const long long row = static_cast<long long>(blockIdx.x) * kRowsPerCta + threadIdx.x / kThreads;
  const bool live = row < rows;
  const int vecs = cols >> 3;
  const uint4* xr = x + (live ? row : 0) * vecs;
  uint4 v[kVec];
#pragma unroll
  for (int i = 0; i < kVec; ++i) {
    const int idx = i * kThreads + lane;
    v[i] = (live && idx < vecs) ? load_stream(xr + idx) : make_uint4(0, 0, 0, 0);
  }
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < kVec; ++i) {
    const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float a = bf16_lo(w[e]), b = bf16_hi(w[e]);
      ss = fmaf(a, a, ss);
      ss = fmaf(b, b, ss);
    }
  }
  ss = row_reduce<kThreads, false>(ss, scratch);
  // x / sqrt(ss / cols + eps): an all-zero row with eps == 0 gives 0 * inf = NaN as 0/0 does.
  const float denom = sqrtf(ss / static_cast<float>(cols) + eps);
  const float inv = 1.0f / denom;
  uint4* yr = y + (live ? row : 0) * vecs;
#pragma unroll
  for (int i = 0; i < kVec; ++i) {
    const int idx = i * kThreads + lane;
    if (live && idx < vecs) {
      const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
      uint32_t o[4];
      if (kHasGain) {
        const uint4 gv = __ldg(gain + idx);
        const uint32_t g[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
        for (int e = 0; e < 4; ++e)
          o[e] = pack_bf16x2(bf16_lo(w[e]) * inv * bf16_lo(g[e]),
                             bf16_hi(w[e]) * inv * bf16_hi(g[e]));
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) o[e] = pack_bf16x2(bf16_lo(w[e]) * inv, bf16_hi(w[e]) * inv);
      }
      store_stream(yr + idx, make_uint4(o[0], o[1], o[2], o[3]));
    }
  }
}

template <int kThreads, int kVec>
__global__ void __launch_bounds__(kThreads > kRowBlock ? kThreads : kRowBlock)
softmax_rows_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, long long rows, int cols) {
  constexpr int kBlock = kThreads > kRowBlock ? kThreads : kRowBlock;
  constexpr int kRowsPerCta = kBlock / kThreads;
  __shared__ float scratch[kBlock / 32];
  grid_dependents_may_launch();
  grid_dependency_wait();   // the previous kernel of the stream may have produced x
  const int lane = threadIdx.x % kThreads;
  const long long row = static_cast<long long>(blockIdx.x) * kRowsPerCta + threadIdx.x / kThreads;
  const bool live = row < rows;
  const int vecs = cols >> 3;
  const uint4* xr = x + (live ? row : 0) * vecs;
  uint4 v[kVec];
#pragma unroll
  for (int i = 0; i < kVec; ++i) {
    const int idx = i * kThreads + lane;
    // Padding lanes hold -inf pairs (0xFF80 is BF16 -inf) so they vanish from max and sum.
    v[i] = (live && idx < vecs) ? load_stream(xr + idx)
                                : make_uint4(0xFF80FF80u, 0xFF80FF80u, 0xFF80FF80u, 0xFF80FF80u);
  }
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < kVec; ++i) {
    const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
    for (int e = 0; e < 4; ++e) m = fmaxf(m, fmaxf(bf16_lo(w[e]), bf16_hi(w[e])));
  }
  m = row_reduce<kThreads, true>(m, scratch);
  // exp(x - m) = exp2((x - m) * log2 e); a row whose maximum is +-inf yields NaN like the
  // reference's inf - inf does.
  constexpr float kLog2e = 1.4426950408889634f;
  float s = 0.0f;
  float e_lo[kVec][4], e_hi[kVec][4];
#pragma unroll
  for (int i = 0; i < kVec; ++i) {
    const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      e_lo[i][e] = exp2f((bf16_lo(w[e]) - m) * kLog2e);
      e_hi[i][e] = exp2f((bf16_hi(w[e]) - m) * kLog2e);
      s += e_lo[i][e] + e_hi[i][e];
    }
  }
  s = row_reduce<kThreads, false>(s, scratch);
  const float inv = 1.0f / s;
  uint4* yr = y + (live ? row : 0) * vecs;
#pragma unroll
  for (int i = 0; i < kVec; ++i) {
    const int idx = i * kThreads + lane;
    if (live && idx < vecs) {
      uint32_t o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) o[e] = pack_bf16x2(e_lo[i][e] * inv, e_hi[i][e] * inv);
      store_stream(yr + idx, make_uint4(o[0], o[1], o[2], o[3]));
    }
  }
}

// Picks lanes per row and vectors per lane: one warp up to 1024 columns, then four vectors per
// lane with as many warps as the row needs (4096 columns -> 128 lanes, 8192 -> 256).
struct RowShape {
  int threads, vec;
};
RowShape row_shape(long long cols) {
  const int vecs = int(cols / 8);
  if (vecs <= 32) return {32, 1};
  if (vecs <= 64) return {32, 2};
  if (vecs <= 128) return {32, 4};
  if (vecs <= 256) return {64, 4};
  if (vecs <= 512) return {128, 4};
  return {256, 4};
}

int check_rows(const char* what, const void* x, const void* y, long long rows, long long cols) {
  if (!x || !y) return fail(TRINITY_SM100_E_INVALID, "%s: null pointer", what);
  if (rows <= 0 || cols <= 0) return fail(TRINITY_SM100_E_INVALID, "%s: empty extent", what);
  if (cols % 8) return fail(TRINITY_SM100_E_UNSUPPORTED, "%s: cols (%lld) must be a multiple of 8", what, cols);
  if (cols > 8192)
    return fail(TRINITY_SM100_E_UNSUPPORTED, "%s: cols (%lld) above the 8192 a CTA keeps in registers", what, cols);
  if (!aligned16(x) || !aligned16(y))
    return fail(TRINITY_SM100_E_INVALID, "%s: pointers must be 16-byte aligned", what);
  if (rows > INT32_MAX) return fail(TRINITY_SM100_E_UNSUPPORTED, "%s: too many rows", what);
  return 0;
}

}  // namespace
}  // namespace trinity_sm100

using namespace trinity_sm100;

extern "C" int trinity_sm100_rmsnorm_bf16(const void* x, const void* gain, void* y, int64_t rows,
                                          int64_t cols, float eps, void* stream_handle) {
  if (int rc = check_rows("rmsnorm", x, y, rows, cols)) return rc;
  if (gain && !aligned16(gain))
    return fail(TRINITY_SM100_E_INVALID, "rmsnorm: gain must be 16-byte aligned");
  if (int rc = require_sm100(nullptr)) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  const uint4* xp = static_cast<const uint4*>(x);
  const uint4* gp = static_cast<const uint4*>(gain);
  uint4* yp = static_cast<uint4*>(y);
  const RowShape shape = row_shape(cols);
  cudaError_t launch_error = cudaSuccess;
#define TRINITY_RMS(T, V)                                                                        \
  {                                                                                              \
    constexpr int block = (T) > kRowBlock ? (T) : kRowBlock;                                     \
    const unsigned grid = unsigned((rows + block / (T) - 1) / (block / (T)));                    \
    KernelLaunch launch(dim3(grid), dim3(block), 0, stream);                                     \
    if (gain)                                                                                    \
      launch_error = cudaLaunchKernelEx(&launch.config, rmsnorm_rows_kernel<T, V, true>, xp, gp, yp, \
                                        static_cast<long long>(rows), int(cols), eps);          \
    else                                                                                         \
      launch_error = cudaLaunchKernelEx(&launch.config, rmsnorm_rows_kernel<T, V, false>, xp, gp, yp, \
                                        static_cast<long long>(rows), int(cols), eps);          \
  }
  if (shape.threads == 32 && shape.vec == 1) TRINITY_RMS(32, 1)
  else if (shape.threads == 32 && shape.vec == 2) TRINITY_RMS(32, 2)
  else if (shape.threads == 32) TRINITY_RMS(32, 4)
  else if (shape.threads == 64) TRINITY_RMS(64, 4)
  else if (shape.threads == 128) TRINITY_RMS(128, 4)
  else TRINITY_RMS(256, 4)
#undef TRINITY_RMS
  if (launch_error != cudaSuccess)
    return fail(TRINITY_SM100_E_CUDA, "rmsnorm_rows launch: %s", cudaGetErrorString(launch_error));
  count_launch();
  return check_launch("rmsnorm_rows");
}

extern "C" int trinity_sm100_softmax_bf16(const void* x, void* y, int64_t rows, int64_t cols,
                                          void* stream_handle) {
  if (int rc = check_rows("softmax", x, y, rows, cols)) return rc;
  if (int rc = require_sm100(nullptr)) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  const uint4* xp = static_cast<const uint4*>(x);
  uint4* yp = static_cast<uint4*>(y);
  const RowShape shape = row_shape(cols);
  cudaError_t launch_error = cudaSuccess;
#define TRINITY_SMX(T, V)                                                                  \
  {                                                                                        \
    constexpr int block = (T) > kRowBlock ? (T) : kRowBlock;                               \
    const unsigned grid = unsigned((rows + block / (T) - 1) / (block / (T)));              \
    KernelLaunch launch(dim3(grid), dim3(block), 0, stream);                               \
    launch_error = cudaLaunchKernelEx(&launch.config, softmax_rows_kernel<T, V>, xp, yp,   \
                                      static_cast<long long>(rows), int(cols));            \
  }
  if (shape.threads == 32 && shape.vec == 1) TRINITY_SMX(32, 1)
  else if (shape.threads == 32 && shape.vec == 2) TRINITY_SMX(32, 2)
  else if (shape.threads == 32) TRINITY_SMX(32, 4)
  else if (shape.threads == 64) TRINITY_SMX(64, 4)
  else if (shape.threads == 128) TRINITY_SMX(128, 4)
  else TRINITY_SMX(256, 4)
#undef TRINITY_SMX
  if (launch_error != cudaSuccess)
    return fail(TRINITY_SM100_E_CUDA, "softmax_rows launch: %s", cudaGetErrorString(launch_error));
  count_launch();
  return check_launch("softmax_rows");
}
