// Bandwidth-bound row kernels: RMSNorm (eps, optional gain) and stable row softmax.
//
// One warp owns one row and keeps it in registers, so every element is read from HBM once and
// written once: algorithmic traffic is rows*cols*2 B in + rows*cols*2 B out (+ cols*2 B gain).
// Loads and stores are 128-bit, coalesced (a warp covers 512 contiguous bytes per access) and
// carry streaming cache hints; all loads of a row are issued before the first use so each warp
// has cols*2 bytes in flight.  Reductions are FP32 warp shuffles.
#include "host_common.h"
#include "sm100_ptx.cuh"

namespace trinity_sm100 {
namespace {

constexpr int kRowWarps = 8;  // rows per CTA

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

// kVec = 16-byte vectors per lane; the row spans up to kVec*256 columns (cols % 8 == 0).
template <int kVec, bool kHasGain>
__global__ void __launch_bounds__(kRowWarps * 32)
rmsnorm_rows_kernel(const uint4* __restrict__ x, const uint4* __restrict__ gain,
                    uint4* __restrict__ y, long long rows, int cols, float eps) {
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * kRowWarps + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int vecs = cols >> 3;
  const uint4* xr = x + row * vecs;
  uint4 v[kVec];
#pragma unroll
  for (int i = 0; i < kVec; ++i) {
    const int idx = i * 32 + lane;
    v[i] = idx < vecs ? load_stream(xr + idx) : make_uint4(0, 0, 0, 0);
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
  ss = warp_sum(ss);
  // x / sqrt(ss / cols + eps): an all-zero row with eps == 0 gives 0 * inf = NaN as 0/0 does.
  const float denom = sqrtf(ss / static_cast<float>(cols) + eps);
  const float inv = 1.0f / denom;
  uint4* yr = y + row * vecs;
#pragma unroll
  for (int i = 0; i < kVec; ++i) {
    const int idx = i * 32 + lane;
    if (idx < vecs) {
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

template <int kVec>
__global__ void __launch_bounds__(kRowWarps * 32)
softmax_rows_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, long long rows, int cols) {
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * kRowWarps + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int vecs = cols >> 3;
  const uint4* xr = x + row * vecs;
  uint4 v[kVec];
#pragma unroll
  for (int i = 0; i < kVec; ++i) {
    const int idx = i * 32 + lane;
    // Padding lanes hold -inf pairs (0xFF80 is BF16 -inf) so they vanish from max and sum.
    v[i] = idx < vecs ? load_stream(xr + idx)
                      : make_uint4(0xFF80FF80u, 0xFF80FF80u, 0xFF80FF80u, 0xFF80FF80u);
  }
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < kVec; ++i) {
    const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
    for (int e = 0; e < 4; ++e) m = fmaxf(m, fmaxf(bf16_lo(w[e]), bf16_hi(w[e])));
  }
  m = warp_max(m);
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
  s = warp_sum(s);
  const float inv = 1.0f / s;
  uint4* yr = y + row * vecs;
#pragma unroll
  for (int i = 0; i < kVec; ++i) {
    const int idx = i * 32 + lane;
    if (idx < vecs) {
      uint32_t o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) o[e] = pack_bf16x2(e_lo[i][e] * inv, e_hi[i][e] * inv);
      store_stream(yr + idx, make_uint4(o[0], o[1], o[2], o[3]));
    }
  }
}

int row_vectors(long long cols) { return int((cols + 255) / 256); }

int check_rows(const char* what, const void* x, const void* y, long long rows, long long cols) {
  if (!x || !y) return fail(TRINITY_SM100_E_INVALID, "%s: null pointer", what);
  if (rows <= 0 || cols <= 0) return fail(TRINITY_SM100_E_INVALID, "%s: empty extent", what);
  if (cols % 8) return fail(TRINITY_SM100_E_UNSUPPORTED, "%s: cols (%lld) must be a multiple of 8", what, cols);
  if (cols > 8192)
    return fail(TRINITY_SM100_E_UNSUPPORTED, "%s: cols (%lld) above the 8192 a warp keeps in registers", what, cols);
  if (!aligned16(x) || !aligned16(y))
    return fail(TRINITY_SM100_E_INVALID, "%s: pointers must be 16-byte aligned", what);
  if ((rows + kRowWarps - 1) / kRowWarps > INT32_MAX)
    return fail(TRINITY_SM100_E_UNSUPPORTED, "%s: too many rows", what);
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
  const unsigned grid = unsigned((rows + kRowWarps - 1) / kRowWarps);
  const uint4* xp = static_cast<const uint4*>(x);
  const uint4* gp = static_cast<const uint4*>(gain);
  uint4* yp = static_cast<uint4*>(y);
#define TRINITY_RMS(V)                                                                          \
  if (gain)                                                                                     \
    rmsnorm_rows_kernel<V, true><<<grid, kRowWarps * 32, 0, stream>>>(xp, gp, yp, rows, int(cols), eps); \
  else                                                                                          \
    rmsnorm_rows_kernel<V, false><<<grid, kRowWarps * 32, 0, stream>>>(xp, gp, yp, rows, int(cols), eps)
  const int v = row_vectors(cols);
  if (v <= 1) { TRINITY_RMS(1); }
  else if (v <= 2) { TRINITY_RMS(2); }
  else if (v <= 4) { TRINITY_RMS(4); }
  else if (v <= 8) { TRINITY_RMS(8); }
  else if (v <= 16) { TRINITY_RMS(16); }
  else { TRINITY_RMS(32); }
#undef TRINITY_RMS
  count_launch();
  return check_launch("rmsnorm_rows");
}

extern "C" int trinity_sm100_softmax_bf16(const void* x, void* y, int64_t rows, int64_t cols,
                                          void* stream_handle) {
  if (int rc = check_rows("softmax", x, y, rows, cols)) return rc;
  if (int rc = require_sm100(nullptr)) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  const unsigned grid = unsigned((rows + kRowWarps - 1) / kRowWarps);
  const uint4* xp = static_cast<const uint4*>(x);
  uint4* yp = static_cast<uint4*>(y);
#define TRINITY_SMX(V) softmax_rows_kernel<V><<<grid, kRowWarps * 32, 0, stream>>>(xp, yp, rows, int(cols))
  const int v = row_vectors(cols);
  if (v <= 1) { TRINITY_SMX(1); }
  else if (v <= 2) { TRINITY_SMX(2); }
  else if (v <= 4) { TRINITY_SMX(4); }
  else if (v <= 8) { TRINITY_SMX(8); }
  else if (v <= 16) { TRINITY_SMX(16); }
  else { TRINITY_SMX(32); }
#undef TRINITY_SMX
  count_launch();
  return check_launch("softmax_rows");
}
