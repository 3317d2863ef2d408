// Generic FP32 pointwise evaluation and row reduce-sum: the primitives the reference's SIMT
// provider offers for plans that are not fused into a larger region.
//
//   pointwise:  out[r,c] = f(operand_0[r,c], operand_1[r | c | r,c], ..., constants)
//               f is a postfix program over + - * / sqr sqrt sigmoid relu exp max, evaluated in
//               FP32 with a single rounding at the store
//   row_reduce: y[r] = sum_c g(x[r,c]), g = identity or square, FP32 accumulate and output
//
// Both are HBM-bound: each thread handles eight consecutive columns with one 128-bit access per
// BF16 operand (two for FP32); algorithmic traffic is the operand bytes plus the output bytes.
#include "host_common.h"
#include "sm100_ptx.cuh"

namespace trinity_sm100 {
namespace {

constexpr int kPwThreads = 256;
constexpr int kPwStack = 6;

struct PwOperand {
  const void* data;
  int dtype;      // 0 bf16, 1 fp32
  int broadcast;  // 0 full, 1 per row, 2 per column
};
struct PwParams {
  PwOperand operands[TRINITY_SM100_PW_MAX_OPERANDS];
  void* out;
  int out_dtype;
  long long rows, cols;
  int length;
  uint32_t program[TRINITY_SM100_PW_MAX_PROGRAM];
};

__device__ __forceinline__ float pw_load_scalar(const PwOperand& o, long long r, long long c,
                                                long long cols) {
  const long long idx = o.broadcast == 1 ? r : o.broadcast == 2 ? c : r * cols + c;
  return o.dtype == 1 ? static_cast<const float*>(o.data)[idx]
                      : __bfloat162float(static_cast<const __nv_bfloat16*>(o.data)[idx]);
}

// Loads eight consecutive columns (c .. c+7) of an operand; `vector` promises c % 8 == 0,
// cols % 8 == 0 and a 16-byte aligned base.
__device__ __forceinline__ void pw_load8(const PwOperand& o, long long r, long long c,
                                         long long cols, int valid, bool vector, float (&v)[8]) {
  if (o.broadcast == 1) {
    const float x = pw_load_scalar(o, r, 0, cols);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = x;
    return;
  }
  if (vector && valid == 8) {
    const long long idx = o.broadcast == 2 ? c : r * cols + c;
    if (o.dtype == 1) {
      const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(o.data) + idx);
      const float4 a = p[0], b = p[1];
      v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
      const uint4 a = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(o.data) + idx);
      const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        v[2 * e] = bf16_lo(w[e]);
        v[2 * e + 1] = bf16_hi(w[e]);
      }
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = i < valid ? pw_load_scalar(o, r, c + i, cols) : 0.0f;
}

__global__ void __launch_bounds__(kPwThreads) pointwise_kernel(const PwParams p, int vector) {
  grid_dependents_may_launch();
  grid_dependency_wait();
  const long long groups_per_row = (p.cols + 7) / 8;
  const long long total = p.rows * groups_per_row;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long g = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; g < total;
       g += stride) {
    const long long r = g / groups_per_row;
    const long long c = (g % groups_per_row) * 8;
    const int valid = int(p.cols - c < 8 ? p.cols - c : 8);
    float stack[kPwStack][8];
    int top = 0;
    for (int pc = 0; pc < p.length; ++pc) {
      const uint32_t word = p.program[pc];
      const uint32_t op = word & 0xFFu;
      if (op == TRINITY_SM100_PW_OPERAND) {
        pw_load8(p.operands[(word >> 8) & 0xFFu], r, c, p.cols, valid, vector != 0, stack[top]);
        ++top;
      } else if (op == TRINITY_SM100_PW_CONST) {
        const float x = __uint_as_float(p.program[++pc]);
#pragma unroll
        for (int i = 0; i < 8; ++i) stack[top][i] = x;
        ++top;
      } else if (op >= TRINITY_SM100_PW_SQR) {  // unary
        float(&a)[8] = stack[top - 1];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float x = a[i];
          a[i] = op == TRINITY_SM100_PW_SQR       ? x * x
                 : op == TRINITY_SM100_PW_SQRT    ? sqrtf(x)
                 : op == TRINITY_SM100_PW_SIGMOID ? 1.0f / (1.0f + expf(-x))
                 : op == TRINITY_SM100_PW_RELU    ? (x < 0.0f ? 0.0f : x)
                                                  : expf(x);
        }
      } else {  // binary: a (op) b with b on top
        float(&a)[8] = stack[top - 2];
        const float(&b)[8] = stack[top - 1];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          a[i] = op == TRINITY_SM100_PW_ADD   ? a[i] + b[i]
                 : op == TRINITY_SM100_PW_SUB ? a[i] - b[i]
                 : op == TRINITY_SM100_PW_MUL ? a[i] * b[i]
                 : op == TRINITY_SM100_PW_DIV ? a[i] / b[i]
                                              : fmaxf(a[i], b[i]);
        }
        --top;
      }
    }
    const float(&y)[8] = stack[0];
    const long long idx = r * p.cols + c;
    if (vector && valid == 8) {
      if (p.out_dtype == 1) {
        float4* o = reinterpret_cast<float4*>(static_cast<float*>(p.out) + idx);
        o[0] = make_float4(y[0], y[1], y[2], y[3]);
        o[1] = make_float4(y[4], y[5], y[6], y[7]);
      } else {
        *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + idx) =
            make_uint4(pack_bf16x2(y[0], y[1]), pack_bf16x2(y[2], y[3]), pack_bf16x2(y[4], y[5]),
                       pack_bf16x2(y[6], y[7]));
      }
    } else {
      for (int i = 0; i < valid; ++i) {
        if (p.out_dtype == 1) static_cast<float*>(p.out)[idx + i] = y[i];
        else static_cast<__nv_bfloat16*>(p.out)[idx + i] = __float2bfloat16(y[i]);
      }
    }
  }
}

// One warp per row; lanes stride over 8-column groups, FP32 accumulation, shuffle tree.
__global__ void __launch_bounds__(256) row_reduce_sum_kernel(const void* x, int dtype, float* y,
                                                             long long rows, long long cols,
                                                             int square, int vector) {
  grid_dependents_may_launch();
  grid_dependency_wait();
  const long long row = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  PwOperand o{x, dtype, 0};
  float acc = 0.0f;
  for (long long c = lane * 8ll; c < cols; c += 256) {
    float v[8];
    const int valid = int(cols - c < 8 ? cols - c : 8);
    pw_load8(o, row, c, cols, valid, vector != 0, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc += square ? v[i] * v[i] : v[i];
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) y[row] = acc;
}

bool vector_ok(const void* p, int dtype) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0 && dtype >= 0; }

}  // namespace
}  // namespace trinity_sm100

using namespace trinity_sm100;

extern "C" int trinity_sm100_pointwise(const trinity_sm100_pointwise_args* args, void* stream_handle) {
  if (!args) return fail(TRINITY_SM100_E_INVALID, "pointwise: null argument block");
  const trinity_sm100_pointwise_args& a = *args;
  if (!a.out || a.rows <= 0 || a.cols <= 0)
    return fail(TRINITY_SM100_E_INVALID, "pointwise: null output or empty extent");
  if (a.operand_count < 0 || a.operand_count > TRINITY_SM100_PW_MAX_OPERANDS)
    return fail(TRINITY_SM100_E_INVALID, "pointwise: operand count %d", a.operand_count);
  if (a.program_length <= 0 || a.program_length > TRINITY_SM100_PW_MAX_PROGRAM)
    return fail(TRINITY_SM100_E_INVALID, "pointwise: program length %d", a.program_length);
  PwParams p;
  bool vector = a.cols % 8 == 0 && vector_ok(a.out, a.out_dtype);
  for (int i = 0; i < TRINITY_SM100_PW_MAX_OPERANDS; ++i) p.operands[i] = {nullptr, 0, 0};
  for (int i = 0; i < a.operand_count; ++i) {
    const auto& o = a.operands[i];
    if (!o.data || o.dtype < 0 || o.dtype > 1 || o.broadcast < 0 || o.broadcast > 2)
      return fail(TRINITY_SM100_E_INVALID, "pointwise: operand %d invalid", i);
    p.operands[i] = {o.data, o.dtype, o.broadcast};
    if (o.broadcast != 1) vector = vector && vector_ok(o.data, o.dtype);
  }
  // Validate the program: stack discipline and operand indices.
  int depth = 0;
  for (int pc = 0; pc < a.program_length; ++pc) {
    const uint32_t word = a.program[pc], op = word & 0xFFu;
    if (op == TRINITY_SM100_PW_OPERAND) {
      if (int((word >> 8) & 0xFFu) >= a.operand_count)
        return fail(TRINITY_SM100_E_INVALID, "pointwise: program reads operand %u", (word >> 8) & 0xFFu);
      ++depth;
    } else if (op == TRINITY_SM100_PW_CONST) {
      if (++pc >= a.program_length) return fail(TRINITY_SM100_E_INVALID, "pointwise: truncated constant");
      ++depth;
    } else if (op >= TRINITY_SM100_PW_SQR && op <= TRINITY_SM100_PW_EXP) {
      if (depth < 1) return fail(TRINITY_SM100_E_INVALID, "pointwise: stack underflow");
    } else if (op >= TRINITY_SM100_PW_ADD && op <= TRINITY_SM100_PW_MAX) {
      if (depth < 2) return fail(TRINITY_SM100_E_INVALID, "pointwise: stack underflow");
      --depth;
    } else {
      return fail(TRINITY_SM100_E_INVALID, "pointwise: unknown opcode %u", op);
    }
    if (depth > kPwStack) return fail(TRINITY_SM100_E_UNSUPPORTED, "pointwise: expression too deep");
  }
  if (depth != 1) return fail(TRINITY_SM100_E_INVALID, "pointwise: program leaves %d values", depth);
  p.out = a.out;
  p.out_dtype = a.out_dtype;
  p.rows = a.rows;
  p.cols = a.cols;
  p.length = a.program_length;
  for (int i = 0; i < a.program_length; ++i) p.program[i] = a.program[i];
  int sm_count = 0;
  if (int rc = require_sm100(&sm_count)) return rc;
  const long long groups = a.rows * ((a.cols + 7) / 8);
  long long blocks = (groups + kPwThreads - 1) / kPwThreads;
  const long long cap = static_cast<long long>(sm_count) * 16;
  if (blocks > cap) blocks = cap;
  KernelLaunch launch(dim3(unsigned(blocks)), dim3(kPwThreads), 0, static_cast<cudaStream_t>(stream_handle));
  cudaError_t e = cudaLaunchKernelEx(&launch.config, pointwise_kernel, p, vector ? 1 : 0);
  if (e != cudaSuccess) return fail(TRINITY_SM100_E_CUDA, "pointwise launch: %s", cudaGetErrorString(e));
  count_launch();
  return check_launch("pointwise");
}

extern "C" int trinity_sm100_row_reduce_sum(const void* x, int32_t x_dtype, void* y, int64_t rows,
                                            int64_t cols, int32_t square, void* stream_handle) {
  if (!x || !y || rows <= 0 || cols <= 0)
    return fail(TRINITY_SM100_E_INVALID, "row_reduce_sum: null pointer or empty extent");
  if (x_dtype < 0 || x_dtype > 1) return fail(TRINITY_SM100_E_INVALID, "row_reduce_sum: dtype");
  if (int rc = require_sm100(nullptr)) return rc;
  const bool vector = cols % 8 == 0 && vector_ok(x, x_dtype);
  const unsigned grid = unsigned((rows + 7) / 8);
  KernelLaunch launch(dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream_handle));
  cudaError_t e = cudaLaunchKernelEx(&launch.config, row_reduce_sum_kernel, x, int(x_dtype), static_cast<float*>(y),
                                     static_cast<long long>(rows), static_cast<long long>(cols), int(square),
                                     vector ? 1 : 0);
  if (e != cudaSuccess) return fail(TRINITY_SM100_E_CUDA, "row_reduce_sum launch: %s", cudaGetErrorString(e));
  count_launch();
  return check_launch("row_reduce_sum");
}

// ------------------------------------------------------------------ plumbing for program.so
extern "C" int trinity_sm100_prepare_device(int32_t* device_index) {
  int device = 0;
  cudaError_t e = cudaFree(nullptr);  // make sure the primary context exists
  if (e == cudaSuccess) e = cudaGetDevice(&device);
  if (e != cudaSuccess) return fail(TRINITY_SM100_E_CUDA, "prepare: %s", cudaGetErrorString(e));
  if (int rc = require_sm100(nullptr)) return rc;
  if (int rc = gemm_prepare_device()) return rc;
  if (int rc = mla_prepare_device()) return rc;
  if (device_index) *device_index = device;
  return 0;
}

extern "C" int trinity_sm100_current_device(int32_t* device_index) {
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return fail(TRINITY_SM100_E_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (device_index) *device_index = device;
  return 0;
}

extern "C" int trinity_sm100_stream_synchronize(void* stream_handle) {
  cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream_handle));
  if (e != cudaSuccess)
    return fail(TRINITY_SM100_E_CUDA, "cudaStreamSynchronize: %s (%d)", cudaGetErrorString(e), int(e));
  return 0;
}
