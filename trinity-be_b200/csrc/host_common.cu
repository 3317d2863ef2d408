// Library-wide host state: error text, launch counter, device status word, tensor maps.
#include "host_common.h"

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "sm100_ptx.cuh"

namespace trinity_sm100 {

namespace {
thread_local char t_error[512] = "";
std::atomic<uint64_t> g_launches{0};

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                 const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                 const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
  static EncodeTiled fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) !=
            cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiled>(p);
  }();
  return fn;
}

CUtensorMapDataType map_dtype(int elem_bytes) {
  return elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
}
}  // namespace

int fail(int code, const char* format, ...) {
  va_list args;
  va_start(args, format);
  vsnprintf(t_error, sizeof(t_error), format, args);
  va_end(args);
  return code;
}

int require_sm100(int* sm_count) {
  static std::mutex mutex;
  static int cached_major[64];
  static int cached_sms[64];
  static bool known[64];
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess)
    return fail(TRINITY_SM100_E_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (device < 0 || device >= 64) return fail(TRINITY_SM100_E_DEVICE, "device index %d", device);
  std::lock_guard<std::mutex> lock(mutex);
  if (!known[device]) {
    int major = 0, sms = 0;
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (e != cudaSuccess)
      return fail(TRINITY_SM100_E_CUDA, "cudaDeviceGetAttribute: %s", cudaGetErrorString(e));
    cached_major[device] = major;
    cached_sms[device] = sms;
    known[device] = true;
  }
  if (cached_major[device] != 10)
    return fail(TRINITY_SM100_E_DEVICE,
                "device %d has compute capability major %d; this library is sm_100a only", device,
                cached_major[device]);
  if (sm_count) *sm_count = cached_sms[device];
  return 0;
}

int opt_in_shared_memory(const void* kernel, int bytes, unsigned long long* done_mask, const char* what) {
  static std::mutex mutex;
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return fail(TRINITY_SM100_E_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (device < 0 || device >= 64) return fail(TRINITY_SM100_E_DEVICE, "device index %d", device);
  const unsigned long long bit = 1ull << device;
  if (__atomic_load_n(done_mask, __ATOMIC_ACQUIRE) & bit) return 0;
  std::lock_guard<std::mutex> lock(mutex);
  if (*done_mask & bit) return 0;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess)
    return fail(TRINITY_SM100_E_CUDA, "%s: shared memory opt-in (%d B): %s", what, bytes, cudaGetErrorString(e));
  __atomic_fetch_or(done_mask, bit, __ATOMIC_RELEASE);
  return 0;
}

void count_launch(unsigned n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess)
    return fail(TRINITY_SM100_E_CUDA, "%s launch: %s", what, cudaGetErrorString(e));
  return 0;
}

bool dependent_launch_enabled() {
  const char* v = getenv("TRINITY_SM100_DEPENDENT_LAUNCH");
  return !(v && v[0] == '0');
}

KernelLaunch::KernelLaunch(dim3 grid, dim3 block, size_t shared_bytes, cudaStream_t stream, unsigned cluster_x) {
  config = cudaLaunchConfig_t{};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = shared_bytes;
  config.stream = stream;
  unsigned count = 0;
  if (cluster_x > 1) {
    attributes[count].id = cudaLaunchAttributeClusterDimension;
    attributes[count].val.clusterDim.x = cluster_x;
    attributes[count].val.clusterDim.y = 1;
    attributes[count].val.clusterDim.z = 1;
    ++count;
  }
  if (dependent_launch_enabled()) {
    attributes[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[count].val.programmaticStreamSerializationAllowed = 1;
    ++count;
  }
  config.attrs = attributes;
  config.numAttrs = count;
}

int make_tensor_map_2d(CUtensorMap* map, const void* base, int elem_bytes, uint64_t inner,
                       uint64_t outer, uint64_t row_pitch_bytes, uint32_t box_inner,
                       uint32_t box_outer, bool swizzle128) {
  EncodeTiled fn = encode_tiled();
  if (!fn) return fail(TRINITY_SM100_E_CUDA, "cuTensorMapEncodeTiled entry point unavailable");
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_pitch_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t elem_strides[2] = {1, 1};
  CUresult r = fn(map, map_dtype(elem_bytes), 2, const_cast<void*>(base), dims, strides, box,
                  elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(TRINITY_SM100_E_CUDA,
                "cuTensorMapEncodeTiled(2d %llu x %llu, pitch %llu, box %u x %u) -> %d",
                (unsigned long long)inner, (unsigned long long)outer,
                (unsigned long long)row_pitch_bytes, box_inner, box_outer, int(r));
  return 0;
}

int make_tensor_map_3d(CUtensorMap* map, const void* base, int elem_bytes, uint64_t inner,
                       uint64_t mid, uint64_t outer, uint64_t mid_pitch_bytes,
                       uint64_t outer_pitch_bytes, uint32_t box_inner, uint32_t box_mid,
                       uint32_t box_outer, int swizzle_bytes) {
  EncodeTiled fn = encode_tiled();
  if (!fn) return fail(TRINITY_SM100_E_CUDA, "cuTensorMapEncodeTiled entry point unavailable");
  cuuint64_t dims[3] = {inner, mid, outer};
  cuuint64_t strides[2] = {mid_pitch_bytes, outer_pitch_bytes};
  cuuint32_t box[3] = {box_inner, box_mid, box_outer};
  cuuint32_t elem_strides[3] = {1, 1, 1};
  CUresult r = fn(map, map_dtype(elem_bytes), 3, const_cast<void*>(base), dims, strides, box,
                  elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle_bytes == 128  ? CU_TENSOR_MAP_SWIZZLE_128B
                  : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                        : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(TRINITY_SM100_E_CUDA, "cuTensorMapEncodeTiled(3d) -> %d", int(r));
  return 0;
}

}  // namespace trinity_sm100

using namespace trinity_sm100;

extern "C" int trinity_sm100_device_status(uint32_t* status, int clear) {
  if (!status) return fail(TRINITY_SM100_E_INVALID, "status pointer is null");
  unsigned int value = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&value, g_device_status, sizeof(value));
  if (e != cudaSuccess)
    return fail(TRINITY_SM100_E_CUDA, "reading device status: %s", cudaGetErrorString(e));
  *status = value;
  if (clear && value) {
    unsigned int zero = 0;
    e = cudaMemcpyToSymbol(g_device_status, &zero, sizeof(zero));
    if (e != cudaSuccess)
      return fail(TRINITY_SM100_E_CUDA, "clearing device status: %s", cudaGetErrorString(e));
  }
  return 0;
}

extern "C" int trinity_sm100_set_wait_budget(uint64_t cycles) {
  long long value = cycles == 0 ? kDefaultWaitBudgetCycles
                                : (cycles > uint64_t(INT64_MAX) ? INT64_MAX : static_cast<long long>(cycles));
  cudaError_t e = cudaMemcpyToSymbol(g_wait_budget_cycles, &value, sizeof(value));
  if (e != cudaSuccess)
    return fail(TRINITY_SM100_E_CUDA, "setting the wait budget: %s", cudaGetErrorString(e));
  return 0;
}

extern "C" int trinity_sm100_abi_version(void) { return TRINITY_SM100_ABI_VERSION; }
extern "C" const char* trinity_sm100_last_error(void) { return t_error; }
extern "C" uint64_t trinity_sm100_launch_count(void) {
  return g_launches.load(std::memory_order_relaxed);
}
