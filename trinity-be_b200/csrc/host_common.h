// Host-side helpers shared by the kernel launchers: error text, device checks, the launch
// counter and TMA tensor-map construction through the driver entry point (no libcuda link).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/trinity_sm100.h"

namespace trinity_sm100 {

// Records a formatted message for trinity_sm100_last_error() and returns `code`.
int fail(int code, const char* format, ...);

// Ensures the current device is compute capability 10.x; caches the SM count per device.
int require_sm100(int* sm_count);

void count_launch(unsigned n = 1);

// Checks cudaGetLastError() after a launch; `what` names the kernel.
int check_launch(const char* what);

// Opts `kernel` into `bytes` of dynamic shared memory on the current device, once per device:
// bit d of `*done_mask` records that device d has it.  Safe to call from several threads.
int opt_in_shared_memory(const void* kernel, int bytes, unsigned long long* done_mask, const char* what);

// Per-device set-up that trinity_sm100_prepare_device runs so that later launches (possibly under
// stream capture) make no attribute or symbol-address calls: the kernels' shared-memory opt-ins
// and the device address of the built-in MLA scratch array.
int gemm_prepare_device();
int mla_prepare_device();

// Launch configuration of the single-GPU kernels: optional cluster width, and (unless
// TRINITY_SM100_DEPENDENT_LAUNCH=0) programmatic dependent launch, with which the kernel's thread
// blocks may start while the previous kernel of the stream is still draining.  Every kernel
// launched this way runs only its set-up (barriers, tensor memory, descriptor prefetch) before
// `griddepcontrol.wait`, which returns once the previous kernel has completed and its writes are
// visible; nothing before the wait reads or writes memory another kernel produces.
struct KernelLaunch {
  cudaLaunchConfig_t config;
  cudaLaunchAttribute attributes[2];
  KernelLaunch(dim3 grid, dim3 block, size_t shared_bytes, cudaStream_t stream, unsigned cluster_x = 1);
};
bool dependent_launch_enabled();

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// 2-D tiled tensor map over a row-major matrix: `inner` contiguous elements per row,
// `outer` rows, `row_pitch_bytes` between rows; box = box_inner x box_outer elements.
// swizzle128 selects the 128-byte shared-memory swizzle (box_inner * elem_bytes must be 128).
int make_tensor_map_2d(CUtensorMap* map, const void* base, int elem_bytes, uint64_t inner,
                       uint64_t outer, uint64_t row_pitch_bytes, uint32_t box_inner,
                       uint32_t box_outer, bool swizzle128);

// 3-D variant: dims (inner, mid, outer) with byte pitches for mid and outer; swizzle_bytes is
// 0, 64 or 128 (the box's inner extent in bytes must equal a non-zero swizzle width).
int make_tensor_map_3d(CUtensorMap* map, const void* base, int elem_bytes, uint64_t inner,
                       uint64_t mid, uint64_t outer, uint64_t mid_pitch_bytes,
                       uint64_t outer_pitch_bytes, uint32_t box_inner, uint32_t box_mid,
                       uint32_t box_outer, int swizzle_bytes);

}  // namespace trinity_sm100
