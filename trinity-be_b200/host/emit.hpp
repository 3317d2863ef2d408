// Emission for the sm_100a provider: region recognition over a PhysicalPlan, launch planning
// with closed-form coverage checks, buffer requirements and the host shim source.
#pragma once

#include <string>
#include <vector>

#include "plan.hpp"

namespace trinity::host {

struct BufferRequirement {
  int slot;
  std::vector<std::string> input_names;
  std::string output_name;  // empty = not the output
  bool is_output = false;
  std::vector<int64_t> shape, strides;
  DType dtype;
  int64_t bytes;
  int alignment;
  bool external;
  bool symmetric = false;   // multi-GPU plans: every rank's copy is mapped into every process
};

// One kernel-library call of the generated launch list.
struct Launch {
  std::string kernel;             // library entry point, e.g. "trinity_sm100_gemm_bf16"
  std::string code;               // C++ statements of the call (use `bindings[slot]`, `stream`)
  std::vector<int> operations;    // plan operations this launch implements
  int shared_memory_bytes = 0;
  int block_threads = 128;
};

struct CudaSource {
  bool persistent = false;   // mode 2 (multi-GPU, PersistentLaunch) instead of mode 1 (streamed)
  std::string code;
  std::string requirements_json;
  std::vector<Launch> launches;
  std::vector<BufferRequirement> buffers;
};

CudaSource emit(const PhysicalPlan& plan);

// Per-operation candidates and rejections as JSON (the role of emit::kernel_candidates,
// src/emit/candidate.rs:107-207).
std::string kernel_candidates_json(const PhysicalPlan& plan);

}  // namespace trinity::host
