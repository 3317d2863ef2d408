// Native runtime for compiled plans: private-copy loader with ABI layout check, modules,
// executions with completion events, CUDA-Graph capture / replay, and a retire queue that keeps
// resources of still-running work alive.
//
// Behaviour follows the reference runtime (src/native/core.hpp:45-217, src/native/runtime.cpp):
//  * the artifact is copied to a private file before dlopen so two loads have independent
//    statics; any difference in the descriptor's struct layout is refused
//  * prepare is idempotent per module and paired with release before dlclose
//  * an execution remembers its binding pointers; run() on a second stream while work is
//    pending is ResourceBusy; a launch failure marks the execution failed for good
//  * while its stream is being captured, run() records no events and never synchronises
//  * wait(timeout) polls the tail event once per millisecond and gives up with code -1001,
//    leaving resources pinned
// PyTorch is not involved here: tensors are validated in the Python layer, this layer sees
// device pointers and stream handles.
#include "runtime.hpp"

#include <cuda_runtime_api.h>
#include <dlfcn.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <thread>

namespace trinity::host {

namespace {

[[noreturn]] void cuda_fail(const char* what, cudaError_t e, bool submitted = false) {
  abi::ErrorInfo info{abi::driver, abi::launch, int(e), submitted ? 1u : 0u, abi::none, 0};
  throw RuntimeFailure(std::string(what) + ": " + cudaGetErrorString(e), info);
}
void cuda_check(const char* what, cudaError_t e) {
  if (e != cudaSuccess) cuda_fail(what, e);
}

struct DeviceGuard {
  int previous = -1;
  explicit DeviceGuard(int device) {
    cuda_check("cudaGetDevice", cudaGetDevice(&previous));
    if (previous != device) cuda_check("cudaSetDevice", cudaSetDevice(device));
    else previous = -1;
  }
  ~DeviceGuard() {
    if (previous >= 0) cudaSetDevice(previous);
  }
};

// ------------------------------------------------------------------ retire queue
// Owners dropped while GPU work is pending hand their resources here; a background thread
// polls the completion event every 5 ms and reclaims afterwards.
class RetireQueue {
 public:
  static RetireQueue& instance() {
    static RetireQueue* q = new RetireQueue();  // leaked on purpose: outlives static teardown
    return *q;
  }
  void defer(int device, cudaEvent_t event, std::function<void()> reclaim) {
    std::lock_guard<std::mutex> lock(mutex_);
    items_.push_back({device, event, std::move(reclaim)});
    if (!started_) {
      started_ = true;
      std::thread([this] { loop(); }).detach();
    }
    cv_.notify_one();
  }
  size_t collect() {
    std::vector<Item> ready;
    {
      std::lock_guard<std::mutex> lock(mutex_);
      for (size_t i = 0; i < items_.size();) {
        if (!items_[i].event || cudaEventQuery(items_[i].event) != cudaErrorNotReady) {
          ready.push_back(std::move(items_[i]));
          items_.erase(items_.begin() + long(i));
        } else {
          ++i;
        }
      }
    }
    for (auto& item : ready) {
      if (item.event) cudaEventDestroy(item.event);
      item.reclaim();
    }
    std::lock_guard<std::mutex> lock(mutex_);
    return items_.size();
  }
  size_t pending() {
    std::lock_guard<std::mutex> lock(mutex_);
    return items_.size();
  }

 private:
  struct Item {
    int device;
    cudaEvent_t event;
    std::function<void()> reclaim;
  };
  void loop() {
    for (;;) {
      {
        std::unique_lock<std::mutex> lock(mutex_);
        cv_.wait(lock, [this] { return !items_.empty(); });
      }
      collect();
      std::this_thread::sleep_for(std::chrono::milliseconds(5));
    }
  }
  std::mutex mutex_;
  std::condition_variable cv_;
  std::vector<Item> items_;
  bool started_ = false;
};

bool copy_file(const std::string& from, const std::string& to) {
  std::ifstream in(from, std::ios::binary);
  std::ofstream out(to, std::ios::binary);
  if (!in || !out) return false;
  out << in.rdbuf();
  return bool(out);
}

}  // namespace

// ------------------------------------------------------------------ Library
Library::Library(const std::string& path, unsigned mode) {
  const char* tmp = getenv("TMPDIR");
  std::string pattern = std::string(tmp && *tmp ? tmp : "/tmp") + "/trinity-module-XXXXXX";
  std::vector<char> dir(pattern.begin(), pattern.end());
  dir.push_back('\0');
  if (!mkdtemp(dir.data())) throw std::invalid_argument("cannot create a private module directory");
  directory_ = dir.data();
  copy_ = directory_ + "/program.so";
  if (!copy_file(path, copy_)) {
    cleanup();
    throw std::invalid_argument("cannot copy artifact library " + path);
  }
  handle_ = dlopen(copy_.c_str(), RTLD_NOW | RTLD_LOCAL);
  if (!handle_) {
    std::string why = dlerror();
    cleanup();
    throw std::invalid_argument("dlopen failed: " + why);
  }
  auto sym = [&](const char* name) {
    void* p = dlsym(handle_, name);
    if (!p) {
      cleanup();
      throw std::invalid_argument(std::string("artifact does not export ") + name);
    }
    return p;
  };
  abi_ = reinterpret_cast<AbiFn>(sym("trinity_abi"));
  prepare_ = reinterpret_cast<PrepareFn>(sym("trinity_prepare"));
  launch_ = sym("trinity_launch");
  status_ = sym("trinity_status");
  release_ = reinterpret_cast<ReleaseFn>(sym("trinity_release"));
  const abi::Descriptor* d = abi_();
  const abi::Descriptor mine = abi::describe(mode, nullptr, 0);
  bool ok = d && d->version == abi::version && d->mode == mode && d->pointer_size == mine.pointer_size &&
            d->error_size == mine.error_size && d->error_alignment == mine.error_alignment &&
            d->launch_size == mine.launch_size && d->launch_alignment == mine.launch_alignment &&
            d->field_count == mine.field_count &&
            !memcmp(d->offsets, mine.offsets, sizeof mine.offsets) &&
            !memcmp(d->error_offsets, mine.error_offsets, sizeof mine.error_offsets) && d->requirements &&
            d->requirements_size <= (16u << 20);
  if (!ok) {
    cleanup();
    throw std::invalid_argument("artifact ABI descriptor differs from this runtime (version, mode or struct layout)");
  }
  requirements_.assign(d->requirements, d->requirements_size);
}

void Library::cleanup() {
  if (handle_) dlclose(handle_);
  handle_ = nullptr;
  if (!copy_.empty()) unlink(copy_.c_str());
  if (!directory_.empty()) rmdir(directory_.c_str());
  copy_.clear();
  directory_.clear();
}

Library::~Library() {
  if (prepared_) {
    abi::ErrorInfo info{};
    release_(&info);
  }
  cleanup();
}

unsigned Library::prepare() {
  if (prepared_) return workers_;
  abi::ErrorInfo info{};
  unsigned workers = 0;
  const int rc = prepare_(&workers, &info);
  if (rc) throw RuntimeFailure("trinity_prepare failed with code " + std::to_string(rc), info);
  prepared_ = true;
  workers_ = workers;
  return workers;
}

void Library::release() {
  if (!prepared_) return;
  abi::ErrorInfo info{};
  const int rc = release_(&info);
  if (rc) throw RuntimeFailure("trinity_release failed with code " + std::to_string(rc), info);  // stays prepared: retry later
  prepared_ = false;
}

// ------------------------------------------------------------------ Module
Module::Module(const std::string& path, int device, unsigned mode) : device_(device), mode_(mode) {
  if (mode != 1 && mode != 2) throw std::invalid_argument("artifact mode must be 1 (streamed) or 2 (persistent)");
  DeviceGuard guard(device);
  cuda_check("cudaFree(0)", cudaFree(nullptr));
  int runtime = 0;
  cuda_check("cudaRuntimeGetVersion", cudaRuntimeGetVersion(&runtime));
  if (runtime < 12080) throw std::invalid_argument("CUDA runtime 12.8 or newer is required for sm_100a");
  library_ = std::make_unique<Library>(path, mode);
}

Module::~Module() {
  try {
    if (library_) {
      DeviceGuard guard(device_);
      library_.reset();
    }
  } catch (...) {
  }
}

unsigned Module::prepare() {
  std::lock_guard<std::recursive_mutex> lock(mutex_);
  if (!library_) throw std::invalid_argument("module is closed");
  DeviceGuard guard(device_);
  return library_->prepare();
}

void Module::close() {
  std::lock_guard<std::recursive_mutex> lock(mutex_);
  if (!library_) return;
  if (executions_ > 0) throw ResourceBusy("module has live executions");
  DeviceGuard guard(device_);
  library_->release();
  library_.reset();
}

// ------------------------------------------------------------------ Execution
Execution::Execution(std::shared_ptr<Module> module, std::vector<void*> bindings, void* ready_stream,
                     void* workspace, size_t workspace_bytes, unsigned workers)
    : module_(std::move(module)), bindings_(std::move(bindings)), workspace_(workspace),
      workspace_bytes_(workspace_bytes), workers_(workers) {
  std::lock_guard<std::recursive_mutex> lock(module_->mutex_);
  if (!module_->library_ || !module_->library_->prepared()) throw std::invalid_argument("module is not prepared");
  if ((module_->mode_ == 2) != (workspace != nullptr))
    throw std::invalid_argument("a persistent module needs a workspace, a streamed one has none");
  DeviceGuard guard(module_->device_);
  for (size_t i = 0; i < bindings_.size(); ++i)
    if (!bindings_[i]) throw std::invalid_argument("binding " + std::to_string(i) + " is null");
  cuda_check("cudaEventCreate", cudaEventCreateWithFlags(&ready_, cudaEventDisableTiming));
  cuda_check("cudaEventCreate", cudaEventCreateWithFlags(&tail_, cudaEventDisableTiming));
  // Work already queued on the preparing stream (fills of the inputs) must precede the first run.
  cuda_check("cudaEventRecord", cudaEventRecord(ready_, static_cast<cudaStream_t>(ready_stream)));
  ++module_->executions_;
}

Execution::~Execution() {
  try {
    close(false);
  } catch (...) {
  }
}

void Execution::validate() const {
  if (closed_) throw std::invalid_argument("execution is closed");
  if (failed_) throw RuntimeFailure("execution failed earlier and cannot run again", failure_);
}

bool Execution::pending() const {
  return recorded_ && cudaEventQuery(tail_) == cudaErrorNotReady;
}

void Execution::run(void* stream_handle) {
  std::lock_guard<std::recursive_mutex> lock(module_->mutex_);
  validate();
  if (graph_owner_ && !graph_active_) throw ResourceBusy("execution is owned by a graph");
  DeviceGuard guard(module_->device_);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
  cuda_check("cudaStreamIsCapturing", cudaStreamIsCapturing(stream, &capture));
  const bool capturing = capture != cudaStreamCaptureStatusNone;
  if (capturing && !graph_active_) throw ResourceBusy("run inside a foreign stream capture; use Graph.capture");
  if (!capturing && pending() && stream != last_stream_)
    throw ResourceBusy("execution has pending work on another stream");
  if (!capturing) cuda_check("cudaStreamWaitEvent", cudaStreamWaitEvent(stream, ready_, 0));
  abi::ErrorInfo info{};
  int rc;
  if (module_->mode_ == 2) {
    abi::PersistentLaunch launch{};
    launch.bindings = bindings_.data();
    launch.binding_count = bindings_.size();
    launch.workspace = workspace_;
    launch.workspace_bytes = workspace_bytes_;
    launch.stream = stream_handle;
    launch.worker_count = workers_;
    launch.delay_rank = -1;
    launch.delay_task = -1;
    launch.delay_cycles = 0;
    auto fn = reinterpret_cast<int (*)(abi::PersistentLaunch const*, abi::ErrorInfo*)>(module_->library_->launch_symbol());
    rc = fn(&launch, &info);
  } else {
    abi::StreamedLaunch launch{bindings_.data(), bindings_.size(), stream_handle};
    auto fn = reinterpret_cast<int (*)(abi::StreamedLaunch const*, abi::ErrorInfo*)>(module_->library_->launch_symbol());
    rc = fn(&launch, &info);
  }
  if (rc) {
    failed_ = true;
    failure_ = info;
    // One entry point may launch several kernels and fail after the first, so work can be in
    // flight whatever `submitted` says: the tail is recorded on every failure outside a capture
    // (as src/native/runtime.cpp:232-238 does) and close() then waits for it.
    if (!capturing) {
      cudaEventRecord(tail_, stream);
      recorded_ = true;
      last_stream_ = stream;
    }
    throw RuntimeFailure("trinity_launch failed with code " + std::to_string(rc), info);
  }
  if (!capturing) {
    cuda_check("cudaEventRecord", cudaEventRecord(tail_, stream));
    recorded_ = true;
    last_stream_ = stream;
  } else {
    captured_ = true;
  }
}

void Execution::wait(double timeout_seconds) {
  cudaEvent_t tail;
  cudaStream_t stream;
  {
    std::lock_guard<std::recursive_mutex> lock(module_->mutex_);
    if (closed_ || !recorded_) return;
    tail = tail_;
    stream = last_stream_;
  }
  DeviceGuard guard(module_->device_);
  const auto start = std::chrono::steady_clock::now();
  for (;;) {
    const cudaError_t q = cudaEventQuery(tail);
    if (q == cudaSuccess) break;
    if (q != cudaErrorNotReady) cuda_fail("cudaEventQuery", q, true);
    if (timeout_seconds >= 0 &&
        std::chrono::duration<double>(std::chrono::steady_clock::now() - start).count() > timeout_seconds) {
      abi::ErrorInfo info{abi::runtime, abi::completion, -1001, 1u, abi::none, 0};
      throw RuntimeFailure("timed out waiting for completion; resources stay pinned", info);
    }
    std::this_thread::sleep_for(std::chrono::milliseconds(1));
  }
  std::lock_guard<std::recursive_mutex> lock(module_->mutex_);
  if (module_->library_) {
    abi::ErrorInfo info{};
    int rc;
    if (module_->mode_ == 2) {
      auto fn = reinterpret_cast<int (*)(void const*, void*, abi::ErrorInfo*)>(module_->library_->status_symbol());
      rc = fn(workspace_, stream, &info);
    } else {
      auto fn = reinterpret_cast<int (*)(void*, abi::ErrorInfo*)>(module_->library_->status_symbol());
      rc = fn(stream, &info);
    }
    if (rc) {
      failed_ = true;
      failure_ = info;
      throw RuntimeFailure("trinity_status reported code " + std::to_string(rc), info);
    }
  }
}

void Execution::close(bool wait_first) {
  if (closed_) return;
  if (graph_owner_) throw ResourceBusy("execution is owned by a graph");
  if (wait_first) {
    // An execution whose launch or completion failed still closes (its resources are released or
    // handed to the retire queue) and then reports the failure, as src/native/runtime.cpp:285-293
    // does: the caller learns that its results are not valid, and nothing stays pinned.
    try {
      wait(-1);
      if (failed_) throw RuntimeFailure("execution failed earlier", failure_);
    } catch (...) {
      reclaim();
      throw;
    }
  }
  reclaim();
}

void Execution::reclaim() {
  std::lock_guard<std::recursive_mutex> lock(module_->mutex_);
  if (closed_) return;
  DeviceGuard guard(module_->device_);
  closed_ = true;
  cudaEventDestroy(ready_);
  std::shared_ptr<Module> module = module_;
  if (pending()) {
    // Work is still running: the module (and through it the loaded library) stays referenced
    // until the tail event completes.
    RetireQueue::instance().defer(module->device_, tail_, [module] {
      std::lock_guard<std::recursive_mutex> l(module->mutex_);
      --module->executions_;
    });
  } else {
    cudaEventDestroy(tail_);
    --module->executions_;
  }
}

// ------------------------------------------------------------------ Graph
Graph::Graph(std::vector<std::shared_ptr<Execution>> executions, int device) : executions_(std::move(executions)), device_(device) {
  for (size_t i = 0; i < executions_.size(); ++i) {
    auto& e = executions_[i];
    std::lock_guard<std::recursive_mutex> lock(e->module_->mutex_);
    e->validate();
    if (e->graph_owner_) throw ResourceBusy("execution already belongs to a graph");
    if (e->module_->device_ != device) throw std::invalid_argument("graph executions must share one device");
    if (e->pending()) throw ResourceBusy("execution has pending work");
    for (size_t j = 0; j < i; ++j)
      if (executions_[j] == e) throw std::invalid_argument("duplicate execution in graph");
  }
  for (auto& e : executions_) e->graph_owner_ = this;
}

Graph::~Graph() {
  try {
    close();
  } catch (...) {
  }
}

void Graph::begin(void* stream_handle, bool capture) {
  DeviceGuard guard(device_);
  if (closed_) throw std::invalid_argument("graph is closed");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  if (!stream) throw std::invalid_argument("graph capture needs a non-default stream");
  cudaStreamCaptureStatus status = cudaStreamCaptureStatusNone;
  cuda_check("cudaStreamIsCapturing", cudaStreamIsCapturing(stream, &status));
  if (status != cudaStreamCaptureStatusNone) throw ResourceBusy("stream is already capturing");
  for (auto& e : executions_) {
    e->graph_active_ = true;
    e->captured_ = false;
  }
  if (capture) {
    const cudaError_t err = cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal);
    if (err != cudaSuccess) {
      for (auto& e : executions_) e->graph_active_ = false;
      cuda_fail("cudaStreamBeginCapture", err);
    }
    capturing_ = true;
  }
  stream_ = stream;
}

void Graph::end_warmup() {
  DeviceGuard guard(device_);
  for (auto& e : executions_) e->graph_active_ = false;
  cuda_check("cudaStreamSynchronize", cudaStreamSynchronize(stream_));
}

void Graph::abort() {
  DeviceGuard guard(device_);
  if (capturing_) {
    cudaGraph_t partial = nullptr;
    const cudaError_t err = cudaStreamEndCapture(stream_, &partial);
    if (partial) cudaGraphDestroy(partial);
    capturing_ = false;
    for (auto& e : executions_) e->graph_active_ = false;
    if (err != cudaSuccess && err != cudaErrorStreamCaptureInvalidated) {
      abi::ErrorInfo info{abi::driver, abi::configure, -1002, 0u, abi::none, 0};
      throw RuntimeFailure("capture could not be ended; the device is unusable for capture in this process", info);
    }
    return;
  }
  for (auto& e : executions_) e->graph_active_ = false;
}

void Graph::end_capture() {
  DeviceGuard guard(device_);
  if (!capturing_) throw std::invalid_argument("graph is not capturing");
  cudaGraph_t graph = nullptr;
  const cudaError_t err = cudaStreamEndCapture(stream_, &graph);
  capturing_ = false;
  for (auto& e : executions_) e->graph_active_ = false;
  if (err != cudaSuccess) {
    if (graph) cudaGraphDestroy(graph);
    abi::ErrorInfo info{abi::driver, abi::configure, int(err), 0u, abi::none, 0};
    throw RuntimeFailure(std::string("cudaStreamEndCapture: ") + cudaGetErrorString(err), info);
  }
  for (auto& e : executions_)
    if (!e->captured_) {
      cudaGraphDestroy(graph);
      throw std::invalid_argument("a graph execution was not run during capture");
    }
  const cudaError_t ierr = cudaGraphInstantiate(&exec_, graph, 0);
  cudaGraphDestroy(graph);
  cuda_check("cudaGraphInstantiate", ierr);
  cuda_check("cudaEventCreate", cudaEventCreateWithFlags(&tail_, cudaEventDisableTiming));
}

void Graph::replay(void* stream_handle) {
  DeviceGuard guard(device_);
  if (closed_ || !exec_) throw std::invalid_argument("graph is not ready");
  for (auto& e : executions_) e->validate();
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  if (recorded_ && cudaEventQuery(tail_) == cudaErrorNotReady && stream != last_stream_)
    throw ResourceBusy("graph has pending work on another stream");
  cuda_check("cudaGraphLaunch", cudaGraphLaunch(exec_, stream));
  cuda_check("cudaEventRecord", cudaEventRecord(tail_, stream));
  recorded_ = true;
  last_stream_ = stream;
}

void Graph::wait(double timeout_seconds) {
  if (!recorded_ || closed_) return;
  DeviceGuard guard(device_);
  const auto start = std::chrono::steady_clock::now();
  for (;;) {
    const cudaError_t q = cudaEventQuery(tail_);
    if (q == cudaSuccess) return;
    if (q != cudaErrorNotReady) cuda_fail("cudaEventQuery", q, true);
    if (timeout_seconds >= 0 &&
        std::chrono::duration<double>(std::chrono::steady_clock::now() - start).count() > timeout_seconds) {
      abi::ErrorInfo info{abi::runtime, abi::completion, -1001, 1u, abi::none, 0};
      throw RuntimeFailure("timed out waiting for graph completion; resources stay pinned", info);
    }
    std::this_thread::sleep_for(std::chrono::milliseconds(1));
  }
}

void Graph::close() {
  if (closed_) return;
  DeviceGuard guard(device_);
  if (capturing_) abort();
  closed_ = true;
  std::vector<std::shared_ptr<Execution>> executions = executions_;
  for (auto& e : executions) {
    e->graph_owner_ = nullptr;
    e->graph_active_ = false;
  }
  cudaGraphExec_t exec = exec_;
  exec_ = nullptr;
  if (recorded_ && cudaEventQuery(tail_) == cudaErrorNotReady) {
    // Replays still running: keep the executable graph and its executions until they finish.
    RetireQueue::instance().defer(device_, tail_, [exec, executions] {
      if (exec) cudaGraphExecDestroy(exec);
    });
  } else {
    if (tail_) cudaEventDestroy(tail_);
    if (exec) cudaGraphExecDestroy(exec);
  }
  tail_ = nullptr;
}

size_t collect_local() { return RetireQueue::instance().collect(); }
size_t retire_pending() { return RetireQueue::instance().pending(); }

}  // namespace trinity::host
