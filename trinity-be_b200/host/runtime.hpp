// Runtime types for compiled plans (see runtime.cpp for behaviour).
#pragma once

#include <functional>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/trinity_abi.h"

struct CUevent_st;
struct CUstream_st;
struct CUgraphExec_st;

namespace trinity::host {

// A call into the artifact, the driver or a completion wait failed.
struct RuntimeFailure : std::runtime_error {
  abi::ErrorInfo info;
  RuntimeFailure(const std::string& what, const abi::ErrorInfo& i) : std::runtime_error(what), info(i) {}
};
// The object is in use (live children, pending work on another stream, owned by a graph).
struct ResourceBusy : std::runtime_error {
  using std::runtime_error::runtime_error;
};

class Library {
 public:
  Library(const std::string& path, unsigned mode);
  ~Library();
  Library(const Library&) = delete;
  unsigned prepare();
  void release();
  bool prepared() const { return prepared_; }
  const std::string& requirements() const { return requirements_; }
  void* launch_symbol() const { return launch_; }
  void* status_symbol() const { return status_; }
  const std::string& private_copy() const { return copy_; }

 private:
  using AbiFn = const abi::Descriptor* (*)();
  using PrepareFn = int (*)(unsigned*, abi::ErrorInfo*);
  using ReleaseFn = int (*)(abi::ErrorInfo*);
  void cleanup();
  std::string directory_, copy_, requirements_;
  void* handle_ = nullptr;
  AbiFn abi_ = nullptr;
  PrepareFn prepare_ = nullptr;
  ReleaseFn release_ = nullptr;
  void* launch_ = nullptr;
  void* status_ = nullptr;
  bool prepared_ = false;
  unsigned workers_ = 0;
};

class Execution;
class Graph;

class Module {
 public:
  Module(const std::string& path, int device, unsigned mode);
  ~Module();
  unsigned prepare();
  void close();
  bool closed() const { return !library_; }
  int device() const { return device_; }
  unsigned mode() const { return mode_; }
  const std::string& requirements() const { return library_->requirements(); }
  int live_executions() const { return executions_; }

 private:
  friend class Execution;
  friend class Graph;
  std::recursive_mutex mutex_;
  std::unique_ptr<Library> library_;
  int device_;
  unsigned mode_;
  int executions_ = 0;
};

class Execution {
 public:
  // workspace / workspace_bytes / workers: only for persistent (mode 2) modules
  Execution(std::shared_ptr<Module> module, std::vector<void*> bindings, void* ready_stream,
            void* workspace = nullptr, size_t workspace_bytes = 0, unsigned workers = 1);
  ~Execution();
  void run(void* stream);
  void wait(double timeout_seconds);  // negative = no limit
  void close(bool wait_first);
  void reclaim();   // the closing part of close(): events destroyed or deferred, module released
  bool closed() const { return closed_; }
  bool failed() const { return failed_; }
  const abi::ErrorInfo& failure() const { return failure_; }

 private:
  friend class Graph;
  void validate() const;
  bool pending() const;
  std::shared_ptr<Module> module_;
  std::vector<void*> bindings_;
  void* workspace_ = nullptr;
  size_t workspace_bytes_ = 0;
  unsigned workers_ = 1;
  CUevent_st* ready_ = nullptr;
  CUevent_st* tail_ = nullptr;
  CUstream_st* last_stream_ = nullptr;
  bool recorded_ = false, closed_ = false, failed_ = false, captured_ = false;
  bool graph_active_ = false;
  Graph* graph_owner_ = nullptr;
  abi::ErrorInfo failure_{};
};

class Graph {
 public:
  Graph(std::vector<std::shared_ptr<Execution>> executions, int device);
  ~Graph();
  void begin(void* stream, bool capture);  // warm-up iteration (capture == false) or the capture
  void end_warmup();
  void end_capture();
  void abort();
  void replay(void* stream);
  void wait(double timeout_seconds);
  void close();
  bool closed() const { return closed_; }

 private:
  std::vector<std::shared_ptr<Execution>> executions_;
  int device_;
  CUstream_st* stream_ = nullptr;
  CUstream_st* last_stream_ = nullptr;
  CUgraphExec_st* exec_ = nullptr;
  CUevent_st* tail_ = nullptr;
  bool capturing_ = false, closed_ = false, recorded_ = false;
};

size_t collect_local();   // reclaim finished deferred work now; returns what is still pending
size_t retire_pending();

}  // namespace trinity::host
