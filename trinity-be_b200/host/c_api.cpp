// C surface of the host library: exception-to-error-code translation over opaque handles.
#include <cuda_runtime_api.h>

#include <cstring>
#include <memory>

#include "../../include/trinity_host.h"
#include "artifact.hpp"
#include "emit.hpp"
#include "plan.hpp"
#include "runtime.hpp"

using namespace trinity::host;

namespace trinity::host {
extern std::string g_include_dir;
extern std::string g_library_dir;
}  // namespace trinity::host

struct th_builder { PlanBuilder builder; };
struct th_plan { PhysicalPlan plan; std::string metadata, symbols, structure; };
struct th_source { CudaSource source; };
struct th_artifact { Artifact artifact; bool closed = false, persisted = false; };
struct th_module { std::shared_ptr<Module> module; std::string requirements; };
struct th_execution { std::shared_ptr<Execution> execution; };
struct th_graph { std::unique_ptr<Graph> graph; };

namespace {
thread_local int t_kind = TH_OK;
thread_local std::string t_message;
thread_local std::string t_diagnostics;
thread_local int32_t t_info[6] = {0, 0, 0, 0, 0, 0};
thread_local std::string t_text;

void set_error(int kind, const std::string& message) {
  t_kind = kind;
  t_message = message;
}

template <class F>
auto guarded(F&& fn, decltype(fn()) failure) -> decltype(fn()) {
  t_kind = TH_OK;
  try {
    return fn();
  } catch (const PlanError& e) {
    set_error(int(e.kind), e.what());
  } catch (const SyntaxError& e) {
    set_error(TH_VALUE_ERROR, e.what());
  } catch (const CompileFailure& e) {
    set_error(TH_COMPILE_ERROR, e.what());
    t_diagnostics = e.diagnostics_json;
  } catch (const RuntimeFailure& e) {
    set_error(TH_RUNTIME_FAILURE, e.what());
    t_info[0] = int32_t(e.info.domain); t_info[1] = int32_t(e.info.stage); t_info[2] = e.info.code;
    t_info[3] = int32_t(e.info.submitted); t_info[4] = int32_t(e.info.cleanup_domain); t_info[5] = e.info.cleanup_code;
  } catch (const ResourceBusy& e) {
    set_error(TH_RESOURCE_BUSY, e.what());
  } catch (const std::invalid_argument& e) {
    set_error(TH_VALUE_ERROR, e.what());
  } catch (const std::exception& e) {
    set_error(TH_RUNTIME_ERROR, e.what());
  }
  return failure;
}
}  // namespace

extern "C" {

int th_last_error_kind(void) { return t_kind; }
const char* th_last_error_message(void) { return t_message.c_str(); }
void th_last_error_info(int32_t out[6]) { memcpy(out, t_info, sizeof t_info); }
const char* th_last_error_diagnostics(void) { return t_diagnostics.c_str(); }

void th_configure(const char* include_dir, const char* library_dir) {
  if (include_dir) g_include_dir = include_dir;
  if (library_dir) g_library_dir = library_dir;
}

// ---------------------------------------------------------------- planning
th_builder* th_builder_new(int world_size, const char* target) {
  return guarded([&]() -> th_builder* { return new th_builder{PlanBuilder(world_size, parse_target(target ? target : "hopper"))}; }, nullptr);
}
void th_builder_free(th_builder* b) { delete b; }
int th_builder_add_value(th_builder* b, const char* dtype, const int64_t* shape, int rank, const char* storage,
                         const char* name) {
  return guarded([&] {
    return b->builder.add_value(parse_dtype(dtype), std::vector<int64_t>(shape, shape + rank), parse_storage(storage),
                                name ? name : "");
  }, -1);
}
int th_builder_bind_input(th_builder* b, const char* name, int value) {
  return guarded([&] { b->builder.bind_input(name, value); return 0; }, -1);
}
int th_builder_add_operation(th_builder* b, const int* inflows, int n_in, const int* outflows, int n_out,
                             const char* expression) {
  return guarded([&] {
    return b->builder.add_operation(std::vector<int>(inflows, inflows + n_in), std::vector<int>(outflows, outflows + n_out),
                                    expression);
  }, -1);
}
int th_builder_add_loop(th_builder* b, const char* kind, const char* variable, const char* start, const char* stop,
                        const char* step, const int* body, int n_body) {
  return guarded([&] { return b->builder.add_loop(kind, variable, start, stop, step, std::vector<int>(body, body + n_body)); }, -1);
}
th_plan* th_builder_build(th_builder* b, const int* statements, int n, const char* output_name, int output) {
  return guarded([&]() -> th_plan* {
    return new th_plan{b->builder.build(std::vector<int>(statements, statements + n), output_name, output), "", "", ""};
  }, nullptr);
}
void th_plan_free(th_plan* p) { delete p; }
const char* th_plan_metadata_json(th_plan* p) {
  p->metadata = p->plan.metadata_json();
  return p->metadata.c_str();
}
const char* th_plan_symbols_json(th_plan* p) {
  std::string s = "[";
  bool first = true;
  for (auto& name : p->plan.symbols()) {
    s += (first ? "\"" : ",\"") + json_escape(name) + "\"";
    first = false;
  }
  p->symbols = s + "]";
  return p->symbols.c_str();
}
const char* th_plan_structure(th_plan* p) {
  p->structure = p->plan.structure_text();
  return p->structure.c_str();
}
uint64_t th_plan_hash(th_plan* p) { return p->plan.hash(); }
int th_plan_world_size(th_plan* p) { return p->plan.world_size; }
th_plan* th_plan_bind_symbols(th_plan* p, const char* const* names, const int64_t* values, int n) {
  return guarded([&]() -> th_plan* {
    std::map<std::string, int64_t> bindings;
    for (int i = 0; i < n; ++i) bindings[names[i]] = values[i];
    return new th_plan{p->plan.bind_symbols(bindings), "", "", ""};
  }, nullptr);
}
int th_lower_ir(const char* text, const char* const* symbol_names, const int64_t* symbol_values, int n_symbols,
                const char* const* tensor_names, const char* const* tensor_dtypes, int n_tensors, const char* target,
                int world_size, th_plan** out, int capacity) {
  return guarded([&] {
    std::map<std::string, int64_t> symbols;
    for (int i = 0; i < n_symbols; ++i) symbols[symbol_names[i]] = symbol_values[i];
    std::map<std::string, std::string> dtypes;
    for (int i = 0; i < n_tensors; ++i) dtypes[tensor_names[i]] = tensor_dtypes[i];
    std::vector<PhysicalPlan> plans = lower_ir(text, symbols, dtypes, parse_target(target ? target : "hopper"), world_size);
    if (int(plans.size()) > capacity) invalid("lower_ir produced more plans than the caller can take");
    for (size_t i = 0; i < plans.size(); ++i) out[i] = new th_plan{std::move(plans[i]), "", "", ""};
    return int(plans.size());
  }, -1);
}

// ---------------------------------------------------------------- emission
th_source* th_emit(th_plan* p) {
  return guarded([&]() -> th_source* { return new th_source{emit(p->plan)}; }, nullptr);
}
void th_source_free(th_source* s) { delete s; }
const char* th_source_code(th_source* s) { return s->source.code.c_str(); }
const char* th_source_requirements_json(th_source* s) { return s->source.requirements_json.c_str(); }
int th_source_launch_count(th_source* s) { return int(s->source.launches.size()); }
const char* th_kernel_candidates_json(th_plan* p) {
  t_text = kernel_candidates_json(p->plan);
  return t_text.c_str();
}

// ---------------------------------------------------------------- compile
th_artifact* th_compile(th_source* s, const char* host_compiler, const char* library_dir) {
  return guarded([&]() -> th_artifact* {
    CompileConfig config;
    if (host_compiler) config.host_compiler = host_compiler;
    if (library_dir) config.library_dir = library_dir;
    return new th_artifact{compile(s->source, config)};
  }, nullptr);
}
int th_artifact_close(th_artifact* a) {
  if (!a->closed && !a->persisted) remove_artifact_directory(a->artifact.directory);
  a->closed = true;
  return 0;
}
void th_artifact_free(th_artifact* a) {
  if (!a) return;
  th_artifact_close(a);
  delete a;
}
const char* th_artifact_directory(th_artifact* a) { return a->artifact.directory.c_str(); }
const char* th_artifact_path(th_artifact* a) { return a->artifact.artifact_path.c_str(); }
const char* th_artifact_manifest_json(th_artifact* a) { return a->artifact.manifest_json.c_str(); }
const char* th_artifact_diagnostics_json(th_artifact* a) { return a->artifact.diagnostics_json.c_str(); }
const char* th_artifact_code(th_artifact* a) { return a->artifact.code.c_str(); }
const char* th_artifact_persist(th_artifact* a) {
  a->persisted = true;
  return a->artifact.directory.c_str();
}

// ---------------------------------------------------------------- runtime
const char* th_library_probe(const char* path, int mode) {
  return guarded([&]() -> const char* {
    Library library(path, unsigned(mode));
    t_text = library.requirements();
    return t_text.c_str();
  }, nullptr);
}
th_module* th_module_load(const char* path, int device, int mode) {
  return guarded([&]() -> th_module* {
    auto m = std::make_shared<Module>(path, device, unsigned(mode));
    return new th_module{m, m->requirements()};
  }, nullptr);
}
void th_module_free(th_module* m) { delete m; }
const char* th_module_requirements_json(th_module* m) { return m->requirements.c_str(); }
int th_module_prepare(th_module* m, unsigned* maximum_workers) {
  return guarded([&] {
    const unsigned w = m->module->prepare();
    if (maximum_workers) *maximum_workers = w;
    return 0;
  }, -1);
}
int th_module_close(th_module* m) { return guarded([&] { m->module->close(); return 0; }, -1); }
int th_module_live_executions(th_module* m) { return m->module->live_executions(); }
th_execution* th_execution_create(th_module* m, void* const* bindings, size_t count, void* ready_stream) {
  return guarded([&]() -> th_execution* {
    return new th_execution{std::make_shared<Execution>(m->module, std::vector<void*>(bindings, bindings + count), ready_stream)};
  }, nullptr);
}
th_execution* th_execution_create_persistent(th_module* m, void* const* bindings, size_t count, void* workspace,
                                             size_t workspace_bytes, unsigned workers, void* ready_stream) {
  return guarded([&]() -> th_execution* {
    return new th_execution{std::make_shared<Execution>(m->module, std::vector<void*>(bindings, bindings + count),
                                                        ready_stream, workspace, workspace_bytes, workers)};
  }, nullptr);
}
void th_execution_free(th_execution* e) { delete e; }
int th_execution_run(th_execution* e, void* stream) { return guarded([&] { e->execution->run(stream); return 0; }, -1); }
int th_execution_wait(th_execution* e, double timeout) { return guarded([&] { e->execution->wait(timeout); return 0; }, -1); }
int th_execution_close(th_execution* e, int wait) { return guarded([&] { e->execution->close(wait != 0); return 0; }, -1); }
int th_execution_closed(th_execution* e) { return e->execution->closed() ? 1 : 0; }
th_graph* th_graph_create(th_execution* const* executions, size_t count, int device) {
  return guarded([&]() -> th_graph* {
    std::vector<std::shared_ptr<Execution>> list;
    for (size_t i = 0; i < count; ++i) list.push_back(executions[i]->execution);
    return new th_graph{std::make_unique<Graph>(std::move(list), device)};
  }, nullptr);
}
void th_graph_free(th_graph* g) { delete g; }
int th_graph_begin(th_graph* g, void* stream, int capture) { return guarded([&] { g->graph->begin(stream, capture != 0); return 0; }, -1); }
int th_graph_end_warmup(th_graph* g) { return guarded([&] { g->graph->end_warmup(); return 0; }, -1); }
int th_graph_end_capture(th_graph* g) { return guarded([&] { g->graph->end_capture(); return 0; }, -1); }
int th_graph_abort(th_graph* g) { return guarded([&] { g->graph->abort(); return 0; }, -1); }
int th_graph_replay(th_graph* g, void* stream) { return guarded([&] { g->graph->replay(stream); return 0; }, -1); }
int th_graph_wait(th_graph* g, double timeout) { return guarded([&] { g->graph->wait(timeout); return 0; }, -1); }
int th_graph_close(th_graph* g) { return guarded([&] { g->graph->close(); return 0; }, -1); }
size_t th_collect_local(void) { return collect_local(); }
size_t th_retire_pending(void) { return retire_pending(); }
int th_cuda_runtime_version(void) {
  int v = 0;
  cudaRuntimeGetVersion(&v);
  return v;
}

}  // extern "C"
