/*
 * trinity_host.h -- C ABI of the host library (planner, emitter, artifact builder, runtime).
 *
 * The reference exposes the same functionality to Python through a PyO3 module (`_compiler`,
 * src/python.rs:726-753) and a pybind11 module (`_native`, src/native/bindings.cpp:12-90);
 * here both are one plain C surface over opaque handles so any FFI can bind it.
 * Functions that return a pointer return NULL on failure; functions that return int return 0
 * on success and non-zero on failure; th_last_error_* then describe the failure for the
 * calling thread.  Returned strings are owned by the handle they came from, or by the library
 * for th_last_error_message, and stay valid until the next call on that handle / thread.
 */
#ifndef TRINITY_HOST_H
#define TRINITY_HOST_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define TRINITY_HOST_API __attribute__((visibility("default")))
#else
#define TRINITY_HOST_API
#endif

/* Error classes; they map onto the exceptions the reference's Python package raises. */
enum th_error_kind {
  TH_OK = 0,
  TH_VALUE_ERROR = 1,        /* ValueError: invalid plan, invalid execution, bad argument        */
  TH_NOT_IMPLEMENTED = 2,    /* NotImplementedError: no provider, unsupported execution          */
  TH_RUNTIME_ERROR = 3,      /* RuntimeError                                                     */
  TH_TYPE_ERROR = 4,         /* TypeError                                                        */
  TH_RUNTIME_FAILURE = 5,    /* trinity_lowering.RuntimeFailure (carries ErrorInfo fields)       */
  TH_RESOURCE_BUSY = 6,      /* trinity_lowering.ResourceBusy                                    */
  TH_COMPILE_ERROR = 7       /* trinity_lowering.CompileError (carries diagnostics JSON)         */
};
TRINITY_HOST_API int th_last_error_kind(void);
TRINITY_HOST_API const char* th_last_error_message(void);
/* domain, stage, code, submitted, cleanup_domain, cleanup_code of the last RuntimeFailure */
TRINITY_HOST_API void th_last_error_info(int32_t out[6]);
TRINITY_HOST_API const char* th_last_error_diagnostics(void);

/* Where trinity_abi.h / trinity_sm100.h and libtrinity_sm100.so live. */
TRINITY_HOST_API void th_configure(const char* include_dir, const char* library_dir);

/* ---- planning (src/analysis/plan/builder.rs:26-94, src/python.rs:326-440) ---------------- */
typedef struct th_builder th_builder;
typedef struct th_plan th_plan;
TRINITY_HOST_API th_builder* th_builder_new(int world_size, const char* target);
TRINITY_HOST_API void th_builder_free(th_builder*);
TRINITY_HOST_API int th_builder_add_value(th_builder*, const char* dtype, const int64_t* shape, int rank,
                                          const char* storage, const char* name_or_null);
TRINITY_HOST_API int th_builder_bind_input(th_builder*, const char* name, int value);
TRINITY_HOST_API int th_builder_add_operation(th_builder*, const int* inflows, int n_in, const int* outflows,
                                              int n_out, const char* expression);
TRINITY_HOST_API int th_builder_add_loop(th_builder*, const char* kind, const char* variable, const char* start,
                                         const char* stop, const char* step, const int* body, int n_body);
TRINITY_HOST_API th_plan* th_builder_build(th_builder*, const int* statements, int n, const char* output_name,
                                           int output);
TRINITY_HOST_API void th_plan_free(th_plan*);
TRINITY_HOST_API const char* th_plan_metadata_json(th_plan*);
TRINITY_HOST_API const char* th_plan_symbols_json(th_plan*);
TRINITY_HOST_API const char* th_plan_structure(th_plan*);
TRINITY_HOST_API uint64_t th_plan_hash(th_plan*);
TRINITY_HOST_API int th_plan_world_size(th_plan*);
/* bindings_json: {"name": integer, ...} */
TRINITY_HOST_API th_plan* th_plan_bind_symbols(th_plan*, const char* const* names, const int64_t* values, int n);
/* lower_ir (src/analysis/plan/ir.rs:85-128): returns the number of plans, -1 on failure */
TRINITY_HOST_API int th_lower_ir(const char* text, const char* const* symbol_names, const int64_t* symbol_values,
                                 int n_symbols, const char* const* tensor_names, const char* const* tensor_dtypes,
                                 int n_tensors, const char* target, int world_size, th_plan** out, int capacity);

/* ---- emission (src/emit/mod.rs:67-69, src/emit/candidate.rs:107-207) ---------------------- */
typedef struct th_source th_source;
TRINITY_HOST_API th_source* th_emit(th_plan*);
TRINITY_HOST_API void th_source_free(th_source*);
TRINITY_HOST_API const char* th_source_code(th_source*);
TRINITY_HOST_API const char* th_source_requirements_json(th_source*);
TRINITY_HOST_API int th_source_launch_count(th_source*);
TRINITY_HOST_API const char* th_kernel_candidates_json(th_plan*);

/* ---- compile (src/compile/cuda/mod.rs:24-118, src/compile/cuda/artifact.rs:13-68) --------- */
typedef struct th_artifact th_artifact;
TRINITY_HOST_API th_artifact* th_compile(th_source*, const char* host_compiler_or_null,
                                         const char* library_dir_or_null);
TRINITY_HOST_API void th_artifact_free(th_artifact*); /* removes the directory unless persisted */
TRINITY_HOST_API const char* th_artifact_directory(th_artifact*);
TRINITY_HOST_API const char* th_artifact_path(th_artifact*);
TRINITY_HOST_API const char* th_artifact_manifest_json(th_artifact*);
TRINITY_HOST_API const char* th_artifact_diagnostics_json(th_artifact*);
TRINITY_HOST_API const char* th_artifact_code(th_artifact*);
TRINITY_HOST_API int th_artifact_close(th_artifact*);
TRINITY_HOST_API const char* th_artifact_persist(th_artifact*);

/* ---- runtime (src/native/runtime.cpp, src/native/core.hpp) --------------------------------- */
typedef struct th_module th_module;
typedef struct th_execution th_execution;
typedef struct th_graph th_graph;
/* Loader check without touching CUDA: private copy, dlopen, five symbols, descriptor layout
 * (src/native/core.hpp:60-99).  Returns the embedded requirements JSON or NULL. */
TRINITY_HOST_API const char* th_library_probe(const char* library_path, int mode);
TRINITY_HOST_API th_module* th_module_load(const char* library_path, int device, int mode);
TRINITY_HOST_API void th_module_free(th_module*);
TRINITY_HOST_API const char* th_module_requirements_json(th_module*);
TRINITY_HOST_API int th_module_prepare(th_module*, unsigned* maximum_workers);
TRINITY_HOST_API int th_module_close(th_module*);
TRINITY_HOST_API int th_module_live_executions(th_module*);
TRINITY_HOST_API th_execution* th_execution_create(th_module*, void* const* bindings, size_t count,
                                                   void* ready_stream);
/* Persistent (mode 2, multi-GPU) modules: the execution also owns the artifact's workspace, whose
 * first bytes hold the peer table (src/native/abi.h:27-40, src/native/runtime.cpp:215-221). */
TRINITY_HOST_API th_execution* th_execution_create_persistent(th_module*, void* const* bindings, size_t count,
                                                              void* workspace, size_t workspace_bytes,
                                                              unsigned workers, void* ready_stream);
TRINITY_HOST_API void th_execution_free(th_execution*);
TRINITY_HOST_API int th_execution_run(th_execution*, void* stream);
TRINITY_HOST_API int th_execution_wait(th_execution*, double timeout_seconds);
TRINITY_HOST_API int th_execution_close(th_execution*, int wait);
TRINITY_HOST_API int th_execution_closed(th_execution*);
TRINITY_HOST_API th_graph* th_graph_create(th_execution* const* executions, size_t count, int device);
TRINITY_HOST_API void th_graph_free(th_graph*);
TRINITY_HOST_API int th_graph_begin(th_graph*, void* stream, int capture);
TRINITY_HOST_API int th_graph_end_warmup(th_graph*);
TRINITY_HOST_API int th_graph_end_capture(th_graph*);
TRINITY_HOST_API int th_graph_abort(th_graph*);
TRINITY_HOST_API int th_graph_replay(th_graph*, void* stream);
TRINITY_HOST_API int th_graph_wait(th_graph*, double timeout_seconds);
TRINITY_HOST_API int th_graph_close(th_graph*);
TRINITY_HOST_API size_t th_collect_local(void);
TRINITY_HOST_API size_t th_retire_pending(void);
TRINITY_HOST_API int th_cuda_runtime_version(void);

#ifdef __cplusplus
}
#endif
#endif /* TRINITY_HOST_H */
