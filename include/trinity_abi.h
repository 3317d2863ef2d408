/*
 * trinity_abi.h -- the five-symbol host ABI of a compiled plan ("program.so").
 *
 * Layout-compatible, field for field, with the reference's artifact ABI
 * (youngchan2/Trinity-BE, src/native/abi.h:11-85): an artifact built against this header is
 * accepted by the reference loader's layout check (src/native/core.hpp:80-97) and vice versa.
 * This text is embedded verbatim into every generated program and shared with the loader.
 *
 * A program exports exactly:
 *   trinity::abi::Descriptor const* trinity_abi();
 *   int trinity_prepare(unsigned* maximum_workers, trinity::abi::ErrorInfo*);
 *   int trinity_launch(trinity::abi::StreamedLaunch const*, trinity::abi::ErrorInfo*);   // mode 1
 *   int trinity_status(void* stream, trinity::abi::ErrorInfo*);                          // mode 1
 *   int trinity_release(trinity::abi::ErrorInfo*);
 * (mode 2 programs take PersistentLaunch in trinity_launch and an extra workspace pointer in
 *  trinity_status; src/native/runtime.cpp:215-221,246-251).
 * Every function returns 0 on success and otherwise the value it stored in ErrorInfo::code.
 */
#ifndef TRINITY_B200_PROGRAM_ABI_H
#define TRINITY_B200_PROGRAM_ABI_H

#include <cstddef>
#include <cstdint>
#include <type_traits>

namespace trinity {
namespace abi {

constexpr std::uint32_t version = 1;

/* Who failed, and while doing what. */
enum Domain : std::uint32_t { none = 0, generated = 1, runtime = 2, driver = 3, transport = 4 };
enum Stage : std::uint32_t {
  idle = 0, validate = 1, prepare = 2, configure = 3, registration = 4, initialization = 5,
  launch = 6, completion = 7, release = 8
};

struct ErrorInfo {
  std::uint32_t domain;
  std::uint32_t stage;
  std::int32_t code;
  std::uint32_t submitted;       /* non-zero: GPU work may already be in flight */
  std::uint32_t cleanup_domain;
  std::int32_t cleanup_code;
};

struct StreamedLaunch {
  void* const* bindings;         /* dense array of device pointers in buffer-slot order */
  std::size_t binding_count;
  void* stream;                  /* cudaStream_t */
};

struct PersistentLaunch {
  void* const* bindings;
  std::size_t binding_count;
  void* workspace;
  std::size_t workspace_bytes;
  void* stream;
  unsigned worker_count;
  int delay_rank;
  int delay_task;
  unsigned long long delay_cycles;
};

struct Descriptor {
  std::uint32_t version, mode, pointer_size, error_size, error_alignment;
  std::uint32_t launch_size, launch_alignment, field_count;
  std::uint32_t offsets[9];
  std::uint32_t error_offsets[6];
  char const* requirements;      /* JSON text, not NUL-terminated by contract */
  std::size_t requirements_size;
};

static_assert(std::is_standard_layout<ErrorInfo>::value && std::is_standard_layout<Descriptor>::value &&
                  std::is_standard_layout<StreamedLaunch>::value &&
                  std::is_standard_layout<PersistentLaunch>::value,
              "ABI structs must be standard layout");

/* Fills a descriptor that describes this compilation unit's view of the structs above. */
inline Descriptor describe(unsigned mode, char const* requirements, std::size_t size) {
  Descriptor d = {};
  d.version = version;
  d.mode = mode;
  d.pointer_size = sizeof(void*);
  d.error_size = sizeof(ErrorInfo);
  d.error_alignment = alignof(ErrorInfo);
  d.requirements = requirements;
  d.requirements_size = size;
  d.error_offsets[0] = offsetof(ErrorInfo, domain);
  d.error_offsets[1] = offsetof(ErrorInfo, stage);
  d.error_offsets[2] = offsetof(ErrorInfo, code);
  d.error_offsets[3] = offsetof(ErrorInfo, submitted);
  d.error_offsets[4] = offsetof(ErrorInfo, cleanup_domain);
  d.error_offsets[5] = offsetof(ErrorInfo, cleanup_code);
  if (mode == 1) {
    d.launch_size = sizeof(StreamedLaunch);
    d.launch_alignment = alignof(StreamedLaunch);
    d.field_count = 3;
    d.offsets[0] = offsetof(StreamedLaunch, bindings);
    d.offsets[1] = offsetof(StreamedLaunch, binding_count);
    d.offsets[2] = offsetof(StreamedLaunch, stream);
  } else {
    d.launch_size = sizeof(PersistentLaunch);
    d.launch_alignment = alignof(PersistentLaunch);
    d.field_count = 9;
    d.offsets[0] = offsetof(PersistentLaunch, bindings);
    d.offsets[1] = offsetof(PersistentLaunch, binding_count);
    d.offsets[2] = offsetof(PersistentLaunch, workspace);
    d.offsets[3] = offsetof(PersistentLaunch, workspace_bytes);
    d.offsets[4] = offsetof(PersistentLaunch, stream);
    d.offsets[5] = offsetof(PersistentLaunch, worker_count);
    d.offsets[6] = offsetof(PersistentLaunch, delay_rank);
    d.offsets[7] = offsetof(PersistentLaunch, delay_task);
    d.offsets[8] = offsetof(PersistentLaunch, delay_cycles);
  }
  return d;
}

/* Stores an outcome and returns its code; a zero code clears the domain. */
inline int report(ErrorInfo* out, Domain domain, int code, Stage stage, bool submitted = false) {
  if (out) {
    out->domain = code ? domain : none;
    out->stage = stage;
    out->code = code;
    out->submitted = submitted ? 1u : 0u;
    out->cleanup_domain = none;
    out->cleanup_code = 0;
  }
  return code;
}

}  // namespace abi
}  // namespace trinity

#endif /* TRINITY_B200_PROGRAM_ABI_H */
