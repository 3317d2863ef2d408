// Minimal program.so for loader tests: the five symbols with a COPY-free launch that only
// records calls.  Compile-time switches corrupt one aspect of the descriptor:
//   -DBAD_VERSION   descriptor.version is wrong
//   -DBAD_OFFSET    one launch-field offset is wrong
//   -DNO_STATUS     trinity_status is not exported
// A run-time switch makes one entry point fail on the host, with the codes of the reference's
// fixture (python/tests/fixtures/cuda_library.cu:16-19, :33-52 there):
//   TRINITY_FIXTURE_FAILURE=prepare | launch | release  ->  code 17 | 719 (submitted) | 19
#include <cstdlib>
#include <cstring>

#include "trinity_abi.h"

using namespace trinity::abi;

static const char kRequirements[] =
    "{\"target\":\"sm100\",\"world_size\":1,\"buffers\":[{\"value\":0,\"input_names\":[\"X\"],"
    "\"output_name\":\"Y\",\"shape\":[4],\"dtype\":\"fp32\",\"strides\":[1],\"bytes\":16,\"alignment\":4,"
    "\"external\":true,\"symmetric\":false}],\"workspace_bytes\":0,\"workspace_alignment\":1,"
    "\"workspace_symmetric\":false,\"cooperative_launch\":false,\"shared_memory_bytes\":0,"
    "\"block_threads\":128,\"nvshmem\":false,\"nvls\":false}";

static int launches = 0;

static bool fault(const char* mode) {
  const char* value = std::getenv("TRINITY_FIXTURE_FAILURE");
  return value && std::strcmp(value, mode) == 0;
}

#define EXPORT extern "C" __attribute__((visibility("default")))

EXPORT Descriptor const* trinity_abi() {
  static Descriptor d = describe(1, kRequirements, sizeof(kRequirements) - 1);
#ifdef BAD_VERSION
  d.version = 7;
#endif
#ifdef BAD_OFFSET
  d.offsets[2] += 8;
#endif
  return &d;
}
EXPORT int trinity_prepare(unsigned* workers, ErrorInfo* e) {
  *workers = 1;
  return report(e, driver, fault("prepare") ? 17 : 0, prepare);
}
EXPORT int trinity_launch(StreamedLaunch const*, ErrorInfo* e) {
  ++launches;
  return report(e, runtime, fault("launch") ? 719 : 0, launch, true);
}
#ifndef NO_STATUS
EXPORT int trinity_status(void*, ErrorInfo* e) { return report(e, none, 0, completion); }
#endif
EXPORT int trinity_release(ErrorInfo* e) { return report(e, driver, fault("release") ? 19 : 0, release); }
EXPORT int fixture_launches() { return launches; }
