// Entry points whose kernels are being written: they refuse every call.
#include "host_common.h"
using namespace trinity_sm100;
extern "C" size_t trinity_sm100_mla_scratch_bytes(int32_t, int32_t, int32_t, int32_t) { return 0; }
extern "C" int trinity_sm100_mla_default_splits(int32_t, int32_t) { return 1; }
extern "C" int trinity_sm100_mla_decode_bf16(const trinity_sm100_mla*, void*) {
  return fail(TRINITY_SM100_E_UNSUPPORTED, "mla decode kernel not built yet");
}
extern "C" size_t trinity_sm100_allreduce_flag_words(void) { return 0; }
extern "C" int trinity_sm100_allreduce_bf16(const trinity_sm100_allreduce*, void*) {
  return fail(TRINITY_SM100_E_UNSUPPORTED, "all-reduce kernel not built yet");
}
