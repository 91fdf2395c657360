// placeholder: attention entry points (kernel lands next)
#include "common.cuh"
extern "C" {
int oasr_b200_fmha(void*, const void*, const void*, const void*, const void*, int64_t, int64_t, int64_t,
                   const int32_t*, const int32_t*, const int32_t*, int64_t, int64_t, int64_t, int64_t, int64_t,
                   int64_t, int64_t, int64_t, double, int, int, void*) {
  return ob::set_error(OASR_ERR_UNSUPPORTED, "fmha: not built yet");
}
int oasr_b200_fmha_varlen(void*, const void*, const void*, const void*, const void*, const void*, int,
                          const int32_t*, const int32_t*, int64_t, int64_t, int64_t, int64_t, int64_t, double, int,
                          void*) {
  return ob::set_error(OASR_ERR_UNSUPPORTED, "fmha_varlen: not built yet");
}
}
