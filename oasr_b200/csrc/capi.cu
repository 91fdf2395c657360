// Library-level entry points: version, per-thread error message, device status word.
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "device_status.cuh"

namespace ob {

static thread_local char g_err[1024] = {0};

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

static unsigned long long g_launches = 0;  // kernels launched through this library (host-side count)

int check_launch(const char* what) {
  ++g_launches;
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    return set_error(OASR_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  }
  return OASR_OK;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// One status word per device, living in device memory for the life of the
// library.  Kernels with bounded waits OR a code into it when a wait gives up.
__device__ uint32_t g_device_status_word = 0;

uint32_t* device_status_ptr() {
  static uint32_t* ptrs[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (ptrs[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_device_status_word) != cudaSuccess) return nullptr;
    ptrs[dev] = static_cast<uint32_t*>(p);
  }
  return ptrs[dev];
}

namespace conv2_pair { extern int g_enabled; }
namespace gemm { extern int g_force_bn; extern int g_use_pairs; extern int g_lsm_path; }
extern int g_dw_path;
extern int g_fmha_relpos_path;
unsigned long long* g_trace_buffer = nullptr;   // diagnostics: device buffer that instrumented kernels stamp their phases into
int g_pdl = 1;  // programmatic stream serialisation for the kernels launched through launch_pdl (a kernel's set-up runs while the
                // previous one drains): offline step 6.29 against 6.38 ms with every GEMM-shaped kernel on it; neutral on the
                // graph-replayed streaming step (2.91 ms) and on the FastConformer step (51.5 ms)
extern int g_fmha_chunk_path;
extern int g_fused_addnorm;
extern int g_qkv_dup;
namespace conv1_mma { extern int g_enabled; }

}  // namespace ob

extern "C" {

int oasr_b200_set_tunable(const char* name, int value) {
  if (name && std::strcmp(name, "gemm_bn") == 0) {
    if (value != 0 && value != 64 && value != 128 && value != 256)
      return ob::set_error(OASR_ERR_INVALID, "gemm_bn must be 0, 64, 128 or 256 (got %d)", value);
    ob::gemm::g_force_bn = value;
    return OASR_OK;
  }
  if (name && std::strcmp(name, "lsm_path") == 0) {
    if (value < 0 || value > 2) return ob::set_error(OASR_ERR_INVALID, "lsm_path must be 0, 1 or 2 (got %d)", value);
    ob::gemm::g_lsm_path = value;
    return OASR_OK;
  }
  if (name && std::strcmp(name, "gemm_pairs") == 0) {
    ob::gemm::g_use_pairs = value != 0;
    return OASR_OK;
  }
  if (name && std::strcmp(name, "fmha_chunk_path") == 0) {
    ob::g_fmha_chunk_path = value != 0;
    return OASR_OK;
  }
  if (name && std::strcmp(name, "fmha_relpos_path") == 0) {
    ob::g_fmha_relpos_path = value != 0;
    return OASR_OK;
  }
  if (name && std::strcmp(name, "qkv_dup") == 0) {
    ob::g_qkv_dup = value != 0;
    return OASR_OK;
  }
  if (name && std::strcmp(name, "pdl") == 0) {
    ob::g_pdl = value != 0;
    return OASR_OK;
  }
  if (name && std::strcmp(name, "conv2_pairs") == 0) {
    ob::conv2_pair::g_enabled = value != 0;
    return OASR_OK;
  }
  if (name && std::strcmp(name, "fused_addnorm") == 0) {
    if (value < 0 || value > 2) return ob::set_error(OASR_ERR_INVALID, "fused_addnorm must be 0, 1 or 2 (got %d)", value);
    ob::g_fused_addnorm = value;
    return OASR_OK;
  }
  if (name && std::strcmp(name, "conv1_mma") == 0) {
    ob::conv1_mma::g_enabled = value != 0;
    return OASR_OK;
  }
  if (name && std::strcmp(name, "dwconv_path") == 0) {
    ob::g_dw_path = value;
    return OASR_OK;
  }
  return ob::set_error(OASR_ERR_INVALID, "unknown tunable '%s'", name ? name : "(null)");
}

unsigned long long oasr_b200_launch_count(void) { return ob::g_launches; }

int oasr_b200_trace_buffer(void* device_buffer) {
  ob::g_trace_buffer = static_cast<unsigned long long*>(device_buffer);
  return OASR_OK;
}

const char* oasr_b200_version(void) { return "oasr_b200 0.1.0 sm_100a"; }

const char* oasr_b200_last_error(void) { return ob::g_err; }

int oasr_b200_device_status(uint32_t* word, void* stream) {
  uint32_t* dptr = ob::device_status_ptr();
  if (dptr == nullptr) return ob::set_error(OASR_ERR_CUDA, "device status word is not addressable");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint32_t h = 0;
  cudaError_t e = cudaMemcpyAsync(&h, dptr, sizeof(h), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return ob::set_error(OASR_ERR_CUDA, "device status read: %s", cudaGetErrorString(e));
  if (word) *word = h;
  if (h != 0) {
    cudaMemsetAsync(dptr, 0, sizeof(h), s);
    cudaStreamSynchronize(s);
    return ob::set_error(OASR_ERR_DEVICE_WAIT, "a kernel gave up a bounded wait (status word 0x%08x)", h);
  }
  return OASR_OK;
}

}  // extern "C"
