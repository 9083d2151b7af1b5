// Error state and version of libb200seq (a library of its own: it is built without the quantized-LLaMA kernels).
#include "seq_common.cuh"

namespace b2l {

static thread_local char g_seq_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_seq_err, sizeof(g_seq_err), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
  set_error("%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
  (void)cudaGetLastError();
  return (int)e;
}

int sm_count() {
  int dev = 0, v = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
  return v;
}

}  // namespace b2l

extern "C" int b2l_seq_version(void) { return 100; }
extern "C" const char* b2l_seq_last_error(void) { return b2l::g_seq_err; }

extern "C" int b2l_seq_zero_slot(void* state, size_t slot_bytes, int slot, b2l_stream_t stream) {
  B2L_CHECK_ARG(state != nullptr && slot >= 0, "b2l_seq_zero_slot: null pointer or negative slot");
  if (slot_bytes == 0) return 0;
  B2L_CUDA(cudaMemsetAsync(static_cast<char*>(state) + (size_t)slot * slot_bytes, 0, slot_bytes, (cudaStream_t)stream));
  return 0;
}
