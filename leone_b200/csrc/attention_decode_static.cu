// The allocation-free variant of the split-KV decode attention: see leone_static.h for who it
// is for, what it costs and how calls share its scratch.  The kernels are the ones of
// attention_tiled.cu, compiled into this library a second time; only where the scratch comes
// from differs.
#include <stdio.h>

#include "attention_tiled.cu"
#include "leone_static.h"

// The scratch itself.  In host code this name is only a handle for the runtime; its device
// address is looked up below and that pointer is what the kernels get.
static __device__ __align__(256) float leone_static_scratch[LEONE_STATIC_SCRATCH_FLOATS];

namespace {

constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {nullptr};

void set_error(char* error, int error_len, const char* text) {
  if (error != nullptr && error_len > 0) snprintf(error, (size_t)error_len, "%s", text);
}

// Once per device, with that device current: the array's address on this device.
int scratch_for_current_device(float** ptr, char* error, int error_len) {
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess || device < 0 || device >= kMaxDevices) {
    set_error(error, error_len, "leone_attention_decode_static: cannot tell the current device");
    return LEONE_STATIC_SETUP_FAILED;
  }
  if (g_scratch_ptr[device] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, leone_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      char text[160];
      snprintf(text, sizeof(text), "leone_attention_decode_static: cudaGetSymbolAddress failed: %s",
               cudaGetErrorString(e));
      set_error(error, error_len, text);
      return LEONE_STATIC_SETUP_FAILED;
    }
    g_scratch_ptr[device] = p;
  }
  *ptr = g_scratch_ptr[device];
  return 0;
}

}  // namespace

extern "C" int leone_attention_decode_static(const void* qkv, int row_stride, void* out,
                                             int out_stride, const void* k_pool, const void* v_pool,
                                             const int* block_table, int table_width,
                                             const int* q_start, const int* ctx_len, int n_seqs,
                                             int n_q, int n_kv, int d, float scale, int window,
                                             int page_tokens, int num_pages, int splits, int* status,
                                             char* error, int error_len, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (splits < 1 || n_q <= 0 || d <= 0) {
    set_error(error, error_len, "leone_attention_decode_static: sizes must be positive");
    return kRefusedSize;
  }
  const long long need = leone_attention_decode_scratch(n_seqs, n_q, d, splits);
  if (need > (long long)LEONE_STATIC_SCRATCH_FLOATS) {
    char text[200];
    snprintf(text, sizeof(text),
             "leone_attention_decode_static: %d sequences x %d heads x %d splits x (%d + 2) = %lld "
             "floats of scratch, the static array holds %d",
             n_seqs, n_q, splits, d, need, (int)LEONE_STATIC_SCRATCH_FLOATS);
    set_error(error, error_len, text);
    return LEONE_STATIC_TOO_LARGE;
  }
  float* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch, error, error_len);
  if (rc != 0) return rc;
  const int code = leone_attention_decode(qkv, row_stride, out, out_stride, k_pool, v_pool,
                                          block_table, table_width, q_start, ctx_len, n_seqs, n_q,
                                          n_kv, d, scale, window, page_tokens, num_pages, splits,
                                          scratch, status, stream);
  if (code < 0) set_error(error, error_len, "leone_attention_decode_static: the kernel refuses these sizes");
  if (code > 0) {
    char text[160];
    snprintf(text, sizeof(text), "leone_attention_decode_static: launch failed: %s",
             cudaGetErrorString((cudaError_t)code));
    set_error(error, error_len, text);
  }
  return code;
}
