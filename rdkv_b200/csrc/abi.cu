// Library-level entry points of the C ABI: version, error text, struct size.
#include "rdkv_common.cuh"

extern "C" int rdkv_version(void) { return 1; }

extern "C" int rdkv_sizeof_layer_view(void) { return (int)sizeof(rdkv_layer_view); }
extern "C" int rdkv_sizeof_tail_args(void) { return (int)sizeof(rdkv_tail_args); }

extern "C" int rdkv_last_cuda_error(void) { return rdkv::g_last_cuda_error; }

extern "C" const char* rdkv_last_error_string(int status) {
  switch (status) {
    case RDKV_OK: return "ok";
    case RDKV_ERR_BAD_ARG: return "bad argument (null pointer, negative extent or unsupported dtype)";
    case RDKV_ERR_BAD_SHAPE: return "unsupported shape (head_dim, group size or channel padding)";
    case RDKV_ERR_TOO_LARGE: return "extent exceeds what the kernel or its scratch can hold";
    case RDKV_ERR_LAUNCH: return "CUDA launch failed (see rdkv_last_cuda_error)";
    case RDKV_ERR_NO_DEVICE: return "no CUDA device";
    default: return "unknown status";
  }
}
