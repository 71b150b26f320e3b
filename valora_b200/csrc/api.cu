// Library-level entry points: version, error strings, device binding.
#include "common.cuh"

extern "C" int vlr_version(void) { return 1; }

extern "C" int vlr_set_device(int device) {
  cudaError_t e = cudaSetDevice(device);
  return e == cudaSuccess ? VLR_OK : static_cast<int>(e);
}

extern "C" const char* vlr_error_string(int code) {
  switch (code) {
    case VLR_OK: return "ok";
    case VLR_ERR_NULL: return "a required pointer is NULL";
    case VLR_ERR_SHAPE: return "unsupported feature sizes or ranks";
    case VLR_ERR_DTYPE: return "dtype must be VLR_F16 or VLR_BF16";
    case VLR_ERR_ALIGN: return "a pointer or row pitch is not 16-byte aligned";
    case VLR_ERR_WORKSPACE: return "workspace too small";
    case VLR_ERR_RANGE: return "a count or capacity is out of range";
    case VLR_ERR_DRIVER: return "tensor-map encoding unavailable or failed";
    case VLR_ERR_UNSUPPORTED: return "not implemented in this build";
    case VLR_ERR_STATIC_LIMIT:
      return "batch exceeds the built-in scratch of vlr_pack_static (at most 8192 tokens and 1024 adapters)";
    default: break;
  }
  if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
  return "unknown error";
}
