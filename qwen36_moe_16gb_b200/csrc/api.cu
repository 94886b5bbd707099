// Probes of the b200moe C ABI: callable without a CUDA context.
#include "common.cuh"

#ifndef B200MOE_BUILD_ID
#define B200MOE_BUILD_ID "b200moe sm_100a " __DATE__ " " __TIME__
#endif

extern "C" int b200moe_abi_version(void) { return B200MOE_ABI_VERSION; }

extern "C" const char* b200moe_build_id(void) { return B200MOE_BUILD_ID; }

extern "C" const char* b200moe_error_string(int code) {
  switch (code) {
    case B200MOE_OK: return "ok";
    case B200MOE_E_NULL: return "b200moe: a required pointer is null";
    case B200MOE_E_SHAPE: return "b200moe: a size is outside what the kernels support";
    case B200MOE_E_ALIGN: return "b200moe: a pointer or stride is not 16-byte aligned";
    case B200MOE_E_WORKSPACE: return "b200moe: workspace too small";
    case B200MOE_E_DEVICE: return "b200moe: the current device is not sm_100";
    case B200MOE_E_STATIC_LIMIT:
      return "b200moe: M * top_k * intermediate needs more scratch than the static array holds "
             "(B200MOE_STATIC_SCRATCH_BYTES); use b200moe_decode_experts with a caller workspace";
    default: break;
  }
  if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
  return "b200moe: unknown error code";
}

// ---- host banks: page-lock a filled host buffer and look up the address the GPU reads it at ----------------
extern "C" int b200moe_host_register(void* addr, int64_t nbytes) {
  if (!addr || nbytes <= 0) return B200MOE_E_NULL;
  const cudaError_t e = cudaHostRegister(addr, (size_t)nbytes, cudaHostRegisterPortable | cudaHostRegisterMapped);
  return e == cudaSuccess ? 0 : (int)e;
}

extern "C" int b200moe_host_unregister(void* addr) {
  if (!addr) return B200MOE_E_NULL;
  const cudaError_t e = cudaHostUnregister(addr);
  return e == cudaSuccess ? 0 : (int)e;
}

extern "C" int b200moe_host_device_ptr(void* host_addr, void** device_addr) {
  if (!host_addr || !device_addr) return B200MOE_E_NULL;
  const cudaError_t e = cudaHostGetDevicePointer(device_addr, host_addr, 0);
  return e == cudaSuccess ? 0 : (int)e;
}
