// bf16 instantiation of the GEMV kernels (gemv_kernels.cuh)
#include "gemv_kernels.cuh"

MUI_STATUS_ACCESSOR(gemv_bf16)

mui_status_t mui_launch_gemv_bf16(cudaStream_t stream, int mode, const GemvArgs& a, int nb, unsigned flags,
                                  const MuiDeviceInfo* dev) {
  return launch_gemv_dt<__nv_bfloat16>(stream, mode, a, nb, flags, dev);
}
