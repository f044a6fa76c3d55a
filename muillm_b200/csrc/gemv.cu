// Entry point of the GEMV-shaped kernels: validated arguments in, one launch (or two half-batch launches) out. The
// kernels live in gemv_kernels.cuh and are instantiated per element type in gemv_f16.cu / gemv_bf16.cu.
#include "gemv_kernels.cuh"

mui_status_t mui_launch_gemv_f16(cudaStream_t stream, int mode, const GemvArgs& a, int nb, unsigned flags,
                                 const MuiDeviceInfo* dev);
mui_status_t mui_launch_gemv_bf16(cudaStream_t stream, int mode, const GemvArgs& a, int nb, unsigned flags,
                                  const MuiDeviceInfo* dev);

// Launches MODE 0 (linear) or MODE 1 (gate/up) on validated arguments; a.w8_fmt < 0 means 16-bit weights.
mui_status_t mui_launch_gemv16(cudaStream_t stream, mui_dtype_t dtype, int mode, const GemvArgs& a_in, unsigned flags) {
  const MuiDeviceInfo* dev = mui_current_device_info();
  if (!dev) return MUI_ERR_CUDA;
  GemvArgs a = a_in;
  if (a.trace == nullptr) a.trace = mui_trace_next_record(mode == 0 ? 1 : 2);
  const int nb = a.B <= 1 ? 1 : (a.B <= 2 ? 2 : (a.B <= 4 ? 4 : 8));
  // The pipeline stages a batch's activations chunk by chunk. The plain-load kernel (odd K, unaligned pointers, the
  // per-group 8-bit format, or when forced) stages whole rows: when those cannot fit, it runs the batch in two
  // halves (the weights are then streamed twice).
  const int kstep = (a.w8_fmt < 0) ? 16 : 32;
  const bool pipeline_ok = !(flags & MUI_FLAG_FORCE_GENERIC) && (a.K % kstep) == 0 &&
                           ((reinterpret_cast<uintptr_t>(a.W) & 15) == 0) &&
                           (mode == 0 || (reinterpret_cast<uintptr_t>(a.W2) & 15) == 0) &&
                           (a.w8_fmt < 0 || a.w8_fmt == MUI_W8_SYM_ROW) &&
                           ((reinterpret_cast<uintptr_t>(a.x) & 15) == 0) &&
                           (a.norm_w == nullptr || (reinterpret_cast<uintptr_t>(a.norm_w) & 15) == 0);
  // per-group 8-bit format: its pipeline kernel stages whole rows; a batch that leaves it fewer than two weight stages
  // runs as two half batches on that kernel (two passes at pipeline speed beat one pass of the plain-load kernel)
  bool gm_split = false;
  if (a.w8_fmt == MUI_W8_GROUP_MIN && a.B > 1 && a.moe_mode == GEMV_MOE_NONE && !a.use_comm &&
      !(flags & MUI_FLAG_FORCE_GENERIC) && a.group_shift >= 5 && a.group_shift <= 11 && (a.K % 16) == 0 &&
      ((reinterpret_cast<uintptr_t>(a.W) & 15) == 0) && ((reinterpret_cast<uintptr_t>(a.x) & 15) == 0)) {
    const int out_tile = (mode == 1 && a.w8_pack) ? 32 : 16;
    const int fixed = gm_layout(0, nb, a.Kp, a.K >> a.group_shift, out_tile).total;
    gm_split = (226 * 1024 - fixed) / GM_STAGE_BYTES < 2;
  }
  if (gm_split ||
      (a.B > 1 && a.moe_mode == GEMV_MOE_NONE && !pipeline_ok && (size_t)nb * (a.Kp + 8) * 2 > 150 * 1024)) {
    const int h = a.B / 2;
    GemvArgs lo = a, hi = a;
    lo.trace = hi.trace = nullptr;
    for (int i = 0; i < 3; ++i) lo.pf_frac[i] = 0;
    lo.B = h;
    hi.B = a.B - h;
    hi.x = reinterpret_cast<const unsigned char*>(a.x) + (size_t)h * a.K * 2;
    if (a.y) hi.y = reinterpret_cast<unsigned char*>(a.y) + (size_t)h * a.N * 2;
    if (a.y_f32) hi.y_f32 = a.y_f32 + (size_t)h * a.N;
    if (a.residual) hi.residual = reinterpret_cast<const unsigned char*>(a.residual) + (size_t)h * a.N * 2;
    mui_status_t st = mui_launch_gemv16(stream, dtype, mode, lo, flags);
    if (st != MUI_OK) return st;
    return mui_launch_gemv16(stream, dtype, mode, hi, flags);
  }
  if (dtype == MUI_F16) return mui_launch_gemv_f16(stream, mode, a, nb, flags, dev);
  return mui_launch_gemv_bf16(stream, mode, a, nb, flags, dev);
}
