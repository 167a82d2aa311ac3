// Allocation-free C entry point. It has no counterpart in the reference code base.
//
// Who needs it: host programs that drive these kernels without a tensor allocator and may not call cudaMalloc at
// the point of use - for example a C training loop that reserved all device memory up front for its own arena, or a
// runtime in which a device allocation would stall every stream. The regular RMSNorm backward needs a scratch
// buffer for per-CTA partial sums of the weight gradient; this variant keeps that scratch inside the library.
//
//   int b200_rmsnorm_bwd_noalloc(dy, h, w, rstd, dres, dh, dw, accumulate_dw, T, H, stream, error_message, len)
//
//   dy, h, dres (optional, may be NULL), dh : bf16 [T, H], contiguous     w : bf16 [H]     rstd : fp32 [T]
//   dw : fp32 [H]; overwritten, or added to when accumulate_dw != 0       stream : cudaStream_t (as void*)
//   returns 0 on success; otherwise a non-zero code and a NUL-terminated explanation in error_message.
//
// Limits and rules:
//   * dy, h, w, rstd, dh and dw must not be NULL (code 6); dy, h, w, dres, dh and dw must be 16-byte aligned and rstd
//     4-byte aligned (code 7): the kernels use 16-byte accesses, so a bad pointer is refused here, before any launch.
//   * H must be a multiple of 8 and at most B200_NOALLOC_RMSNORM_MAX_H; larger rows are rejected (code 2).
//   * The scratch is one array of B200_NOALLOC_RMSNORM_MAX_ROWS x B200_NOALLOC_RMSNORM_MAX_H floats (5 MiB) in the
//     library image; every GPU that loads the library holds it until the process exits.
//   * The first call on each device resolves the array's device address (with that device current). Make that first
//     call outside of any stream capture.
//   * No cudaMalloc / cudaFree / allocating library routine is called. All calls on a device share the one scratch
//     array and it keeps the previous call's contents: each call overwrites every element it later reads, so nothing
//     needs clearing, but two calls whose kernels overlap on the GPU (different streams) race on it - serialise them.
#pragma once

#define B200_NOALLOC_RMSNORM_MAX_ROWS 160
#define B200_NOALLOC_RMSNORM_MAX_H 8192

#ifdef __cplusplus
extern "C" {
#endif

int b200_rmsnorm_bwd_noalloc(const void* dy, const void* h, const void* w, const float* rstd, const void* dres, void* dh,
                             float* dw, int accumulate_dw, int T, int H, void* stream, char* error_message,
                             int error_message_len);

#ifdef __cplusplus
}
#endif
