// RMSNorm backward that allocates nothing. This entry point has no counterpart in the
// reference project; it exists for callers of this library that must not allocate.
//
// Who cannot allocate, and why. tx_rmsnorm_bwd needs a [partials, D] fp32 scratch that its
// caller provides. The Python wrappers take that from torch's caching allocator, which a
// caller outside Python does not have: a native host thread of the runtime that drives the
// library through its C symbols, or a program that links the library without torch. What is
// left to such a caller is cudaMalloc, which synchronises the device and fails once the
// caching allocator has taken the HBM for its own pools (the normal state of a training job
// sized for the whole card). A caller that already runs inside a step whose memory plan is
// fixed is in the same position. For them the scratch lives in the library's own image.
//
// Contract.
//  * Same arguments, same kernels and same results as tx_rmsnorm_bwd without dw_partial.
//  * D must be a multiple of 8 and at most tx_rmsnorm_bwd_static_max_d() (4096); a larger D
//    is rejected with TX_STATIC_ERR_TOO_LARGE before anything is launched. T is unlimited.
//  * The scratch is one file-scope device array per device, 296 x 4096 fp32 = 4.6 MiB,
//    part of the module image. The first call on a device looks its address up (with that
//    device current) and keeps it; that look-up may load the module, so make the first call
//    during start-up, before any stream capture begins.
//  * No cudaMalloc / cudaFree / allocating library routine is called, torch's included.
//  * Nothing in the scratch has to be zero on entry: the first launch of a call writes every
//    word that its second launch reads.
//  * Every call on a device shares the one array. Calls on the same stream are ordered and
//    safe; calls that can overlap (different streams, or threads on different streams)
//    race on it and give wrong dw. Serialise them, or use tx_rmsnorm_bwd with own scratch.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  TX_STATIC_OK = 0,
  TX_STATIC_ERR_BAD_SHAPE = 1,    // D not a multiple of 8, or T < 0
  TX_STATIC_ERR_TOO_LARGE = 2,    // D > tx_rmsnorm_bwd_static_max_d()
  TX_STATIC_ERR_DEVICE = 3,       // current device unknown or its ordinal >= 64
  TX_STATIC_ERR_SYMBOL = 4,       // the address look-up of the scratch array failed
  TX_STATIC_ERR_LAUNCH = 400      // a kernel launch was refused
};

int tx_rmsnorm_bwd_static_max_d(void);
const char* tx_rmsnorm_bwd_static_strerror(int code);
int tx_rmsnorm_bwd_static(const void* x, const void* w, const void* dy, const float* rstd, const void* dres,
                          void* dx, float* dw, int dw_accumulate, int T, int D, float eps, float w_offset,
                          cudaStream_t stream);

#ifdef __cplusplus
}
#endif
