// LayerNorm backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference; it exists for hosts of this library that run inside a
// fixed memory budget or an allocation-free region - an inference server that pre-sized every buffer at start-up,
// a real-time loop, a plug-in whose embedding application owns the allocator - where a cudaMalloc (or a framework
// allocator call that may fall through to one) is either forbidden or stalls the device.
//
// It computes exactly what ffb_layernorm_bwd computes (dx, dgamma, dbeta of LayerNorm over the last dimension),
// but the per-block partial sums for dgamma / dbeta, which ffb_layernorm_bwd takes as a caller-allocated workspace,
// live in a file-scope device array inside the library:
//
//     capacity : FFB_LN_NOALLOC_BLOCKS (148) blocks x 2 x FFB_LN_NOALLOC_MAX_C (1024) floats = 1,212,416 bytes,
//                held by every GPU that loads the library until the process exits.
//     limit    : C <= FFB_LN_NOALLOC_MAX_C; a larger C is refused with FFB_LN_NOALLOC_TOO_WIDE (nothing is launched)
//                and a one-line message on stderr.  rows is unlimited (blocks walk rows with a grid stride).
//
// The call performs no cudaMalloc / cudaFree and calls no allocating library routine; the caller passes every
// input and output buffer.  The first call on a device resolves the array's device address
// (cudaGetSymbolAddress) with that device current - make that first call outside any stream capture.  All calls
// share the one array, which still holds the previous call's partial sums.  What a call accumulates into is cleared
// first (cudaMemsetAsync on the given stream); the bf16 kernels for C = 64 / 128 / 256 skip that memset because every
// block of theirs stores (not adds) each of its partial sums before the final reduction reads them, so stale contents
// are overwritten.  Two calls that overlap on the GPU (different streams, or different host threads on one device)
// race on the array - serialise them.
#pragma once

#define FFB_LN_NOALLOC_BLOCKS 148
#define FFB_LN_NOALLOC_MAX_C 1024
#define FFB_LN_NOALLOC_TOO_WIDE (-3)

#ifdef __cplusplus
extern "C" {
#endif

// dtype: 0 = fp32, 1 = fp16, 2 = bf16 (dy, x, gamma, dx, dgamma, dbeta share it); mean / rstd: fp32 [rows] as saved
// by ffb_layernorm_fwd.  Returns 0, FFB_LN_NOALLOC_TOO_WIDE, -2 (bad dtype) or -1 (CUDA error).
int ffb_layernorm_bwd_noalloc(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, void* dx,
                              void* dgamma, void* dbeta, long long rows, int C, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
