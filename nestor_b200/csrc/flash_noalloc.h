// Attention backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference implementation; it exists for
// embedders of this library.
//
// Who needs it: code that runs where a device allocation is off the table — a serving or
// training process whose memory was handed out up front to a fixed pool, a step that has
// just hit an out-of-memory condition and must still finish a backward pass, a plugin
// running inside somebody else's framework that forbids allocator calls on its hot path,
// or latency-critical code that cannot afford the device-wide synchronisation an
// allocation may imply. The regular entry point `nb_flash_bwd` needs one scratch buffer
// (`delta`, rows x heads floats) from its caller, which in practice means an allocation
// per call; this variant keeps that scratch in a fixed array inside the library instead.
//
// Contract
//   * Same argument block as `nb_flash_bwd` (`struct NbFlashBwdArgs`, flash.h); the `delta`
//     field is ignored. Inputs and outputs still belong to the caller.
//   * The scratch is one file-scope device array of NB_FLASH_NOALLOC_MAX_FLOATS floats
//     (4 MiB). Every GPU that loads the library holds it until the process exits.
//     A call with rows * heads above that limit is refused with
//     NB_FLASH_NOALLOC_TOO_LARGE and does nothing.
//   * The first call on each device looks up the array's device address (with that device
//     current). Make that first call outside of any stream capture. Threads that make a
//     device's first call at the same time all store the same address, which is harmless.
//   * The call itself performs no cudaMalloc / cudaFree and calls no allocating library
//     routine.
//   * All calls on a device share the one array and it keeps whatever the last call left
//     in it. Each call overwrites the part it uses before reading it, so nothing has to be
//     cleared between calls — but two calls whose kernels can overlap on the GPU (different
//     streams, no ordering between them) race on it. Serialise them.
#pragma once
#include <cuda_runtime.h>
#include "flash.h"   // struct NbFlashBwdArgs, nb_flash_bwd

#ifdef __cplusplus
extern "C" {
#endif

#define NB_FLASH_NOALLOC_MAX_FLOATS (1 << 20)
#define NB_FLASH_NOALLOC_TOO_LARGE (-100)
#define NB_FLASH_NOALLOC_SETUP_FAILED (-101)

// Returns 0 on success, NB_FLASH_NOALLOC_TOO_LARGE / NB_FLASH_NOALLOC_SETUP_FAILED, or the
// code `nb_flash_bwd` would return.
int nb_flash_bwd_noalloc(const struct NbFlashBwdArgs* args, cudaStream_t stream);

// Human-readable reason for the last non-zero return of nb_flash_bwd_noalloc on this thread.
const char* nb_flash_bwd_noalloc_error(void);

#ifdef __cplusplus
}
#endif
