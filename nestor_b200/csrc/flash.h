// Public C interface of the packed varlen causal attention kernels (flash_fwd.cu, flash_bwd.cu).
//
// All tensors are bf16 with a contiguous last dimension; head h of a row occupies columns h*hd .. h*hd+hd-1.
// `seg_start` holds nseg + 1 ascending row offsets: attention is causal inside [seg_start[s], seg_start[s+1])
// and never crosses segments. `status` points at a device int that a kernel sets to a nonzero code when one of its
// bounded waits gives up. Entry points return 0, a negative argument error, or a cudaError_t value.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

struct NbFlashArgs {
  const void* Q; const void* K; const void* V;   // row pitch `ld_qkv` elements (shared by the three)
  long ld_qkv;
  void* O; long ldo;                             // [rows, H*hd]
  float* lse;                                    // [rows, H] log-sum-exp of the scaled scores, log2 domain
  const int* seg_start; int nseg;
  int rows, H, hd;
  float scale;                                   // logit scale (the models use 1/hd)
  int* status;
  int max_tiles;                                 // upper bound on q tiles: ceil(rows/128) + nseg
  int lazy_rescale;                              // flag bits: 2 = probabilities through tensor memory (head dims <= 64); bit 0 unused
};

struct NbFlashBwdArgs {
  const void* Q; const void* K; const void* V; long ld_qkv;    // saved forward operands (shared row pitch)
  const void* O; long ld_o;
  const void* dO; long ld_do;
  const float* lse; float* delta;                              // [rows, H] each; delta is scratch the call fills
  void* dQ; void* dK; void* dV; long ld_dqkv;
  const int* seg_start; int nseg;
  int rows, H, hd;
  float scale;
  int* status;
  int max_tiles;                                               // ceil(rows/128) + nseg
};

int nb_flash_fwd(const struct NbFlashArgs* args, cudaStream_t stream);
int nb_flash_bwd(const struct NbFlashBwdArgs* args, cudaStream_t stream);

// sizeof the two argument blocks as this library was compiled: bindings that mirror the structs check their layout.
int nb_flash_args_size(void);
int nb_flash_bwd_args_size(void);

#ifdef __cplusplus
}
#endif
