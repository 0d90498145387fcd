#!/usr/bin/env bash
# Runtime flags every launcher exports before `nestor_cli`. Each can be preset in the environment.
# The kernel path has one implementation per op, so there are no fast-path switches here; what remains
# are the flags that change semantics, parameter layout, memory behaviour or the loop.
export NESTOR_BF16="${NESTOR_BF16:-1}"                                # bf16 compute copy, fp32 masters
export NESTOR_DENSE_NO_ROUTER="${NESTOR_DENSE_NO_ROUTER:-1}"          # single-choice routers are frozen and skipped
export NESTOR_STACKED_EXPERT_BANKS="${NESTOR_STACKED_EXPERT_BANKS:-1}" # checkpoint layout of the expert banks
export NESTOR_MUON_SHARD="${NESTOR_MUON_SHARD:-1}"                    # one owner rank per Muon matrix
export NESTOR_ZERO1="${NESTOR_ZERO1:-1}"                              # AdamW state sharded like Muon (owner of an arena range updates it)
export NESTOR_FSDP_BANKS="${NESTOR_FSDP_BANKS:-0}"                      # expert banks read from their owner ranks inside the bank GEMMs (slower than replicated banks on 2 GPUs; saves no memory yet)
export NESTOR_ACTIVATION_CHECKPOINT="${NESTOR_ACTIVATION_CHECKPOINT:-0}" # recompute ladder, rung 1: every layer is a recomputed region
export NESTOR_ACTIVATION_CHECKPOINT_SPLIT="${NESTOR_ACTIVATION_CHECKPOINT_SPLIT:-0}" # attention half and expert half are separate regions
export NESTOR_ACTIVATION_CHECKPOINT_LEAN="${NESTOR_ACTIVATION_CHECKPOINT_LEAN:-0}"   # alias of the split (a half's inputs are [T, d] tensors only)
export NESTOR_ACTIVATION_CHECKPOINT_BLOCK="${NESTOR_ACTIVATION_CHECKPOINT_BLOCK:-0}" # the whole block is one outer region
export NESTOR_EXPERT_HALF_CHUNKS="${NESTOR_EXPERT_HALF_CHUNKS:-0}"     # expert half over n row chunks, one region each
export NESTOR_ACTIVATION_OFFLOAD="${NESTOR_ACTIVATION_OFFLOAD:-0}"     # saved activations parked in pinned host memory
export NESTOR_FUSED_HEAD_CE="${NESTOR_FUSED_HEAD_CE:-1}"              # chunked head + cross-entropy, no [T, V] logits
export NESTOR_CE_CHUNK_ROWS="${NESTOR_CE_CHUNK_ROWS:-4096}"
export NESTOR_RUNAHEAD="${NESTOR_RUNAHEAD:-0}"                        # host may run this many steps ahead of the GPU
export NESTOR_DDP_BROADCAST_BUFFERS="${NESTOR_DDP_BROADCAST_BUFFERS:-1}" # rank 0's balancing biases win each step
export NESTOR_B200_CUDA_GRAPH="${NESTOR_B200_CUDA_GRAPH:-1}"          # replay the micro-batch as one CUDA graph
export NESTOR_B200_GRAD_TRANSPORT="${NESTOR_B200_GRAD_TRANSPORT:-fused}" # fused peer-memory all-reduce | nccl
export NESTOR_MFU_PEAK_TFLOPS="${NESTOR_MFU_PEAK_TFLOPS:-2250}"       # B200 dense bf16
# Recipe and bookkeeping switches that are read when set (unset = the registered recipe):
#   NESTOR_MUP_ROUTER_BASE_LR=1 / NESTOR_MUP_ROUTER_BASE_INIT=1  routers at the base AdamW rate / drawn at initializer_range
#                                (only differ from the default under matrix_optimizer="adamw")
#   NESTOR_DROP_MUP=1            ignore every optimizer tag: one AdamW group at the base rate
#   NESTOR_MFU_FLOPS_PER_STEP=x  pin the FLOPs of one rank's forward + backward micro-batch used by the MFU metric
#   NESTOR_BF16_MASTER           accepted; bf16 compute with fp32 masters is the only bf16 mode here
#   NESTOR_B200_NVLS=0           keep the in-kernel collectives on plain peer loads / stores (no multimem)
#   NESTOR_B200_STRICT=1         a shape beyond a kernel's built-in limit raises instead of running the PyTorch statement
#   NESTOR_B200_BOUNDS_CHECK=1   load the index-checking build of the kernel library
#   NESTOR_B200_POINTWISE_BANK=0 banks of pointwise (non-SwiGLU) experts run the PyTorch statement instead of the grouped kernels
#   NESTOR_DEPTH_READ_KEEP_H=0   do not keep the depth-read mixture for the backward (one [T, d] fp32 row per read)
