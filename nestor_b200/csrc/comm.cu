// In-kernel collectives over NVLink peer memory (symmetric buffers mapped into every rank).
//
//   allreduce_push : every rank owns 1/W of the range; the owner loads its slice from all
//                    peers (plain peer loads over NVLink), sums in fp32, scales, and stores
//                    the result into every rank's buffer (plus an optional bf16 mirror).
//                    Traffic per rank: (W-1)/W in, (W-1)/W out — the all-reduce minimum.
//   param_push     : after a sharded optimizer step each rank stores its updated master
//                    range into every peer's fp32 master buffer and bf16 compute buffer
//                    (all-gather fused with the compute-dtype cast).
//
// Synchronisation: block b of every rank meets block b of its peers at a start barrier
// (the peers' kernels are running, hence everything stream-ordered before them is done)
// and at an end barrier (all stores into this rank's buffers have landed before its
// kernel completes). Flags live in the symmetric signal pad, carry a monotonically
// increasing epoch (never reset), and are written with release / read with acquire
// semantics at system scope. Every wait is bounded: when the budget runs out the kernel
// records kTimeoutPeer in the status word and returns; the host turns that into an error.
//
// Replaces DDP's bucketed NCCL all-reduce (nestor/utils/distributed.py:436-443), the per-owner
// reduce / broadcast of the bf16-master path (nestor/scaling/bf16_master.py:142-172) and
// `_broadcast_muon_params` (nestor/scaling/muon.py:410-433) of the reference.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nbc {

constexpr int kMaxWorld = 8;
constexpr int kTimeoutPeer = 5;

struct Peers {
  void* buf[kMaxWorld];        // fp32 buffer of every rank (index = rank)
  void* aux[kMaxWorld];        // optional second buffer of every rank (bf16 mirror / compute copy)
  uint32_t* sig[kMaxWorld];    // signal pad of every rank
  int world, rank;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Block `blockIdx.x` of every rank meets here. Slot layout: sig[dst][(phase*gridDim.x + block)*kMaxWorld + src].
// Returns false (and sets *status) when a peer does not show up within `budget` polls.
__device__ bool block_barrier(const Peers& P, int phase, uint32_t epoch, long budget, int* status) {
  __shared__ int s_ok;
  __syncthreads();
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < P.world) {
    const int peer = threadIdx.x;
    const long slot = (long(phase) * gridDim.x + blockIdx.x) * kMaxWorld;
    __threadfence_system();
    st_release_sys(P.sig[peer] + slot + P.rank, epoch);
    const uint32_t* mine = P.sig[P.rank] + slot + peer;
    bool ok = false;
    for (long i = 0; i < budget; ++i) {
      if (int32_t(ld_acquire_sys(mine) - epoch) >= 0) { ok = true; break; }
      __nanosleep(100);
    }
    if (!ok) { s_ok = 0; atomicCAS(status, 0, kTimeoutPeer); }
  }
  __syncthreads();
  return s_ok != 0;
}

// store_all = 1: all-reduce (the owner of a slice writes the sum into every replica). store_all = 0:
// reduce-scatter (the sum stays with the owner, whose slice [own_lo, own_hi) is given explicitly so that it can
// follow the optimizer's ownership ranges; the other ranks' copies of that slice are only read).
__global__ void __launch_bounds__(512, 1)
allreduce_push_kernel(Peers P, long offset, long numel, float scale, int write_mirror, uint32_t epoch, long budget,
                      int* status, int store_all, long own_lo, long own_hi) {
  if (!block_barrier(P, 0, epoch, budget, status)) return;
  // this rank's slice of [0, numel), in float4 units
  const long n4 = numel / 4;
  const long per = (n4 + P.world - 1) / P.world;
  const long lo = store_all ? per * P.rank : own_lo / 4, hi = store_all ? min(n4, lo + per) : own_hi / 4;
  // kUnroll float4 per thread and iteration: every peer load of the batch is issued before the first add, so
  // (world - 1) * kUnroll NVLink reads are in flight per thread
  constexpr int kUnroll = 8;
  const long stride = long(gridDim.x) * blockDim.x;
  for (long i0 = lo + long(blockIdx.x) * blockDim.x + threadIdx.x; i0 < hi; i0 += stride * kUnroll) {
    float4 acc[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int p = 0; p < kMaxWorld; ++p) {
      if (p < P.world) {
        const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(P.buf[p]) + offset);
        float4 v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const long i = i0 + u * stride;
          v[u] = i < hi ? src[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) { acc[u].x += v[u].x; acc[u].y += v[u].y; acc[u].z += v[u].z; acc[u].w += v[u].w; }
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const long i = i0 + u * stride;
      if (i >= hi) break;
      float4 a = acc[u];
      a.x *= scale; a.y *= scale; a.z *= scale; a.w *= scale;
      __nv_bfloat162 b0 = __floats2bfloat162_rn(a.x, a.y), b1 = __floats2bfloat162_rn(a.z, a.w);
      const uint2 packed = make_uint2(*reinterpret_cast<uint32_t*>(&b0), *reinterpret_cast<uint32_t*>(&b1));
#pragma unroll
      for (int p = 0; p < kMaxWorld; ++p) {
        if (p < P.world && (store_all || p == P.rank)) {
          reinterpret_cast<float4*>(reinterpret_cast<float*>(P.buf[p]) + offset)[i] = a;
          if (write_mirror)
            reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(P.aux[p]) + offset)[i] = packed;
        }
      }
    }
  }
  block_barrier(P, 1, epoch, budget, status);
}

// Store the bf16 rounding of master[lo:hi) into every rank's compute buffer and, with `push_master`, the fp32 values
// into every peer's master as well. Without it a rank's fp32 masters outside its own range go stale, which nothing on
// the training path reads (they are brought up to date from their owners when a checkpoint is written): the push then
// moves 2 bytes per parameter instead of 6.
__global__ void __launch_bounds__(512, 1)
param_push_kernel(Peers P, long lo, long hi, uint32_t epoch, long budget, int* status, int push_master) {
  if (!block_barrier(P, 2, epoch, budget, status)) return;
  const long lo4 = lo / 4, hi4 = hi / 4;
  const long stride = long(gridDim.x) * blockDim.x;
  const float4* src = reinterpret_cast<const float4*>(P.buf[P.rank]);
  for (long i = lo4 + long(blockIdx.x) * blockDim.x + threadIdx.x; i < hi4; i += stride) {
    const float4 v = src[i];
    __nv_bfloat162 b0 = __floats2bfloat162_rn(v.x, v.y), b1 = __floats2bfloat162_rn(v.z, v.w);
    const uint2 packed = make_uint2(*reinterpret_cast<uint32_t*>(&b0), *reinterpret_cast<uint32_t*>(&b1));
#pragma unroll
    for (int p = 0; p < kMaxWorld; ++p) {
      if (p < P.world) {
        if (push_master && p != P.rank) reinterpret_cast<float4*>(P.buf[p])[i] = v;
        if (P.aux[p]) reinterpret_cast<uint2*>(P.aux[p])[i] = packed;
      }
    }
  }
  block_barrier(P, 3, epoch, budget, status);
}

// ------------------------------------------------------------------------------------------------
// NVLS variants: the symmetric buffers are also mapped through one NVLink multicast address each. A
// `multimem.ld_reduce` on that address returns the sum of every rank's copy, added inside the NVSwitch (each GPU
// receives one reduced stream instead of world - 1 peer streams), and a `multimem.st` writes every rank's copy at once
// (the owner sends one stream instead of world - 1). Same barriers, same bounded waits, same status word.
__device__ __forceinline__ float4 mm_ld_reduce_f32x4(const float* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ void mm_st_f32x4(float* mc, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
               :: "l"(mc), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ void mm_st_bf16x4(__nv_bfloat16* mc, uint2 packed) {
  asm volatile("multimem.st.relaxed.sys.global.v2.bf16x2 [%0], {%1,%2};" :: "l"(mc), "r"(packed.x), "r"(packed.y) : "memory");
}

// Reduce-scatter (store_all = 0: the sum of [own_lo, own_hi) lands in this rank's buffer only) or all-reduce
// (store_all = 1: every rank reduces its 1/world slice of [offset, offset + numel) and multicasts the result).
// `mc_buf` / `mc_aux` are the multicast addresses of the fp32 buffer and of the optional bf16 mirror.
__global__ void __launch_bounds__(512, 1)
allreduce_nvls_kernel(Peers P, float* mc_buf, __nv_bfloat16* mc_aux, long offset, long numel, float scale, int write_mirror,
                      uint32_t epoch, long budget, int* status, int store_all, long own_lo, long own_hi) {
  if (!block_barrier(P, 0, epoch, budget, status)) return;
  const long n4 = numel / 4;
  const long per = (n4 + P.world - 1) / P.world;
  const long lo = store_all ? per * P.rank : own_lo / 4, hi = store_all ? min(n4, lo + per) : own_hi / 4;
  constexpr int kUnroll = 8;
  const long stride = long(gridDim.x) * blockDim.x;
  float* mine = reinterpret_cast<float*>(P.buf[P.rank]) + offset;
  __nv_bfloat16* mine_aux = reinterpret_cast<__nv_bfloat16*>(P.aux[P.rank]) + offset;
  for (long i0 = lo + long(blockIdx.x) * blockDim.x + threadIdx.x; i0 < hi; i0 += stride * kUnroll) {
    float4 v[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const long i = i0 + u * stride;
      v[u] = i < hi ? mm_ld_reduce_f32x4(mc_buf + offset + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const long i = i0 + u * stride;
      if (i >= hi) break;
      float4 a = v[u];
      a.x *= scale; a.y *= scale; a.z *= scale; a.w *= scale;
      __nv_bfloat162 b0 = __floats2bfloat162_rn(a.x, a.y), b1 = __floats2bfloat162_rn(a.z, a.w);
      const uint2 packed = make_uint2(*reinterpret_cast<uint32_t*>(&b0), *reinterpret_cast<uint32_t*>(&b1));
      if (store_all) {
        mm_st_f32x4(mc_buf + offset + 4 * i, a);
        if (write_mirror) mm_st_bf16x4(mc_aux + offset + 4 * i, packed);
      } else {
        reinterpret_cast<float4*>(mine)[i] = a;
        if (write_mirror) reinterpret_cast<uint2*>(mine_aux)[i] = packed;
      }
    }
  }
  block_barrier(P, 1, epoch, budget, status);
}

// Parameter push through the multicast mapping: one store per element reaches every replica (this rank's included,
// which rewrites its own master with the value just read).
__global__ void __launch_bounds__(512, 1)
param_push_nvls_kernel(Peers P, float* mc_master, __nv_bfloat16* mc_compute, long lo, long hi, uint32_t epoch, long budget,
                       int* status, int push_master) {
  if (!block_barrier(P, 2, epoch, budget, status)) return;
  const long lo4 = lo / 4, hi4 = hi / 4;
  const long stride = long(gridDim.x) * blockDim.x;
  const float4* src = reinterpret_cast<const float4*>(P.buf[P.rank]);
  for (long i = lo4 + long(blockIdx.x) * blockDim.x + threadIdx.x; i < hi4; i += stride) {
    const float4 v = src[i];
    __nv_bfloat162 b0 = __floats2bfloat162_rn(v.x, v.y), b1 = __floats2bfloat162_rn(v.z, v.w);
    const uint2 packed = make_uint2(*reinterpret_cast<uint32_t*>(&b0), *reinterpret_cast<uint32_t*>(&b1));
    if (push_master) mm_st_f32x4(mc_master + 4 * i, v);
    if (mc_compute) mm_st_bf16x4(mc_compute + 4 * i, packed);
  }
  block_barrier(P, 3, epoch, budget, status);
}

// Single-GPU exercise of the bounded wait: spins on a flag nothing sets and reports the timeout.
__global__ void wait_timeout_probe_kernel(uint32_t* flag, uint32_t expect, long budget, int* status) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    bool ok = false;
    for (long i = 0; i < budget; ++i) {
      if (int32_t(ld_acquire_sys(flag) - expect) >= 0) { ok = true; break; }
      __nanosleep(100);
    }
    if (!ok) atomicCAS(status, 0, kTimeoutPeer);
  }
}

}  // namespace nbc

extern "C" {

struct NbPeers {
  void* buf[8]; void* aux[8]; void* sig[8];
  int world, rank;
};

static int max_blocks() {
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 1;
  }
  return sms;
}

// Launches are one block per SM at most (512 threads, one block resident per SM): every block of every rank must be
// running for the in-kernel barriers to complete.
int nb_comm_max_blocks(void) { return max_blocks(); }

static nbc::Peers to_peers(const NbPeers* a) {
  nbc::Peers P;
  for (int i = 0; i < 8; ++i) { P.buf[i] = a->buf[i]; P.aux[i] = a->aux[i]; P.sig[i] = reinterpret_cast<uint32_t*>(a->sig[i]); }
  P.world = a->world; P.rank = a->rank;
  return P;
}

// numel and offset in fp32 elements, both multiples of 4. `blocks` must be equal on every rank and at most the SM count
// (nb_comm_max_blocks).
int nb_allreduce_push(const NbPeers* a, long offset, long numel, float scale, int write_mirror, unsigned epoch, long budget,
                      int blocks, int* status, cudaStream_t st) {
  if (a->world < 1 || a->world > 8 || (numel % 4) || (offset % 4) || blocks < 1 || blocks > max_blocks()) return -1;
  nbc::allreduce_push_kernel<<<blocks, 512, 0, st>>>(to_peers(a), offset, numel, scale, write_mirror, epoch, budget, status,
                                                     1, 0, 0);
  return int(cudaGetLastError());
}

// Reduce-scatter: this rank sums [lo, hi) (fp32 elements, multiples of 4) of every replica into its own buffer
// (x scale). Every rank passes its own range; ranges may differ in size and must not overlap.
int nb_reduce_scatter_push(const NbPeers* a, long lo, long hi, float scale, int write_mirror, unsigned epoch, long budget,
                           int blocks, int* status, cudaStream_t st) {
  if (a->world < 1 || a->world > 8 || (lo % 4) || (hi % 4) || hi < lo || blocks < 1 || blocks > max_blocks()) return -1;
  nbc::allreduce_push_kernel<<<blocks, 512, 0, st>>>(to_peers(a), 0, 0, scale, write_mirror, epoch, budget, status, 0, lo, hi);
  return int(cudaGetLastError());
}

// push_master = 0 requires a compute buffer (aux) on every rank: it is then the only thing written.
int nb_param_push(const NbPeers* a, long lo, long hi, unsigned epoch, long budget, int blocks, int* status, int push_master,
                  cudaStream_t st) {
  if (a->world < 1 || a->world > 8 || (lo % 4) || (hi % 4) || blocks < 1 || blocks > max_blocks()) return -1;
  if (!push_master) for (int r = 0; r < a->world; ++r) if (!a->aux[r]) return -2;
  nbc::param_push_kernel<<<blocks, 512, 0, st>>>(to_peers(a), lo, hi, epoch, budget, status, push_master);
  return int(cudaGetLastError());
}

// NVLS forms of the three collectives: `mc_buf` / `mc_aux` are the multicast addresses of the buffers whose per-rank
// addresses are in `a->buf` / `a->aux` (mc_aux may be null when no mirror / compute copy is written).
int nb_allreduce_nvls(const NbPeers* a, void* mc_buf, void* mc_aux, long offset, long numel, float scale, int write_mirror,
                      unsigned epoch, long budget, int blocks, int* status, cudaStream_t st) {
  if (a->world < 1 || a->world > 8 || !mc_buf || (numel % 4) || (offset % 4) || blocks < 1 || blocks > max_blocks()) return -1;
  if (write_mirror && !mc_aux) return -1;
  nbc::allreduce_nvls_kernel<<<blocks, 512, 0, st>>>(to_peers(a), static_cast<float*>(mc_buf), static_cast<__nv_bfloat16*>(mc_aux),
                                                     offset, numel, scale, write_mirror, epoch, budget, status, 1, 0, 0);
  return int(cudaGetLastError());
}

int nb_reduce_scatter_nvls(const NbPeers* a, void* mc_buf, long lo, long hi, float scale, int write_mirror, unsigned epoch,
                           long budget, int blocks, int* status, cudaStream_t st) {
  if (a->world < 1 || a->world > 8 || !mc_buf || (lo % 4) || (hi % 4) || hi < lo || blocks < 1 || blocks > max_blocks()) return -1;
  nbc::allreduce_nvls_kernel<<<blocks, 512, 0, st>>>(to_peers(a), static_cast<float*>(mc_buf), nullptr, 0, 0, scale, write_mirror,
                                                     epoch, budget, status, 0, lo, hi);
  return int(cudaGetLastError());
}

int nb_param_push_nvls(const NbPeers* a, void* mc_master, void* mc_compute, long lo, long hi, unsigned epoch, long budget,
                       int blocks, int* status, int push_master, cudaStream_t st) {
  if (a->world < 1 || a->world > 8 || !mc_master || (lo % 4) || (hi % 4) || blocks < 1 || blocks > max_blocks()) return -1;
  if (!push_master && !mc_compute) return -2;
  nbc::param_push_nvls_kernel<<<blocks, 512, 0, st>>>(to_peers(a), static_cast<float*>(mc_master),
                                                      static_cast<__nv_bfloat16*>(mc_compute), lo, hi, epoch, budget, status,
                                                      push_master);
  return int(cudaGetLastError());
}

int nb_wait_timeout_probe(void* flag, unsigned expect, long budget, int* status, cudaStream_t st) {
  nbc::wait_timeout_probe_kernel<<<1, 32, 0, st>>>(reinterpret_cast<uint32_t*>(flag), expect, budget, status);
  return int(cudaGetLastError());
}

}  // extern "C"
