// Multi-tensor optimizer kernels: one launch updates every tensor of a parameter group.
//
// A group is described by a device table of tensors (up to four base pointers and an element count each) and a
// chunk list (tensor index, first element); each block owns one chunk of kChunk elements. Three operations:
//   adamw    : p *= 1 - lr*wd;  m = lerp(m, g, 1-b1);  v = b2*v + (1-b2)*g*g;
//              p -= (lr / bc1) * m / (sqrt(v) / sqrt(bc2) + eps)            (the reference's foreach sequence)
//   momentum : buf = mu*buf + g;  dir = nesterov ? g + mu*buf : buf           (Muon, before Newton-Schulz)
//   axpy     : p = p*decay + alpha*u   with u fp32 or bf16                    (Muon, after Newton-Schulz)
//
// Replaces the torch._foreach_* chains of the reference optimizer (nestor/scaling/muon.py:588-651 for Muon,
// :667-710 for AdamW): about a dozen multi-tensor launches per group become one.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nbo {

constexpr int kChunk = 16384;

struct Entry { void* p[4]; long numel; };

enum Op : int { kAdamW = 0, kMomentum = 1, kAxpyF32 = 2, kAxpyBf16 = 3 };

struct Scalars { float s[8]; };

template <int OP>
__global__ void __launch_bounds__(256) multi_tensor_kernel(const Entry* __restrict__ table, const int2* __restrict__ chunks,
                                                           Scalars sc) {
  const int2 ch = chunks[blockIdx.x];
  const Entry e = table[ch.x];
  const long base = long(ch.y) * kChunk;
  const long end = min(e.numel, base + kChunk);
  for (long i = base + threadIdx.x; i < end; i += blockDim.x) {
    if (OP == kAdamW) {
      float* p = reinterpret_cast<float*>(e.p[0]);
      const float g = reinterpret_cast<const float*>(e.p[1])[i];
      float* m = reinterpret_cast<float*>(e.p[2]);
      float* v = reinterpret_cast<float*>(e.p[3]);
      // s: 0 decay factor, 1 (1 - b1), 2 b2, 3 (1 - b2), 4 1/sqrt(bc2), 5 eps, 6 lr/bc1
      float pv = p[i] * sc.s[0];
      float mv = m[i]; mv = mv + sc.s[1] * (g - mv);
      float vv = v[i] * sc.s[2] + sc.s[3] * g * g;
      const float denom = sqrtf(vv) * sc.s[4] + sc.s[5];
      pv -= sc.s[6] * mv / denom;
      p[i] = pv; m[i] = mv; v[i] = vv;
    } else if (OP == kMomentum) {
      const float g = reinterpret_cast<const float*>(e.p[0])[i];
      float* buf = reinterpret_cast<float*>(e.p[1]);
      float* dir = reinterpret_cast<float*>(e.p[2]);
      // s: 0 mu, 1 nesterov flag
      const float b = sc.s[0] * buf[i] + g;
      buf[i] = b;
      dir[i] = sc.s[1] != 0.f ? g + sc.s[0] * b : b;
    } else {
      float* p = reinterpret_cast<float*>(e.p[0]);
      // s: 0 decay factor, 1 alpha
      const float u = OP == kAxpyF32 ? reinterpret_cast<const float*>(e.p[1])[i]
                                     : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(e.p[1])[i]);
      p[i] = p[i] * sc.s[0] + sc.s[1] * u;
    }
  }
}

// Loss-free balancing nudge for every router at once: bias += rate * sign(mean(c) - c), one warp per router.
// `counts` is the flat tensor of all routers' summed selection counts; a router's slice starts at `offset`.
struct BiasEntry { float* bias; long offset; int n; float rate; };

__global__ void __launch_bounds__(128) bias_update_kernel(const BiasEntry* __restrict__ table, int n_routers,
                                                          const float* __restrict__ counts) {
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= n_routers) return;
  const BiasEntry e = table[r];
  const float* c = counts + e.offset;
  float sum = 0.f;
  for (int i = lane; i < e.n; i += 32) sum += c[i];
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, s);
  const float mean = sum / float(e.n);
  for (int i = lane; i < e.n; i += 32) {
    const float d = mean - c[i];
    e.bias[i] += e.rate * (d > 0.f ? 1.f : (d < 0.f ? -1.f : 0.f));
  }
}

}  // namespace nbo

extern "C" {

// table: device array of {bias pointer, offset into counts, n, rate} (24 bytes per router)
int nb_bias_update(const void* table, int n_routers, const float* counts, cudaStream_t st) {
  if (n_routers <= 0) return 0;
  nbo::bias_update_kernel<<<(n_routers + 3) / 4, 128, 0, st>>>(reinterpret_cast<const nbo::BiasEntry*>(table), n_routers, counts);
  return int(cudaGetLastError());
}

int nb_multi_tensor_chunk() { return nbo::kChunk; }

// table: device array of {ptr, ptr, ptr, ptr, numel} (5 x 8 bytes per tensor); chunks: device int32 pairs.
int nb_multi_tensor(int op, const void* table, const void* chunks, int n_chunks, const float* scalars, cudaStream_t st) {
  if (n_chunks <= 0) return 0;
  nbo::Scalars sc;
  for (int i = 0; i < 8; ++i) sc.s[i] = scalars[i];
  const nbo::Entry* t = reinterpret_cast<const nbo::Entry*>(table);
  const int2* c = reinterpret_cast<const int2*>(chunks);
  switch (op) {
    case nbo::kAdamW: nbo::multi_tensor_kernel<nbo::kAdamW><<<n_chunks, 256, 0, st>>>(t, c, sc); break;
    case nbo::kMomentum: nbo::multi_tensor_kernel<nbo::kMomentum><<<n_chunks, 256, 0, st>>>(t, c, sc); break;
    case nbo::kAxpyF32: nbo::multi_tensor_kernel<nbo::kAxpyF32><<<n_chunks, 256, 0, st>>>(t, c, sc); break;
    case nbo::kAxpyBf16: nbo::multi_tensor_kernel<nbo::kAxpyBf16><<<n_chunks, 256, 0, st>>>(t, c, sc); break;
    default: return -1;
  }
  return int(cudaGetLastError());
}

}  // extern "C"
