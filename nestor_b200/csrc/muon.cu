// Newton-Schulz orthogonalisation (Muon): the pointwise ends of the iteration.
//
// The five iterations  A = X X^T;  B = b A + c A A;  X <- a X + B X  are three launches each of the grouped tcgen05
// GEMM (gemm.cu, groups = matrices of one shape, the two polynomial steps in its `alpha * acc + beta * E1`
// epilogue). The kernels here bracket them:
//   ns_prepare : fp32 [batch, m, n] -> bf16 [batch, mp, np] in the wide orientation (transposed when m > n),
//                divided by the Frobenius norm of the bf16-rounded matrix (+1e-7); padding rows / columns (up to
//                the 8-element alignment the tensor maps need) are written as zeros, which the iteration keeps zero.
//   ns_finish  : bf16 [batch, mp, np] -> bf16 [batch, m, n] (back to the parameter's orientation, padding dropped).
//
// Replaces `zeropower_via_newtonschulz5` and its batched form (nestor/scaling/muon.py:83-151) of the reference,
// which run on cuBLAS bmm.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nbm {

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < (blockDim.x >> 5) ? red[lane] : 0.f;
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) t += __shfl_xor_sync(0xffffffffu, t, s);
    if (lane == 0) red[0] = t;
  }
  __syncthreads();
  return red[0];
}

// One block per matrix. `rows` x `cols` is the wide orientation (rows <= cols) of the m x n input.
__global__ void __launch_bounds__(512) ns_prepare_kernel(const float* __restrict__ g, __nv_bfloat16* __restrict__ x, int m,
                                                         int n, int transpose, int mp, int np, long x_batch_stride) {
  __shared__ float red[32];
  const float* src = g + long(blockIdx.x) * m * n;
  __nv_bfloat16* dst = x + long(blockIdx.x) * x_batch_stride;
  float ss = 0.f;
  for (long i = threadIdx.x; i < long(m) * n; i += blockDim.x) {
    const float v = __bfloat162float(__float2bfloat16(src[i]));
    ss += v * v;
  }
  const float inv = 1.f / (sqrtf(block_sum(ss, red)) + 1e-7f);
  const int rows = transpose ? n : m, cols = transpose ? m : n;
  for (long i = threadIdx.x; i < long(mp) * np; i += blockDim.x) {
    const int r = int(i / np), c = int(i - long(r) * np);
    float v = 0.f;
    if (r < rows && c < cols) v = __bfloat162float(__float2bfloat16(transpose ? src[long(c) * n + r] : src[long(r) * n + c])) * inv;
    dst[i] = __float2bfloat16(v);
  }
}

__global__ void __launch_bounds__(512) ns_finish_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                                        int m, int n, int transpose, int np, long x_batch_stride) {
  const __nv_bfloat16* src = x + long(blockIdx.x) * x_batch_stride;
  __nv_bfloat16* dst = out + long(blockIdx.x) * m * n;
  for (long i = threadIdx.x; i < long(m) * n; i += blockDim.x) {
    const int r = int(i / n), c = int(i - long(r) * n);
    dst[i] = transpose ? src[long(c) * np + r] : src[long(r) * np + c];
  }
}

}  // namespace nbm

extern "C" {

// g: fp32 [batch, m, n] contiguous. x: bf16 [batch, mp, np] (mp, np >= the wide dims, multiples of 8).
int nb_ns_prepare(const float* g, void* x, int batch, int m, int n, int mp, int np, cudaStream_t st) {
  if (batch <= 0) return 0;
  const int transpose = m > n ? 1 : 0;
  const int rows = transpose ? n : m, cols = transpose ? m : n;
  if (mp < rows || np < cols || (mp % 8) || (np % 8)) return -1;
  nbm::ns_prepare_kernel<<<batch, 512, 0, st>>>(g, reinterpret_cast<__nv_bfloat16*>(x), m, n, transpose, mp, np, long(mp) * np);
  return int(cudaGetLastError());
}

int nb_ns_finish(const void* x, void* out, int batch, int m, int n, int mp, int np, cudaStream_t st) {
  if (batch <= 0) return 0;
  nbm::ns_finish_kernel<<<batch, 512, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<__nv_bfloat16*>(out),
                                               m, n, m > n ? 1 : 0, np, long(mp) * np);
  return int(cudaGetLastError());
}

}  // extern "C"
