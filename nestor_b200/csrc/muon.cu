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

// A matrix is split over `gridDim.y` blocks (a 640 x 640 matrix on one block ran at one SM's pace; a bucket of a few
// matrices left most of the chip idle). `rows` x `cols` is the wide orientation (rows <= cols) of the m x n input.
// Pass 1: each block sums the squares of the bf16-rounded values of its slice into partial[matrix][block].
__global__ void __launch_bounds__(256) ns_sumsq_kernel(const float* __restrict__ g, float* __restrict__ partial, long numel) {
  __shared__ float red[32];
  const float* src = g + long(blockIdx.x) * numel;
  const long per = (numel + gridDim.y - 1) / gridDim.y;
  const long lo = long(blockIdx.y) * per, hi = lo + per < numel ? lo + per : numel;
  float ss = 0.f;
  for (long i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float v = __bfloat162float(__float2bfloat16(src[i]));
    ss += v * v;
  }
  ss = block_sum(ss, red);
  if (threadIdx.x == 0) partial[long(blockIdx.x) * gridDim.y + blockIdx.y] = ss;
}

// Pass 2: every block adds the matrix's partial sums in the same fixed order (the result does not depend on the
// schedule), then scales, casts and orients its slice of output rows; padding is written as zeros.
__global__ void __launch_bounds__(256) ns_prepare_kernel(const float* __restrict__ g, const float* __restrict__ partial,
                                                         __nv_bfloat16* __restrict__ x, int m, int n, int transpose, int mp,
                                                         int np, long x_batch_stride) {
  const float* src = g + long(blockIdx.x) * m * n;
  __nv_bfloat16* dst = x + long(blockIdx.x) * x_batch_stride;
  float total = 0.f;
  for (int i = 0; i < int(gridDim.y); ++i) total += partial[long(blockIdx.x) * gridDim.y + i];
  const float inv = 1.f / (sqrtf(total) + 1e-7f);
  const int rows = transpose ? n : m, cols = transpose ? m : n;
  const int per = (mp + gridDim.y - 1) / gridDim.y;
  const int r0 = blockIdx.y * per, r1 = min(mp, r0 + per);
  for (int r = r0; r < r1; ++r)
    for (int c = threadIdx.x; c < np; c += blockDim.x) {
      float v = 0.f;
      if (r < rows && c < cols) v = __bfloat162float(__float2bfloat16(transpose ? src[long(c) * n + r] : src[long(r) * n + c])) * inv;
      dst[long(r) * np + c] = __float2bfloat16(v);
    }
}

__global__ void __launch_bounds__(256) ns_finish_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                                        int m, int n, int transpose, int np, long x_batch_stride) {
  const __nv_bfloat16* src = x + long(blockIdx.x) * x_batch_stride;
  __nv_bfloat16* dst = out + long(blockIdx.x) * m * n;
  const int per = (m + gridDim.y - 1) / gridDim.y;
  const int r0 = blockIdx.y * per, r1 = min(m, r0 + per);
  for (int r = r0; r < r1; ++r)
    for (int c = threadIdx.x; c < n; c += blockDim.x)
      dst[long(r) * n + c] = transpose ? src[long(c) * np + r] : src[long(r) * np + c];
}

}  // namespace nbm

extern "C" {

// Blocks per matrix: enough to put about four blocks on every SM for the whole batch, at most 32.
static int ns_splits(int batch) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int s = (4 * sms + batch - 1) / batch;
  return s < 1 ? 1 : (s > 32 ? 32 : s);
}

// g: fp32 [batch, m, n] contiguous. x: bf16 [batch, mp, np] (mp, np >= the wide dims, multiples of 8).
// scratch: fp32 [batch * 32] partial sums of squares.
int nb_ns_prepare(const float* g, void* x, int batch, int m, int n, int mp, int np, float* scratch, cudaStream_t st) {
  if (batch <= 0) return 0;
  const int transpose = m > n ? 1 : 0;
  const int rows = transpose ? n : m, cols = transpose ? m : n;
  if (mp < rows || np < cols || (mp % 8) || (np % 8) || !scratch) return -1;
  const dim3 grid(batch, ns_splits(batch));
  nbm::ns_sumsq_kernel<<<grid, 256, 0, st>>>(g, scratch, long(m) * n);
  nbm::ns_prepare_kernel<<<grid, 256, 0, st>>>(g, scratch, reinterpret_cast<__nv_bfloat16*>(x), m, n, transpose, mp, np,
                                               long(mp) * np);
  return int(cudaGetLastError());
}

int nb_ns_finish(const void* x, void* out, int batch, int m, int n, int mp, int np, cudaStream_t st) {
  if (batch <= 0) return 0;
  const dim3 grid(batch, ns_splits(batch));
  nbm::ns_finish_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<__nv_bfloat16*>(out),
                                              m, n, m > n ? 1 : 0, np, long(mp) * np);
  return int(cudaGetLastError());
}

}  // extern "C"
