// Bandwidth-bound companions of the GEMM and attention kernels: row gathers for token
// dispatch, weighted slot combines, in-place RoPE on packed q/k, the cross-entropy
// gradient over a logits chunk, and the fused depth-read + RMSNorm.
//
// Every kernel is a pure gather (no atomics): each output element has exactly one writer,
// which is what makes the backward passes deterministic. Counterparts in the reference:
// Triton pack / dispatch / combine kernels (nestor/backbones/triton_packed.py:112-169,
// triton_expert.py:270-344), RoPE epilogue (triton_packed.py:171-322), chunked CE
// (nestor/train/losses.py:177-209), depth read (nestor/backbones/attention_residual.py:488-718).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nb {

// Index checking for the gather-style kernels, compiled in with -DNESTOR_BOUNDS_CHECK (a separate library build, see
// csrc/build.py): an index outside [0, limit) is recorded once in `g_bounds` (code, kernel, index, row) and the access
// is skipped, so a bad plan shows up as a status the host can read and never as a wild read. The normal build compiles
// none of this.
#ifdef NESTOR_BOUNDS_CHECK
__device__ int g_bounds[4] = {0, 0, 0, 0};
__device__ __forceinline__ bool index_ok(long idx, long limit, int kernel_id, long row) {
  if (limit <= 0 || (idx >= 0 && idx < limit)) return true;
  if (atomicCAS(&g_bounds[0], 0, 7) == 0) { g_bounds[1] = kernel_id; g_bounds[2] = int(idx); g_bounds[3] = int(row); }
  return false;
}
#define NB_INDEX_OK(idx, limit, kernel_id, row) index_ok(idx, limit, kernel_id, row)
#else
#define NB_INDEX_OK(idx, limit, kernel_id, row) true
#endif


__device__ __forceinline__ float bf(const __nv_bfloat16 x) { return __bfloat162float(x); }

// out[r, :] = bf16(src[idx[r] / div, :])   (src fp32 or bf16, row pitch lds)
template <typename TIn>
__global__ void gather_rows_kernel(const TIn* __restrict__ src, long lds, const int* __restrict__ idx, int div,
                                   __nv_bfloat16* __restrict__ out, long ldo, int rows, int d, long src_rows) {
  int r = blockIdx.x * blockDim.y + threadIdx.y;
  if (r >= rows) return;
  if (!NB_INDEX_OK(idx[r] / div, src_rows, 1, r)) return;
  const TIn* s = src + long(idx[r] / div) * lds;
  __nv_bfloat16* o = out + long(r) * ldo;
  for (int c = threadIdx.x * 8; c < d; c += blockDim.x * 8) {
    uint32_t w[4];
    if constexpr (sizeof(TIn) == 4) {
      float4 a = *reinterpret_cast<const float4*>(s + c), b = *reinterpret_cast<const float4*>(s + c + 4);
      __nv_bfloat162 t0 = __floats2bfloat162_rn(a.x, a.y), t1 = __floats2bfloat162_rn(a.z, a.w);
      __nv_bfloat162 t2 = __floats2bfloat162_rn(b.x, b.y), t3 = __floats2bfloat162_rn(b.z, b.w);
      w[0] = *reinterpret_cast<uint32_t*>(&t0); w[1] = *reinterpret_cast<uint32_t*>(&t1);
      w[2] = *reinterpret_cast<uint32_t*>(&t2); w[3] = *reinterpret_cast<uint32_t*>(&t3);
      *reinterpret_cast<uint4*>(o + c) = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
      *reinterpret_cast<uint4*>(o + c) = *reinterpret_cast<const uint4*>(s + c);
    }
  }
}

// out[t, g, :] = sum_{e < group} round_bf16(y[idx[(t*G + g)*group + e], :] * w[(t*G + g)*group + e])   (fp32 out)
// With w == nullptr the weight is 1. `accumulate` adds into out instead of overwriting; `round_products`
// rounds each weighted row to bf16 before the fp32 sum (the expert-combine contract).
// `out_bf16` stores the fp32 sums rounded to bf16 (no accumulate): the data gradient that goes back into a bf16 stream.
__global__ void combine_rows_kernel(const __nv_bfloat16* __restrict__ y, long ldy, const int* __restrict__ idx,
                                    const float* __restrict__ w, int group, float* __restrict__ out, long ldo,
                                    int n_out, int d, int accumulate, int round_products, long y_rows, int out_bf16) {
  int o = blockIdx.x * blockDim.y + threadIdx.y;
  if (o >= n_out) return;
  float* dst = out + long(o) * ldo;
  for (int c = threadIdx.x * 8; c < d; c += blockDim.x * 8) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int e = 0; e < group; ++e) {
      int s = o * group + e;
      float ww = w ? w[s] : 1.f;
      if (!NB_INDEX_OK(idx[s], y_rows, 2, s)) continue;
      uint4 q = *reinterpret_cast<const uint4*>(y + long(idx[s]) * ldy + c);
      const __nv_bfloat16* v = reinterpret_cast<const __nv_bfloat16*>(&q);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += round_products ? bf(__float2bfloat16(bf(v[i]) * ww)) : bf(v[i]) * ww;
    }
    if (out_bf16) {
      __nv_bfloat162 t0 = __floats2bfloat162_rn(acc[0], acc[1]), t1 = __floats2bfloat162_rn(acc[2], acc[3]);
      __nv_bfloat162 t2 = __floats2bfloat162_rn(acc[4], acc[5]), t3 = __floats2bfloat162_rn(acc[6], acc[7]);
      __nv_bfloat16* d16 = reinterpret_cast<__nv_bfloat16*>(out) + long(o) * ldo + c;
      *reinterpret_cast<uint4*>(d16) = make_uint4(*reinterpret_cast<uint32_t*>(&t0), *reinterpret_cast<uint32_t*>(&t1),
                                                  *reinterpret_cast<uint32_t*>(&t2), *reinterpret_cast<uint32_t*>(&t3));
      continue;
    }
    float4* d4 = reinterpret_cast<float4*>(dst + c);
    if (accumulate) {
      float4 a = d4[0], b = d4[1];
      d4[0] = make_float4(a.x + acc[0], a.y + acc[1], a.z + acc[2], a.w + acc[3]);
      d4[1] = make_float4(b.x + acc[4], b.y + acc[5], b.z + acc[6], b.w + acc[7]);
    } else {
      d4[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
      d4[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
  }
}

// Backward of the weighted combine, one warp per sorted row r (slot s = slot_of_row[r]):
//   dy[r, :] = bf16(g[s / group, :] * w[s]);   dw[s] = <g[s / group, :], y[r, :]>
__global__ void combine_bwd_kernel(const float* __restrict__ g, long ldg, const __nv_bfloat16* __restrict__ y, long ldy,
                                   const int* __restrict__ slot_of_row, const float* __restrict__ w, int group,
                                   __nv_bfloat16* __restrict__ dy, long lddy, float* __restrict__ dw, int rows, int d,
                                   const float* __restrict__ g2, const float* __restrict__ g3, long ldg2, int g2_div,
                                   float g2_scale, long slots) {
  int r = blockIdx.x * blockDim.y + threadIdx.y;
  if (r >= rows) return;
  int s = slot_of_row[r];
  if (!NB_INDEX_OK(s, slots, 3, r)) return;
  float ww = w ? w[s] : 1.f;
  const float* gr = g + long(s / group) * ldg;
  // optional second gradient of the same output, shared by `g2_div` consecutive slots (the mean over a token's slots
  // that feeds the next depth read): added here instead of by a separate pass over the [slots, d] gradient
  const float* g2r = g2 ? g2 + long(s / g2_div) * ldg2 : nullptr;
  const float* g3r = g3 ? g3 + long(s / g2_div) * ldg2 : nullptr;
  const __nv_bfloat16* yr = y + long(r) * ldy;
  __nv_bfloat16* dr = dy + long(r) * lddy;
  float dot = 0.f;
  for (int c = threadIdx.x * 8; c < d; c += 32 * 8) {
    float4 a = *reinterpret_cast<const float4*>(gr + c), b = *reinterpret_cast<const float4*>(gr + c + 4);
    float gv[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    if (g2r) {
      float4 e = *reinterpret_cast<const float4*>(g2r + c), f = *reinterpret_cast<const float4*>(g2r + c + 4);
      gv[0] += e.x * g2_scale; gv[1] += e.y * g2_scale; gv[2] += e.z * g2_scale; gv[3] += e.w * g2_scale;
      gv[4] += f.x * g2_scale; gv[5] += f.y * g2_scale; gv[6] += f.z * g2_scale; gv[7] += f.w * g2_scale;
    }
    if (g3r) {
      float4 e = *reinterpret_cast<const float4*>(g3r + c), f = *reinterpret_cast<const float4*>(g3r + c + 4);
      gv[0] += e.x * g2_scale; gv[1] += e.y * g2_scale; gv[2] += e.z * g2_scale; gv[3] += e.w * g2_scale;
      gv[4] += f.x * g2_scale; gv[5] += f.y * g2_scale; gv[6] += f.z * g2_scale; gv[7] += f.w * g2_scale;
    }
    uint32_t o[4];
    if (dw) {
      uint4 q = *reinterpret_cast<const uint4*>(yr + c);
      const __nv_bfloat16* v = reinterpret_cast<const __nv_bfloat16*>(&q);
#pragma unroll
      for (int i = 0; i < 8; ++i) dot += gv[i] * bf(v[i]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 t = __floats2bfloat162_rn(gv[2 * i] * ww, gv[2 * i + 1] * ww);
      o[i] = *reinterpret_cast<uint32_t*>(&t);
    }
    *reinterpret_cast<uint4*>(dr + c) = make_uint4(o[0], o[1], o[2], o[3]);
  }
  if (dw) {
#pragma unroll
    for (int sft = 16; sft > 0; sft >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, sft);
    if (threadIdx.x == 0) dw[s] = dot;
  }
}

// In-place rotate-half RoPE on the q and k column ranges of a packed [rows, ld] bf16 buffer.
// One warp per row; `sign` = +1 forward, -1 for the gradient (inverse rotation).
__global__ void rope_kernel(__nv_bfloat16* __restrict__ buf, long ld, const int* __restrict__ pos, int rows, int H,
                            int hd, int k_offset, float log2_base, float sign) {
  int r = blockIdx.x * blockDim.y + threadIdx.y;
  if (r >= rows) return;
  const int half = hd / 2;
  const float p = float(pos[r]);
  __nv_bfloat16* row = buf + long(r) * ld;
  for (int i = threadIdx.x; i < 2 * H * half; i += 32) {
    int part = i / (H * half), rem = i - part * H * half;
    int h = rem / half, j = rem - h * half;
    float inv_freq = exp2f(-log2_base * (2.f * j) / hd);
    float sn, cs;
    sincosf(p * inv_freq, &sn, &cs);
    sn *= sign;
    __nv_bfloat16* x = row + part * k_offset + h * hd;
    float x1 = bf(x[j]), x2 = bf(x[j + half]);
    x[j] = __float2bfloat16(x1 * cs - x2 * sn);
    x[j + half] = __float2bfloat16(x2 * cs + x1 * sn);
  }
}

// Re-pitch heads: dst[r, h, 0:min(hs, hd)] = src[r, h, 0:min(hs, hd)], zero where hd > hs, and zero the columns
// [nheads * hd, dst_cols) of every row. Pads head dims that are not multiples of 8 (30, 60) to the next multiple
// for the TMA-fed attention kernels and strips the padding again; hs and hd are even, pairs move as 32-bit words.
__global__ void repack_heads_kernel(const __nv_bfloat16* __restrict__ src, long ld_src, __nv_bfloat16* __restrict__ dst,
                                    long ld_dst, int rows, int nheads, int hs, int hd, int dst_cols) {
  const int pairs = dst_cols / 2, hp = hd / 2, sp = hs / 2;
  for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < long(rows) * pairs; i += long(gridDim.x) * blockDim.x) {
    const long r = i / pairs;
    const int c = int(i - r * pairs);
    const int h = c / hp, j = c - h * hp;
    uint32_t v = 0u;
    if (h < nheads && j < sp) v = reinterpret_cast<const uint32_t*>(src + r * ld_src + h * hs)[j];
    reinterpret_cast<uint32_t*>(dst + r * ld_dst)[c] = v;
  }
}

// Cross-entropy over a chunk of bf16 logits [n, ld] with per-(row, tile) (max, sumexp) partials:
// loss[row] = lse - logit[target]; logits are overwritten by (softmax - onehot) (zero for ignored rows).
__global__ void ce_grad_kernel(__nv_bfloat16* __restrict__ logits, long ld, int V, const float2* __restrict__ part,
                               int n_tiles, const long* __restrict__ targets, long ignore_index,
                               float* __restrict__ loss, int n) {
  int r = blockIdx.x;
  if (r >= n) return;
  __shared__ float s_lse;
  if (threadIdx.x < 32) {
    float m = -INFINITY;
    for (int t = threadIdx.x; t < n_tiles; t += 32) m = fmaxf(m, part[long(r) * n_tiles + t].x);
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, s));
    float sum = 0.f;
    for (int t = threadIdx.x; t < n_tiles; t += 32) {
      float2 q = part[long(r) * n_tiles + t];
      sum += q.y * __expf(q.x - m);
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, s);
    if (threadIdx.x == 0) s_lse = m + __logf(sum);
  }
  __syncthreads();
  const float lse = s_lse;
  const long tgt = targets[r];
  const bool valid = tgt != ignore_index;
  __nv_bfloat16* row = logits + long(r) * ld;
  if (threadIdx.x == 0) loss[r] = valid ? lse - bf(row[tgt]) : 0.f;
  __syncthreads();
  for (int c = threadIdx.x * 8; c < V; c += blockDim.x * 8) {
    uint4 q = *reinterpret_cast<uint4*>(row + c);
    __nv_bfloat16* v = reinterpret_cast<__nv_bfloat16*>(&q);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float g = valid ? __expf(bf(v[i]) - lse) - ((c + i) == tgt ? 1.f : 0.f) : 0.f;
      v[i] = __float2bfloat16((c + i) < V ? g : 0.f);
    }
    *reinterpret_cast<uint4*>(row + c) = q;
  }
}

// Fused depth read + RMSNorm, one warp per token (d <= 32 * 8 * DEPTH_VEC ... handled by a strided loop):
//   r_i = rsqrt(mean(s_i^2) + eps_read);  z_i = r_i <s_i, q> / sqrt(d);  w = softmax_i(z) * gain_i
//   h = sum_i (w_i r_i) s_i;   out = bf16(h * rsqrt(mean(h^2) + eps_norm) * gamma)
// Online over sources: one pass, running (max, denominator, accumulator). Saves per-(token, source)
// (r_i, u_i = <s_i, q>) and per-token rstd for the backward.
constexpr int kMaxSources = 48;
constexpr int kMaxDepthDim = 1280;     // widest model dim of the fused depth read (10 float4 per lane)
struct SourceList { const float* ptr[kMaxSources]; };

template <int NV>   // d == NV * 32 * 4 is not required; each lane owns NV float4 chunks at stride 32
__global__ void depth_read_norm_fwd_kernel(SourceList src, int n, const float* __restrict__ query,
                                           const float* __restrict__ gains, const float* __restrict__ gamma,
                                           float eps_read, float eps_norm, __nv_bfloat16* __restrict__ out,
                                           float* __restrict__ h_out, float* __restrict__ stats, float* __restrict__ rstd_out,
                                           int T, int d) {
  int t = blockIdx.x * blockDim.y + threadIdx.y;
  if (t >= T) return;
  const int lane = threadIdx.x;
  const int nchunk = d / 4;
  float4 qv[NV], acc[NV];
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    int c = lane + 32 * v;
    qv[v] = c < nchunk ? reinterpret_cast<const float4*>(query)[c] : make_float4(0, 0, 0, 0);
    acc[v] = make_float4(0, 0, 0, 0);
  }
  const float inv_sqrt_d = rsqrtf(float(d));
  float m = -INFINITY, den = 0.f;
  for (int i = 0; i < n; ++i) {
    const float4* s = reinterpret_cast<const float4*>(src.ptr[i] + long(t) * d);
    float4 sv[NV];
    float ss = 0.f, dot = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      int c = lane + 32 * v;
      sv[v] = c < nchunk ? s[c] : make_float4(0, 0, 0, 0);
      ss += sv[v].x * sv[v].x + sv[v].y * sv[v].y + sv[v].z * sv[v].z + sv[v].w * sv[v].w;
      dot += sv[v].x * qv[v].x + sv[v].y * qv[v].y + sv[v].z * qv[v].z + sv[v].w * qv[v].w;
    }
#pragma unroll
    for (int sft = 16; sft > 0; sft >>= 1) {
      ss += __shfl_xor_sync(0xffffffffu, ss, sft);
      dot += __shfl_xor_sync(0xffffffffu, dot, sft);
    }
    float r = rsqrtf(ss / d + eps_read);
    float z = r * dot * inv_sqrt_d;
    float m_new = fmaxf(m, z);
    float a = __expf(m - m_new), e = __expf(z - m_new);
    float coef = e * gains[i] * r;
    den = den * a + e;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      acc[v].x = acc[v].x * a + coef * sv[v].x; acc[v].y = acc[v].y * a + coef * sv[v].y;
      acc[v].z = acc[v].z * a + coef * sv[v].z; acc[v].w = acc[v].w * a + coef * sv[v].w;
    }
    m = m_new;
    if (lane == 0 && stats) { stats[(long(t) * n + i) * 2] = r; stats[(long(t) * n + i) * 2 + 1] = dot; }
  }
  float inv_den = 1.f / den, hs = 0.f;
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    acc[v].x *= inv_den; acc[v].y *= inv_den; acc[v].z *= inv_den; acc[v].w *= inv_den;
    hs += acc[v].x * acc[v].x + acc[v].y * acc[v].y + acc[v].z * acc[v].z + acc[v].w * acc[v].w;
  }
#pragma unroll
  for (int sft = 16; sft > 0; sft >>= 1) hs += __shfl_xor_sync(0xffffffffu, hs, sft);
  float rstd = rsqrtf(hs / d + eps_norm);
  if (lane == 0 && rstd_out) rstd_out[t] = rstd;
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    int c = lane + 32 * v;
    if (c < nchunk) {
      if (h_out) reinterpret_cast<float4*>(h_out + long(t) * d)[c] = acc[v];
      if (out) {
        float4 g = reinterpret_cast<const float4*>(gamma)[c];
        __nv_bfloat162 a = __floats2bfloat162_rn(acc[v].x * rstd * g.x, acc[v].y * rstd * g.y);
        __nv_bfloat162 b = __floats2bfloat162_rn(acc[v].z * rstd * g.z, acc[v].w * rstd * g.w);
        uint2 w = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
        reinterpret_cast<uint2*>(out + long(t) * d)[c] = w;
      }
    }
  }
}

}  // namespace nb

// SM count of the current device (grids of the grid-stride kernels are sized from it).
static int nb_pointwise_sms() {
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 1;
  }
  return sms;
}

extern "C" {

// 1 in a library built with -DNESTOR_BOUNDS_CHECK, 0 otherwise.
int nb_bounds_check_enabled(void) {
#ifdef NESTOR_BOUNDS_CHECK
  return 1;
#else
  return 0;
#endif
}

// Copies {code, kernel (1 gather_rows, 2 combine_rows, 3 combine_bwd), bad index, row} of the first recorded violation
// to `host4` and clears the record (synchronises the device). Zeros in a normal build.
int nb_bounds_check_read(int* host4) {
  host4[0] = host4[1] = host4[2] = host4[3] = 0;
#ifdef NESTOR_BOUNDS_CHECK
  cudaError_t e = cudaMemcpyFromSymbol(host4, nb::g_bounds, 4 * sizeof(int));
  if (e != cudaSuccess) return int(e);
  const int zero[4] = {0, 0, 0, 0};
  e = cudaMemcpyToSymbol(nb::g_bounds, zero, sizeof(zero));
  return int(e);
#else
  return 0;
#endif
}

// `src_rows` / `y_rows` / `slots` below bound the indices (0 = unknown); they are only looked at by a checking build.
int nb_gather_rows(const void* src, int src_is_f32, long lds, const int* idx, int div, void* out, long ldo, int rows,
                   int d, long src_rows, cudaStream_t st) {
  if (d % 8) return -1;
  dim3 block(32, 8), grid((rows + 7) / 8);
  if (src_is_f32)
    nb::gather_rows_kernel<float><<<grid, block, 0, st>>>((const float*)src, lds, idx, div, (__nv_bfloat16*)out, ldo, rows, d,
                                                          src_rows);
  else
    nb::gather_rows_kernel<__nv_bfloat16><<<grid, block, 0, st>>>((const __nv_bfloat16*)src, lds, idx, div,
                                                                  (__nv_bfloat16*)out, ldo, rows, d, src_rows);
  return int(cudaGetLastError());
}

int nb_combine_rows(const void* y, long ldy, const int* idx, const float* w, int group, float* out, long ldo, int n_out,
                    int d, int accumulate, int round_products, long y_rows, int out_bf16, cudaStream_t st) {
  if (d % 8 || (out_bf16 && (accumulate || ldo % 8))) return -1;
  dim3 block(32, 8), grid((n_out + 7) / 8);
  nb::combine_rows_kernel<<<grid, block, 0, st>>>((const __nv_bfloat16*)y, ldy, idx, w, group, out, ldo, n_out, d, accumulate,
                                                 round_products && w != nullptr, y_rows, out_bf16);
  return int(cudaGetLastError());
}

int nb_combine_bwd(const float* g, long ldg, const void* y, long ldy, const int* slot_of_row, const float* w, int group,
                   void* dy, long lddy, float* dw, int rows, int d, const float* g2, const float* g3, long ldg2, int g2_div,
                   float g2_scale, long slots, cudaStream_t st) {
  if (d % 8 || ((g2 || g3) && g2_div < 1)) return -1;
  dim3 block(32, 8), grid((rows + 7) / 8);
  nb::combine_bwd_kernel<<<grid, block, 0, st>>>(g, ldg, (const __nv_bfloat16*)y, ldy, slot_of_row, w, group,
                                                (__nv_bfloat16*)dy, lddy, dw, rows, d, g2, g3, ldg2, g2_div, g2_scale, slots);
  return int(cudaGetLastError());
}

// src [rows, nheads * hs] (pitch ld_src) -> dst [rows, dst_cols] (pitch ld_dst) with head stride hd; see the kernel.
int nb_repack_heads(const void* src, long ld_src, void* dst, long ld_dst, int rows, int nheads, int hs, int hd,
                    int dst_cols, cudaStream_t st) {
  if ((hs | hd | dst_cols) & 1 || dst_cols < nheads * hd || (ld_src & 1) || (ld_dst & 1) || rows < 0) return -1;
  if (rows == 0) return 0;
  long n = long(rows) * (dst_cols / 2);
  const long cap = long(nb_pointwise_sms()) * 16;
  int blocks = int(n / 256 + 1 < cap ? n / 256 + 1 : cap);
  nb::repack_heads_kernel<<<blocks, 256, 0, st>>>((const __nv_bfloat16*)src, ld_src, (__nv_bfloat16*)dst, ld_dst, rows,
                                                  nheads, hs, hd, dst_cols);
  return int(cudaGetLastError());
}

int nb_rope(void* buf, long ld, const int* pos, int rows, int H, int hd, int k_offset, float base, float sign,
            cudaStream_t st) {
  dim3 block(32, 8), grid((rows + 7) / 8);
  nb::rope_kernel<<<grid, block, 0, st>>>((__nv_bfloat16*)buf, ld, pos, rows, H, hd, k_offset, log2f(base), sign);
  return int(cudaGetLastError());
}

int nb_ce_grad(void* logits, long ld, int V, const void* part, int n_tiles, const long* targets, long ignore_index,
               float* loss, int n, cudaStream_t st) {
  if (ld % 8) return -1;
  nb::ce_grad_kernel<<<n, 256, 0, st>>>((__nv_bfloat16*)logits, ld, V, (const float2*)part, n_tiles, targets,
                                        ignore_index, loss, n);
  return int(cudaGetLastError());
}

int nb_depth_read_norm(const float* const* sources, int n, const float* query, const float* gains, const float* gamma,
                       float eps_read, float eps_norm, void* out, float* h_out, float* stats, float* rstd, int T, int d,
                       cudaStream_t st) {
  if (n < 1 || n > nb::kMaxSources || d % 4) return -1;
  nb::SourceList sl;
  for (int i = 0; i < n; ++i) sl.ptr[i] = sources[i];
  dim3 block(32, 4), grid((T + 3) / 4);
  int nv = (d / 4 + 31) / 32;
#define NB_DR(NV) nb::depth_read_norm_fwd_kernel<NV><<<grid, block, 0, st>>>(sl, n, query, gains, gamma, eps_read, \
      eps_norm, (__nv_bfloat16*)out, h_out, stats, rstd, T, d)
  if (nv <= 1) NB_DR(1); else if (nv <= 2) NB_DR(2); else if (nv <= 4) NB_DR(4); else if (nv <= 5) NB_DR(5);
  else if (nv <= 8) NB_DR(8); else if (nv <= 10) NB_DR(10); else return -2;
#undef NB_DR
  return int(cudaGetLastError());
}

}  // extern "C"

// ----------------------------------------------------------------------------------------------
// Backward of the fused depth read + RMSNorm. One warp per token (grid-stride), three sweeps
// over the token's sources (they stay L1/L2-resident between sweeps):
//   1. rebuild h = sum_i a_i s_i from the saved (r_i, u_i); turn dn into dh through the norm
//   2. t_i = <dh, s_i> for every source
//   3. ds_i = a_i dh + du_i q - dr_i r_i^3 s_i / d   written to its own [T, d] slab
// Parameter gradients (query, gains, gamma) are reduced per block and added atomically.
namespace nb {

struct GradList { float* ptr[kMaxSources]; };

template <int NV>
__global__ void depth_read_norm_bwd_kernel(SourceList src, GradList dsrc, int n, const float* __restrict__ query,
                                           const float* __restrict__ gains, const float* __restrict__ gamma,
                                           const float* __restrict__ stats, const float* __restrict__ rstd_in,
                                           const __nv_bfloat16* __restrict__ dn, const float* __restrict__ dh_in,
                                           float* __restrict__ partial, int has_gamma, int T, int d,
                                           unsigned long long acc_mask, const float* __restrict__ h_saved) {
  // Parameter gradients leave the kernel as one partial row per block, [dquery (d) | dgamma (d) | dgains (64)],
  // summed by depth_param_reduce_kernel: thousands of warps adding atomically into the same 2d + n addresses
  // serialised in L2 and cost more than the rest of the kernel.
  // bit i of acc_mask: the gradient of source i is added to what dsrc[i] already holds (a buffer shared by every
  // reader of that source) instead of overwriting it
  __shared__ float s_w[4][kMaxSources], s_t[4][kMaxSources];
  const int lane = threadIdx.x, wy = threadIdx.y;
  const int nchunk = d / 4;
  const float inv_sqrt_d = rsqrtf(float(d));
  // The norm-weight gradient accumulates in this warp's row of s_red (one read-modify-write per token) instead of
  // registers: the kernel is bound by memory latency at low occupancy, and 20 registers fewer is one more block per SM.
  __shared__ float s_red[4][kMaxDepthDim];
  float4* gg_acc = reinterpret_cast<float4*>(&s_red[wy][0]);
  float4 qv[NV], gq[NV];
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    int c = lane + 32 * v;
    qv[v] = c < nchunk ? reinterpret_cast<const float4*>(query)[c] : make_float4(0, 0, 0, 0);
    gq[v] = make_float4(0, 0, 0, 0);
    if (c < nchunk) gg_acc[c] = make_float4(0, 0, 0, 0);
  }
  float dgain_acc[2] = {0.f, 0.f};   // lane owns sources lane and lane + 32
  for (int t = blockIdx.x * blockDim.y + wy; t < T; t += gridDim.x * blockDim.y) {
    // softmax weights from the saved statistics
    float zmax = -INFINITY;
    for (int i = lane; i < n; i += 32) {
      float r = stats[(long(t) * n + i) * 2], u = stats[(long(t) * n + i) * 2 + 1];
      zmax = fmaxf(zmax, r * u * inv_sqrt_d);
    }
#pragma unroll
    for (int sft = 16; sft > 0; sft >>= 1) zmax = fmaxf(zmax, __shfl_xor_sync(0xffffffffu, zmax, sft));
    float zsum = 0.f;
    for (int i = lane; i < n; i += 32) {
      float r = stats[(long(t) * n + i) * 2], u = stats[(long(t) * n + i) * 2 + 1];
      float e = __expf(r * u * inv_sqrt_d - zmax);
      s_w[wy][i] = e; zsum += e;
    }
#pragma unroll
    for (int sft = 16; sft > 0; sft >>= 1) zsum += __shfl_xor_sync(0xffffffffu, zsum, sft);
    __syncwarp();
    const float inv_z = 1.f / zsum;
    // sweep 1: h, read back when the forward kept it (one row instead of a pass over all the sources), else rebuilt
    float4 h[NV];
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int c = lane + 32 * v;
      h[v] = (h_saved && c < nchunk) ? reinterpret_cast<const float4*>(h_saved + long(t) * d)[c] : make_float4(0, 0, 0, 0);
    }
    for (int i = 0; i < n && !h_saved; ++i) {
      float a = s_w[wy][i] * inv_z * gains[i] * stats[(long(t) * n + i) * 2];
      const float4* s = reinterpret_cast<const float4*>(src.ptr[i] + long(t) * d);
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        int c = lane + 32 * v;
        if (c < nchunk) { float4 x = s[c]; h[v].x += a * x.x; h[v].y += a * x.y; h[v].z += a * x.z; h[v].w += a * x.w; }
      }
    }
    // dn -> dh through y = h * rstd * gamma
    float4 dh[NV];
    if (dn) {
      const float rstd = rstd_in[t];
      float dot = 0.f;
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        int c = lane + 32 * v;
        dh[v] = make_float4(0, 0, 0, 0);
        if (c < nchunk) {
          uint2 raw = reinterpret_cast<const uint2*>(dn + long(t) * d)[c];
          __nv_bfloat162 p0 = *reinterpret_cast<__nv_bfloat162*>(&raw.x), p1 = *reinterpret_cast<__nv_bfloat162*>(&raw.y);
          float4 g = reinterpret_cast<const float4*>(gamma)[c];
          float4 dy = make_float4(bf(p0.x), bf(p0.y), bf(p1.x), bf(p1.y));
          float4 ga = gg_acc[c];
          ga.x += dy.x * h[v].x * rstd; ga.y += dy.y * h[v].y * rstd;
          ga.z += dy.z * h[v].z * rstd; ga.w += dy.w * h[v].w * rstd;
          gg_acc[c] = ga;
          dh[v] = make_float4(dy.x * g.x, dy.y * g.y, dy.z * g.z, dy.w * g.w);
          dot += dh[v].x * h[v].x + dh[v].y * h[v].y + dh[v].z * h[v].z + dh[v].w * h[v].w;
        }
      }
#pragma unroll
      for (int sft = 16; sft > 0; sft >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, sft);
      const float k2 = dot * rstd * rstd * rstd / d;
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        dh[v].x = dh[v].x * rstd - h[v].x * k2; dh[v].y = dh[v].y * rstd - h[v].y * k2;
        dh[v].z = dh[v].z * rstd - h[v].z * k2; dh[v].w = dh[v].w * rstd - h[v].w * k2;
      }
    } else {
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        int c = lane + 32 * v;
        dh[v] = c < nchunk ? reinterpret_cast<const float4*>(dh_in + long(t) * d)[c] : make_float4(0, 0, 0, 0);
      }
    }
    // sweep 2: t_i = <dh, s_i>, two sources at a time (their loads are in flight together, their reductions interleave)
    int i2 = 0;
    for (; i2 + 1 < n; i2 += 2) {
      const float4* s0 = reinterpret_cast<const float4*>(src.ptr[i2] + long(t) * d);
      const float4* s1 = reinterpret_cast<const float4*>(src.ptr[i2 + 1] + long(t) * d);
      float a0 = 0.f, a1 = 0.f;
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        int c = lane + 32 * v;
        if (c < nchunk) {
          float4 x = s0[c], y = s1[c];
          a0 += dh[v].x * x.x + dh[v].y * x.y + dh[v].z * x.z + dh[v].w * x.w;
          a1 += dh[v].x * y.x + dh[v].y * y.y + dh[v].z * y.z + dh[v].w * y.w;
        }
      }
#pragma unroll
      for (int sft = 16; sft > 0; sft >>= 1) {
        a0 += __shfl_xor_sync(0xffffffffu, a0, sft);
        a1 += __shfl_xor_sync(0xffffffffu, a1, sft);
      }
      if (lane == 0) { s_t[wy][i2] = a0; s_t[wy][i2 + 1] = a1; }
    }
    for (int i = i2; i < n; ++i) {
      const float4* s = reinterpret_cast<const float4*>(src.ptr[i] + long(t) * d);
      float acc = 0.f;
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        int c = lane + 32 * v;
        if (c < nchunk) { float4 x = s[c]; acc += dh[v].x * x.x + dh[v].y * x.y + dh[v].z * x.z + dh[v].w * x.w; }
      }
#pragma unroll
      for (int sft = 16; sft > 0; sft >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, sft);
      if (lane == 0) s_t[wy][i] = acc;
    }
    __syncwarp();
    float mix = 0.f;   // sum_j w_j dw_j
    for (int i = lane; i < n; i += 32)
      mix += s_w[wy][i] * inv_z * s_t[wy][i] * gains[i] * stats[(long(t) * n + i) * 2];
#pragma unroll
    for (int sft = 16; sft > 0; sft >>= 1) mix += __shfl_xor_sync(0xffffffffu, mix, sft);
    for (int i = lane, slot = 0; i < n; i += 32, ++slot)
      dgain_acc[slot] += s_t[wy][i] * s_w[wy][i] * inv_z * stats[(long(t) * n + i) * 2];
    // sweep 3: ds_i
    for (int i = 0; i < n; ++i) {
      const float r = stats[(long(t) * n + i) * 2], u = stats[(long(t) * n + i) * 2 + 1];
      const float w = s_w[wy][i] * inv_z, ti = s_t[wy][i], g = gains[i];
      const float dz = w * (ti * g * r - mix);
      const float dr = ti * w * g + dz * u * inv_sqrt_d;
      const float du = dz * r * inv_sqrt_d;
      const float a = w * g * r, cs = -dr * r * r * r / d;
      const float4* s = reinterpret_cast<const float4*>(src.ptr[i] + long(t) * d);
      float4* o = reinterpret_cast<float4*>(dsrc.ptr[i] + long(t) * d);
      // all loads of the source row (and of the gradient row it is added to) first: a store between two loads
      // would make the second wait, since the compiler cannot know that the rows do not overlap
      const bool add = (acc_mask >> i) & 1ull;
      float4 x[NV], old[NV];
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        const int c = lane + 32 * v;
        x[v] = c < nchunk ? s[c] : make_float4(0, 0, 0, 0);
      }
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        const int c = lane + 32 * v;
        old[v] = (add && c < nchunk) ? o[c] : make_float4(0, 0, 0, 0);
      }
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        const int c = lane + 32 * v;
        if (c < nchunk) {
          o[c] = make_float4(a * dh[v].x + du * qv[v].x + cs * x[v].x + old[v].x, a * dh[v].y + du * qv[v].y + cs * x[v].y + old[v].y,
                             a * dh[v].z + du * qv[v].z + cs * x[v].z + old[v].z, a * dh[v].w + du * qv[v].w + cs * x[v].w + old[v].w);
          gq[v].x += du * x[v].x; gq[v].y += du * x[v].y; gq[v].z += du * x[v].z; gq[v].w += du * x[v].w;
        }
      }
    }
    __syncwarp();
  }
  // parameter gradients: sum the block's four warps through shared memory, write the block's partial row
  const int tid = wy * 32 + lane, stride = 2 * d + 64;
  float* prow = partial + long(blockIdx.x) * stride;
  __syncthreads();                                   // every warp's gamma row is complete
  if (has_gamma)
    for (int j = tid; j < d; j += 128) prow[d + j] = s_red[0][j] + s_red[1][j] + s_red[2][j] + s_red[3][j];
  __syncthreads();
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    int c = lane + 32 * v;
    if (c < nchunk) gg_acc[c] = gq[v];
  }
  __syncthreads();
  for (int j = tid; j < d; j += 128) prow[j] = s_red[0][j] + s_red[1][j] + s_red[2][j] + s_red[3][j];
  __syncthreads();
  s_red[wy][lane] = dgain_acc[0]; s_red[wy][lane + 32] = dgain_acc[1];
  __syncthreads();
  if (tid < 64) prow[2 * d + tid] = s_red[0][tid] + s_red[1][tid] + s_red[2][tid] + s_red[3][tid];
}

// Column sums of the [nblk, 2d + 64] partial rows -> dquery [d], dgamma [d] (optional), dgains [n].
__global__ void depth_param_reduce_kernel(const float* __restrict__ partial, int nblk, int d, int n,
                                          float* __restrict__ dquery, float* __restrict__ dgains,
                                          float* __restrict__ dgamma) {
  __shared__ float s_acc[8][32];
  const int stride = 2 * d + 64;
  const int col = blockIdx.x * 32 + threadIdx.x;
  float acc = 0.f;
  if (col < stride)
    for (int r = threadIdx.y; r < nblk; r += 8) acc += partial[long(r) * stride + col];
  s_acc[threadIdx.y][threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.y == 0 && col < stride) {
    float t = 0.f;
#pragma unroll
    for (int r = 0; r < 8; ++r) t += s_acc[r][threadIdx.x];
    if (col < d) dquery[col] = t;
    else if (col < 2 * d) { if (dgamma) dgamma[col - d] = t; }
    else if (col - 2 * d < n) dgains[col - 2 * d] = t;
  }
}

}  // namespace nb

extern "C" int nb_depth_read_norm_bwd(const float* const* sources, float* const* dsources, int n, const float* query,
                                      const float* gains, const float* gamma, const float* stats, const float* rstd,
                                      const void* dn, const float* dh, float* dquery, float* dgains, float* dgamma, int T,
                                      int d, unsigned long long acc_mask, float* scratch, const float* h_saved,
                                      cudaStream_t st) {
  // scratch: fp32 [8 * SMs * (2d + 64)] per-block partial sums of the parameter gradients
  if (n < 1 || n > nb::kMaxSources || d % 4 || d > nb::kMaxDepthDim || !scratch) return -1;
  nb::SourceList sl; nb::GradList gl;
  for (int i = 0; i < n; ++i) { sl.ptr[i] = sources[i]; gl.ptr[i] = dsources[i]; }
  dim3 block(32, 4);
  int blocks = (T + 3) / 4;
  if (blocks > nb_pointwise_sms() * 8) blocks = nb_pointwise_sms() * 8;
  int nv = (d / 4 + 31) / 32;
#define NB_DRB(NV) nb::depth_read_norm_bwd_kernel<NV><<<blocks, block, 0, st>>>(sl, gl, n, query, gains, gamma, stats, rstd, \
      (const __nv_bfloat16*)dn, dh, scratch, dgamma != nullptr, T, d, acc_mask, h_saved)
  if (nv <= 1) NB_DRB(1); else if (nv <= 2) NB_DRB(2); else if (nv <= 4) NB_DRB(4); else if (nv <= 5) NB_DRB(5);
  else if (nv <= 8) NB_DRB(8); else if (nv <= 10) NB_DRB(10); else return -2;
#undef NB_DRB
  nb::depth_param_reduce_kernel<<<(2 * d + 64 + 31) / 32, dim3(32, 8), 0, st>>>(scratch, blocks, d, n, dquery, dgains, dgamma);
  return int(cudaGetLastError());
}

// ----------------------------------------------------------------------------------------------
// Residual-stream bookkeeping of a column layer, one pass each (float4 per thread over [T, d]).
namespace nb {

__device__ __forceinline__ float rbf(float x) { return __bfloat162float(__float2bfloat16(x)); }
__device__ __forceinline__ float4 f4add(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }
__device__ __forceinline__ float4 f4scale(float4 a, float s) { return make_float4(a.x * s, a.y * s, a.z * s, a.w * s); }

// mid[t] = running[t] + mean_j attn[t, j]
__global__ void mid_source_kernel(const float4* __restrict__ running, const float4* __restrict__ attn,
                                  float4* __restrict__ mid, long n4, int d4, int k) {
  long i = blockIdx.x * long(blockDim.x) + threadIdx.x;
  if (i >= n4) return;
  long t = i / d4; int c = int(i - t * d4);
  float4 acc = make_float4(0, 0, 0, 0);
  for (int j = 0; j < k; ++j) acc = f4add(acc, attn[(t * k + j) * d4 + c]);
  acc = f4scale(acc, 1.f / k);
  if (running) acc = f4add(acc, running[i]);
  mid[i] = acc;
}

// streams'[t,j] = streams[t,j] + attn[t,j] + rbf(p1[t]*priv[t,j]) + rbf(p0[t]*pub[t]);  running' = running + mean_j(update)
__global__ void layer_combine_kernel(const float4* __restrict__ attn, const float4* __restrict__ priv,
                                     const float4* __restrict__ pub, const float* __restrict__ path,
                                     const float4* __restrict__ streams, const float4* __restrict__ running,
                                     float4* __restrict__ streams_out, float4* __restrict__ running_out, long n4, int d4,
                                     int k) {
  long i = blockIdx.x * long(blockDim.x) + threadIdx.x;
  if (i >= n4) return;
  long t = i / d4; int c = int(i - t * d4);
  float p0 = path ? path[2 * t] : 1.f, p1 = path ? path[2 * t + 1] : 1.f;
  float4 pb = pub[i];
  if (path) pb = make_float4(rbf(p0 * pb.x), rbf(p0 * pb.y), rbf(p0 * pb.z), rbf(p0 * pb.w));
  float4 mean = make_float4(0, 0, 0, 0);
  for (int j = 0; j < k; ++j) {
    long o = (t * k + j) * d4 + c;
    float4 u = f4add(attn[o], pb);
    if (priv) {
      float4 pv = priv[o];
      u = f4add(u, make_float4(rbf(p1 * pv.x), rbf(p1 * pv.y), rbf(p1 * pv.z), rbf(p1 * pv.w)));
    }
    mean = f4add(mean, u);
    streams_out[o] = streams ? f4add(streams[o], u) : u;
  }
  mean = f4scale(mean, 1.f / k);
  running_out[i] = running ? f4add(running[i], mean) : mean;
}

// Backward: du[t,j] = ds[t,j] + dr[t]/k;  d_attn = du (optional: a consumer that can add dr[t]/k itself reads ds);
// d_priv = p1*du;  d_pub = p0*sum_j du;
// d_path (per token, warp-reduced over d): dp1 = sum_{j,c} du*priv, dp0 = sum_c (sum_j du)*pub. One warp per token.
__global__ void layer_combine_bwd_kernel(const float* __restrict__ ds, const float* __restrict__ dr,
                                         const float* __restrict__ priv, const float* __restrict__ pub,
                                         const float* __restrict__ path, float* __restrict__ d_attn,
                                         float* __restrict__ d_priv, float* __restrict__ d_pub, float* __restrict__ d_path,
                                         int T, int d, int k) {
  int t = blockIdx.x * blockDim.y + threadIdx.y;
  if (t >= T) return;
  const int lane = threadIdx.x;
  float p0 = path ? path[2 * t] : 1.f, p1 = path ? path[2 * t + 1] : 1.f;
  float a0 = 0.f, a1 = 0.f;
  const float inv_k = 1.f / k;
  for (int c = lane * 4; c < d; c += 128) {
    float4 r = dr ? *reinterpret_cast<const float4*>(dr + long(t) * d + c) : make_float4(0, 0, 0, 0);
    r = f4scale(r, inv_k);
    float4 sum = make_float4(0, 0, 0, 0);
    for (int j = 0; j < k; ++j) {
      long o = (long(t) * k + j) * d + c;
      float4 u = ds ? f4add(*reinterpret_cast<const float4*>(ds + o), r) : r;
      if (d_attn) *reinterpret_cast<float4*>(d_attn + o) = u;
      sum = f4add(sum, u);
      if (priv) {
        float4 pv = *reinterpret_cast<const float4*>(priv + o);
        a1 += u.x * pv.x + u.y * pv.y + u.z * pv.z + u.w * pv.w;
        *reinterpret_cast<float4*>(d_priv + o) = f4scale(u, p1);
      }
    }
    float4 pb = *reinterpret_cast<const float4*>(pub + long(t) * d + c);
    a0 += sum.x * pb.x + sum.y * pb.y + sum.z * pb.z + sum.w * pb.w;
    *reinterpret_cast<float4*>(d_pub + long(t) * d + c) = f4scale(sum, p0);
  }
  if (d_path) {
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) { a0 += __shfl_xor_sync(0xffffffffu, a0, s); a1 += __shfl_xor_sync(0xffffffffu, a1, s); }
    if (lane == 0) { d_path[2 * t] = a0; d_path[2 * t + 1] = a1; }
  }
}

// Block exit: agg[t] = mean_j s[t,j]; dev[j][t] = s[t,j] - agg[t]   (dev is source-major so every export is contiguous)
__global__ void block_exit_kernel(const float4* __restrict__ s, float4* __restrict__ dev, float4* __restrict__ agg,
                                  long n4, int d4, int k) {
  long i = blockIdx.x * long(blockDim.x) + threadIdx.x;
  if (i >= n4) return;
  long t = i / d4; int c = int(i - t * d4);
  float4 m = make_float4(0, 0, 0, 0);
  for (int j = 0; j < k; ++j) m = f4add(m, s[(t * k + j) * d4 + c]);
  m = f4scale(m, 1.f / k);
  agg[i] = m;
  for (int j = 0; j < k; ++j) {
    float4 v = s[(t * k + j) * d4 + c];
    dev[long(j) * n4 + i] = make_float4(v.x - m.x, v.y - m.y, v.z - m.z, v.w - m.w);
  }
}
// d_s[t,j] = d_dev[j][t] - mean_j' d_dev[j'][t] + d_agg[t]/k
__global__ void block_exit_bwd_kernel(const float4* __restrict__ d_dev, const float4* __restrict__ d_agg,
                                      float4* __restrict__ d_s, long n4, int d4, int k) {
  long i = blockIdx.x * long(blockDim.x) + threadIdx.x;
  if (i >= n4) return;
  long t = i / d4; int c = int(i - t * d4);
  float4 m = make_float4(0, 0, 0, 0);
  if (d_dev) for (int j = 0; j < k; ++j) m = f4add(m, d_dev[long(j) * n4 + i]);
  float4 corr = d_agg ? f4add(f4scale(m, -1.f / k), f4scale(d_agg[i], 1.f / k)) : f4scale(m, -1.f / k);
  for (int j = 0; j < k; ++j) {
    float4 v = d_dev ? d_dev[long(j) * n4 + i] : make_float4(0, 0, 0, 0);
    d_s[(t * k + j) * d4 + c] = f4add(v, corr);
  }
}

}  // namespace nb

extern "C" {
int nb_mid_source(const float* running, const float* attn, float* mid, int T, int d, int k, cudaStream_t st) {
  long n4 = long(T) * d / 4;
  nb::mid_source_kernel<<<unsigned((n4 + 255) / 256), 256, 0, st>>>((const float4*)running, (const float4*)attn, (float4*)mid, n4, d / 4, k);
  return int(cudaGetLastError());
}
int nb_layer_combine(const float* attn, const float* priv, const float* pub, const float* path, const float* streams,
                     const float* running, float* streams_out, float* running_out, int T, int d, int k, cudaStream_t st) {
  long n4 = long(T) * d / 4;
  nb::layer_combine_kernel<<<unsigned((n4 + 255) / 256), 256, 0, st>>>(
      (const float4*)attn, (const float4*)priv, (const float4*)pub, path, (const float4*)streams, (const float4*)running,
      (float4*)streams_out, (float4*)running_out, n4, d / 4, k);
  return int(cudaGetLastError());
}
int nb_layer_combine_bwd(const float* ds, const float* dr, const float* priv, const float* pub, const float* path,
                         float* d_attn, float* d_priv, float* d_pub, float* d_path, int T, int d, int k, cudaStream_t st) {
  dim3 block(32, 8), grid((T + 7) / 8);
  nb::layer_combine_bwd_kernel<<<grid, block, 0, st>>>(ds, dr, priv, pub, path, d_attn, d_priv, d_pub, d_path, T, d, k);
  return int(cudaGetLastError());
}
int nb_block_exit(const float* s, float* dev, float* agg, int T, int d, int k, cudaStream_t st) {
  long n4 = long(T) * d / 4;
  nb::block_exit_kernel<<<unsigned((n4 + 255) / 256), 256, 0, st>>>((const float4*)s, (float4*)dev, (float4*)agg, n4, d / 4, k);
  return int(cudaGetLastError());
}
int nb_block_exit_bwd(const float* d_dev, const float* d_agg, float* d_s, int T, int d, int k, cudaStream_t st) {
  long n4 = long(T) * d / 4;
  nb::block_exit_bwd_kernel<<<unsigned((n4 + 255) / 256), 256, 0, st>>>((const float4*)d_dev, (const float4*)d_agg, (float4*)d_s, n4, d / 4, k);
  return int(cudaGetLastError());
}
}
