// Varlen causal flash attention forward for sm_100a (tcgen05 + TMEM + TMA).
//
// Rows of Q/K/V are packed by segment (the members of one attention column in one
// sequence, in token order); attention is causal inside a segment and segments never
// mix. One CTA owns one (q tile of 128 rows, head) pair and walks the kv tiles of its
// segment up to the diagonal:
//     S  = Q K^T            tcgen05.mma, K-major operands, fp32 in TMEM (double-buffered)
//     P  = exp2(S*c - m)    softmax warps: one thread per q row, online max / sum
//     Oj = P V              tcgen05.mma, A = P (bf16, written to swizzled smem), B = V (MN-major)
//     O  = O*alpha + Oj     in registers
// Heads are `hd` wide (any multiple of 8 up to 128); tiles are zero-extended to a multiple
// of 16 by TMA out-of-bounds fill (the tensor map's innermost extent is `hd`).
// Tiles start at the segment's first row, so a q or kv tile may run past the segment end;
// the causal mask hides such kv rows from valid q rows and the store masks such q rows.
//
// Replaces torch's varlen_attn / SDPA calls of the reference (nestor/backbones/nestor.py:6357,
// :6213, :5802) including its 1/head_dim logit scale (:3201).
#include "sm100.cuh"
#include "flash.h"

namespace nb {

constexpr int FQ = 128;      // q rows per CTA
constexpr int FK = 64;      // kv rows per tile: with 64 the CTA needs 192 TMEM columns and 64 KB of shared memory,
                            // so two CTAs share an SM and one's softmax overlaps the other's loads and MMAs
constexpr int kMaxSeg = 1024;

struct FlashParams {
  int nseg, H, hd, rows;
  const int* seg_start;        // [nseg + 1]
  float scale_log2;            // softmax scale * log2(e)
  __nv_bfloat16* O; long ldo;  // [rows, H*hd]
  float* lse;                  // [rows, H] log2-domain logsumexp of scaled scores
  int* status;
};

__device__ __forceinline__ void st_p_chunk(uint8_t* pbase, int row, int col0, const uint32_t* w) {
  // 8 bf16 (16 B) of row `row`, columns col0..col0+7, into the 128B-swizzled K-major P tile
  int blk = col0 >> 6, ch = (col0 & 63) >> 3;
  uint8_t* dst = pbase + blk * 16384 + row * 128 + ((ch ^ (row & 7)) << 4);
  *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
}

// HDN: N of the P.V product, 64 (hd <= 64) or 128. LAZY: O stays in TMEM across kv tiles and is rescaled only when a
// row maximum moves by more than 2^8 (otherwise O is folded into registers after every tile).
template <int HDN, bool LAZY>
__global__ void __launch_bounds__(192, HDN == 64 ? 2 : 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const FlashParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ uint64_t q_full, kv_full[2], kv_empty[2], s_full[2], p_ready, o_full;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_abort;
  __shared__ int s_tile[4];   // seg begin, seg end, q0, valid

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y;
  const int nkb = (p.hd + 63) / 64;                 // 64-column blocks per operand tile
  const int hd16 = (p.hd + 15) & ~15;   // reduction width of Q K^T
  const uint32_t tile_bytes = uint32_t(nkb) * 16384;   // Q tile: 128 rows, 64-column blocks of 16 KB
  const uint32_t ktile_bytes = uint32_t(nkb) * 8192;   // K / V tile: 64 rows, 64-column blocks of 8 KB
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + tile_bytes;          // 2 stages
  uint8_t* sV = sK + 2 * ktile_bytes;     // 2 stages
  uint8_t* sP = sV + 2 * ktile_bytes;     // 128 rows x 64 kv columns: one 16 KB block

  if (threadIdx.x == 0) {
    // locate this CTA's q tile: tiles are numbered segment by segment, heaviest (last) q tile first
    int t = blockIdx.x, found = 0, b = 0, e = 0, q0 = 0;
    for (int s = 0; s < p.nseg; ++s) {
      b = p.seg_start[s]; e = p.seg_start[s + 1];
      int nt = (e - b + FQ - 1) / FQ;
      if (t < nt) { q0 = b + (nt - 1 - t) * FQ; found = 1; break; }
      t -= nt;
    }
    s_tile[0] = b; s_tile[1] = e; s_tile[2] = q0; s_tile[3] = found;
    s_abort = 0;
    mbar_init(&q_full, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); mbar_init(&s_full[i], 1); }
    mbar_init(&p_ready, 4); mbar_init(&o_full, 1);
    fence_barrier_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV);
  }
  __syncthreads();
  if (!s_tile[3]) return;                          // grid is an upper bound on the tile count
  if (warp == 1) { tmem_alloc(&tmem_slot, 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t tS0 = tmem, tO = tmem + 2 * FK;        // S double-buffered in columns [0, 128), O from 128
  const int seg_b = s_tile[0], seg_e = s_tile[1], q0 = s_tile[2];
  const int ntiles = (min(q0 + FQ, seg_e) - seg_b + FK - 1) / FK;   // kv tiles up to and including the diagonal
  volatile int* abort_flag = &s_abort;

  if (warp == 0) {
    if (elect_one()) {
      mbar_expect_tx(&q_full, tile_bytes);
      for (int b = 0; b < nkb; ++b) tma_load_3d(sQ + b * 16384, &tmQ, &q_full, b * 64, head, q0);
      for (int j = 0; j < ntiles; ++j) {
        int s = j & 1;
        if (!mbar_wait(&kv_empty[s], ((j >> 1) & 1) ^ 1, abort_flag, p.status, kTimeoutEmpty)) break;
        mbar_expect_tx(&kv_full[s], 2 * ktile_bytes);
        int r0 = seg_b + j * FK;
        for (int b = 0; b < nkb; ++b) {
          tma_load_3d(sK + s * ktile_bytes + b * 8192, &tmK, &kv_full[s], b * 64, head, r0);
          tma_load_3d(sV + s * ktile_bytes + b * 8192, &tmV, &kv_full[s], b * 64, head, r0);
        }
      }
    }
  } else if (warp == 1) {
    // Descriptors are computed by the whole warp (warp-uniform values stay in uniform registers, where the MMA
    // instruction reads them) and advance by additions on the 16-byte-unit address field; one elected lane
    // issues. All lanes poll the barriers together, so no shuffle sits between a wait and the issue.
    const uint32_t idesc_s = make_idesc(FQ, FK, 0, 0);
    const uint32_t idesc_o = make_idesc(FQ, HDN, 0, 1);
    const uint64_t q_desc = sdesc_kmajor(smem_u32(sQ));
    const uint64_t p_desc = sdesc_kmajor(smem_u32(sP));
    const int ks = hd16 / 16;
    bool ok = true;
    auto issue_s = [&](int j) {
      // S_j = Q K_j^T into buffer j&1
      const int s = j & 1;
      ok = mbar_wait(&kv_full[s], (j >> 1) & 1, abort_flag, p.status, kTimeoutFull);
      if (!ok) return;
      const uint64_t k_desc = sdesc_kmajor(smem_u32(sK + s * ktile_bytes));
      const uint32_t d_addr = tS0 + s * FK;
      if (elect_one()) {
        for (int k = 0; k < ks; ++k) {
          // (64-column block, 32 B per K step) in 16-byte units; blocks are 16 KB apart in Q, 8 KB in K
          const uint32_t qoff = (k >> 2) * 1024 + (k & 3) * 2, koff = (k >> 2) * 512 + (k & 3) * 2;
          umma_bf16(d_addr, q_desc + qoff, k_desc + koff, idesc_s, k != 0);
        }
        umma_commit(&s_full[s]);
      }
      __syncwarp();
    };
    ok = mbar_wait(&q_full, 0, abort_flag, p.status, kTimeoutFull);
    if (ok) issue_s(0);
    for (int j = 0; j < ntiles && ok; ++j) {
      if (j + 1 < ntiles) { issue_s(j + 1); if (!ok) break; }
      ok = mbar_wait(&p_ready, j & 1, abort_flag, p.status, kTimeoutTmemEmpty);
      if (!ok) break;
      tc_fence_after();
      const int s = j & 1;
      const uint64_t v_desc = sdesc_mnmajor(smem_u32(sV + s * ktile_bytes), 8192);
      if (elect_one()) {
#pragma unroll
        for (int k = 0; k < FK / 16; ++k)
          umma_bf16(tO, p_desc + (k & 3) * 2, v_desc + k * 128, idesc_o, LAZY ? (j | k) != 0 : k != 0);   // lazy mode: O accumulates in TMEM over the kv tiles
        umma_commit(&kv_empty[s]);
        umma_commit(&o_full);
      }
      __syncwarp();
    }
  } else {
    // ---------------------------------------------------------------- softmax + output
    const int q = warp & 3;
    const int r = q * 32 + lane;               // row inside the q tile
    const int qrow = q0 + r;
    const uint32_t lane_off = uint32_t(q * 32) << 16;
    float m = -INFINITY, l = 0.f;
    float o[LAZY ? 1 : HDN];     // eager mode: running output in registers
    bool ok = true;
    if constexpr (LAZY) {
      // O stays in TMEM and is accumulated by the MMAs across kv tiles, relative to a reference maximum m that is
      // only moved (and O rescaled in TMEM) when some row of the warp finds a score more than 2^8 above it: the
      // probabilities stay below 256, exact enough in bf16, and most tiles skip the 2 x HDN TMEM round trip.
      for (int j = 0; j < ntiles; ++j) {
        int s = j & 1;
        if (!mbar_wait(&s_full[s], (j >> 1) & 1, abort_flag, p.status, kTimeoutTmemFull)) { ok = false; break; }
        tc_fence_after();
        const uint32_t ts = tS0 + s * FK + lane_off;
        const int kv0 = seg_b + j * FK;
        const int lim = min(FK, qrow - kv0 + 1);     // columns < lim are visible (causal); the diagonal spans two tiles
        // pass 1: row max
        float mx = m;
        for (int c = 0; c < FK; c += 32) {
          float v[32];
          tmem_ld32(ts + c, v); tmem_ld_wait();
  #pragma unroll
          for (int i = 0; i < 32; ++i) if (c + i < lim) mx = fmaxf(mx, v[i] * p.scale_log2);
        }
        // the previous tile's P.V must have retired before P is overwritten (and before O is touched)
        if (j > 0) {
          if (!mbar_wait(&o_full, (j - 1) & 1, abort_flag, p.status, kTimeoutTmemFull)) { ok = false; break; }
          tc_fence_after();
        }
        const bool moved = mx > m + 8.f || (m == -INFINITY && mx != -INFINITY);
        if (__any_sync(0xffffffffu, moved)) {
          const float f = (m == -INFINITY) ? 0.f : exp2f(m - mx);     // 1 for rows whose maximum did not move
          if (j > 0) {
  #pragma unroll
            for (int c = 0; c < HDN; c += 32) {
              float v[32];
              tmem_ld32(tO + lane_off + c, v); tmem_ld_wait();
  #pragma unroll
              for (int i = 0; i < 32; ++i) v[i] *= f;
              tmem_st32(tO + lane_off + c, v);
            }
            tmem_st_wait();
          }
          l *= f;
          m = mx;
        }
        const float m_use = (m == -INFINITY) ? 0.f : m;
        // pass 2: probabilities -> bf16 -> swizzled smem
        float rs = 0.f;
        for (int c = 0; c < FK; c += 32) {
          float v[32];
          tmem_ld32(ts + c, v); tmem_ld_wait();
          uint32_t w[16];
  #pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float p0 = (c + i < lim) ? exp2f(v[i] * p.scale_log2 - m_use) : 0.f;
            float p1 = (c + i + 1 < lim) ? exp2f(v[i + 1] * p.scale_log2 - m_use) : 0.f;
            __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
            rs += __bfloat162float(pk.x) + __bfloat162float(pk.y);
            w[i >> 1] = *reinterpret_cast<uint32_t*>(&pk);
          }
  #pragma unroll
          for (int g = 0; g < 4; ++g) st_p_chunk(sP, r, c + g * 8, w + g * 4);
        }
        l += rs;
        fence_async_smem();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_ready);
      }
    } else {
  #pragma unroll
      for (int i = 0; i < HDN; ++i) o[i] = 0.f;
      for (int j = 0; j < ntiles; ++j) {
        int s = j & 1;
        if (!mbar_wait(&s_full[s], (j >> 1) & 1, abort_flag, p.status, kTimeoutTmemFull)) { ok = false; break; }
        tc_fence_after();
        const uint32_t ts = tS0 + s * FK + lane_off;
        const int kv0 = seg_b + j * FK;
        const int lim = min(FK, qrow - kv0 + 1);     // columns < lim are visible (causal); the diagonal spans two tiles
        // pass 1: row max
        float mx = m;
        for (int c = 0; c < FK; c += 32) {
          float v[32];
          tmem_ld32(ts + c, v); tmem_ld_wait();
  #pragma unroll
          for (int i = 0; i < 32; ++i) if (c + i < lim) mx = fmaxf(mx, v[i] * p.scale_log2);
        }
        const float m_new = mx;
        const float alpha = (m == -INFINITY) ? 0.f : exp2f(m - m_new);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        // fold the previous tile's P.V into the running output before P is overwritten
        if (j > 0) {
          if (!mbar_wait(&o_full, (j - 1) & 1, abort_flag, p.status, kTimeoutTmemFull)) { ok = false; break; }
          tc_fence_after();
  #pragma unroll
          for (int c = 0; c < HDN; c += 16) {
            float v[16];
            tmem_ld16(tO + lane_off + c, v); tmem_ld_wait();
  #pragma unroll
            for (int i = 0; i < 16; ++i) o[c + i] = (o[c + i] + v[i]) * alpha;
          }
        }
        // pass 2: probabilities -> bf16 -> swizzled smem
        float rs = 0.f;
        for (int c = 0; c < FK; c += 32) {
          float v[32];
          tmem_ld32(ts + c, v); tmem_ld_wait();
          uint32_t w[16];
  #pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float p0 = (c + i < lim) ? exp2f(v[i] * p.scale_log2 - m_use) : 0.f;
            float p1 = (c + i + 1 < lim) ? exp2f(v[i + 1] * p.scale_log2 - m_use) : 0.f;
            __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
            rs += __bfloat162float(pk.x) + __bfloat162float(pk.y);
            w[i >> 1] = *reinterpret_cast<uint32_t*>(&pk);
          }
  #pragma unroll
          for (int g = 0; g < 4; ++g) st_p_chunk(sP, r, c + g * 8, w + g * 4);
        }
        l = l * alpha + rs;
        m = m_new;
        fence_async_smem();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_ready);
      }
    }
    if (ok && mbar_wait(&o_full, (ntiles - 1) & 1, abort_flag, p.status, kTimeoutTmemFull)) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const bool row_ok = qrow < seg_e;
      __nv_bfloat16* dst = p.O + long(qrow) * p.ldo + head * p.hd;
#pragma unroll
      for (int c = 0; c < HDN; c += 16) {
        {
          float v[16];
          tmem_ld16(tO + lane_off + c, v); tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int i = 0; i < 16; i += 8) {
              if (c + i < p.hd) {
                uint32_t w[4];
#pragma unroll
                for (int e = 0; e < 4; ++e)
                  w[e] = LAZY ? pack_bf16(v[i + 2 * e] * inv, v[i + 2 * e + 1] * inv)
                              : pack_bf16((o[c + i + 2 * e] + v[i + 2 * e]) * inv, (o[c + i + 2 * e + 1] + v[i + 2 * e + 1]) * inv);
                *reinterpret_cast<uint4*>(dst + c + i) = make_uint4(w[0], w[1], w[2], w[3]);
              }
            }
          }
        }
      }
      if (row_ok) p.lse[long(qrow) * p.H + head] = (l > 0.f) ? m + log2f(l) : -INFINITY;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 256); }
}

}  // namespace nb

#include <string.h>

namespace {
typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                             const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                             CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn flash_encode_fn() {
  static EncodeFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess || !ptr) return nullptr;
    fn = reinterpret_cast<EncodeFn>(ptr);
  }
  return fn;
}
}  // namespace

// [rows, H, hd] view of a bf16 buffer: element (r, h, c) at base + r*row_pitch + h*hd + c.
// Box = 64 columns x 1 head x 128 rows; columns past `hd` read as zero.
extern "C" int nb_head_map_rows(CUtensorMap* m, const void* base, long rows, int H, int hd, long row_pitch_elems,
                                int box_rows) {
  EncodeFn fn = flash_encode_fn();
  if (!fn) return 1;
  cuuint64_t gd[3] = {cuuint64_t(hd), cuuint64_t(H), cuuint64_t(rows)};
  cuuint64_t gs[2] = {cuuint64_t(hd) * 2, cuuint64_t(row_pitch_elems) * 2};
  cuuint32_t bx[3] = {64, 1, cuuint32_t(box_rows)};
  cuuint32_t es[3] = {1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), gd, gs, bx, es,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 2;
}

extern "C" int nb_head_map(CUtensorMap* m, const void* base, long rows, int H, int hd, long row_pitch_elems) {
  return nb_head_map_rows(m, base, rows, H, hd, row_pitch_elems, 128);
}

extern "C" {

int nb_flash_args_size(void) { return int(sizeof(NbFlashArgs)); }

int nb_flash_fwd(const NbFlashArgs* a, cudaStream_t stream) {
  using namespace nb;
  if (a->hd % 8 || a->hd < 8 || a->hd > 128) return -1;
  if (a->nseg < 1 || a->nseg > kMaxSeg) return -2;
  CUtensorMap tq, tk, tv;
  if (nb_head_map(&tq, a->Q, a->rows, a->H, a->hd, a->ld_qkv)) return -10;
  if (nb_head_map_rows(&tk, a->K, a->rows, a->H, a->hd, a->ld_qkv, FK)) return -11;
  if (nb_head_map_rows(&tv, a->V, a->rows, a->H, a->hd, a->ld_qkv, FK)) return -12;
  FlashParams p;
  p.nseg = a->nseg; p.H = a->H; p.hd = a->hd; p.rows = a->rows; p.seg_start = a->seg_start;
  p.scale_log2 = a->scale * 1.4426950408889634f;
  p.O = reinterpret_cast<__nv_bfloat16*>(a->O); p.ldo = a->ldo; p.lse = a->lse; p.status = a->status;
  const int nkb = (a->hd + 63) / 64;
  size_t smem = size_t(nkb) * (16384 + 4 * 8192) + 16384 + 1024;
  dim3 grid(a->max_tiles, a->H);
#define NB_FWD(HDN, LAZY)                                                                                          \
  do {                                                                                                             \
    static SmemAttr attr;                                                                                          \
    if (int e = attr.ensure(flash_fwd_kernel<HDN, LAZY>, smem)) return e;                                          \
    flash_fwd_kernel<HDN, LAZY><<<grid, 192, smem, stream>>>(tq, tk, tv, p);                                       \
  } while (0)
  if (a->hd <= 64) { if (a->lazy_rescale) NB_FWD(64, true); else NB_FWD(64, false); }
  else { if (a->lazy_rescale) NB_FWD(128, true); else NB_FWD(128, false); }
#undef NB_FWD
  return int(cudaGetLastError());
}

}  // extern "C"
