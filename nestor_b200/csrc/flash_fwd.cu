// Varlen causal flash attention forward for sm_100a (tcgen05 + TMEM + TMA).
//
// Rows of Q/K/V are packed by segment (the members of one attention column in one
// sequence, in token order); attention is causal inside a segment and segments never
// mix. One CTA owns one (q tile of 128 rows, head) pair and walks the kv tiles of its
// segment up to the diagonal:
//     S  = Q K^T            tcgen05.mma, K-major operands, fp32 in TMEM (double-buffered)
//     P  = exp2(S*c - m)    softmax warps: one thread per q row, online max / sum
//     O += P V              tcgen05.mma, B = V (MN-major); A = P in bf16, handed over through tensor memory
//                           (tcgen05.st, A operand read from TMEM) for head dims <= 64, else through a swizzled
//                           shared-memory tile; O stays in TMEM and is rescaled lazily (see the kernel)
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
constexpr int KVS = 3;      // K/V ring depth: a stage is refilled when the P.V product that read it retires (a tile takes
                            // about 1 us to land; with 2 stages that latency sat in every iteration)
constexpr int FK = 64;      // kv rows per tile: with 64 the CTA needs 192 TMEM columns and 64 KB of shared memory,
                            // so two CTAs share an SM and one's softmax overlaps the other's loads and MMAs

// Phase timing (clock64 sums per role, written by the CTAs of head 0) is compiled in only with -DNB_FLASH_DIAG.
#ifdef NB_FLASH_DIAG
#define FD_T(var) const long long var = clock64()
#define FD_ADD(slot, a, b) diag[slot] += (b) - (a)
#else
#define FD_T(var)
#define FD_ADD(slot, a, b)
#endif

struct FlashParams {
  int nseg, H, hd, rows;
  const int* seg_start;        // [nseg + 1]
  float scale_log2;            // softmax scale * log2(e)
  __nv_bfloat16* O; long ldo;  // [rows, H*hd]
  float* lse;                  // [rows, H] log2-domain logsumexp of scaled scores
  int* status;
  int p_tmem;                  // probabilities handed to the P V product through tensor memory instead of shared memory
  long long* diag;             // NB_FLASH_DIAG builds: [grid.x][16] cycle sums
};

__device__ __forceinline__ void st_p_chunk(uint8_t* pbase, int row, int col0, const uint32_t* w) {
  // 8 bf16 (16 B) of row `row`, columns col0..col0+7, into the 128B-swizzled K-major P tile
  int blk = col0 >> 6, ch = (col0 & 63) >> 3;
  uint8_t* dst = pbase + blk * 16384 + row * 128 + ((ch ^ (row & 7)) << 4);
  *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
}

// HDN: N of the P.V product, 64 (hd <= 64) or 128. The output accumulator stays in TMEM across kv tiles (the P.V
// MMAs accumulate into it) relative to a per-row reference maximum that only moves, with a rescale of the
// accumulator in TMEM, when some row of the warp finds a score more than 2^8 above it: probabilities stay below 256,
// exact enough in bf16, and most tiles skip the TMEM round trip of the accumulator.
//
// The softmax loop is written for instruction count, which is what bounds it at head dims this small (a 128 x 64
// score tile is ~100 tensor-core cycles but 8192 exponentials): one TMEM read of the score row into registers, the
// row maximum on raw scores with three-input max, the scale-and-shift as packed two-float FMAs, causal masking only
// on the (at most two) kv tiles that cross the diagonal.
template <int HDN>
__global__ void __launch_bounds__(192, HDN == 64 ? 2 : 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const FlashParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ uint64_t q_full, kv_full[KVS], kv_empty[KVS], s_full[2], s_empty[2], p_ready[2], o_full[2];
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
  uint8_t* sK = sQ + tile_bytes;            // KVS stages
  uint8_t* sV = sK + KVS * ktile_bytes;     // KVS stages
  uint8_t* sP = sV + KVS * ktile_bytes;     // 2 x (128 rows x 64 kv columns: one 16 KB block), alternating by kv tile

  if (warp == 0) {
    // locate this CTA's q tile: tiles are numbered segment by segment, heaviest (last) q tile first
    int b = 0, e = 0, local = 0, nt = 0;
    const bool found = find_segment_tile(p.seg_start, p.nseg, FQ, blockIdx.x, b, e, local, nt);
    if (lane == 0) {
      s_tile[0] = b; s_tile[1] = e; s_tile[2] = b + (nt - 1 - local) * FQ; s_tile[3] = found ? 1 : 0;
      s_abort = 0;
      mbar_init(&q_full, 1);
      for (int i = 0; i < KVS; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); }
      for (int i = 0; i < 2; ++i) {
        mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 4); mbar_init(&o_full[i], 1); mbar_init(&p_ready[i], 4);
      }
      fence_barrier_init();
      prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV);
    }
  }
  __syncthreads();
  if (!s_tile[3]) return;                          // grid is an upper bound on the tile count
  if (warp == 1) { tmem_alloc(&tmem_slot, 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t tS0 = tmem, tO = tmem + 2 * FK;        // S double-buffered in columns [0, 128), O from 128
  const uint32_t tP0 = tmem + 2 * FK + 64;              // bf16 P, 32 columns per buffer, in [192, 256) (head dims <= 64)
  const int seg_b = s_tile[0], seg_e = s_tile[1], q0 = s_tile[2];
  const int ntiles = (min(q0 + FQ, seg_e) - seg_b + FK - 1) / FK;   // kv tiles up to and including the diagonal
  volatile int* abort_flag = &s_abort;

  // Issuing a tcgen05.mma costs its thread some 50 cycles and a commit about as much, and a 128 x 64 tile of this
  // kernel needs seven small MMAs, so the two products are issued by different warps, which run ahead of each other
  // independently: warp 1 issues S = Q K^T as soon as a K tile has landed and the score buffer is drained; warp 0
  // issues P V when the probabilities are written and, since it is the one that learns when a K/V stage is free
  // again, also refills that stage.
  if (warp == 0) {
    const uint32_t idesc_o = make_idesc(FQ, HDN, 0, 1);
    const uint64_t p_desc = sdesc_kmajor(smem_u32(sP));
    const bool el = elect_one();
    auto load_kv = [&](int j) {
      const int s = j % KVS, r0 = seg_b + j * FK;
      mbar_expect_tx(&kv_full[s], 2 * ktile_bytes);
      for (int b = 0; b < nkb; ++b) {
        tma_load_3d(sK + s * ktile_bytes + b * 8192, &tmK, &kv_full[s], b * 64, head, r0);
        tma_load_3d(sV + s * ktile_bytes + b * 8192, &tmV, &kv_full[s], b * 64, head, r0);
      }
    };
    if (el) {
      mbar_expect_tx(&q_full, tile_bytes);
      for (int b = 0; b < nkb; ++b) tma_load_3d(sQ + b * 16384, &tmQ, &q_full, b * 64, head, q0);
      for (int j = 0; j < ntiles && j < KVS; ++j) load_kv(j);
    }
    __syncwarp();
#ifdef NB_FLASH_DIAG
    long long diag[4] = {0, 0, 0, 0};
#endif
    bool ok = true;
    for (int j = 0; j < ntiles && ok; ++j) {
      const int s = j % KVS;
      FD_T(u0);
      // One barrier per P buffer. With a single barrier a softmax warp that runs one tile ahead (it may, the buffers
      // alternate) would supply the fourth arrival of tile j with its arrival for tile j + 1 while a slower warp is
      // still writing its rows of P_j, and the product below would read those rows before they exist. On barrier
      // j & 1 an early arrival is impossible: a warp reaches tile j + 2 only after P_j V_j has retired.
      ok = mbar_wait(&p_ready[j & 1], (j >> 1) & 1, abort_flag, p.status, kTimeoutTmemEmpty);
      if (!ok) break;
      // (the V tile landed before S_j was issued, which precedes these probabilities; waiting on its barrier here as
      // well makes this warp an observer of the copy in its own right)
      ok = mbar_wait(&kv_full[s], (j / KVS) & 1, abort_flag, p.status, kTimeoutFull);
      if (!ok) break;
      tc_fence_after();
      FD_T(u1); FD_ADD(0, u0, u1);
      const uint64_t v_desc = sdesc_mnmajor(smem_u32(sV + s * ktile_bytes), 8192);
      const uint64_t pj_desc = p_desc + uint64_t((j & 1) * (16384 >> 4));
      if (el) {
#pragma unroll
        for (int k = 0; k < FK / 16; ++k) {
          // O accumulates in TMEM over the kv tiles
          if (p.p_tmem) umma_bf16_ts(tO, tP0 + (j & 1) * (FK / 2) + k * 8, v_desc + k * 128, idesc_o, (j | k) != 0);
          else umma_bf16(tO, pj_desc + (k & 3) * 2, v_desc + k * 128, idesc_o, (j | k) != 0);
        }
        umma_commit(&kv_empty[s]);
        umma_commit(&o_full[j & 1]);      // P buffer j & 1 may be rewritten; with the last tile: O is final
      }
      __syncwarp();
      FD_T(u2); FD_ADD(1, u1, u2);
      if (j + KVS < ntiles) {
        // refill this stage once the product just issued has read it
        ok = mbar_wait(&kv_empty[s], (j / KVS) & 1, abort_flag, p.status, kTimeoutEmpty);
        if (!ok) break;
        if (el) load_kv(j + KVS);
        __syncwarp();
      }
      FD_T(u3); FD_ADD(2, u2, u3);
    }
#ifdef NB_FLASH_DIAG
    if (p.diag && head == 0 && lane == 0) for (int i = 0; i < 3; ++i) p.diag[blockIdx.x * 16 + 8 + i] = diag[i];
#endif
  } else if (warp == 1) {
    // Descriptors are computed by the whole warp (warp-uniform values stay in uniform registers, where the MMA
    // instruction reads them) and advance by additions on the 16-byte-unit address field; one elected lane
    // issues. All lanes poll the barriers together, so no shuffle sits between a wait and the issue.
    const uint32_t idesc_s = make_idesc(FQ, FK, 0, 0);
    const uint64_t q_desc = sdesc_kmajor(smem_u32(sQ));
    const int ks = hd16 / 16;
#ifdef NB_FLASH_DIAG
    long long diag[4] = {0, 0, 0, 0};
#endif
    bool ok = mbar_wait(&q_full, 0, abort_flag, p.status, kTimeoutFull);
    for (int j = 0; j < ntiles && ok; ++j) {
      // S_j = Q K_j^T into score buffer j & 1, once the softmax warps have read tile j - 2 out of it
      const int s = j % KVS, sb = j & 1;
      FD_T(u0);
      ok = mbar_wait(&kv_full[s], (j / KVS) & 1, abort_flag, p.status, kTimeoutFull);
      if (!ok) break;
      FD_T(u1); FD_ADD(0, u0, u1);
      if (j >= 2) {
        ok = mbar_wait(&s_empty[sb], ((j - 2) >> 1) & 1, abort_flag, p.status, kTimeoutTmemEmpty);
        if (!ok) break;
        tc_fence_after();
      }
      FD_T(u2); FD_ADD(1, u1, u2);
      const uint64_t k_desc = sdesc_kmajor(smem_u32(sK + s * ktile_bytes));
      const uint32_t d_addr = tS0 + sb * FK;
      if (elect_one()) {
        for (int k = 0; k < ks; ++k) {
          // (64-column block, 32 B per K step) in 16-byte units; blocks are 16 KB apart in Q, 8 KB in K
          const uint32_t qoff = (k >> 2) * 1024 + (k & 3) * 2, koff = (k >> 2) * 512 + (k & 3) * 2;
          umma_bf16(d_addr, q_desc + qoff, k_desc + koff, idesc_s, k != 0);
        }
        umma_commit(&s_full[sb]);
      }
      __syncwarp();
      FD_T(u3); FD_ADD(2, u2, u3);
    }
#ifdef NB_FLASH_DIAG
    if (p.diag && head == 0 && lane == 0) for (int i = 0; i < 3; ++i) p.diag[blockIdx.x * 16 + 12 + i] = diag[i];
#endif
  } else {
    // ---------------------------------------------------------------- softmax + output
    const int q = warp & 3;
    const int r = q * 32 + lane;               // row inside the q tile
    const int qrow = q0 + r;
    const uint32_t lane_off = uint32_t(q * 32) << 16;
    float m = -INFINITY;                       // reference maximum of this row (scaled, log2 domain)
    uint64_t l2 = f2_pack(0.f, 0.f);           // running sum of probabilities, two partial sums
    const uint64_t scale2 = f2_pack(p.scale_log2, p.scale_log2);
    bool ok = true;
#ifdef NB_FLASH_DIAG
    long long diag[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#endif
    for (int j = 0; j < ntiles; ++j) {
      const int s = j & 1;
      FD_T(t0);
      if (!mbar_wait(&s_full[s], (j >> 1) & 1, abort_flag, p.status, kTimeoutTmemFull)) { ok = false; break; }
      tc_fence_after();
      FD_T(t1); FD_ADD(0, t0, t1);
      const uint32_t ts = tS0 + s * FK + lane_off;
      const int kv0 = seg_b + j * FK;
      float sv[FK];
      tmem_ld32(ts, sv); tmem_ld32(ts + 32, sv + 32);
      tmem_ld_wait32x2(sv, sv + 32);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[s]);     // the score buffer may take tile j + 2
      FD_T(t2); FD_ADD(1, t1, t2);
      if (kv0 + FK - 1 > q0) {
        // the tile crosses the diagonal for some row of the q tile: hide columns past this row's own position
        const int lim = qrow - kv0 + 1;
#pragma unroll
        for (int i = 0; i < FK; ++i) sv[i] = i < lim ? sv[i] : -INFINITY;
      }
      // four independent chains, then one merge: the exponentials below all wait for this value
      float m0 = fmax3(sv[0], sv[1], sv[2]), m1 = fmax3(sv[3], sv[4], sv[5]), m2 = fmax3(sv[6], sv[7], sv[8]),
            m3 = fmax3(sv[9], sv[10], sv[11]);
#pragma unroll
      for (int i = 12; i + 7 < FK; i += 8) {
        m0 = fmax3(m0, sv[i], sv[i + 1]); m1 = fmax3(m1, sv[i + 2], sv[i + 3]);
        m2 = fmax3(m2, sv[i + 4], sv[i + 5]); m3 = fmax3(m3, sv[i + 6], sv[i + 7]);
      }
      m0 = fmax3(m0, sv[FK - 4], sv[FK - 3]); m1 = fmax3(m1, sv[FK - 2], sv[FK - 1]);
      const float mr = fmaxf(fmax3(m0, m1, m2), m3);
      const float mx = fmaxf(m, mr * p.scale_log2);
      FD_T(t3); FD_ADD(2, t2, t3);
      // P buffer j & 1 was last read by the P.V product of tile j - 2
      if (j > 1) {
        if (!mbar_wait(&o_full[j & 1], ((j - 2) >> 1) & 1, abort_flag, p.status, kTimeoutTmemFull)) { ok = false; break; }
      }
      FD_T(t4); FD_ADD(3, t3, t4);
      const bool moved = mx > m + 8.f || (m == -INFINITY && mx != -INFINITY);
      if (__any_sync(0xffffffffu, moved)) {
        const float f = (m == -INFINITY) ? 0.f : ex2_approx(m - mx);     // 1 for rows whose maximum did not move
        if (j > 0) {
          // O is rescaled in place: the previous tile's P.V must have retired (the next one is issued only after this
          // warp's arrival below)
          if (!mbar_wait(&o_full[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag, p.status, kTimeoutTmemFull)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < HDN; c += 32) {
            float v[32];
            tmem_ld32(tO + lane_off + c, v); tmem_ld_wait32(v);
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] *= f;
            tmem_st32(tO + lane_off + c, v);
          }
          tmem_st_wait();
        }
        l2 = f2_mul(l2, f2_pack(f, f));
        m = mx;
      }
      FD_T(t5); FD_ADD(4, t4, t5);
      const float neg_m = (m == -INFINITY) ? 0.f : -m;
      const uint64_t neg2 = f2_pack(neg_m, neg_m);
      if (p.p_tmem) {
        // probabilities -> bf16 pairs -> this row's lane of the P buffer in tensor memory
        uint32_t pw[FK / 2];
#pragma unroll
        for (int c = 0; c < FK; c += 2) {
          float t0, t1;
          f2_unpack(f2_fma(f2_pack(sv[c], sv[c + 1]), scale2, neg2), t0, t1);
          const float p0 = ex2_approx(t0), p1 = ex2_approx(t1);
          l2 = f2_add(l2, f2_pack(p0, p1));
          pw[c >> 1] = pack_bf16(p0, p1);
        }
        tmem_st32(tP0 + (j & 1) * (FK / 2) + lane_off, reinterpret_cast<const float*>(pw));
        tmem_st_wait();
      } else
      // probabilities -> bf16 -> swizzled smem, 8 columns (one 16-byte chunk) at a time
#pragma unroll
      for (int c = 0; c < FK; c += 8) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
          float t0, t1;
          f2_unpack(f2_fma(f2_pack(sv[c + i], sv[c + i + 1]), scale2, neg2), t0, t1);
          const float p0 = ex2_approx(t0), p1 = ex2_approx(t1);
          l2 = f2_add(l2, f2_pack(p0, p1));
          w[i >> 1] = pack_bf16(p0, p1);
        }
        st_p_chunk(sP + (j & 1) * 16384, r, c, w);
      }
      FD_T(t6); FD_ADD(5, t5, t6);
      fence_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[j & 1]);
      FD_T(t7); FD_ADD(6, t6, t7);
    }
#ifdef NB_FLASH_DIAG
    if (p.diag && head == 0 && warp == 2 && lane == 0) {
      for (int i = 0; i < 7; ++i) p.diag[blockIdx.x * 16 + i] = diag[i];
      p.diag[blockIdx.x * 16 + 7] = ntiles;
    }
#endif
    if (ok && mbar_wait(&o_full[(ntiles - 1) & 1], ((ntiles - 1) >> 1) & 1, abort_flag, p.status, kTimeoutTmemFull)) {
      tc_fence_after();
      float la, lb;
      f2_unpack(l2, la, lb);
      const float l = la + lb;
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const bool row_ok = qrow < seg_e;
      __nv_bfloat16* dst = p.O + long(qrow) * p.ldo + head * p.hd;
#pragma unroll
      for (int c = 0; c < HDN; c += 16) {
        float v[16];
        tmem_ld16(tO + lane_off + c, v); tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 16; i += 8) {
            if (c + i < p.hd) {
              uint32_t w[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) w[e] = pack_bf16(v[i + 2 * e] * inv, v[i + 2 * e + 1] * inv);
              *reinterpret_cast<uint4*>(dst + c + i) = make_uint4(w[0], w[1], w[2], w[3]);
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

#ifdef NB_FLASH_DIAG
long long* nb_flash_diag_buffer = nullptr;
extern "C" void nb_flash_set_diag(long long* buf) { nb_flash_diag_buffer = buf; }
#endif

extern "C" {

int nb_flash_args_size(void) { return int(sizeof(NbFlashArgs)); }

int nb_flash_fwd(const NbFlashArgs* a, cudaStream_t stream) {
  using namespace nb;
  if (a->hd % 8 || a->hd < 8 || a->hd > 128) return -1;
  if (a->nseg < 1) return -2;
  CUtensorMap tq, tk, tv;
  if (nb_head_map(&tq, a->Q, a->rows, a->H, a->hd, a->ld_qkv)) return -10;
  if (nb_head_map_rows(&tk, a->K, a->rows, a->H, a->hd, a->ld_qkv, FK)) return -11;
  if (nb_head_map_rows(&tv, a->V, a->rows, a->H, a->hd, a->ld_qkv, FK)) return -12;
  FlashParams p;
  p.nseg = a->nseg; p.H = a->H; p.hd = a->hd; p.rows = a->rows; p.seg_start = a->seg_start;
  p.scale_log2 = a->scale * 1.4426950408889634f;
  p.O = reinterpret_cast<__nv_bfloat16*>(a->O); p.ldo = a->ldo; p.lse = a->lse; p.status = a->status;
  p.diag = nullptr;
  p.p_tmem = (a->lazy_rescale & 2) && a->hd <= 64 ? 1 : 0;
#ifdef NB_FLASH_DIAG
  p.diag = nb_flash_diag_buffer;
#endif
  const int nkb = (a->hd + 63) / 64;
  size_t smem = size_t(nkb) * (16384 + 2 * KVS * 8192) + 2 * 16384 + 1024;
  dim3 grid(a->max_tiles, a->H);
#define NB_FWD(HDN)                                                                                 \
  do {                                                                                              \
    static SmemAttr attr;                                                                           \
    if (int e = attr.ensure(flash_fwd_kernel<HDN>, smem)) return e;                                 \
    flash_fwd_kernel<HDN><<<grid, 192, smem, stream>>>(tq, tk, tv, p);                              \
  } while (0)
  if (a->hd <= 64) NB_FWD(64); else NB_FWD(128);
#undef NB_FWD
  return int(cudaGetLastError());
}

}  // extern "C"
