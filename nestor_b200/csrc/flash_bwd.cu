// Varlen causal flash attention backward for sm_100a (tcgen05 + TMEM + TMA).
//
// Two launches of one templated kernel, both recomputing the probabilities from the saved
// log-sum-exp (log2 domain):
//   MODE 0 (dK, dV): a CTA owns a kv tile of 128 rows and walks the q tiles at or below it.
//       S^T = K Q^T,  dP^T = V dO^T              (tcgen05, K-major operands, fp32 in TMEM)
//       P^T = exp2(S^T c - lse[q]),  dS^T = P^T (dP^T - delta[q])   (one thread per kv row)
//       dV += P^T dO,  dK += dS^T Q               (A from swizzled smem, B = dO / Q read MN-major)
//   MODE 1 (dQ): a CTA owns a q tile and walks the kv tiles up to the diagonal.
//       S = Q K^T,  dP = dO V^T,  dS = P (dP - delta[q]),  dQ += dS K
// delta[q] = sum_c dO[q, c] O[q, c] comes from `attn_delta_kernel`. Gradients of the scaled
// scores are folded back with the softmax scale when dQ / dK are stored.
// The same shared-memory tile serves as a K-major operand of the score products and as an
// MN-major operand of the accumulate products, so every tile is fetched once.
// The MMA warp issues the score products of tile it + 1 as soon as the softmax warps have read tile it's scores out
// of TMEM, and the accumulate products of tile it when its dS / P^T tiles are written: the two chains overlap.
#include "sm100.cuh"
#include "flash.h"

namespace nb {

constexpr int BT = 128;     // rows of the resident tile (kv tile in MODE 0, q tile in MODE 1)
constexpr int BX = 64;      // rows of a streamed tile: half a resident tile, so that score + dP accumulators take 128
                            // TMEM columns, a CTA needs 256 columns and < 100 KB of shared memory, and two CTAs share an SM

struct FlashBwdParams {
  int nseg, H, hd, rows, stages;
  const int* seg_start;
  float scale_log2, scale;
  const float* lse;      // [rows, H]
  const float* delta;    // [rows, H]
  __nv_bfloat16* out1; __nv_bfloat16* out2; long ldo;   // MODE 0: dK, dV; MODE 1: dQ
  int* status;
};

__device__ __forceinline__ void st_tile_chunk(uint8_t* base, int row, int col0, const uint32_t* w) {
  int blk = col0 >> 6, ch = (col0 & 63) >> 3;
  *reinterpret_cast<uint4*>(base + blk * 16384 + row * 128 + ((ch ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
}

template <int MODE, int HDN>
__global__ void __launch_bounds__(320, HDN == 64 ? 2 : 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tmR1, const __grid_constant__ CUtensorMap tmR2,
                 const __grid_constant__ CUtensorMap tmX1, const __grid_constant__ CUtensorMap tmX2,
                 const FlashBwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ uint64_t r_full, x_full[3], x_empty[3], sc_full, sc_empty, ds_ready, acc_done;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_abort;
  __shared__ int s_tile[4];
  __shared__ __align__(16) float s_lse[8][32], s_delta[8][32];   // negated; the 32 columns of each softmax warp (no cross-warp barrier)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y;
  const int nkb = (p.hd + 63) / 64;
  const int hd16 = (p.hd + 15) & ~15;
  const uint32_t tile_bytes = uint32_t(nkb) * 16384;   // resident tile: 128 rows, 64-column blocks of 16 KB
  const uint32_t xtile_bytes = uint32_t(nkb) * 8192;   // streamed tile: 64 rows, 64-column blocks of 8 KB
  const int stages = p.stages;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sR1 = smem;
  uint8_t* sR2 = sR1 + tile_bytes;
  uint8_t* sX = sR2 + tile_bytes;                       // stages x (X1, X2)
  uint8_t* sDS = sX + stages * 2 * xtile_bytes;         // 16 KB: dS (or dS^T), 128 rows x 64 streamed columns
  uint8_t* sPT = sDS + 16384;                           // 16 KB: P^T (MODE 0 only)

  if (warp == 0) {
    int b = 0, e = 0, local = 0, nt = 0;
    const bool found = find_segment_tile(p.seg_start, p.nseg, BT, blockIdx.x, b, e, local, nt);
    if (lane == 0) {
      // heaviest first: MODE 0 the earliest kv tile, MODE 1 the last q tile
      s_tile[0] = b; s_tile[1] = e; s_tile[2] = (MODE == 0) ? b + local * BT : b + (nt - 1 - local) * BT; s_tile[3] = found ? 1 : 0;
      s_abort = 0;
      mbar_init(&r_full, 1);
      for (int i = 0; i < 3; ++i) { mbar_init(&x_full[i], 1); mbar_init(&x_empty[i], 1); }
      mbar_init(&sc_full, 1); mbar_init(&sc_empty, 8); mbar_init(&ds_ready, 8); mbar_init(&acc_done, 1);
      fence_barrier_init();
      prefetch_tmap(&tmR1); prefetch_tmap(&tmR2); prefetch_tmap(&tmX1); prefetch_tmap(&tmX2);
    }
  }
  __syncthreads();
  if (!s_tile[3]) return;
  constexpr uint32_t kTmemCols = HDN == 64 ? 256 : 512;   // S 64 + dP 64 + accumulators 2 x HDN
  if (warp == 1) { tmem_alloc(&tmem_slot, kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t tS = tmem, tDP = tmem + BX, tA1 = tmem + 2 * BX, tA2 = tmem + 2 * BX + HDN;
  const int seg_b = s_tile[0], seg_e = s_tile[1], r0 = s_tile[2];
  // streamed tiles: MODE 0 -> q tiles r0, r0+128, ... below seg_e; MODE 1 -> kv tiles seg_b .. r0
  const int x_first = (MODE == 0) ? r0 : seg_b;
  // MODE 0: q rows r0 .. seg_e; MODE 1: kv rows seg_b .. r0 + 127 (up to and including the diagonal tile)
  const int niter = (MODE == 0) ? (seg_e - r0 + BX - 1) / BX : (min(r0 + BT, seg_e) - seg_b + BX - 1) / BX;
  volatile int* abort_flag = &s_abort;

  if (warp == 0) {
    if (elect_one()) {
      mbar_expect_tx(&r_full, 2 * tile_bytes);
      for (int b = 0; b < nkb; ++b) {
        tma_load_3d(sR1 + b * 16384, &tmR1, &r_full, b * 64, head, r0);
        tma_load_3d(sR2 + b * 16384, &tmR2, &r_full, b * 64, head, r0);
      }
      for (int it = 0; it < niter; ++it) {
        int s = it % stages;
        if (!mbar_wait(&x_empty[s], ((it / stages) & 1) ^ 1, abort_flag, p.status, kTimeoutEmpty)) break;
        mbar_expect_tx(&x_full[s], 2 * xtile_bytes);
        int x0 = x_first + it * BX;
        uint8_t* d = sX + s * 2 * xtile_bytes;
        for (int b = 0; b < nkb; ++b) {
          tma_load_3d(d + b * 8192, &tmX1, &x_full[s], b * 64, head, x0);
          tma_load_3d(d + xtile_bytes + b * 8192, &tmX2, &x_full[s], b * 64, head, x0);
        }
      }
    }
  } else if (warp == 1) {
    // Warp-uniform descriptor arithmetic, one elected lane issues (see flash_fwd.cu).
    const uint32_t idesc_sc = make_idesc(BT, BX, 0, 0);
    const uint32_t idesc_acc = make_idesc(BT, HDN, 0, 1);
    const uint64_t r1_desc = sdesc_kmajor(smem_u32(sR1)), r2_desc = sdesc_kmajor(smem_u32(sR2));
    const uint64_t ds_desc = sdesc_kmajor(smem_u32(sDS)), pt_desc = sdesc_kmajor(smem_u32(sPT));
    const int ks = hd16 / 16;
    bool ok = mbar_wait(&r_full, 0, abort_flag, p.status, kTimeoutFull);
    // The score products of tile it + 1 are issued as soon as the softmax warps have read tile it's scores out of
    // TMEM (sc_empty), i.e. while they are still computing on them; the accumulate products of tile it follow when its
    // dS / P^T tiles are written (ds_ready). One iteration then costs the longer of the two chains instead of their
    // sum. `ss` / `sph` walk the ring for the score products, `s` / `ph` for the accumulate products.
    int s = 0, ss = 0; uint32_t sph = 0;
    auto issue_scores = [&](int stage) {
      uint8_t* x1 = sX + stage * 2 * xtile_bytes;
      uint8_t* x2 = x1 + xtile_bytes;
      const uint64_t x1_k = sdesc_kmajor(smem_u32(x1)), x2_k = sdesc_kmajor(smem_u32(x2));
      if (elect_one()) {
        for (int k = 0; k < ks; ++k) {   // 64-column blocks are 16 KB apart in the resident tile, 8 KB in the streamed one
          const uint32_t roff = (k >> 2) * 1024 + (k & 3) * 2, xoff = (k >> 2) * 512 + (k & 3) * 2;
          umma_bf16(tS, r1_desc + roff, x1_k + xoff, idesc_sc, k != 0);
        }
        for (int k = 0; k < ks; ++k) {
          const uint32_t roff = (k >> 2) * 1024 + (k & 3) * 2, xoff = (k >> 2) * 512 + (k & 3) * 2;
          umma_bf16(tDP, r2_desc + roff, x2_k + xoff, idesc_sc, k != 0);
        }
        umma_commit(&sc_full);
      }
      __syncwarp();
    };
    if (ok && niter > 0) {
      ok = mbar_wait(&x_full[0], 0, abort_flag, p.status, kTimeoutFull);
      if (ok) issue_scores(0);
      if (++ss == stages) { ss = 0; sph ^= 1; }
    }
    for (int it = 0; it < niter && ok; ++it) {
      if (it + 1 < niter) {
        // tile it's scores have left TMEM: the next tile's products may overwrite them
        ok = mbar_wait(&sc_empty, it & 1, abort_flag, p.status, kTimeoutTmemEmpty);
        if (!ok) break;
        ok = mbar_wait(&x_full[ss], sph, abort_flag, p.status, kTimeoutFull);
        if (!ok) break;
        tc_fence_after();
        issue_scores(ss);
        if (++ss == stages) { ss = 0; sph ^= 1; }
      }
      uint8_t* x1 = sX + s * 2 * xtile_bytes;
      uint8_t* x2 = x1 + xtile_bytes;
      const uint64_t x1_mn = sdesc_mnmajor(smem_u32(x1), 8192), x2_mn = sdesc_mnmajor(smem_u32(x2), 8192);
      ok = mbar_wait(&ds_ready, it & 1, abort_flag, p.status, kTimeoutTmemEmpty);
      if (!ok) break;
      tc_fence_after();
      if (elect_one()) {
#pragma unroll
        for (int k = 0; k < BX / 16; ++k) {
          const uint32_t aoff = (k & 3) * 2;
          if (MODE == 0) {
            umma_bf16(tA1, pt_desc + aoff, x2_mn + k * 128, idesc_acc, (it | k) != 0);  // dV += P^T dO
            umma_bf16(tA2, ds_desc + aoff, x1_mn + k * 128, idesc_acc, (it | k) != 0);  // dK += dS^T Q
          } else {
            umma_bf16(tA1, ds_desc + aoff, x1_mn + k * 128, idesc_acc, (it | k) != 0);  // dQ += dS K
          }
        }
        umma_commit(&x_empty[s]);
        umma_commit(&acc_done);
      }
      __syncwarp();
      if (++s == stages) s = 0;
    }
  } else {
    // Eight warps: warp w reads TMEM lane quarter w % 4 (its 32 rows of the resident tile); the two warps of a quarter
    // split the streamed tile's 64 columns, so every row is worked on by two threads. Nothing here is bound by a
    // unit's throughput (exponential pipe ~30 %, issue slots ~30 % with one thread per row); what matters is how many
    // independent instruction streams the schedulers can switch between while TMEM reads, exponentials and
    // shared-memory stores are in flight.
    const int q4 = warp & 3;
    const int half = (warp - 2) >> 2;               // which 32 streamed columns
    const int r = q4 * 32 + lane;
    const int grow = r0 + r;                        // global row owned by this thread
    const uint32_t lane_off = uint32_t(q4 * 32) << 16;
    const int c0 = half * 32;
    float* nlse_c = s_lse[warp - 2];
    float* ndel_c = s_delta[warp - 2];
    float my_nlse = 0.f, my_ndelta = 0.f;
    if (MODE == 1 && grow < p.rows) { my_nlse = -p.lse[long(grow) * p.H + head]; my_ndelta = -p.delta[long(grow) * p.H + head]; }
    const uint64_t my_nlse2 = f2_pack(my_nlse, my_nlse), my_ndelta2 = f2_pack(my_ndelta, my_ndelta);
    const uint64_t scale2 = f2_pack(p.scale_log2, p.scale_log2);
    bool ok = true;
    float pre_l = 0.f, pre_d = 0.f;
    auto fetch_stats = [&](int xbase) {
      const int xr = xbase + c0 + lane;
      const bool in = xr < seg_e;
      pre_l = in ? -p.lse[long(xr) * p.H + head] : -INFINITY;   // exp2(-inf) = 0 for rows past the segment
      pre_d = in ? -p.delta[long(xr) * p.H + head] : 0.f;
    };
    if (MODE == 0) fetch_stats(x_first);
    for (int it = 0; it < niter; ++it) {
      const int x0 = x_first + it * BX;
      if (MODE == 0) {
        // the streamed q rows' (negated) log-sum-exp and delta: this iteration's values were fetched during the previous
        // one, the next iteration's are requested now, so their latency never sits between two tiles
        __syncwarp();
        nlse_c[lane] = pre_l; ndel_c[lane] = pre_d;
        __syncwarp();
        if (it + 1 < niter) fetch_stats(x0 + BX);
      }
      if (!mbar_wait(&sc_full, it & 1, abort_flag, p.status, kTimeoutTmemFull)) { ok = false; break; }
      tc_fence_after();
      // does any (row of the resident tile, column of the streamed tile) pair fall on the hidden side of the diagonal?
      const bool diag = (MODE == 0) ? (x0 < r0 + BT - 1) : (x0 + BX - 1 > r0);
      float sv[32], dv[32];
      tmem_ld32(tS + lane_off + c0, sv); tmem_ld32(tDP + lane_off + c0, dv);
      tmem_ld_wait32x2(sv, dv);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sc_empty);          // the next tile's score products may overwrite S and dP
      // phase 1: scaled, shifted scores and (dP - delta), two columns per instruction
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        const uint64_t nl2 = (MODE == 0) ? *reinterpret_cast<const uint64_t*>(nlse_c + i) : my_nlse2;
        const uint64_t nd2 = (MODE == 0) ? *reinterpret_cast<const uint64_t*>(ndel_c + i) : my_ndelta2;
        f2_unpack(f2_fma(f2_pack(sv[i], sv[i + 1]), scale2, nl2), sv[i], sv[i + 1]);
        f2_unpack(f2_add(f2_pack(dv[i], dv[i + 1]), nd2), dv[i], dv[i + 1]);
      }
      // phase 2: probabilities (independent exponentials back to back)
#pragma unroll
      for (int i = 0; i < 32; ++i) sv[i] = ex2_approx(sv[i]);
      if (diag) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const bool vis = (MODE == 0) ? (x0 + c0 + i) >= grow : (x0 + c0 + i) <= grow;
          sv[i] = vis ? sv[i] : 0.f;
        }
      }
      // phase 3: dS = P (dP - delta), both rounded to bf16 into the swizzled operand tiles
      uint32_t wp[16], wd[16];
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        float d0, d1;
        f2_unpack(f2_mul(f2_pack(sv[i], sv[i + 1]), f2_pack(dv[i], dv[i + 1])), d0, d1);
        wd[i >> 1] = pack_bf16(d0, d1);
        if (MODE == 0) wp[i >> 1] = pack_bf16(sv[i], sv[i + 1]);
      }
      // the dS / P^T tiles are free once the previous iteration's accumulate products have retired (they have been
      // running under the arithmetic above)
      if (it > 0 && !mbar_wait(&acc_done, (it - 1) & 1, abort_flag, p.status, kTimeoutTmemFull)) { ok = false; break; }
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        st_tile_chunk(sDS, r, c0 + 8 * g, wd + 4 * g);
        if (MODE == 0) st_tile_chunk(sPT, r, c0 + 8 * g, wp + 4 * g);
      }
      fence_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ds_ready);
    }
    if (ok && mbar_wait(&acc_done, (niter - 1) & 1, abort_flag, p.status, kTimeoutTmemFull)) {
      tc_fence_after();
      const bool row_ok = grow < seg_e;
      const long o = long(grow) * p.ldo + head * p.hd;
      // the two warps of a lane quarter take alternating 16-column groups of the accumulators
#pragma unroll
      for (int c = 16 * half; c < HDN; c += 32) {
        if (c >= p.hd) break;
        float a1[16], a2[16];
        tmem_ld16(tA1 + lane_off + c, a1);
        if (MODE == 0) tmem_ld16(tA2 + lane_off + c, a2);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 16; i += 8) {
            if (c + i < p.hd) {
              uint32_t w[4];
              if (MODE == 0) {
#pragma unroll
                for (int e = 0; e < 4; ++e) w[e] = pack_bf16(a2[i + 2 * e] * p.scale, a2[i + 2 * e + 1] * p.scale);
                *reinterpret_cast<uint4*>(p.out1 + o + c + i) = make_uint4(w[0], w[1], w[2], w[3]);     // dK
#pragma unroll
                for (int e = 0; e < 4; ++e) w[e] = pack_bf16(a1[i + 2 * e], a1[i + 2 * e + 1]);
                *reinterpret_cast<uint4*>(p.out2 + o + c + i) = make_uint4(w[0], w[1], w[2], w[3]);     // dV
              } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) w[e] = pack_bf16(a1[i + 2 * e] * p.scale, a1[i + 2 * e + 1] * p.scale);
                *reinterpret_cast<uint4*>(p.out1 + o + c + i) = make_uint4(w[0], w[1], w[2], w[3]);     // dQ
              }
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, kTmemCols); }
}

// delta[row, h] = sum_c dO[row, h, c] * O[row, h, c]; one warp per (row, head).
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ dO, const __nv_bfloat16* __restrict__ O, long ld_do,
                                  long ld_o, float* __restrict__ delta, int rows, int H, int hd) {
  int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= rows * H) return;
  int row = w / H, h = w - row * H;
  const __nv_bfloat16* a = dO + long(row) * ld_do + h * hd;
  const __nv_bfloat16* b = O + long(row) * ld_o + h * hd;
  float acc = 0.f;
  for (int c = lane; c < hd; c += 32) acc += __bfloat162float(a[c]) * __bfloat162float(b[c]);
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (lane == 0) delta[w] = acc;
}

}  // namespace nb

extern "C" int nb_head_map(CUtensorMap* m, const void* base, long rows, int H, int hd, long row_pitch_elems);
extern "C" int nb_head_map_rows(CUtensorMap* m, const void* base, long rows, int H, int hd, long row_pitch_elems, int box_rows);

extern "C" {

int nb_flash_bwd_args_size(void) { return int(sizeof(NbFlashBwdArgs)); }

int nb_flash_bwd(const NbFlashBwdArgs* a, cudaStream_t stream) {
  using namespace nb;
  if (a->hd % 8 || a->hd < 8 || a->hd > 128) return -1;
  // resident tiles are fetched in boxes of 128 rows, streamed tiles in boxes of 64 rows
  CUtensorMap tq, tk, tv, tdo, xq, xk, xv, xdo;
  if (nb_head_map(&tq, a->Q, a->rows, a->H, a->hd, a->ld_qkv)) return -10;
  if (nb_head_map(&tk, a->K, a->rows, a->H, a->hd, a->ld_qkv)) return -11;
  if (nb_head_map(&tv, a->V, a->rows, a->H, a->hd, a->ld_qkv)) return -12;
  if (nb_head_map(&tdo, a->dO, a->rows, a->H, a->hd, a->ld_do)) return -13;
  if (nb_head_map_rows(&xq, a->Q, a->rows, a->H, a->hd, a->ld_qkv, BX)) return -14;
  if (nb_head_map_rows(&xk, a->K, a->rows, a->H, a->hd, a->ld_qkv, BX)) return -15;
  if (nb_head_map_rows(&xv, a->V, a->rows, a->H, a->hd, a->ld_qkv, BX)) return -16;
  if (nb_head_map_rows(&xdo, a->dO, a->rows, a->H, a->hd, a->ld_do, BX)) return -17;
  {
    long warps = long(a->rows) * a->H;
    int threads = 256;
    long blocks = (warps * 32 + threads - 1) / threads;
    attn_delta_kernel<<<unsigned(blocks), threads, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(a->dO), reinterpret_cast<const __nv_bfloat16*>(a->O), a->ld_do, a->ld_o,
        a->delta, a->rows, a->H, a->hd);
  }
  FlashBwdParams p;
  p.nseg = a->nseg; p.H = a->H; p.hd = a->hd; p.rows = a->rows; p.seg_start = a->seg_start;
  p.scale = a->scale; p.scale_log2 = a->scale * 1.4426950408889634f;
  p.lse = a->lse; p.delta = a->delta; p.ldo = a->ld_dqkv; p.status = a->status;
  const int nkb = (a->hd + 63) / 64;
  // Streamed-tile ring: two stages next to the two 16 KB operand tiles of the dK/dV pass, three in the dQ pass, which
  // has no P^T tile (both sized so that two CTAs of head dims <= 64 share an SM); two stages for head dims above 64
  // (165 KB, one CTA per SM). At least two are needed: the score products of tile it + 1 are issued while tile it's
  // stage is still being read by its accumulate products.
  dim3 grid(a->max_tiles, a->H);
  size_t smem = 0;
#define NB_LAUNCH(MODE, HDN, R1, R2, X1, X2)                                                                        \
  do {                                                                                                               \
    static SmemAttr attr;                                                                                            \
    p.stages = nkb == 1 ? (MODE == 0 ? 2 : 3) : 2;                                                                   \
    smem = size_t(nkb) * (2 * 16384 + 2 * p.stages * 8192) + (MODE == 0 ? 32768 : 16384) + 1024;                     \
    if (int e = attr.ensure(flash_bwd_kernel<MODE, HDN>, smem)) return e;                                            \
    flash_bwd_kernel<MODE, HDN><<<grid, 320, smem, stream>>>(R1, R2, X1, X2, p);                                     \
  } while (0)
  p.out1 = reinterpret_cast<__nv_bfloat16*>(a->dK); p.out2 = reinterpret_cast<__nv_bfloat16*>(a->dV);
  if (a->hd <= 64) NB_LAUNCH(0, 64, tk, tv, xq, xdo); else NB_LAUNCH(0, 128, tk, tv, xq, xdo);
  p.out1 = reinterpret_cast<__nv_bfloat16*>(a->dQ); p.out2 = nullptr;
  if (a->hd <= 64) NB_LAUNCH(1, 64, tq, tdo, xk, xv); else NB_LAUNCH(1, 128, tq, tdo, xk, xv);
#undef NB_LAUNCH
  return int(cudaGetLastError());
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// Allocation-free variant (see flash_noalloc.h): the `delta` scratch lives in a fixed device array.
#include "flash_noalloc.h"
#include <stdio.h>

static __device__ __align__(256) float g_noalloc_delta[NB_FLASH_NOALLOC_MAX_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_noalloc_ptr[kMaxDevices] = {nullptr};      // device address of g_noalloc_delta, per device
thread_local char g_noalloc_msg[256] = "";
}  // namespace

extern "C" const char* nb_flash_bwd_noalloc_error(void) { return g_noalloc_msg; }

extern "C" int nb_flash_bwd_noalloc(const NbFlashBwdArgs* args, cudaStream_t stream) {
  g_noalloc_msg[0] = 0;
  const long need = long(args->rows) * args->H;
  if (need > NB_FLASH_NOALLOC_MAX_FLOATS) {
    snprintf(g_noalloc_msg, sizeof(g_noalloc_msg),
             "nb_flash_bwd_noalloc: rows * heads = %ld exceeds the built-in scratch of %d floats; "
             "use nb_flash_bwd with a caller-provided delta buffer", need, NB_FLASH_NOALLOC_MAX_FLOATS);
    return NB_FLASH_NOALLOC_TOO_LARGE;
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    snprintf(g_noalloc_msg, sizeof(g_noalloc_msg), "nb_flash_bwd_noalloc: cannot identify the current device (%s)",
             cudaGetErrorString(e));
    return NB_FLASH_NOALLOC_SETUP_FAILED;
  }
  if (!g_noalloc_ptr[dev]) {
    // Set-up, once per device, with that device current: the array's name is only a host-side handle;
    // kernels need its device address.
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_delta);
    if (e != cudaSuccess || !p) {
      snprintf(g_noalloc_msg, sizeof(g_noalloc_msg), "nb_flash_bwd_noalloc: cudaGetSymbolAddress failed (%s)",
               cudaGetErrorString(e));
      return NB_FLASH_NOALLOC_SETUP_FAILED;
    }
    g_noalloc_ptr[dev] = p;
  }
  NbFlashBwdArgs local = *args;
  local.delta = g_noalloc_ptr[dev];   // fully rewritten (rows * heads entries) before it is read
  int rc = nb_flash_bwd(&local, stream);
  if (rc != 0) snprintf(g_noalloc_msg, sizeof(g_noalloc_msg), "nb_flash_bwd_noalloc: nb_flash_bwd returned %d", rc);
  return rc;
}
