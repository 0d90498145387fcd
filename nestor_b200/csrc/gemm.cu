// Persistent grouped GEMM for sm_100a: TMA -> 128B-swizzled shared memory -> tcgen05.mma
// with fp32 accumulators in TMEM -> register epilogue.
//
// One kernel covers every matrix product of the model; it is configured at run time:
//   mode 0 ("row-grouped"): C[r, :] = A[r, :] . B[g(r)]   for rows r packed by group
//        (expert banks, per-column attention projections, plain GEMMs with one group).
//        A tile rows start at the group's first row, so a tile may run past the group's
//        end; those rows are computed and discarded by the masked epilogue.
//   mode 1 ("reduction-grouped", weight gradients): C[g] (+)= A[rows of g]^T . B[rows of g].
//        The last 64-row block of a group is zeroed in shared memory past the group's end
//        before the tensor core reads it.
// Operands are bf16, K-major (rows of K) or MN-major (rows of M/N); see sm100.cuh.
// A second (A2, B2) operand pair extends the reduction (dX = dG.Wg^T + dU.Wu^T in one pass).
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer (+TMEM owner),
// warps 2..5 = epilogue (warp w reads TMEM lanes 32*(w%4)..+31). Two accumulator buffers
// let the epilogue of tile i overlap the main loop of tile i+1.
//
// Replaces the reference's torch._grouped_mm call sites (nestor/backbones/grouped_mm.py:83,
// :417-450; nestor/backbones/nestor.py:6337, :6367) and their Triton pointwise companions.
#include "sm100.cuh"

namespace nb {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kMaxGroups = 256;

enum Epilogue : int {
  kStoreBf16 = 0,     // C bf16 [.., ldc]
  kStoreF32 = 1,      // C fp32
  kAccumF32 = 2,      // C fp32 += acc * alpha
  kSwiGLU = 3,        // tile columns [0,BN/2) = gate, [BN/2,BN) = up: write gate, up and silu(gate)*up (bf16)
  kSwiGLUBwd = 4,     // acc = dH: read gate/up, write dGate, dUp (bf16)
  kStoreBf16Stats = 5 // store bf16 (scaled) and per-(row, n-tile) max / sum-exp partials
};

struct GemmParams {
  int mode, groups, BN, epilogue;
  int M, N, K;              // mode 0: M = total rows. mode 1: M x N output per group, K = total rows
  int K2;                   // second reduction segment (0 = none)
  const int* offsets;       // [groups + 1] device row offsets, or nullptr for uniform groups
  int rows_per_group;       // uniform groups: rows per group
  int a_mn, b_mn;           // operand majors (1 = MN-major)
  int b_grouped;            // B indexed by group (3-D map) or shared
  void* C; long ldc; long c_group_stride;
  void* C2; void* C3;       // extra outputs (SwiGLU: gate/up; stats: partials)
  const void* E1; const void* E2;  // extra inputs (SwiGLU bwd: gate, up)
  long lde;
  float alpha;
  int n_valid;              // stats epilogue: columns >= n_valid are padding (stored as -inf)
  int splits;               // mode 1: each output tile is reduced by `splits` CTAs (atomic fp32 adds)
  int* status;
  int max_tiles;
  unsigned long long* trace;   // optional: per-CTA phase timestamps (ns), 64 slots per CTA (diagnostics)
  int prefetch_dist;           // producer pulls k-block (i + dist) into L2 while loading k-block i (0 = off)
  int prefetch_ops;            // operands to prefetch: 1 = A, 2 = B, 3 = both
};

__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
#define NB_TRACE(slot) do { if (p.trace && (slot) < 64) p.trace[blockIdx.x * 64 + (slot)] = gtime(); } while (0)

struct Tile { int g, m0, n0, row_end, kb, kb2, kb0, valid; };

struct Sched {
  // tile t -> (group, m tile, n tile); identical arithmetic in every warp role.
  int n_tiles, total;
  const int* tstart;  // smem prefix of m-tiles per group (mode 0)
  const int* off;     // smem offsets
};

__device__ __forceinline__ Tile decode_tile(const GemmParams& p, const int* s_off, const int* s_tstart, int t,
                                            int n_tiles) {
  Tile r;
  r.valid = 1;
  r.kb0 = 0;
  if (p.mode == 0) {
    int mt = t / n_tiles, nt = t - mt * n_tiles;
    int lo = 0, hi = p.groups;          // find g with tstart[g] <= mt < tstart[g+1]
    while (hi - lo > 1) {
      int mid = (lo + hi) >> 1;
      if (s_tstart[mid] <= mt) lo = mid; else hi = mid;
    }
    r.g = lo;
    r.m0 = s_off[lo] + (mt - s_tstart[lo]) * BM;
    r.row_end = s_off[lo + 1];
    r.n0 = nt * p.BN;
    r.kb = (p.K + BK - 1) / BK;
    r.kb2 = (p.K2 + BK - 1) / BK;
  } else {
    int m_tiles = (p.M + BM - 1) / BM;
    int per_g = m_tiles * n_tiles * p.splits;
    r.g = t / per_g;
    int rem = t - r.g * per_g;
    int sp = rem % p.splits; rem /= p.splits;
    int mt = rem / n_tiles, nt = rem - mt * n_tiles;
    r.m0 = mt * BM;
    r.n0 = nt * p.BN;
    r.row_end = s_off[r.g + 1];
    int nkb = (s_off[r.g + 1] - s_off[r.g] + BK - 1) / BK;
    int per = (nkb + p.splits - 1) / p.splits;
    r.kb0 = sp * per;
    r.kb = max(0, min(nkb, r.kb0 + per) - r.kb0);
    r.kb2 = 0;
  }
  return r;
}

__global__ void __launch_bounds__(192, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2,
            const GemmParams p, int stages) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ uint64_t full_bar[8], empty_bar[8], tfull_bar[2], tempty_bar[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int s_abort;
  __shared__ int s_off[kMaxGroups + 1];
  __shared__ int s_tstart[kMaxGroups + 1];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t a_bytes = BM * BK * 2;               // 16 KB
  const uint32_t b_bytes = uint32_t(p.BN) * BK * 2;
  const uint32_t stage_bytes = a_bytes + b_bytes;
  const uint32_t tmem_cols = (2 * p.BN <= 32) ? 32 : (2 * p.BN <= 64) ? 64 : (2 * p.BN <= 128) ? 128
                           : (2 * p.BN <= 256) ? 256 : 512;
  const int n_tiles = (p.N + p.BN - 1) / p.BN;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int g = 0; g <= p.groups; ++g)
      s_off[g] = p.offsets ? p.offsets[g] : g * p.rows_per_group;
    int acc = 0;
    for (int g = 0; g < p.groups; ++g) {
      s_tstart[g] = acc;
      acc += (s_off[g + 1] - s_off[g] + BM - 1) / BM;
    }
    s_tstart[p.groups] = acc;
    for (int s = 0; s < stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tfull_bar[b], 1); mbar_init(&tempty_bar[b], 4); }
    fence_barrier_init();
    prefetch_tmap(&tmA); prefetch_tmap(&tmB);
    if (p.K2) { prefetch_tmap(&tmA2); prefetch_tmap(&tmB2); }
  }
  if (warp == 1) { tmem_alloc(&tmem_base_slot, tmem_cols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  int total_tiles;
  if (p.mode == 0) total_tiles = s_tstart[p.groups] * n_tiles;
  else total_tiles = p.groups * ((p.M + BM - 1) / BM) * n_tiles * p.splits;

  volatile int* abort_flag = &s_abort;

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer
    if (elect_one()) {
      // One routine computes the coordinates of a k-block's boxes; `pf` = 0 issues the loads into the stage,
      // otherwise it only pulls the boxes of the operands in the mask (1 = A, 2 = B) into L2.
      auto ld2 = [&](void* dst, const CUtensorMap* m, uint64_t* bar, int x, int y, int pf) {
        if (pf) tma_prefetch_2d(m, x, y); else tma_load_2d(dst, m, bar, x, y);
      };
      auto ld3 = [&](void* dst, const CUtensorMap* m, uint64_t* bar, int x, int y, int z, int pf) {
        if (pf) tma_prefetch_3d(m, x, y, z); else tma_load_3d(dst, m, bar, x, y, z);
      };
      auto issue = [&](const Tile& tl, int kb, uint8_t* sa, uint8_t* sb, uint64_t* bar, int pf) {
        const bool doA = !pf || (pf & 1), doB = !pf || (pf & 2);
        bool second = kb >= tl.kb;
        const CUtensorMap* mA = second ? &tmA2 : &tmA;
        const CUtensorMap* mB = second ? &tmB2 : &tmB;
        int kk = (second ? kb - tl.kb : kb) * BK;
        if (p.mode == 0) {
          if (doA) {
            if (!p.a_mn) ld2(sa, mA, bar, kk, tl.m0, pf);
            else { ld2(sa, mA, bar, tl.m0, kk, pf); ld2(sa + 8192, mA, bar, tl.m0 + 64, kk, pf); }
          }
          if (doB) {
            int bg = p.b_grouped ? tl.g : 0;
            if (!p.b_mn) ld3(sb, mB, bar, kk, tl.n0, bg, pf);
            else if (p.epilogue == kSwiGLU) {
              // B tile = [gate columns | up columns], each half from its own tensor (tmB = gate, tmB2 = up)
              int half = p.BN / 2, c0 = tl.n0 / 2;
              for (int a = 0; a < half / 64; ++a) ld3(sb + a * 8192, &tmB, bar, c0 + a * 64, kk, bg, pf);
              for (int a = 0; a < half / 64; ++a) ld3(sb + (half / 64 + a) * 8192, &tmB2, bar, c0 + a * 64, kk, bg, pf);
            } else {
              for (int a = 0; a < p.BN / 64; ++a) ld3(sb + a * 8192, mB, bar, tl.n0 + a * 64, kk, bg, pf);
            }
          }
        } else {
          int row = s_off[tl.g] + (tl.kb0 + kb) * BK;     // reduction over the group's rows; operands are MN-major
          if (doA) { ld2(sa, mA, bar, tl.m0, row, pf); ld2(sa + 8192, mA, bar, tl.m0 + 64, row, pf); }
          if (doB) for (int a = 0; a < p.BN / 64; ++a) ld2(sb + a * 8192, mB, bar, tl.n0 + a * 64, row, pf);
        }
      };
      const int D = p.prefetch_dist, pf_mask = p.prefetch_ops;
      uint32_t it = 0;
      NB_TRACE(0);
      for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x) {
        Tile tl = decode_tile(p, s_off, s_tstart, t, n_tiles);
        int nkb = tl.kb + tl.kb2;
        Tile nx = tl; int nx_nkb = 0;
        if (D > 0 && t + int(gridDim.x) < total_tiles) {
          nx = decode_tile(p, s_off, s_tstart, t + gridDim.x, n_tiles);
          nx_nkb = nx.kb + nx.kb2;
        }
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          int s = it % stages; uint32_t ph = (it / stages) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.status, kTimeoutEmpty)) break;
          if (it < 12) NB_TRACE(1 + it);
          uint8_t* sa = smem + s * stage_bytes;
          mbar_expect_tx(&full_bar[s], stage_bytes);
          issue(tl, kb, sa, sa + a_bytes, &full_bar[s], 0);
          if (D > 0) {
            int pk = kb + D;
            if (pk < nkb) issue(tl, pk, nullptr, nullptr, nullptr, pf_mask);
            else if (pk - nkb < nx_nkb) issue(nx, pk - nkb, nullptr, nullptr, nullptr, pf_mask);
          }
        }
      }
    }
  } else if (warp == 1) {
    // --------------------------------------------------------------- MMA issuer
    const uint32_t idesc = make_idesc(BM, p.BN, p.a_mn, p.b_mn);
    uint32_t it = 0, tile_i = 0;
    for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x) {
      Tile tl = decode_tile(p, s_off, s_tstart, t, n_tiles);
      int nkb = tl.kb + tl.kb2;
      if (nkb == 0) continue;            // empty reduction: epilogue writes zeros without an accumulator
      uint32_t buf = tile_i & 1, bph = (tile_i >> 1) & 1;
      ++tile_i;
      bool ok = true;
      if (lane == 0) ok = mbar_wait(&tempty_bar[buf], bph ^ 1, abort_flag, p.status, kTimeoutTmemEmpty);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      tc_fence_after();
      if (lane == 0 && tile_i <= 6) NB_TRACE(16 + 4 * (tile_i - 1));
      uint32_t d_addr = tmem_base + buf * p.BN;
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        int s = it % stages; uint32_t ph = (it / stages) & 1;
        if (lane == 0) ok = mbar_wait(&full_bar[s], ph, abort_flag, p.status, kTimeoutFull);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        if (lane == 0 && kb == 0 && tile_i <= 6) NB_TRACE(16 + 4 * (tile_i - 1) + 1);
        uint8_t* sa = smem + s * stage_bytes;
        uint8_t* sb = sa + a_bytes;
        if (p.mode == 1) {
          // zero k-rows past the end of the group (they belong to the next group)
          int row0 = s_off[tl.g] + (tl.kb0 + kb) * BK;
          int valid = tl.row_end - row0;
          if (valid < BK) {
            int natoms = 2 + p.BN / 64;
            for (int a = 0; a < natoms; ++a) {
              uint8_t* base = (a < 2) ? sa + a * 8192 : sb + (a - 2) * 8192;
              for (int r = valid; r < BK; ++r)
                reinterpret_cast<uint32_t*>(base + r * 128)[lane] = 0u;
            }
            fence_async_smem();
            __syncwarp();
          }
        }
        tc_fence_after();
        if (lane == 0) {
          uint32_t a0 = smem_u32(sa), b0 = smem_u32(sb);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            uint64_t ad = p.a_mn ? sdesc_mnmajor(a0 + k * 2048, 8192) : sdesc_kmajor(a0 + k * 32);
            uint64_t bd = p.b_mn ? sdesc_mnmajor(b0 + k * 2048, 8192) : sdesc_kmajor(b0 + k * 32);
            umma_bf16(d_addr, ad, bd, idesc, (kb | k) != 0);
          }
          umma_commit(&empty_bar[s]);              // stage is free once these MMAs retire
          if (kb == nkb - 1) { umma_commit(&tfull_bar[buf]); if (tile_i <= 6) NB_TRACE(16 + 4 * (tile_i - 1) + 2); }
        }
        __syncwarp();
      }
      if (!ok) break;
    }
  } else {
    // ----------------------------------------------------------------- epilogue
    const int q = warp & 3;                      // TMEM lane quarter this warp may read
    uint32_t tile_i = 0;
    for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x) {
      Tile tl = decode_tile(p, s_off, s_tstart, t, n_tiles);
      int nkb = tl.kb + tl.kb2;
      const int row = tl.m0 + q * 32 + lane;
      bool row_ok;
      long c_base;
      if (p.mode == 0) { row_ok = row < tl.row_end; c_base = long(row) * p.ldc; }
      else { row_ok = row < p.M; c_base = long(tl.g) * p.c_group_stride + long(row) * p.ldc; }
      uint32_t buf = 0;
      if (nkb > 0) {
        buf = tile_i & 1; uint32_t bph = (tile_i >> 1) & 1;
        ++tile_i;
        if (!mbar_wait(&tfull_bar[buf], bph, abort_flag, p.status, kTimeoutTmemFull)) break;
        tc_fence_after();
        if (q == 0 && lane == 0 && tile_i <= 6) NB_TRACE(40 + 3 * (tile_i - 1));
      }
      const uint32_t taddr = tmem_base + buf * p.BN + (uint32_t(q * 32) << 16);
      const int ncols = min(p.BN, p.N - tl.n0);
      if (p.epilogue == kSwiGLU) {
        const int half = p.BN / 2, h0 = tl.n0 / 2;
        const int hcols = min(half, p.N / 2 - h0);
        for (int c = 0; c < hcols; c += 16) {
          float g[16], u[16];
          tmem_ld16(taddr + c, g); tmem_ld16(taddr + half + c, u);
          tmem_ld_wait();
          if (row_ok) {
            uint32_t og[8], ou[8], oh[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              // round gate/up to bf16 first: the product must match silu evaluated on the stored values
              float g0 = __bfloat162float(__float2bfloat16(g[2 * j])), g1 = __bfloat162float(__float2bfloat16(g[2 * j + 1]));
              float u0 = __bfloat162float(__float2bfloat16(u[2 * j])), u1 = __bfloat162float(__float2bfloat16(u[2 * j + 1]));
              float s0 = __bfloat162float(__float2bfloat16(g0 / (1.f + __expf(-g0))));
              float s1 = __bfloat162float(__float2bfloat16(g1 / (1.f + __expf(-g1))));
              og[j] = pack_bf16(g0, g1); ou[j] = pack_bf16(u0, u1); oh[j] = pack_bf16(s0 * u0, s1 * u1);
            }
            long o = long(row) * p.ldc + h0 + c;
            int rem = hcols - c;
            __nv_bfloat16* H = reinterpret_cast<__nv_bfloat16*>(p.C) + o;
            __nv_bfloat16* Gp = reinterpret_cast<__nv_bfloat16*>(p.C2) + o;
            __nv_bfloat16* Up = reinterpret_cast<__nv_bfloat16*>(p.C3) + o;
            if (rem >= 16) {
              reinterpret_cast<uint4*>(H)[0] = make_uint4(oh[0], oh[1], oh[2], oh[3]);
              reinterpret_cast<uint4*>(H)[1] = make_uint4(oh[4], oh[5], oh[6], oh[7]);
              reinterpret_cast<uint4*>(Gp)[0] = make_uint4(og[0], og[1], og[2], og[3]);
              reinterpret_cast<uint4*>(Gp)[1] = make_uint4(og[4], og[5], og[6], og[7]);
              reinterpret_cast<uint4*>(Up)[0] = make_uint4(ou[0], ou[1], ou[2], ou[3]);
              reinterpret_cast<uint4*>(Up)[1] = make_uint4(ou[4], ou[5], ou[6], ou[7]);
            } else {  // rem == 8 (all widths are multiples of 8)
              reinterpret_cast<uint4*>(H)[0] = make_uint4(oh[0], oh[1], oh[2], oh[3]);
              reinterpret_cast<uint4*>(Gp)[0] = make_uint4(og[0], og[1], og[2], og[3]);
              reinterpret_cast<uint4*>(Up)[0] = make_uint4(ou[0], ou[1], ou[2], ou[3]);
            }
          }
        }
      } else {
        float run_max = -INFINITY, run_sum = 0.f;
        for (int c0 = 0; c0 < ncols; c0 += 32) {
          // 32 accumulator columns per TMEM round trip (16 when that is all that is left of the tile)
          float v32[32];
          if (nkb > 0) {
            if (ncols - c0 > 16) tmem_ld32(taddr + c0, v32); else tmem_ld16(taddr + c0, v32);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v32[j] = 0.f;
          }
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
          const int c = c0 + 16 * hh;
          float* v = v32 + 16 * hh;
          const int rem = ncols - c;           // <= 0 (past the tile), 8 or >= 16
          if (!row_ok || rem <= 0) continue;
          const long o = c_base + tl.n0 + c;
          if (p.epilogue == kStoreBf16 || p.epilogue == kStoreBf16Stats) {
            if (p.epilogue == kStoreBf16Stats) {
#pragma unroll
              for (int j = 0; j < 16; ++j) if (tl.n0 + c + j >= p.n_valid) v[j] = -INFINITY;
            }
            uint32_t w[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) w[j] = pack_bf16(v[2 * j] * p.alpha, v[2 * j + 1] * p.alpha);
            __nv_bfloat16* Cp = reinterpret_cast<__nv_bfloat16*>(p.C) + o;
            reinterpret_cast<uint4*>(Cp)[0] = make_uint4(w[0], w[1], w[2], w[3]);
            if (rem >= 16) reinterpret_cast<uint4*>(Cp)[1] = make_uint4(w[4], w[5], w[6], w[7]);
            if (p.epilogue == kStoreBf16Stats) {
              const int lim = rem >= 16 ? 16 : 8;
              float m = run_max;
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                float x = __bfloat162float(__float2bfloat16(v[j] * p.alpha));
                v[j] = j < lim ? x : -INFINITY; m = fmaxf(m, v[j]);
              }
              float ssum = run_sum * __expf(run_max - m);
#pragma unroll
              for (int j = 0; j < 16; ++j) ssum += __expf(v[j] - m);
              run_max = m; run_sum = ssum;
            }
          } else if (p.epilogue == kStoreF32) {
            float* Cp = reinterpret_cast<float*>(p.C) + o;
            const int lim = rem >= 16 ? 16 : 8;
#pragma unroll
            for (int j = 0; j < 16; j += 4)
              if (j < lim) reinterpret_cast<float4*>(Cp + j)[0] = make_float4(v[j] * p.alpha, v[j + 1] * p.alpha, v[j + 2] * p.alpha, v[j + 3] * p.alpha);
          } else if (p.epilogue == kAccumF32) {
            if (nkb > 0) {
              float* Cp = reinterpret_cast<float*>(p.C) + o;
              const int lim = rem >= 16 ? 16 : 8;
#pragma unroll
              for (int j = 0; j < 16; j += 4) {
                if (j >= lim) break;
                float4 add = make_float4(v[j] * p.alpha, v[j + 1] * p.alpha, v[j + 2] * p.alpha, v[j + 3] * p.alpha);
                if (p.splits > 1) {
                  atomicAdd(reinterpret_cast<float4*>(Cp + j), add);
                } else {
                  float4 old = reinterpret_cast<float4*>(Cp + j)[0];
                  reinterpret_cast<float4*>(Cp + j)[0] = make_float4(old.x + add.x, old.y + add.y, old.z + add.z, old.w + add.w);
                }
              }
            }
          } else if (p.epilogue == kSwiGLUBwd) {
            // v = dH. dGate = dH * up * s * (1 + g * (1 - s)); dUp = dH * silu(g)   (s = sigmoid(g))
            const long oe = long(row) * p.lde + tl.n0 + c;
            const __nv_bfloat16* Gp = reinterpret_cast<const __nv_bfloat16*>(p.E1) + oe;
            const __nv_bfloat16* Up = reinterpret_cast<const __nv_bfloat16*>(p.E2) + oe;
            __nv_bfloat16* dG = reinterpret_cast<__nv_bfloat16*>(p.C) + o;
            __nv_bfloat16* dU = reinterpret_cast<__nv_bfloat16*>(p.C2) + o;
            const int lim = rem >= 16 ? 16 : 8;
#pragma unroll
            for (int j = 0; j < 16; j += 8) {
              if (j >= lim) break;
              uint4 gq = reinterpret_cast<const uint4*>(Gp + j)[0], uq = reinterpret_cast<const uint4*>(Up + j)[0];
              const __nv_bfloat16* gb = reinterpret_cast<const __nv_bfloat16*>(&gq);
              const __nv_bfloat16* ub = reinterpret_cast<const __nv_bfloat16*>(&uq);
              uint32_t wg[4], wu[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                float r[2][2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                  float gg = __bfloat162float(gb[2 * e + h]), uu = __bfloat162float(ub[2 * e + h]);
                  float dh = __bfloat162float(__float2bfloat16(v[j + 2 * e + h]));
                  float sg = 1.f / (1.f + __expf(-gg));
                  r[h][0] = dh * uu * sg * (1.f + gg * (1.f - sg));
                  r[h][1] = dh * gg * sg;
                }
                wg[e] = pack_bf16(r[0][0], r[1][0]); wu[e] = pack_bf16(r[0][1], r[1][1]);
              }
              reinterpret_cast<uint4*>(dG + j)[0] = make_uint4(wg[0], wg[1], wg[2], wg[3]);
              reinterpret_cast<uint4*>(dU + j)[0] = make_uint4(wu[0], wu[1], wu[2], wu[3]);
            }
          }
        }
          }
        if (p.epilogue == kStoreBf16Stats && row_ok) {
          float2* part = reinterpret_cast<float2*>(p.C2) + long(row) * n_tiles + (tl.n0 / p.BN);
          *part = make_float2(run_max, run_sum);
        }
      }
      if (nkb > 0) {
        tc_fence_before();
        __syncwarp();
        if (q == 0 && lane == 0 && tile_i <= 6) NB_TRACE(40 + 3 * (tile_i - 1) + 1);
        if (lane == 0) mbar_arrive(&tempty_bar[buf]);
      }
    }
  }

  // ----------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, tmem_cols); }
}

}  // namespace nb

// ============================================================================ host side
#include <stdio.h>
#include <string.h>

namespace {

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                             const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                             CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess || !ptr) return nullptr;
    fn = reinterpret_cast<EncodeFn>(ptr);
  }
  return fn;
}

// bf16 tensor of rank 2 or 3 (dims innermost-first), strides in elements for dims 1.. (innermost is contiguous).
int make_map(CUtensorMap* m, const void* base, int rank, const long* dims, const long* strides_elems,
             const int* box) {
  EncodeFn fn = encode_fn();
  if (!fn) return 1;
  cuuint64_t gd[3]; cuuint64_t gs[2]; cuuint32_t bx[3]; cuuint32_t es[3] = {1, 1, 1};
  for (int i = 0; i < rank; ++i) { gd[i] = cuuint64_t(dims[i]); bx[i] = cuuint32_t(box[i]); }
  for (int i = 0; i + 1 < rank; ++i) gs[i] = cuuint64_t(strides_elems[i]) * 2;
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, cuuint32_t(rank), const_cast<void*>(base), gd, gs, bx, es,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 2;
}

int g_num_sms = 0;

}  // namespace

extern "C" {

// Operand descriptor passed from Python: base pointer, rows, cols, row stride, group count and stride (elements).
struct NbOperand {
  const void* ptr;
  long rows, cols, ld, groups, group_stride;
};

struct NbGemmArgs {
  int mode, groups, BN, epilogue;
  int M, N, K, K2;
  const int* offsets; int rows_per_group;
  int a_mn, b_mn, b_grouped;
  NbOperand A, B, A2, B2;
  void* C; long ldc; long c_group_stride;
  void* C2; void* C3; const void* E1; const void* E2; long lde;
  float alpha;
  int n_valid;
  int splits;
  int* status;
  int max_m_tiles;          // upper bound on m tiles over all groups (mode 0)
  int sms;                  // 0 = all
  unsigned long long* trace;
  int prefetch_dist;        // L2 look-ahead of the producer in k-blocks (0 = off)
  int prefetch_ops;         // 1 = A, 2 = B, 3 = both
  int max_stages;           // 0 = as many as fit
};

// Returns 0 on success, a negative code for bad arguments / map failures, or a CUDA error code.
int nb_gemm(const NbGemmArgs* a, cudaStream_t stream) {
  using namespace nb;
  if (a->groups < 1 || a->groups > kMaxGroups) return -1;
  if (a->BN < 16 || a->BN > 256 || a->BN % 16) return -2;
  if ((a->a_mn || a->b_mn) && false) return -3;
  if (a->b_mn && a->BN % 64) return -4;
  if (a->mode == 1 && !(a->a_mn && a->b_mn)) return -5;
  if (a->epilogue == kSwiGLU && (a->BN % 128 || !a->b_mn)) return -6;
  if (!g_num_sms) {
    int dev; cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  CUtensorMap tmA, tmB, tmA2, tmB2;
  memset(&tmA2, 0, sizeof(tmA2)); memset(&tmB2, 0, sizeof(tmB2));
  auto map_a = [&](CUtensorMap* m, const NbOperand& o) -> int {
    long dims[2] = {o.cols, o.rows}; long st[1] = {o.ld};
    int box_k[2] = {BK, BM};            // K-major: 64 k x 128 rows
    int box_mn[2] = {64, BK};           // MN-major: 64 m x 64 k-rows
    return make_map(m, o.ptr, 2, dims, st, a->a_mn ? box_mn : box_k);
  };
  auto map_b = [&](CUtensorMap* m, const NbOperand& o) -> int {
    if (a->mode == 1) {
      long dims[2] = {o.cols, o.rows}; long st[1] = {o.ld};
      int box[2] = {64, BK};
      return make_map(m, o.ptr, 2, dims, st, box);
    }
    long dims[3] = {o.cols, o.rows, o.groups > 0 ? o.groups : 1};
    long st[2] = {o.ld, o.group_stride > 0 ? o.group_stride : o.rows * o.ld};
    int box_k[3] = {BK, a->BN, 1};      // K-major B [N, K]: 64 k x BN rows
    int box_mn[3] = {64, BK, 1};        // MN-major B [K, N]: 64 n x 64 k-rows
    return make_map(m, o.ptr, 3, dims, st, a->b_mn ? box_mn : box_k);
  };
  if (map_a(&tmA, a->A)) return -10;
  if (map_b(&tmB, a->B)) return -11;
  if (a->K2 > 0) { if (map_a(&tmA2, a->A2)) return -12; }
  if (a->K2 > 0 || a->epilogue == kSwiGLU) { if (map_b(&tmB2, a->B2)) return -13; }

  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.mode = a->mode; p.groups = a->groups; p.BN = a->BN; p.epilogue = a->epilogue;
  p.M = a->M; p.N = a->N; p.K = a->K; p.K2 = a->K2; p.offsets = a->offsets; p.rows_per_group = a->rows_per_group;
  p.a_mn = a->a_mn; p.b_mn = a->b_mn; p.b_grouped = a->b_grouped;
  p.C = a->C; p.ldc = a->ldc; p.c_group_stride = a->c_group_stride; p.C2 = a->C2; p.C3 = a->C3;
  p.E1 = a->E1; p.E2 = a->E2; p.lde = a->lde; p.alpha = a->alpha; p.n_valid = a->n_valid > 0 ? a->n_valid : a->N; p.status = a->status;
  p.trace = a->trace;
  p.prefetch_dist = a->prefetch_dist > 0 ? a->prefetch_dist : 0;
  p.prefetch_ops = a->prefetch_ops & 3;
  p.splits = (a->mode == 1 && a->epilogue == kAccumF32 && a->splits > 1) ? a->splits : 1;

  const int n_tiles = (a->N + a->BN - 1) / a->BN;
  long tiles = a->mode == 0 ? long(a->max_m_tiles) * n_tiles
                            : long(a->groups) * ((a->M + BM - 1) / BM) * n_tiles * p.splits;
  if (tiles <= 0) return 0;
  const uint32_t stage_bytes = BM * BK * 2 + a->BN * BK * 2;
  int stages = int((220 * 1024) / stage_bytes);   // 227 KB per CTA minus barriers, offsets and alignment slack
  if (stages > 8) stages = 8;
  if (a->max_stages > 0 && stages > a->max_stages) stages = a->max_stages;
  if (stages < 2) return -7;
  size_t smem = size_t(stages) * stage_bytes + 1024;
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return int(e);
    configured = smem;
  }
  int sms = a->sms > 0 ? a->sms : g_num_sms;
  int grid = int(tiles < sms ? tiles : sms);
  gemm_kernel<<<grid, 192, smem, stream>>>(tmA, tmB, tmA2, tmB2, p, stages);
  return int(cudaGetLastError());
}

}  // extern "C"
