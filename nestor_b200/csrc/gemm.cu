// Persistent grouped GEMM for sm_100a: TMA -> 128B-swizzled shared memory -> tcgen05.mma
// with fp32 accumulators in TMEM -> epilogue through registers and per-warp shared-memory slabs (tiled TMA stores /
// reduce-adds where a warp's 32 rows are whole, masked vector stores at the ragged end of a group).
//
// One kernel covers every matrix product of the model; it is configured at run time:
//   mode 0 ("row-grouped"): C[r, :] = A[r, :] . B[g(r)]   for rows r packed by group
//        (expert banks, per-column attention projections, plain GEMMs with one group).
//        A tile rows start at the group's first row, so a tile may run past the group's
//        end; those rows are computed and discarded by the masked epilogue.
//   mode 1 ("reduction-grouped", weight gradients): C[g] (+)= A[rows of g]^T . B[rows of g].
//        The last 64-row block of a group is zeroed in shared memory past the group's end
//        before the tensor core reads it (in both CTAs' stages when the product runs on a CTA pair).
// Operands are bf16, K-major (rows of K) or MN-major (rows of M/N); see sm100.cuh.
// A second (A2, B2) operand pair extends the reduction (dX = dG.Wg^T + dU.Wu^T in one pass).
//
// Warp roles (352 threads; a gathering launch adds warp 11, see GatherParams): warp 0 = TMA producer of A tiles, warp 10 = TMA producer of B tiles, warp 1 = MMA
// issuer (+TMEM owner), warps 2..9 = epilogue (warp w reads TMEM lanes 32*(w%4)..+31; the two warps of a lane
// quarter take alternating 32-column chunks). Two accumulator buffers let the epilogue of tile i overlap the main
// loop of tile i+1. With PAIR = 1 the kernel runs as clusters of two CTAs on 256-row tiles (cta_group::2): each CTA
// stages its 128 rows of A and half of B, rank 0 issues the MMAs for both and signals both CTAs' barriers.
//
// What bounds it (measured with the trace / debug switches below): shared memory is filled at about 85 bytes per
// clock per SM whatever the number of producer warps, so a 128 x 256 x 64 k-block (48 KB) takes ~560 cycles to
// load against 512 cycles of tensor-core time; pairs cut the bytes per CTA to 32 KB. Short-K products (K of a few
// hundred, outputs as large as the inputs) are bound by DRAM once their operands are cold: with everything resident
// in L2 the expert down projection takes 27 us on the chip, 60 us after an L2 flush.
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
  kStoreBf16Stats = 5,// store bf16 (scaled) and per-(row, n-tile) max / sum-exp partials
  kAxpbyBf16 = 6      // C = alpha * acc + beta * E1 (bf16 in, bf16 out): the Newton-Schulz polynomial steps
};

// All-gather fused into the product (mode 0, grouped B). The groups of B (one or two tensors of the same shape:
// B and, for SwiGLU / two-segment products, B2) are sharded over ranks: rank r holds the current values of groups
// [r * groups_per_rank, (r + 1) * groups_per_rank) in its copy of the weight arena, which every rank maps
// (`src[r]`). A twelfth warp of every CTA of the launch pulls its share of the chunks of every group from the
// group's owner into the local staging tensor that the B tensor maps describe, in group order, with bulk copies
// through a small shared-memory ring, and counts finished chunks in `flags[group]`. (Measured on two GPUs: a CTA that only
// copies moves 11-14 GB/s whatever its ring depth or chunk size, so the copy is spread over all SMs instead of being
// given to a few dedicated CTAs.) The B producers wait (bounded) for a group's count before their first load of
// it, so the product of the early groups overlaps the transfer of the later ones. Nothing waits on another GPU:
// a shard is constant while the products that read it run. The last CTA to leave zeroes the counters for the next
// launch (launches that share `flags` must be stream-ordered).
struct GatherParams {
  const uint8_t* src[8];       // per rank: base address of its weight arena as mapped here
  uint8_t* dst;                // base address of the local staging tensors
  long seg_src_off[2];         // byte offset of group 0 of B / B2 inside an arena
  long seg_dst_off[2];         // byte offset of group 0 of the staged B / B2 from `dst`
  long group_bytes;            // bytes of one group (contiguous, multiple of 16)
  long group_stride_src;       // byte distance between groups in the arena (the staging is dense)
  int nseg;                    // 1 or 2 tensors
  int groups_per_rank;
  int on;                      // 0 = no gather
  int chunk_bytes;             // bulk-copy granularity (multiple of 16)
  int nbuf;                    // shared-memory ring depth per copying lane (chunks), >= 2
  int lanes;                   // lanes of the copy warp that copy (1..4); lanes * nbuf <= 8
  int* flags;                  // [groups] finished chunks per group, then [groups]: CTAs that left
  unsigned wait_polls;         // polls (>= 100 ns each) a B producer spends on a group's counter before it gives up
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
  float alpha, beta;
  int n_valid;              // stats epilogue: columns >= n_valid are padding (stored as -inf)
  int splits;               // mode 1: each output tile is reduced by `splits` CTAs (atomic fp32 adds)
  int* status;
  int max_tiles;
  unsigned long long* trace;   // optional: per-CTA phase timestamps (ns), 64 slots per CTA (diagnostics)
  int prefetch_dist;           // producer pulls k-block (i + dist) into L2 while loading k-block i (0 = off)
  int prefetch_ops;            // operands to prefetch: 1 = A, 2 = B, 3 = both
  int pair;                    // mode 0: CTA pairs (cluster of 2) run 256-row tiles with cta_group::2 MMAs
  int a_atoms, b_atoms;        // MN-major operand read through an "atom" map: one TMA instruction per k-block
  int c_tiled;                 // the output has a tensor map (tmC): whole 32-row chunks leave as tiled stores
  int debug;                   // timing experiments only (results are garbage): 1 = issue no MMAs, 2 = issue no loads, 4 = store nothing
  GatherParams gather;         // fused all-gather of a rank-sharded B operand (gather.on == 0: off)
};

// Timing diagnostics (per-CTA phase timestamps, "issue no MMAs / loads / stores" experiments) are compiled in only
// with -DNB_GEMM_DIAG; the library build leaves them out, so the production kernels carry none of that code.
#ifdef NB_GEMM_DIAG
constexpr bool kDiag = true;
#else
constexpr bool kDiag = false;
#endif

__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
#define NB_TRACE(slot) do { if (kDiag && p.trace && (slot) < 64) p.trace[blockIdx.x * 64 + (slot)] = gtime(); } while (0)

struct Tile { int g, m0, n0, row_end, kb, kb2, kb0, valid; };

struct Sched {
  // tile t -> (group, m tile, n tile); identical arithmetic in every warp role.
  int n_tiles, total;
  const int* tstart;  // smem prefix of m-tiles per group (mode 0)
  const int* off;     // smem offsets
};

// `g_hint` carries the group of the caller's previous tile: a CTA visits tiles in increasing order, so the
// group is found by stepping forward instead of searching.
__device__ __forceinline__ Tile decode_tile(const GemmParams& p, const int* s_off, const int* s_tstart, int t,
                                            int n_tiles, int rank, int& g_hint) {
  Tile r;
  r.valid = 1;
  r.kb0 = 0;
  if (p.mode == 0) {
    int mt = t / n_tiles, nt = t - mt * n_tiles;
    int lo = g_hint;                    // find g with tstart[g] <= mt < tstart[g+1]
    while (lo + 1 < p.groups && s_tstart[lo + 1] <= mt) ++lo;
    g_hint = lo;
    r.g = lo;
    r.m0 = s_off[lo] + (mt - s_tstart[lo]) * (p.pair ? 2 * BM : BM) + rank * BM;   // rank 1 owns the lower half
    r.row_end = s_off[lo + 1];
    r.n0 = nt * p.BN;
    r.kb = (p.K + BK - 1) / BK;
    r.kb2 = (p.K2 + BK - 1) / BK;
  } else {
    const int bm = p.pair ? 2 * BM : BM;             // a pair's tile is 256 output rows; rank 1 owns the lower half
    int m_tiles = (p.M + bm - 1) / bm;
    int per_g = m_tiles * n_tiles * p.splits;
    r.g = t / per_g;
    int rem = t - r.g * per_g;
    int sp = rem % p.splits; rem /= p.splits;
    int mt = rem / n_tiles, nt = rem - mt * n_tiles;
    r.m0 = mt * bm + rank * BM;
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

// Epilogue staging: a warp holds its accumulator chunk one row per lane, but a store instruction in that shape
// touches 32 different 128-byte lines (16 B each) and the load/store unit serialises them. Each warp therefore
// transposes 32 rows x 32 bf16 columns through a private shared-memory slab (row pitch 80 B keeps both the
// row-per-lane writes and the read-back free of bank conflicts) and stores 8 rows x 64 B per instruction.
constexpr int kSlabPitch = 80;
constexpr int kSlabBytes = 32 * kSlabPitch;      // per epilogue warp
constexpr int kSlabBytesF32 = 32 * 128;          // per epilogue warp, fp32 outputs of a reduction-grouped product

// w[16] = this lane's row, 32 bf16 columns (packed pairs). Rows >= rows_ok and 8-column groups >= cols_ok (a
// multiple of 8) are not stored. `dst` points at (row 0 of the slab's 32 rows, first column of the chunk).
__device__ __forceinline__ void store_chunk_bf16(uint8_t* slab, int lane, const uint32_t* w, __nv_bfloat16* dst, long ld,
                                                 int rows_ok, int cols_ok) {
  uint4* mine = reinterpret_cast<uint4*>(slab + lane * kSlabPitch);
  mine[0] = make_uint4(w[0], w[1], w[2], w[3]);
  mine[1] = make_uint4(w[4], w[5], w[6], w[7]);
  mine[2] = make_uint4(w[8], w[9], w[10], w[11]);
  mine[3] = make_uint4(w[12], w[13], w[14], w[15]);
  __syncwarp();
  const int c = lane & 3;                                  // 16-byte column group
  const int r0 = (lane >> 3) + 4 * ((lane >> 2) & 1);      // rows r0, r0 + 8, r0 + 16, r0 + 24
  if (c * 8 < cols_ok) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = r0 + 8 * i;
      if (r < rows_ok)
        *reinterpret_cast<uint4*>(dst + long(r) * ld + c * 8) = *reinterpret_cast<const uint4*>(slab + r * kSlabPitch + c * 16);
    }
  }
  __syncwarp();
}

// The reverse: 32 rows x 32 bf16 columns from global memory (coalesced) into w[16] = this lane's row.
__device__ __forceinline__ void load_chunk_bf16(uint8_t* slab, int lane, uint32_t* w, const __nv_bfloat16* src, long ld,
                                                int rows_ok, int cols_ok) {
  const int c = lane & 3;
  const int r0 = (lane >> 3) + 4 * ((lane >> 2) & 1);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = r0 + 8 * i;
    uint4 x = make_uint4(0u, 0u, 0u, 0u);
    if (r < rows_ok && c * 8 < cols_ok) x = *reinterpret_cast<const uint4*>(src + long(r) * ld + c * 8);
    *reinterpret_cast<uint4*>(slab + r * kSlabPitch + c * 16) = x;
  }
  __syncwarp();
  const uint4* mine = reinterpret_cast<const uint4*>(slab + lane * kSlabPitch);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint4 x = mine[i];
    w[4 * i] = x.x; w[4 * i + 1] = x.y; w[4 * i + 2] = x.z; w[4 * i + 3] = x.w;
  }
  __syncwarp();
}

// The copy warp of a fused all-gather launch (see GatherParams). One thread drives a ring of `nbuf` chunk buffers.
// A buffer is refilled as soon as the store that drains it has read it (`wait_group.read`), so `nbuf - 1` loads
// stay in flight; a chunk is published `kGatherLag` stores later, when its store has completed. Hand-offs between
// the generic and the async proxy are fenced on both sides although the mbarrier (load -> store) and the bulk-group
// completion (store -> this thread) arguably order them already: taking the fences out did not raise the copy rate
// when that was tried, so the loop keeps them and does not depend on that reading of the proxy rules.
constexpr int kGatherLag = 4;
constexpr uint32_t kGatherSpinLimit = 1u << 22;   // default wait budget: polls of >= 100 ns, about half a second
__device__ __noinline__ void gather_role(const GatherParams& g, int groups, uint8_t* smem, uint64_t* bars, int* status,
                                         volatile int* abort_flag) {
  // per-buffer destination and size, and the group of each recent chunk, are computed once when the chunk's load
  // is issued: one thread runs this loop, so its index arithmetic (32-bit, one division per chunk) is on the
  // critical path of the copy
  __shared__ uint8_t* s_dst_all[4][8];
  __shared__ uint32_t s_bytes_all[4][8];
  __shared__ int s_grp_all[4][16];
  // up to four lanes of the warp run the loop independently, each on its own slice of the ring, its own barriers
  // and its own bulk groups: the loop is a chain of waits, so several chains per SM raise the copy rate
  const uint32_t lane = threadIdx.x & 31u, lanes = uint32_t(g.lanes);
  if (lane >= lanes) return;
  const uint32_t nbuf = uint32_t(g.nbuf);
  uint8_t** s_dst = s_dst_all[lane];
  uint32_t* s_bytes = s_bytes_all[lane];
  int* s_grp = s_grp_all[lane];
  bars += lane * nbuf;
  smem += size_t(lane) * nbuf * uint32_t(g.chunk_bytes);
  for (uint32_t b = 0; b < nbuf; ++b) mbar_init(&bars[b], 1);
  fence_barrier_init();
  const uint32_t chunk = uint32_t(g.chunk_bytes);
  const uint32_t per_seg = uint32_t((g.group_bytes + chunk - 1) / chunk);
  const uint32_t per_group = per_seg * uint32_t(g.nseg);
  const uint32_t total = uint32_t(groups) * per_group;
  const uint32_t first = blockIdx.x * lanes + lane, step = gridDim.x * lanes;
  const uint32_t n_mine = first < total ? (total - first + step - 1) / step : 0;
  uint32_t li = 0, lb = 0, lc = first;       // next load: index, buffer, global chunk number
  auto load = [&]() {
    const uint32_t grp = lc / per_group;
    uint32_t rem = lc - grp * per_group;
    const uint32_t seg = rem >= per_seg ? 1u : 0u;
    rem -= seg * per_seg;
    const long off = long(rem) * chunk;
    const long left = g.group_bytes - off;
    const uint32_t bytes = left < long(chunk) ? uint32_t(left) : chunk;
    const uint8_t* src = g.src[grp / uint32_t(g.groups_per_rank)] + g.seg_src_off[seg] + long(grp) * g.group_stride_src + off;
    s_dst[lb] = g.dst + g.seg_dst_off[seg] + long(grp) * g.group_bytes + off;
    s_bytes[lb] = bytes;
    s_grp[li & 15u] = int(grp);
    mbar_expect_tx(&bars[lb], bytes);
    bulk_load(smem + size_t(lb) * chunk, src, bytes, &bars[lb]);
    ++li; lc += step;
    if (++lb == nbuf) lb = 0;
  };
  auto publish = [&](uint32_t i) {
    fence_async_all();
    __threadfence();
    atomicAdd(&g.flags[s_grp[i & 15u]], 1);
  };
  while (li < n_mine && li < nbuf) load();
  uint32_t done = 0, b = 0, ph = 0;      // chunks published; buffer and barrier phase of chunk i
  for (uint32_t i = 0; i < n_mine; ++i) {
    if (!mbar_wait(&bars[b], ph, abort_flag, status, kTimeoutPeer, 32)) break;
    fence_async_smem();
    bulk_store(s_dst[b], smem + size_t(b) * chunk, s_bytes[b]);
    bulk_commit();
    if (i >= 1 && li < n_mine) {
      bulk_wait_read<1>();                      // the store of chunk i - 1 has read its buffer: refill it
      load();
    }
    if (i >= uint32_t(kGatherLag)) {
      bulk_wait<kGatherLag>();
      publish(i - kGatherLag);
      ++done;
    }
    if (++b == nbuf) { b = 0; ph ^= 1u; }
  }
  bulk_wait<0>();        // also on a timeout: no store of this CTA is in flight when it leaves
  if (!*abort_flag) for (; done < n_mine; ++done) publish(done);
}

// Every CTA of a gathering launch counts itself out; the last one clears the counters for the next launch.
__device__ __forceinline__ void gather_leave(const GatherParams& g, int groups) {
  __threadfence();
  if (atomicAdd(&g.flags[groups], 1) == int(gridDim.x) - 1) {
    for (int i = 0; i <= groups; ++i) g.flags[i] = 0;
    __threadfence();
  }
}

// PAIR = 1 is compiled separately: a kernel that contains cta_group::2 instructions can only be launched as
// clusters of two, so the single-CTA variant must not contain them. The epilogue is a template parameter too:
// with every variant in one kernel the eleven warps of a CTA (each in a different code region) thrash the
// instruction cache, which showed as "no instruction" stalls on every role.
// GATHER = 1 adds the copy warp and the per-group waits of the fused all-gather (GatherParams). It is a template
// parameter so that the kernels of ordinary launches contain none of it: with the gather code compiled into every
// variant the weight-gradient product ran 60 % slower (130 vs 81 us on its nestor_200m shape) although it never
// executes that code, and the one-GPU training step lost 5 %.
template <int PAIR, int EPI, int GATHER>
__global__ void __launch_bounds__(GATHER ? 384 : 352, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2,
            const __grid_constant__ CUtensorMap tmC, const __grid_constant__ GemmParams p, int stages) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ uint64_t full_bar[8], empty_bar[8], tfull_bar[2], tempty_bar[2];
  __shared__ uint64_t gather_bar[GATHER ? 8 : 1];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int s_abort;
  __shared__ int s_off[kMaxGroups + 1];
  __shared__ int s_tstart[kMaxGroups + 1];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int pair = PAIR;
  constexpr int n_gather = GATHER;
  const uint32_t rank = pair ? cluster_ctarank() : 0u;   // rank 0 of a pair issues the MMAs
  const int b_cols = pair ? p.BN / 2 : p.BN;             // B columns staged by this CTA
  const uint32_t a_bytes = BM * BK * 2;               // 16 KB
  const uint32_t b_bytes = uint32_t(b_cols) * BK * 2;
  const uint32_t stage_bytes = a_bytes + b_bytes;
  const uint32_t tmem_cols = (2 * p.BN <= 32) ? 32 : (2 * p.BN <= 64) ? 64 : (2 * p.BN <= 128) ? 128
                           : (2 * p.BN <= 256) ? 256 : 512;
  const int n_tiles = (p.N + p.BN - 1) / p.BN;

  // every thread fetches one group offset (one round of loads in flight; a single thread walking up to 257 offsets
  // paid a global-memory latency per group before the first tile could start)
  for (int g = threadIdx.x; g <= p.groups; g += blockDim.x)
    s_off[g] = p.offsets ? p.offsets[g] : g * p.rows_per_group;
  __syncthreads();
  if (threadIdx.x == 0) {
    s_abort = 0;
    int acc = 0;
    for (int g = 0; g < p.groups; ++g) {
      s_tstart[g] = acc;
      acc += pair ? (s_off[g + 1] - s_off[g] + 2 * BM - 1) / (2 * BM) : (s_off[g + 1] - s_off[g] + BM - 1) / BM;
    }
    s_tstart[p.groups] = acc;
    for (int s = 0; s < stages; ++s) { mbar_init(&full_bar[s], 2); mbar_init(&empty_bar[s], 1); }   // full: A and B producers
    // an accumulator is drained by the eight epilogue warps of every CTA that holds a part of it
    for (int b = 0; b < 2; ++b) { mbar_init(&tfull_bar[b], 1); mbar_init(&tempty_bar[b], pair ? 16 : 8); }
    fence_barrier_init();
    prefetch_tmap(&tmA); prefetch_tmap(&tmB);
    if (p.K2) { prefetch_tmap(&tmA2); prefetch_tmap(&tmB2); }
  }
  if (warp == 1) {
    if (pair) { tmem_alloc_pair(&tmem_base_slot, tmem_cols); tmem_relinquish_pair(); }
    else { tmem_alloc(&tmem_base_slot, tmem_cols); tmem_relinquish(); }
  }
  tc_fence_before();
  __syncthreads();
  if (pair) cluster_sync_all();     // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  int total_tiles;
  if (p.mode == 0) total_tiles = s_tstart[p.groups] * n_tiles;
  else total_tiles = p.groups * ((p.M + (pair ? 2 * BM : BM) - 1) / (pair ? 2 * BM : BM)) * n_tiles * p.splits;

  volatile int* abort_flag = &s_abort;
  const int cta = pair ? int(blockIdx.x >> 1) : int(blockIdx.x);       // persistent worker index
  const int n_cta = pair ? int(gridDim.x >> 1) : int(gridDim.x);

  if (warp == 0 || warp == 10) {
    // ------------------------------------------- TMA producers (warp 0: A tiles, warp 10: B tiles)
    const int which = warp == 0 ? 1 : 2;
    {
      // The whole warp runs the loop (coordinates stay warp-uniform); one elected lane issues the instructions.
      const bool el = elect_one();
      // One routine computes the coordinates of a k-block's boxes; `pf` = 0 issues the loads into the stage,
      // otherwise it only pulls the boxes of the operands in the mask (1 = A, 2 = B) into L2.
      // In a pair both CTAs' loads complete on the barrier of rank 0, whose MMA thread consumes both halves.
      auto ld2 = [&](void* dst, const CUtensorMap* m, uint64_t* bar, int x, int y, int pf) {
        if (!el) return;
        if (pf) tma_prefetch_2d(m, x, y);
        else if (pair) tma_load_2d_pair(dst, m, mapa_shared(smem_u32(bar), 0), x, y);
        else tma_load_2d(dst, m, bar, x, y);
      };
      auto ld3 = [&](void* dst, const CUtensorMap* m, uint64_t* bar, int x, int y, int z, int pf) {
        if (!el) return;
        if (pf) tma_prefetch_3d(m, x, y, z);
        else if (pair) tma_load_3d_pair(dst, m, mapa_shared(smem_u32(bar), 0), x, y, z);
        else tma_load_3d(dst, m, bar, x, y, z);
      };
      auto ld4 = [&](void* dst, const CUtensorMap* m, uint64_t* bar, int x, int y, int z, int w, int pf) {
        if (!el || pf) return;
        if (pair) tma_load_4d_pair(dst, m, mapa_shared(smem_u32(bar), 0), x, y, z, w);
        else tma_load_4d(dst, m, bar, x, y, z, w);
      };
      auto issue = [&](const Tile& tl, int kb, uint8_t* sa, uint8_t* sb, uint64_t* bar, int pf) {
        const bool doA = (which & 1) && (!pf || (pf & 1)), doB = (which & 2) && (!pf || (pf & 2));
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
            const int nb0 = tl.n0 + int(rank) * b_cols;    // first B column staged by this CTA
            if (!p.b_mn) ld3(sb, mB, bar, kk, nb0, bg, pf);
            else if (p.b_atoms) {
              // atom map [64, K rows, column atoms, groups]: the whole B stage is one box
              if (EPI == kSwiGLU) {
                int half = p.BN / 2, c0 = tl.n0 / 2;
                if (!pair) {
                  ld4(sb, &tmB, bar, 0, kk, c0 / 64, bg, pf);
                  ld4(sb + (half / 64) * 8192, &tmB2, bar, 0, kk, c0 / 64, bg, pf);
                } else ld4(sb, rank ? &tmB2 : &tmB, bar, 0, kk, c0 / 64, bg, pf);
              } else ld4(sb, mB, bar, 0, kk, nb0 / 64, bg, pf);
            } else if (EPI == kSwiGLU) {
              // B tile = [gate columns | up columns], each half from its own tensor (tmB = gate, tmB2 = up);
              // in a pair rank 0 stages the gate half and rank 1 the up half
              int half = p.BN / 2, c0 = tl.n0 / 2;
              if (!pair) {
                for (int a = 0; a < half / 64; ++a) ld3(sb + a * 8192, &tmB, bar, c0 + a * 64, kk, bg, pf);
                for (int a = 0; a < half / 64; ++a) ld3(sb + (half / 64 + a) * 8192, &tmB2, bar, c0 + a * 64, kk, bg, pf);
              } else {
                const CUtensorMap* mh = rank ? &tmB2 : &tmB;
                for (int a = 0; a < half / 64; ++a) ld3(sb + a * 8192, mh, bar, c0 + a * 64, kk, bg, pf);
              }
            } else {
              for (int a = 0; a < b_cols / 64; ++a) ld3(sb + a * 8192, mB, bar, nb0 + a * 64, kk, bg, pf);
            }
          }
        } else {
          int row = s_off[tl.g] + (tl.kb0 + kb) * BK;     // reduction over the group's rows; operands are MN-major
          if (doA) {
            if (p.a_atoms) { if (!pf) ld3(sa, mA, bar, 0, row, tl.m0 / 64, 0); }
            else { ld2(sa, mA, bar, tl.m0, row, pf); ld2(sa + 8192, mA, bar, tl.m0 + 64, row, pf); }
          }
          if (doB) {
            const int nb0 = tl.n0 + int(rank) * b_cols;    // first B column staged by this CTA
            if (p.b_atoms) { if (!pf) ld3(sb, mB, bar, 0, row, nb0 / 64, 0); }
            else for (int a = 0; a < b_cols / 64; ++a) ld2(sb + a * 8192, mB, bar, nb0 + a * 64, row, pf);
          }
        }
      };
      const int D = p.prefetch_dist, pf_mask = p.prefetch_ops;
      uint32_t it = 0, s = 0, ph = 0;
      int g_hint = 0, g_ready = -1;
      const bool trace_on = kDiag && p.trace != nullptr;
      long long acc_wait = 0, acc_issue = 0;
      if (el && which == 1) NB_TRACE(0);
      for (int t = cta; t < total_tiles && !*abort_flag; t += n_cta) {
        Tile tl = decode_tile(p, s_off, s_tstart, t, n_tiles, rank, g_hint);
        int nkb = tl.kb + tl.kb2;
        if constexpr (GATHER) if (which == 2 && tl.g != g_ready) {
          // first load of a gathered group: wait until the copy CTAs have staged all of its chunks
          const int need = int((p.gather.group_bytes + p.gather.chunk_bytes - 1) / p.gather.chunk_bytes) * p.gather.nseg;
          const volatile int* fl = p.gather.flags + tl.g;
          uint32_t spins = 0;
          while (*fl < need) {
            __nanosleep(100);
            if (++spins > p.gather.wait_polls || *abort_flag) {
              if (!*abort_flag) { *abort_flag = 1; atomicCAS(p.status, 0, int(kTimeoutPeer)); }
              break;
            }
          }
          if (*abort_flag) break;
          __threadfence();
          fence_async_all();
          g_ready = tl.g;
        }
        Tile nx = tl; int nx_nkb = 0;
        if (D > 0 && t + n_cta < total_tiles) {
          { int gh = g_hint; nx = decode_tile(p, s_off, s_tstart, t + n_cta, n_tiles, rank, gh); }
          nx_nkb = nx.kb + nx.kb2;
        }
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          long long c0 = trace_on ? clock64() : 0;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.status, kTimeoutEmpty)) break;
          long long c1 = trace_on ? clock64() : 0;
          if (trace_on && el && which == 1 && it >= 16 && it < 28) NB_TRACE(1 + it - 16);
          uint8_t* sa = smem + s * stage_bytes;
          if (kDiag && (p.debug & 2)) { if (rank == 0 && el) mbar_arrive(&full_bar[s]); }
          else {
            if (el && rank == 0) mbar_expect_tx(&full_bar[s], (which == 1 ? a_bytes : b_bytes) * (pair ? 2u : 1u));
            issue(tl, kb, sa, sa + a_bytes, &full_bar[s], 0);
            if (D > 0) {
              int pk = kb + D;
              if (pk < nkb) issue(tl, pk, nullptr, nullptr, nullptr, pf_mask);
              else if (pk - nkb < nx_nkb) issue(nx, pk - nkb, nullptr, nullptr, nullptr, pf_mask);
            }
          }
          if (trace_on) { acc_wait += c1 - c0; acc_issue += clock64() - c1; }
          if (++s == uint32_t(stages)) { s = 0; ph ^= 1; }
        }
      }
      if (trace_on && el) { const int o = which == 1 ? 13 : 62; p.trace[blockIdx.x * 64 + o] = acc_wait; p.trace[blockIdx.x * 64 + o + 1] = acc_issue; }
    }
  } else if (warp == 1) {
    // --------------------------------------------------------------- MMA issuer
    // One thread feeds the tensor core, so the per-k-block instruction count of this loop is what bounds the
    // kernel: stage index, phase and the operand descriptors advance by additions only (the descriptor's
    // address field is its low 14 bits, in 16-byte units), and all lanes poll the barrier together so that no
    // shuffle or re-convergence sits between the wait and the issue.
    const uint32_t idesc = make_idesc(pair ? 2 * BM : BM, p.BN, p.a_mn, p.b_mn);
    const uint64_t a_desc0 = p.a_mn ? sdesc_mnmajor(0, 8192) : sdesc_kmajor(0);
    const uint64_t b_desc0 = p.b_mn ? sdesc_mnmajor(0, 8192) : sdesc_kmajor(0);
    const uint32_t a_step = p.a_mn ? (2048u >> 4) : (32u >> 4);   // descriptor increment per K = 16 step
    const uint32_t b_step = p.b_mn ? (2048u >> 4) : (32u >> 4);
    const uint32_t smem_enc = smem_u32(smem) >> 4, stage_enc = stage_bytes >> 4, a_enc = a_bytes >> 4;
    const bool trace_on = kDiag && p.trace != nullptr;
    uint32_t s = 0, ph = 0, it = 0, tile_i = 0;
    int g_hint = 0;
    long long acc_wait = 0, acc_issue = 0, acc_commit = 0, acc_tempty = 0;
    for (int t = cta; t < total_tiles && !*abort_flag && rank == 0; t += n_cta) {
      Tile tl = decode_tile(p, s_off, s_tstart, t, n_tiles, 0, g_hint);
      const int nkb = tl.kb + tl.kb2;
      if (nkb == 0) continue;            // empty reduction: epilogue writes zeros without an accumulator
      const uint32_t buf = tile_i & 1, bph = (tile_i >> 1) & 1;
      ++tile_i;
      long long cte = trace_on ? clock64() : 0;
      if (!mbar_wait(&tempty_bar[buf], bph ^ 1, abort_flag, p.status, kTimeoutTmemEmpty)) break;
      if (trace_on) acc_tempty += clock64() - cte;
      tc_fence_after();                  // orders the epilogue's TMEM reads of this buffer before the new MMAs
      const uint32_t d_addr = tmem_base + buf * p.BN;
      // mode 1: only the k-block that holds the group's last rows can be partial; find it once per tile so that
      // the per-k-block path carries no shared-memory reads
      int tail_kb = -1, tail_valid = 0;
      if (p.mode == 1) {
        const int rows_g = tl.row_end - s_off[tl.g];
        if (rows_g % BK) { tail_kb = rows_g / BK - tl.kb0; tail_valid = rows_g % BK; }
      }
      bool ok = true;
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        long long c0 = trace_on ? clock64() : 0;
        ok = mbar_wait(&full_bar[s], ph, abort_flag, p.status, kTimeoutFull);
        if (!ok) break;
        long long c1 = trace_on ? clock64() : 0;
        if (trace_on && lane == 0 && it >= 16 && it < 28) NB_TRACE(16 + it - 16);
        if (kb == tail_kb) {
          // zero k-rows past the end of the group (they belong to the next group)
          const int valid = tail_valid;
          {
            uint8_t* sa = smem + s * stage_bytes;
            uint8_t* sb = sa + a_bytes;
            const int natoms = 2 + b_cols / 64;
            for (int a = 0; a < natoms; ++a) {
              uint8_t* base = (a < 2) ? sa + a * 8192 : sb + (a - 2) * 8192;
              for (int r = valid; r < BK; ++r)
                reinterpret_cast<uint32_t*>(base + r * 128)[lane] = 0u;
              if (pair) {
                // the peer's half of the stage (its A rows, its B columns) sits at the same offsets of its shared
                // memory; its loads have landed too (they complete on this CTA's barrier)
                const uint32_t peer = mapa_shared(smem_u32(base), 1);
                for (int r = valid; r < BK; ++r) st_shared_cluster_u32(peer + uint32_t(r) * 128u + uint32_t(lane) * 4u, 0u);
              }
            }
            if (pair) fence_async_all(); else fence_async_smem();
            __syncwarp();
          }
        }
        // operands are computed by the whole warp (warp-uniform values stay in uniform registers, which is where
        // the MMA instruction wants them); only the instructions themselves are issued by one elected lane
        const uint64_t ad = a_desc0 + (smem_enc + s * stage_enc);
        const uint64_t bd = b_desc0 + (smem_enc + s * stage_enc + a_enc);
        const uint32_t empty_addr = smem_u32(&empty_bar[s]), tfull_addr = smem_u32(&tfull_bar[buf]);
        const uint32_t empty_peer = pair ? mapa_shared(empty_addr, 1) : 0u, tfull_peer = pair ? mapa_shared(tfull_addr, 1) : 0u;
        if (elect_one()) {
          if (!(kDiag && (p.debug & 1))) {
#pragma unroll
            for (int k = 0; k < BK / 16; ++k) {
              if (pair) umma_bf16_pair(d_addr, ad + k * a_step, bd + k * b_step, idesc, (kb | k) != 0);
              else umma_bf16(d_addr, ad + k * a_step, bd + k * b_step, idesc, (kb | k) != 0);
            }
          }
          long long c2 = trace_on ? clock64() : 0;
          // the stage is free once these MMAs retire; in a pair both CTAs' barriers are told
          if (pair) { umma_commit_pair(empty_addr); umma_commit_pair(empty_peer); }
          else umma_commit(&empty_bar[s]);
          if (kb == nkb - 1) {
            if (pair) { umma_commit_pair(tfull_addr); umma_commit_pair(tfull_peer); }
            else umma_commit(&tfull_bar[buf]);
          }
          if (trace_on) {
            acc_wait += c1 - c0; acc_issue += c2 - c1; acc_commit += clock64() - c2;
            if (it >= 16 && it < 28) NB_TRACE(32 + it - 16);
          }
        }
        __syncwarp();
        if (++s == uint32_t(stages)) { s = 0; ph ^= 1; }
      }
      if (!ok) break;
    }
    if (trace_on && acc_issue != 0) {      // only the elected lane accumulated
      unsigned long long* tr = p.trace + blockIdx.x * 64;
      tr[56] = acc_wait; tr[57] = acc_issue; tr[58] = acc_commit; tr[60] = it; tr[61] = acc_tempty;
    }
  } else if (warp == 11) {
    // ----------------------------------------------------------------- copy warp of a gathering launch
    // (`p` is a __grid_constant__ parameter so that handing `p.gather` to the out-of-line copy loop by reference does
    // not make every instantiation keep a local-memory copy of the parameter block and read its fields from there)
    if constexpr (GATHER)
      gather_role(p.gather, p.groups, smem + uint32_t(stages) * stage_bytes + 8 * kSlabBytes, gather_bar, p.status, abort_flag);
  } else {
    // ----------------------------------------------------------------- epilogue
    // Eight warps: warp w reads TMEM lane quarter w % 4 (its 32 rows); the two warps of a quarter split the
    // tile's columns in alternating chunks. TMEM loads are double-buffered in registers: the load of the next
    // chunk is in flight while the current one is converted and stored.
    const int q = warp & 3;
    const int grp = (warp - 2) >> 2;             // column group 0 / 1
    // fp32 outputs of a reduction-grouped product leave through a 32 x 32 fp32 slab and one tiled reduce / store
    constexpr bool kF32Epi = EPI == kStoreF32 || EPI == kAccumF32;
    const bool tiled_out = kF32Epi && p.mode == 1 && p.c_tiled != 0;
    // bf16 outputs of a row-grouped product: a warp whose 32 rows all belong to the tile's group hands its 32 x 32
    // chunk to one tiled store (64-byte rows in the slab, 16-byte groups XOR-swizzled as the map expects); a warp
    // that straddles the end of a group stores row by row through the masked path
    constexpr bool kBf16Tiled = EPI == kStoreBf16 || EPI == kStoreBf16Stats || EPI == kAxpbyBf16;
    const bool c_tiled = kBf16Tiled && p.c_tiled != 0;
    uint8_t* slab = smem + uint32_t(stages) * stage_bytes + (warp - 2) * (tiled_out ? kSlabBytesF32 : kSlabBytes);
    uint32_t tile_i = 0;
    int g_hint = 0;
    const bool trace_on = kDiag && p.trace != nullptr;
    long long e_wait = 0, e_work = 0, e_decode = 0, e_t0 = 0;
    for (int t = cta; t < total_tiles && !*abort_flag; t += n_cta) {
      if (trace_on) e_t0 = clock64();
      Tile tl = decode_tile(p, s_off, s_tstart, t, n_tiles, rank, g_hint);
      const int nkb = tl.kb + tl.kb2;
      const int row = tl.m0 + q * 32 + lane;
      bool row_ok;
      long c_base;
      if (p.mode == 0) { row_ok = row < tl.row_end; c_base = long(row) * p.ldc; }
      else { row_ok = row < p.M; c_base = long(tl.g) * p.c_group_stride + long(row) * p.ldc; }
      if (kDiag && (p.debug & 4)) row_ok = false;           // timing experiment: no global stores
      // the warp's 32 rows start at row_w; the first rows_w of them exist
      const int row_w = tl.m0 + q * 32;
      const int rows_w = (kDiag && (p.debug & 4)) ? 0 : max(0, min(32, (p.mode == 0 ? tl.row_end : p.M) - row_w));
      const long cw_base = (p.mode == 0 ? 0 : long(tl.g) * p.c_group_stride) + long(row_w) * p.ldc;
      uint32_t buf = 0;
      if (nkb > 0) {
        buf = tile_i & 1; uint32_t bph = (tile_i >> 1) & 1;
        ++tile_i;
        // one lane polls (with back-off): a warp spinning on the barrier takes issue slots and shared-memory
        // cycles from the MMA issuer that shares its scheduler
        bool ok = true;
        long long e_t1 = trace_on ? clock64() : 0;
        if (lane == 0) ok = mbar_wait(&tfull_bar[buf], bph, abort_flag, p.status, kTimeoutTmemFull, 32);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        tc_fence_after();
        if (trace_on) { long long e_t2 = clock64(); e_decode += e_t1 - e_t0; e_wait += e_t2 - e_t1; e_t0 = e_t2; }
        if (warp == 4 && lane == 0 && tile_i <= 4) NB_TRACE(48 + 2 * (tile_i - 1));
      }
      const uint32_t taddr = tmem_base + buf * p.BN + (uint32_t(q * 32) << 16);
      const int ncols = min(p.BN, p.N - tl.n0);
      if (EPI == kSwiGLU) {
        const int half = p.BN / 2, h0 = tl.n0 / 2;
        const int hcols = min(half, p.N / 2 - h0);
        const int nch = (hcols + 31) >> 5;       // chunks of 32 gate + 32 up columns, alternating between the groups
        for (int j = grp; j < nch; j += 2) {
          float g[32], u[32];
          const int c = 32 * j;
          if (hcols - c > 16) { tmem_ld32(taddr + c, g); tmem_ld32(taddr + half + c, u); }
          else {
            tmem_ld16(taddr + c, g); tmem_ld16(taddr + half + c, u);
#pragma unroll
            for (int i = 16; i < 32; ++i) { g[i] = 0.f; u[i] = 0.f; }
          }
          tmem_ld_wait();
          uint32_t og[16], ou[16], oh[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            // round gate/up to bf16 first: the product must match silu evaluated on the stored values
            float g0 = __bfloat162float(__float2bfloat16(g[2 * i])), g1 = __bfloat162float(__float2bfloat16(g[2 * i + 1]));
            float u0 = __bfloat162float(__float2bfloat16(u[2 * i])), u1 = __bfloat162float(__float2bfloat16(u[2 * i + 1]));
            float s0 = __bfloat162float(__float2bfloat16(g0 / (1.f + __expf(-g0))));
            float s1 = __bfloat162float(__float2bfloat16(g1 / (1.f + __expf(-g1))));
            og[i] = pack_bf16(g0, g1); ou[i] = pack_bf16(u0, u1); oh[i] = pack_bf16(s0 * u0, s1 * u1);
          }
          const long o = cw_base + h0 + c;
          const int cols_ok = hcols - c;
          store_chunk_bf16(slab, lane, oh, reinterpret_cast<__nv_bfloat16*>(p.C) + o, p.ldc, rows_w, cols_ok);
          store_chunk_bf16(slab, lane, og, reinterpret_cast<__nv_bfloat16*>(p.C2) + o, p.ldc, rows_w, cols_ok);
          store_chunk_bf16(slab, lane, ou, reinterpret_cast<__nv_bfloat16*>(p.C3) + o, p.ldc, rows_w, cols_ok);
        }
      } else {
        float run_max = -INFINITY, run_sum = 0.f;
        const int nch = (ncols + 31) >> 5;       // chunks of 32 columns (the last one may hold 8, 16 or 24)
        auto load = [&](int jj, float* v) {
          if (nkb == 0) return;
          if (ncols - 32 * jj > 16) tmem_ld32(taddr + 32 * jj, v); else tmem_ld16(taddr + 32 * jj, v);
        };
        auto store_bf16 = [&](const uint32_t* w, int c0, int rem) {
          if (kBf16Tiled) { bulk_wait_read<0>(); __syncwarp(); }       // lane 0: the slab's last tiled store has read it
          // (a chunk cut short by the tile's width, not by N, must not spill into the neighbouring tile's columns)
          if (c_tiled && rows_w == 32 && (rem >= 32 || tl.n0 + c0 + rem >= p.N)) {
            uint4* mine = reinterpret_cast<uint4*>(slab + lane * 64);
            const int sw = (lane >> 1) & 3;
#pragma unroll
            for (int j = 0; j < 4; ++j) mine[j ^ sw] = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
            fence_async_smem();
            __syncwarp();
            if (lane == 0) { tma_store_2d(&tmC, slab, tl.n0 + c0, row_w); bulk_commit(); }
          } else {
            store_chunk_bf16(slab, lane, w, reinterpret_cast<__nv_bfloat16*>(p.C) + cw_base + tl.n0 + c0, p.ldc, rows_w, rem);
          }
        };
        auto process = [&](float* v, int c0) {
          const int rem = ncols - c0;            // columns of this chunk that exist: 8, 16, 24 or >= 32
          if (EPI == kStoreBf16 || EPI == kStoreBf16Stats) {
            if (EPI == kStoreBf16Stats) {
#pragma unroll
              for (int j = 0; j < 32; ++j) if (tl.n0 + c0 + j >= p.n_valid || j >= rem) v[j] = -INFINITY;
            }
            uint32_t w[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) w[j] = pack_bf16(v[2 * j] * p.alpha, v[2 * j + 1] * p.alpha);
            store_bf16(w, c0, rem);
            if (EPI == kStoreBf16Stats) {
              float m = run_max;
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                v[j] = __bfloat162float(__float2bfloat16(v[j] * p.alpha));    // statistics of the stored values
                m = fmaxf(m, v[j]);
              }
              if (m != -INFINITY) {
                float ssum = run_sum * __expf(run_max - m);
#pragma unroll
                for (int j = 0; j < 32; ++j) ssum += __expf(v[j] - m);
                run_max = m; run_sum = ssum;
              }
            }
          } else if (EPI == kSwiGLUBwd) {
            // v = dH. dGate = dH * up * s * (1 + g * (1 - s)); dUp = dH * silu(g)   (s = sigmoid(g))
            const long oe = long(row_w) * p.lde + tl.n0 + c0;
            uint32_t gw[16], uw[16], wg[16], wu[16];
            load_chunk_bf16(slab, lane, gw, reinterpret_cast<const __nv_bfloat16*>(p.E1) + oe, p.lde, rows_w, rem);
            load_chunk_bf16(slab, lane, uw, reinterpret_cast<const __nv_bfloat16*>(p.E2) + oe, p.lde, rows_w, rem);
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              float r[2][2];
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const uint32_t gbits = h ? (gw[e] & 0xFFFF0000u) : (gw[e] << 16);
                const uint32_t ubits = h ? (uw[e] & 0xFFFF0000u) : (uw[e] << 16);
                float gg = __uint_as_float(gbits), uu = __uint_as_float(ubits);
                float dh = __bfloat162float(__float2bfloat16(v[2 * e + h]));
                float sg = 1.f / (1.f + __expf(-gg));
                r[h][0] = dh * uu * sg * (1.f + gg * (1.f - sg));
                r[h][1] = dh * gg * sg;
              }
              wg[e] = pack_bf16(r[0][0], r[1][0]); wu[e] = pack_bf16(r[0][1], r[1][1]);
            }
            const long o = cw_base + tl.n0 + c0;
            store_chunk_bf16(slab, lane, wg, reinterpret_cast<__nv_bfloat16*>(p.C) + o, p.ldc, rows_w, rem);
            store_chunk_bf16(slab, lane, wu, reinterpret_cast<__nv_bfloat16*>(p.C2) + o, p.ldc, rows_w, rem);
          } else if (EPI == kAxpbyBf16) {
            // C = alpha * acc + beta * E1 in fp32, one rounding to bf16
            const long oe = long(row_w) * p.lde + tl.n0 + c0;
            uint32_t ew[16], w[16];
            bulk_wait_read<0>(); __syncwarp();           // the slab's last tiled store has read it
            load_chunk_bf16(slab, lane, ew, reinterpret_cast<const __nv_bfloat16*>(p.E1) + oe, p.lde, rows_w, rem);
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const float lo = __uint_as_float(ew[e] << 16), hi = __uint_as_float(ew[e] & 0xFFFF0000u);
              w[e] = pack_bf16(p.alpha * v[2 * e] + p.beta * lo, p.alpha * v[2 * e + 1] + p.beta * hi);
            }
            store_bf16(w, c0, rem);
          } else if (tiled_out) {
            // fp32 outputs [G, M, N] (weight gradients): the lane's row goes to its 128-byte row of the slab, 16-byte
            // groups XOR-swizzled by the row as the tensor map expects, and the 32 x 32 chunk leaves as one tiled
            // reduce-add (or store). Rows past M and columns past N are clipped by the map. Per-lane vector
            // reductions in the accumulator's row-per-lane shape touched 32 cache lines per instruction and cost
            // 12.7 k cycles per 128 x 216 tile.
            if (nkb > 0 || EPI == kStoreF32) {
              bulk_wait_read<0>();                 // lane 0: the previous chunk's operation has read the slab
              __syncwarp();
              float4* mine = reinterpret_cast<float4*>(slab + lane * 128);
#pragma unroll
              for (int j = 0; j < 8; ++j)
                mine[j ^ (lane & 7)] = make_float4(v[4 * j] * p.alpha, v[4 * j + 1] * p.alpha, v[4 * j + 2] * p.alpha,
                                                   v[4 * j + 3] * p.alpha);
              fence_async_smem();
              __syncwarp();
              if (lane == 0 && row_w < p.M) {
                if (EPI == kStoreF32) tma_store_3d(&tmC, slab, tl.n0 + c0, row_w, tl.g);
                else tma_reduce_add_3d(&tmC, slab, tl.n0 + c0, row_w, tl.g);
                bulk_commit();
              }
            }
          } else if (row_ok) {
            // fp32 outputs, row-grouped product: one row per lane
            float* Cp = reinterpret_cast<float*>(p.C) + c_base + tl.n0 + c0;
            if (EPI == kStoreF32) {
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                if (j < rem) reinterpret_cast<float4*>(Cp + j)[0] = make_float4(v[j] * p.alpha, v[j + 1] * p.alpha, v[j + 2] * p.alpha, v[j + 3] * p.alpha);
            } else if (nkb > 0) {                // kAccumF32
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                if (j >= rem) break;
                // a vector reduction (no return value): fire-and-forget, so the epilogue never waits on a load of the
                // old value. Without a split reduction every address is touched once per launch, so the sum is
                // still deterministic.
                float4 add = make_float4(v[j] * p.alpha, v[j + 1] * p.alpha, v[j + 2] * p.alpha, v[j + 3] * p.alpha);
                atomicAdd(reinterpret_cast<float4*>(Cp + j), add);
              }
            }
          }
        };
        float va[32], vb[32];
        if (nkb == 0) {
#pragma unroll
          for (int j = 0; j < 32; ++j) { va[j] = 0.f; vb[j] = 0.f; }
        }
        int j = grp;
        if (j < nch) load(j, va);
        while (j < nch) {
          if (nkb > 0) tmem_ld_wait32(va);
          if (j + 2 < nch) load(j + 2, vb);
          process(va, 32 * j);
          j += 2;
          if (j >= nch) break;
          if (nkb > 0) tmem_ld_wait32(vb);
          if (j + 2 < nch) load(j + 2, va);
          process(vb, 32 * j);
          j += 2;
        }
        if (EPI == kStoreBf16Stats && row_ok) {
          // one (max, sum-exp) partial per row, n-tile and column group
          float2* part = reinterpret_cast<float2*>(p.C2) + (long(row) * n_tiles + (tl.n0 / p.BN)) * 2 + grp;
          *part = make_float2(run_max, run_sum);
        }
      }
      if (nkb > 0) {
        tc_fence_before();
        __syncwarp();
        if (warp == 4 && lane == 0 && tile_i <= 4) NB_TRACE(48 + 2 * (tile_i - 1) + 1);
        if (lane == 0) {
          if (pair) mbar_arrive_cluster(mapa_shared(smem_u32(&tempty_bar[buf]), 0));
          else mbar_arrive(&tempty_bar[buf]);
        }
        if (trace_on) e_work += clock64() - e_t0;
      }
    }
    if (tiled_out || c_tiled) bulk_wait<0>();           // nothing of this CTA's shared memory is still being read when it leaves
    if (trace_on && warp == 4 && lane == 0) {
      unsigned long long* tr = p.trace + blockIdx.x * 64;
      tr[44] = e_decode; tr[45] = e_wait; tr[46] = e_work; tr[47] = tile_i;
    }
  }

  // ----------------------------------------------------------------------- teardown
  // After a wait gave up, tile loads issued before the abort may still be on their way into this CTA's shared memory
  // (at most one per pipeline stage, each a few microseconds): let them land before the CTA gives its memory back.
  if (*abort_flag) for (int i = 0; i < 64; ++i) __nanosleep(1000);
  tc_fence_before();
  __syncthreads();
  if (pair) cluster_sync_all();     // neither CTA leaves (or frees TMEM) while its peer may still signal or read it
  if (warp == 1) {
    tc_fence_after();
    if (pair) tmem_dealloc_pair(tmem_base, tmem_cols); else tmem_dealloc(tmem_base, tmem_cols);
  }
  if constexpr (GATHER) { if (threadIdx.x == 0) gather_leave(p.gather, p.groups); }
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

// bf16 tensor of rank 2 to 4 (dims innermost-first), strides in elements for dims 1.. (innermost is contiguous).
int make_map(CUtensorMap* m, const void* base, int rank, const long* dims, const long* strides_elems,
             const int* box, int elem_bytes = 2, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeFn fn = encode_fn();
  if (!fn) return 1;
  cuuint64_t gd[4]; cuuint64_t gs[3]; cuuint32_t bx[4]; cuuint32_t es[4] = {1, 1, 1, 1};
  for (int i = 0; i < rank; ++i) { gd[i] = cuuint64_t(dims[i]); bx[i] = cuuint32_t(box[i]); }
  for (int i = 0; i + 1 < rank; ++i) gs[i] = cuuint64_t(strides_elems[i]) * cuuint64_t(elem_bytes);
  CUresult r = fn(m, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, cuuint32_t(rank), const_cast<void*>(base), gd, gs, bx, es,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
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
  float beta;               // kAxpbyBf16: weight of E1
  int n_valid;
  int splits;
  int* status;
  int max_m_tiles;          // upper bound on m tiles over all groups (mode 0)
  int sms;                  // 0 = all
  unsigned long long* trace;
  int prefetch_dist;        // L2 look-ahead of the producer in k-blocks (0 = off)
  int prefetch_ops;         // 1 = A, 2 = B, 3 = both
  int max_stages;           // 0 = as many as fit
  int pair;                 // mode 0 only: 256-row tiles on CTA pairs (cta_group::2), each CTA stages half of B
  int debug;                // builds with -DNB_GEMM_DIAG only: 1 = no MMAs, 2 = no loads, 4 = no stores (outputs are garbage)
  // fused all-gather of B (and B2) from rank-sharded weight arenas; see nb::GatherParams. gather_on == 0: off.
  const void* gather_src[8];
  void* gather_dst;
  long gather_seg_src_off[2], gather_seg_dst_off[2];
  long gather_group_bytes, gather_group_stride_src;
  int gather_nseg, gather_groups_per_rank, gather_on, gather_chunk;
  int* gather_flags;        // [groups + 1] ints, zero before the first launch
  int gather_nbuf;          // ring depth per copying lane (chunks)
  int gather_lanes;         // copying lanes of the copy warp (0 = 1)
  unsigned gather_wait_polls;  // 0 = default (about half a second)
  int no_tiled_store;          // 1 = bf16 outputs always leave through the row-masked store path
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
  const int pair = a->pair ? 1 : 0;
  // a pair splits B by columns: MN-major halves must be whole 64-column atoms. Reduction-grouped products (mode 1)
  // take pairs too: each CTA stages its own 128 of the tile's 256 A columns and half of the B columns.
  if (pair && ((a->mode == 0 && a->a_mn) || a->BN % 16 || ((a->b_mn || a->mode == 1) && a->BN % 128))) return -8;
  if (!g_num_sms) {   // the GPUs of one machine are identical: the first device asked answers for all
    int dev; cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  CUtensorMap tmA, tmB, tmA2, tmB2, tmC;
  memset(&tmA2, 0, sizeof(tmA2)); memset(&tmB2, 0, sizeof(tmB2)); memset(&tmC, 0, sizeof(tmC));
  // An MN-major operand [k rows, cols] whose row pitch covers whole 64-column atoms can be viewed as
  // [64, k rows, atoms]: one box then fills every atom of a stage (atom-major in shared memory, as the MMA
  // descriptors expect). Columns past `cols` inside the last atom are whatever the pitch padding holds; they only
  // reach output rows / columns that the epilogue masks. Atoms past the last one are zero-filled.
  auto atoms_ok = [&](const NbOperand& o) { return o.ptr != nullptr && o.ld >= ((o.cols + 63) / 64) * 64; };
  const int a_atoms = a->mode == 1 && atoms_ok(a->A);
  const int b_atoms = (a->mode == 1 || a->b_mn) && atoms_ok(a->B) && (a->epilogue != kSwiGLU || atoms_ok(a->B2));
  auto map_a = [&](CUtensorMap* m, const NbOperand& o) -> int {
    if (a_atoms) {
      long dims[3] = {64, o.rows, (o.cols + 63) / 64}; long st[2] = {o.ld, 64};
      int box[3] = {64, BK, 2};
      return make_map(m, o.ptr, 3, dims, st, box);
    }
    long dims[2] = {o.cols, o.rows}; long st[1] = {o.ld};
    int box_k[2] = {BK, BM};            // K-major: 64 k x 128 rows
    int box_mn[2] = {64, BK};           // MN-major: 64 m x 64 k-rows
    return make_map(m, o.ptr, 2, dims, st, a->a_mn ? box_mn : box_k);
  };
  auto map_b = [&](CUtensorMap* m, const NbOperand& o) -> int {
    if (a->mode == 1) {
      if (b_atoms) {
        long dims[3] = {64, o.rows, (o.cols + 63) / 64}; long st[2] = {o.ld, 64};
        int box[3] = {64, BK, (pair ? a->BN / 2 : a->BN) / 64};
        return make_map(m, o.ptr, 3, dims, st, box);
      }
      long dims[2] = {o.cols, o.rows}; long st[1] = {o.ld};
      int box[2] = {64, BK};
      return make_map(m, o.ptr, 2, dims, st, box);
    }
    if (b_atoms) {
      const int cols_cta = pair ? a->BN / 2 : a->BN;
      long dims[4] = {64, o.rows, (o.cols + 63) / 64, o.groups > 0 ? o.groups : 1};
      long st[3] = {o.ld, 64, o.group_stride > 0 ? o.group_stride : o.rows * o.ld};
      int box[4] = {64, BK, (a->epilogue == kSwiGLU ? (pair ? a->BN / 2 : a->BN / 2) : cols_cta) / 64, 1};
      return make_map(m, o.ptr, 4, dims, st, box);
    }
    long dims[3] = {o.cols, o.rows, o.groups > 0 ? o.groups : 1};
    long st[2] = {o.ld, o.group_stride > 0 ? o.group_stride : o.rows * o.ld};
    int box_k[3] = {BK, pair ? a->BN / 2 : a->BN, 1};   // K-major B [N, K]: 64 k x (this CTA's) rows
    int box_mn[3] = {64, BK, 1};        // MN-major B [K, N]: 64 n x 64 k-rows
    return make_map(m, o.ptr, 3, dims, st, a->b_mn ? box_mn : box_k);
  };
  if (map_a(&tmA, a->A)) return -10;
  if (map_b(&tmB, a->B)) return -11;
  if (a->K2 > 0) { if (map_a(&tmA2, a->A2)) return -12; }
  const bool tiled_out = a->mode == 1 && (a->epilogue == kStoreF32 || a->epilogue == kAccumF32) && !a->no_tiled_store;
  if (tiled_out) {
    // the fp32 output [G, M, N] as a tensor map: 32 x 32 boxes, 128-byte rows swizzled
    if (a->ldc % 4 || a->c_group_stride % 4 || reinterpret_cast<uintptr_t>(a->C) % 16) return -14;
    long dims[3] = {a->N, a->M, a->groups}; long st[2] = {a->ldc, a->groups > 1 ? a->c_group_stride : long(a->M) * a->ldc};
    int box[3] = {32, 32, 1};
    if (make_map(&tmC, a->C, 3, dims, st, box, 4)) return -14;
  }
  int c_tiled = tiled_out ? 1 : 0;
  // bf16 output [rows, N] of a row-grouped product: 32 x 32 boxes, 64-byte rows, 64-byte swizzle
  if (a->mode == 0 && (a->epilogue == kStoreBf16 || a->epilogue == kStoreBf16Stats || a->epilogue == kAxpbyBf16) &&
      a->ldc % 8 == 0 && reinterpret_cast<uintptr_t>(a->C) % 16 == 0 && a->A.rows > 0 && !a->no_tiled_store) {
    long dims[2] = {a->N, a->A.rows}; long st[1] = {a->ldc};
    int box[2] = {32, 32};
    if (make_map(&tmC, a->C, 2, dims, st, box, 2, CU_TENSOR_MAP_SWIZZLE_64B)) return -14;
    c_tiled = 1;
  }
  if (a->K2 > 0 || a->epilogue == kSwiGLU) { if (map_b(&tmB2, a->B2)) return -13; }

  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.mode = a->mode; p.groups = a->groups; p.BN = a->BN; p.epilogue = a->epilogue;
  p.M = a->M; p.N = a->N; p.K = a->K; p.K2 = a->K2; p.offsets = a->offsets; p.rows_per_group = a->rows_per_group;
  p.a_mn = a->a_mn; p.b_mn = a->b_mn; p.b_grouped = a->b_grouped;
  p.C = a->C; p.ldc = a->ldc; p.c_group_stride = a->c_group_stride; p.C2 = a->C2; p.C3 = a->C3;
  p.E1 = a->E1; p.E2 = a->E2; p.lde = a->lde; p.alpha = a->alpha; p.beta = a->beta; p.n_valid = a->n_valid > 0 ? a->n_valid : a->N; p.status = a->status;
  p.trace = a->trace;
  p.prefetch_dist = a->prefetch_dist > 0 ? a->prefetch_dist : 0;
  p.prefetch_ops = a->prefetch_ops & 3;
  p.pair = pair;
  p.a_atoms = a_atoms; p.b_atoms = b_atoms;
  p.debug = a->debug;
  p.c_tiled = c_tiled;
  p.splits = (a->mode == 1 && a->epilogue == kAccumF32 && a->splits > 1) ? a->splits : 1;

  const int n_tiles = (a->N + a->BN - 1) / a->BN;
  // mode 0: max_m_tiles bounds the row tiles over all groups (tiles of 256 rows for pairs)
  long tiles = a->mode == 0 ? long(a->max_m_tiles) * n_tiles
                            : long(a->groups) * ((a->M + (pair ? 2 * BM : BM) - 1) / (pair ? 2 * BM : BM)) * n_tiles * p.splits;
  if (tiles <= 0) return 0;
  const uint32_t stage_bytes = BM * BK * 2 + (pair ? a->BN / 2 : a->BN) * BK * 2;
  size_t ring_bytes = 0;
  if (a->gather_on) {
    if (a->mode != 0 || !a->b_grouped || !a->gather_flags || !a->gather_dst) return -20;
    if (a->gather_nseg < 1 || a->gather_nseg > 2 || a->gather_groups_per_rank < 1) return -21;
    if (a->gather_group_bytes <= 0 || a->gather_group_bytes % 16 || a->gather_group_stride_src % 16) return -22;
    if (a->gather_chunk < 1024 || a->gather_chunk % 1024 || a->gather_chunk > 32768) return -23;
    p.gather.on = 1;
    p.gather.chunk_bytes = a->gather_chunk;
    p.gather.nbuf = a->gather_nbuf;
    p.gather.lanes = a->gather_lanes > 0 ? a->gather_lanes : 1;
    if (p.gather.lanes > 4 || p.gather.nbuf < 2 || p.gather.nbuf * p.gather.lanes > 8 ||
        size_t(p.gather.nbuf) * p.gather.lanes * a->gather_chunk > 64 * 1024) return -25;
    for (int r = 0; r < 8; ++r) p.gather.src[r] = static_cast<const uint8_t*>(a->gather_src[r]);
    p.gather.dst = static_cast<uint8_t*>(a->gather_dst);
    for (int i = 0; i < 2; ++i) {
      if (a->gather_seg_src_off[i] % 16 || a->gather_seg_dst_off[i] % 16) return -22;
      p.gather.seg_src_off[i] = a->gather_seg_src_off[i]; p.gather.seg_dst_off[i] = a->gather_seg_dst_off[i];
    }
    const int owners = (a->groups + a->gather_groups_per_rank - 1) / a->gather_groups_per_rank;
    if (owners > 8) return -26;
    for (int r = 0; r < owners; ++r) if (!a->gather_src[r]) return -26;
    p.gather.group_bytes = a->gather_group_bytes; p.gather.group_stride_src = a->gather_group_stride_src;
    p.gather.nseg = a->gather_nseg; p.gather.groups_per_rank = a->gather_groups_per_rank;
    p.gather.flags = a->gather_flags;
    p.gather.wait_polls = a->gather_wait_polls ? a->gather_wait_polls : kGatherSpinLimit;
    ring_bytes = size_t(p.gather.nbuf) * p.gather.lanes * a->gather_chunk;
  }
  const size_t slab_bytes = tiled_out ? kSlabBytesF32 : kSlabBytes;
  int stages = int((200 * 1024 - ring_bytes - 8 * (slab_bytes - kSlabBytes)) / stage_bytes);   // 227 KB per CTA minus epilogue slabs, barriers, offsets, alignment slack
  if (stages > 8) stages = 8;
  if (a->max_stages > 0 && stages > a->max_stages) stages = a->max_stages;
  if (stages < 2) return -7;
  size_t smem = size_t(stages) * stage_bytes + 1024 + 8 * slab_bytes + ring_bytes;
  typedef void (*KernelFn)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap, const GemmParams, int);
  static const KernelFn kernels[2][7] = {
      {gemm_kernel<0, 0, 0>, gemm_kernel<0, 1, 0>, gemm_kernel<0, 2, 0>, gemm_kernel<0, 3, 0>, gemm_kernel<0, 4, 0>, gemm_kernel<0, 5, 0>,
       gemm_kernel<0, 6, 0>},
      {gemm_kernel<1, 0, 0>, gemm_kernel<1, 1, 0>, gemm_kernel<1, 2, 0>, gemm_kernel<1, 3, 0>, gemm_kernel<1, 4, 0>, gemm_kernel<1, 5, 0>,
       gemm_kernel<1, 6, 0>}};
  // gathering launches: the expert-bank products only (plain store, SwiGLU forward, SwiGLU backward)
  static const KernelFn gather_kernels[2][7] = {
      {gemm_kernel<0, 0, 1>, nullptr, nullptr, gemm_kernel<0, 3, 1>, gemm_kernel<0, 4, 1>, nullptr, nullptr},
      {gemm_kernel<1, 0, 1>, nullptr, nullptr, gemm_kernel<1, 3, 1>, gemm_kernel<1, 4, 1>, nullptr, nullptr}};
  if (a->epilogue < 0 || a->epilogue > 6) return -9;
  if (a->epilogue == kAxpbyBf16 && !a->E1) return -9;
  const int gat = p.gather.on ? 1 : 0;
  const KernelFn kernel = gat ? gather_kernels[pair][a->epilogue] : kernels[pair][a->epilogue];
  if (!kernel) return -27;      // no gathering variant of this epilogue
  static SmemAttr configured[2][2][7];
  if (int e = configured[gat][pair][a->epilogue].ensure(kernel, smem)) return e;
  int sms = a->sms > 0 ? a->sms : g_num_sms;
  const int threads = p.gather.on ? 384 : 352;
  if (p.gather.on) {
    // The B producers of a gathering launch wait for chunks that the copy warps of ALL its CTAs stage, so every CTA
    // of the grid has to be resident at the same time: never launch more than the occupancy calculator grants.
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem) != cudaSuccess || per_sm < 1) return -28;
    if (sms > per_sm * g_num_sms) sms = per_sm * g_num_sms;
  }
  if (!pair) {
    int grid = int(tiles < sms ? tiles : sms);
    kernel<<<grid, threads, smem, stream>>>(tmA, tmB, tmA2, tmB2, tmC, p, stages);
    return int(cudaGetLastError());
  }
  int pairs = sms / 2;
  if (tiles < pairs) pairs = int(tiles);
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(2 * pairs); cfg.blockDim = dim3(threads); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  return int(cudaLaunchKernelEx(&cfg, kernel, tmA, tmB, tmA2, tmB2, tmC, p, stages));
}

}  // extern "C"
