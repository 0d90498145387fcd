// Routing kernels: top-k selection with gates (forward / backward) and the expert dispatch plan.
//
//   route_fwd / route_bwd : one thread per routing problem. A problem is one score vector of E
//       entries (E <= 64): a token's scores of one router, or - with a column selection - the
//       scores of the private experts of one selected column of a token. Selection is top-k of
//       (score + bias) with ties broken towards the lower index; gates come from the raw scores:
//         mode 0 "renorm" : softmax over the k selected scores
//         mode 1 "switch" : the selected entries of the softmax over all E scores
//         mode 2 "all"    : k == E, no selection, softmax over all scores in index order
//       Optionally the gate is multiplied with the gate of the selected column and rounded to bf16
//       (the weight a private expert's output is combined with).
//   plan_hist / plan_scan / plan_place : stable counting sort of (token, slot) pairs by expert id
//       -> order, inverse order and per-expert row offsets, without a device-wide sort.
//
// Replaces the reference's torch.topk / softmax / gather chains in its routers
// (nestor/backbones/nestor.py:558-575, nestor/backbones/batched_router.py:210-224,
// nestor/backbones/expert_pools.py:495-510) and its argsort-based dispatch tables
// (nestor/backbones/grouped_mm.py:245-262, nestor/backbones/triton_dispatch.py).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace nbr {

constexpr int kMaxK = 8;
constexpr int kMaxE = 64;

struct RouteArgs {
  const void* scores; long ld; int is_f32;   // [T, ld] score matrix (bf16 or fp32)
  int col_off;                               // first column of this router family inside a row
  const int* cols; int k_cols;               // optional [T, k_cols] selected columns (problem (t, j) reads block cols[t, j])
  const float* bias;                         // [E] or [n_blocks, E] (with cols); may be null
  int E, k, mode, T;
  const int* idx_in;                         // optional [nprob, k]: replay these selections instead of selecting
  int* idx_out;                              // [nprob, k] selected entries (local index)
  int* id_out;                               // optional [nprob, k] global ids (column * E + local)
  float* gates;                              // [nprob, k] fp32 gates
  const float* colgate;                      // optional [T, k_cols] gates of the selected columns
  __nv_bfloat16* w_out;                      // optional [nprob, k] bf16(bf16(gate) * bf16(colgate))
};

__device__ __forceinline__ float load_score(const void* base, long i, int is_f32) {
  return is_f32 ? reinterpret_cast<const float*>(base)[i] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[i]);
}
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16(x)); }

__global__ void route_fwd_kernel(RouteArgs a) {
  const int kc = a.cols ? a.k_cols : 1;
  const long nprob = long(a.T) * kc;
  const long p = long(blockIdx.x) * blockDim.x + threadIdx.x;
  if (p >= nprob) return;
  const long t = p / kc;
  const int col = a.cols ? a.cols[p] : 0;
  const long s0 = t * a.ld + a.col_off + long(col) * a.E;
  const float* b = a.bias ? a.bias + (a.cols ? long(col) * a.E : 0) : nullptr;
  int sel[kMaxK];
  float sv[kMaxK];
  if (a.mode == 2) {
    for (int j = 0; j < a.k; ++j) sel[j] = j;
  } else if (a.idx_in) {
    for (int j = 0; j < a.k; ++j) sel[j] = a.idx_in[p * a.k + j];
  } else {
    for (int j = 0; j < a.k; ++j) {
      float best = -INFINITY; int bi = 0; bool have = false;
      for (int e = 0; e < a.E; ++e) {
        bool used = false;
        for (int i = 0; i < j; ++i) used |= sel[i] == e;
        if (used) continue;
        float v = load_score(a.scores, s0 + e, a.is_f32) + (b ? b[e] : 0.f);
        if (!have || v > best) { best = v; bi = e; have = true; }     // strict '>' keeps the lower index on ties
      }
      sel[j] = bi;
    }
  }
  float m = -INFINITY;
  for (int j = 0; j < a.k; ++j) { sv[j] = load_score(a.scores, s0 + sel[j], a.is_f32); m = fmaxf(m, sv[j]); }
  float z = 0.f;
  if (a.mode == 1) {
    for (int e = 0; e < a.E; ++e) m = fmaxf(m, load_score(a.scores, s0 + e, a.is_f32));
    for (int e = 0; e < a.E; ++e) z += expf(load_score(a.scores, s0 + e, a.is_f32) - m);
  } else {
    for (int j = 0; j < a.k; ++j) z += expf(sv[j] - m);
  }
  const float cg = a.colgate ? a.colgate[p] : 1.f;
  for (int j = 0; j < a.k; ++j) {
    const float g = expf(sv[j] - m) / z;
    a.idx_out[p * a.k + j] = sel[j];
    if (a.id_out) a.id_out[p * a.k + j] = col * a.E + sel[j];
    a.gates[p * a.k + j] = g;
    if (a.w_out) a.w_out[p * a.k + j] = __float2bfloat16(round_bf16(g) * round_bf16(cg));
  }
}

struct RouteBwdArgs {
  RouteArgs f;                      // forward arguments (scores, layout, selections in idx_out, gates)
  const float* dgates;              // [nprob, k] gradient of the fp32 gates (may be null)
  const __nv_bfloat16* dw;          // [nprob, k] gradient of w_out (may be null)
  void* dscores; long d_ld; int d_is_f32;   // [T, d_ld] dense over this family's columns, pre-zeroed by the caller
  float* dcolgate;                  // optional [T, k_cols]
};

__device__ __forceinline__ void store_score(void* base, long i, int is_f32, float v) {
  if (is_f32) reinterpret_cast<float*>(base)[i] = v;
  else reinterpret_cast<__nv_bfloat16*>(base)[i] = __float2bfloat16(v);
}

__global__ void route_bwd_kernel(RouteBwdArgs a) {
  const RouteArgs& f = a.f;
  const int kc = f.cols ? f.k_cols : 1;
  const long nprob = long(f.T) * kc;
  const long p = long(blockIdx.x) * blockDim.x + threadIdx.x;
  if (p >= nprob) return;
  const long t = p / kc;
  const int col = f.cols ? f.cols[p] : 0;
  const long s0 = t * f.ld + f.col_off + long(col) * f.E;
  const long d0 = t * a.d_ld + long(col) * f.E;
  const float cg = f.colgate ? round_bf16(f.colgate[p]) : 1.f;
  float dg[kMaxK], g[kMaxK];
  int sel[kMaxK];
  float dot = 0.f, dcg = 0.f;
  for (int j = 0; j < f.k; ++j) {
    sel[j] = f.idx_out[p * f.k + j];
    g[j] = f.gates[p * f.k + j];
    float d = a.dgates ? a.dgates[p * f.k + j] : 0.f;
    if (a.dw) {
      const float w = __bfloat162float(a.dw[p * f.k + j]);
      d += w * cg;
      dcg += w * round_bf16(g[j]);
    }
    dg[j] = d;
    dot += g[j] * d;
  }
  if (a.dcolgate) a.dcolgate[p] = dcg;
  if (f.mode == 1) {
    // gate_j = softmax(all)_sel_j: d score_e = p_e * ([e selected] dg_e - sum_j g_j dg_j)
    float m = -INFINITY, z = 0.f;
    for (int e = 0; e < f.E; ++e) m = fmaxf(m, load_score(f.scores, s0 + e, f.is_f32));
    for (int e = 0; e < f.E; ++e) z += expf(load_score(f.scores, s0 + e, f.is_f32) - m);
    for (int e = 0; e < f.E; ++e) {
      const float pe = expf(load_score(f.scores, s0 + e, f.is_f32) - m) / z;
      float d = 0.f;
      for (int j = 0; j < f.k; ++j) if (sel[j] == e) d = dg[j];
      store_score(a.dscores, d0 + e, a.d_is_f32, pe * (d - dot));
    }
  } else {
    for (int j = 0; j < f.k; ++j) store_score(a.dscores, d0 + sel[j], a.d_is_f32, g[j] * (dg[j] - dot));
  }
}

// ------------------------------------------------------------------------------- expert plan
// n elements (flat token*slots + slot order), ids in [0, E), E <= kMaxKeys. Blocks of kPlanBlock elements.
// The same sort builds the packed-attention plan of a block with key = column * B + sequence.
constexpr int kPlanBlock = 1024;
constexpr int kMaxKeys = 256;

// Per-block histogram. hist[blk * E + e].
__global__ void plan_hist_kernel(const int* __restrict__ ids, int n, int E, int* __restrict__ hist) {
  __shared__ int s_h[kMaxKeys];
  if (threadIdx.x < kMaxKeys) s_h[threadIdx.x] = 0;
  __syncthreads();
  const int i = blockIdx.x * kPlanBlock + threadIdx.x;
  if (i < n) atomicAdd(&s_h[ids[i]], 1);
  __syncthreads();
  if (threadIdx.x < E) hist[blockIdx.x * E + threadIdx.x] = s_h[threadIdx.x];
}

// One block: exclusive scan of every expert's counts over the blocks (hist becomes the block's base inside the
// expert's range) and the expert offsets.
__global__ void plan_scan_kernel(int* __restrict__ hist, int nblk, int E, int* __restrict__ offsets) {
  __shared__ int s_tot[kMaxKeys + 1];
  const int e = threadIdx.x;
  if (e < E) {
    int run = 0;
    for (int b = 0; b < nblk; ++b) { int c = hist[b * E + e]; hist[b * E + e] = run; run += c; }
    s_tot[e] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int i = 0; i < E; ++i) { offsets[i] = run; run += s_tot[i]; }
    offsets[E] = run;
  }
}

// Stable placement: element i goes to offsets[e] + base[blk][e] + (number of earlier elements of e in the block).
__global__ void plan_place_kernel(const int* __restrict__ ids, int n, int E, const int* __restrict__ base,
                                  const int* __restrict__ offsets, int* __restrict__ order, int* __restrict__ inv) {
  __shared__ int s_w[kPlanBlock / 32][kMaxKeys];  // per-warp counts, then exclusive prefix over the warps
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int j = threadIdx.x; j < (kPlanBlock / 32) * kMaxKeys; j += blockDim.x) (&s_w[0][0])[j] = 0;
  __syncthreads();
  const int i = blockIdx.x * kPlanBlock + threadIdx.x;
  const bool live = i < n;
  const int e = live ? ids[i] : -1;
  const unsigned peers = __match_any_sync(0xffffffffu, e);
  const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
  if (live && rank_in_warp == 0) s_w[warp][e] = __popc(peers);
  __syncthreads();
  if (threadIdx.x < E) {
    int run = 0;
    for (int w = 0; w < kPlanBlock / 32; ++w) { int c = s_w[w][threadIdx.x]; s_w[w][threadIdx.x] = run; run += c; }
  }
  __syncthreads();
  if (live) {
    const int pos = offsets[e] + base[blockIdx.x * E + e] + s_w[warp][e] + rank_in_warp;
    inv[i] = pos;
    order[pos] = i;
  }
}

// Packed-attention plan from the sort of keys column * B + sequence: per packed row its token, slot and position.
__global__ void column_plan_finish_kernel(const int* __restrict__ order, int rows, int k, const int* __restrict__ pos,
                                          int S, int* __restrict__ tok_of_row, int* __restrict__ slot_of_row,
                                          int* __restrict__ pos_of_row) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const int flat = order[r];
  const int t = flat / k;
  tok_of_row[r] = t;
  slot_of_row[r] = flat - t * k;
  pos_of_row[r] = pos ? max(pos[t], 0) : t % S;
}

// keys[t * k + j] = idx[t, j] * B + t / S
__global__ void column_plan_keys_kernel(const int* __restrict__ idx, int n, int k, int S, int B, int* __restrict__ keys) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  keys[i] = idx[i] * B + (i / k) / S;
}

}  // namespace nbr

extern "C" {

struct NbRouteArgs {
  const void* scores; long ld; int is_f32;
  int col_off;
  const int* cols; int k_cols;
  const float* bias;
  int E, k, mode, T;
  const int* idx_in;
  int* idx_out;
  int* id_out;
  float* gates;
  const float* colgate;
  void* w_out;
};

static nbr::RouteArgs to_route(const NbRouteArgs* a) {
  nbr::RouteArgs r;
  r.scores = a->scores; r.ld = a->ld; r.is_f32 = a->is_f32; r.col_off = a->col_off; r.cols = a->cols; r.k_cols = a->k_cols;
  r.bias = a->bias; r.E = a->E; r.k = a->k; r.mode = a->mode; r.T = a->T; r.idx_in = a->idx_in; r.idx_out = a->idx_out;
  r.id_out = a->id_out; r.gates = a->gates; r.colgate = a->colgate; r.w_out = reinterpret_cast<__nv_bfloat16*>(a->w_out);
  return r;
}

static int route_check(const NbRouteArgs* a) {
  if (a->E < 1 || a->E > nbr::kMaxE || a->k < 1 || a->k > nbr::kMaxK || a->k > a->E || a->T < 0) return -1;
  if (a->mode < 0 || a->mode > 2 || (a->mode == 2 && a->k != a->E)) return -2;
  return 0;
}

int nb_route_fwd(const NbRouteArgs* a, cudaStream_t st) {
  if (int rc = route_check(a)) return rc;
  const long nprob = long(a->T) * (a->cols ? a->k_cols : 1);
  if (nprob == 0) return 0;
  nbr::route_fwd_kernel<<<unsigned((nprob + 127) / 128), 128, 0, st>>>(to_route(a));
  return int(cudaGetLastError());
}

int nb_route_bwd(const NbRouteArgs* a, const float* dgates, const void* dw, void* dscores, long d_ld, int d_is_f32,
                 float* dcolgate, cudaStream_t st) {
  if (int rc = route_check(a)) return rc;
  const long nprob = long(a->T) * (a->cols ? a->k_cols : 1);
  if (nprob == 0) return 0;
  nbr::RouteBwdArgs b;
  b.f = to_route(a); b.dgates = dgates; b.dw = reinterpret_cast<const __nv_bfloat16*>(dw); b.dscores = dscores;
  b.d_ld = d_ld; b.d_is_f32 = d_is_f32; b.dcolgate = dcolgate;
  nbr::route_bwd_kernel<<<unsigned((nprob + 127) / 128), 128, 0, st>>>(b);
  return int(cudaGetLastError());
}

// ids [n] int32 in [0, E). scratch: int32 [ceil(n / 1024) * E]. Outputs: order [n], inv [n], offsets [E + 1].
int nb_expert_plan(const int* ids, int n, int E, int* scratch, int* order, int* inv, int* offsets, cudaStream_t st) {
  if (E < 1 || E > nbr::kMaxKeys || n < 0) return -1;
  const int nblk = (n + nbr::kPlanBlock - 1) / nbr::kPlanBlock;
  if (nblk > 0) nbr::plan_hist_kernel<<<nblk, nbr::kPlanBlock, 0, st>>>(ids, n, E, scratch);
  nbr::plan_scan_kernel<<<1, nbr::kMaxKeys, 0, st>>>(scratch, nblk, E, offsets);
  if (nblk > 0) nbr::plan_place_kernel<<<nblk, nbr::kPlanBlock, 0, st>>>(ids, n, E, scratch, offsets, order, inv);
  return int(cudaGetLastError());
}

// Packed-attention plan of one block. idx [T, k] int32 columns (T = B * S tokens), pos [T] int32 or null.
// keys / order / inv: int32 [T * k]; seg_start: int32 [G * B + 1]; scratch: int32 [ceil(T * k / 1024) * G * B].
int nb_column_plan(const int* idx, int T, int k, int S, int B, int G, const int* pos, int* keys, int* scratch, int* order,
                   int* inv, int* seg_start, int* tok_of_row, int* slot_of_row, int* pos_of_row, cudaStream_t st) {
  const int n = T * k;
  if (G * B > nbr::kMaxKeys || n <= 0) return -1;
  nbr::column_plan_keys_kernel<<<(n + 255) / 256, 256, 0, st>>>(idx, n, k, S, B, keys);
  int rc = nb_expert_plan(keys, n, G * B, scratch, order, inv, seg_start, st);
  if (rc) return rc;
  nbr::column_plan_finish_kernel<<<(n + 255) / 256, 256, 0, st>>>(order, n, k, pos, S, tok_of_row, slot_of_row, pos_of_row);
  return int(cudaGetLastError());
}

}  // extern "C"
