// The block drafter's candidate path: top-K of a (draft-vocabulary) head, exact rerank of the candidates against
// the target's own lm_head rows, and the per-row pick (arg-max, or Gumbel-arg-max with noise keyed by
// (seed, position, token id) so that a replay draws the same drafts).
//
// Roles of the reference's src/kernels/dflash/df_topk.cl (two fixed stages, no atomics), df_rerank.cl (gather the
// candidates' head rows, exact dots, keep the best) and df_select.cl in its per-row form (src/kernels/dflash/
// df_select.cl:1-20; the pairwise "walk" of its second drafter generation needs that drafter's edge tables and is
// not built).  One comparator everywhere: the larger value wins, an equal value goes to the lower id, NaN never
// wins, ids at or above `used` are never candidates; absent candidates are (-inf, kNoIdx).
//
// B200 form: a row of logits (up to ~250k floats = 1 MB) is L2-resident right after the head GEMV wrote it.  The
// top-K is two launches: a warp per ~1k-entry slice keeps its best 16 as a list sorted across its lanes (ballot +
// shuffle-up per insertion), then one CTA per row runs the same routine over the slices' lists.  The rerank is one warp per candidate streaming that head row (bf16, 10 KB at hidden 5120) against the
// drafter's hidden row in shared memory.
#include "common.cuh"

using namespace b2;

namespace {

constexpr int kTopMax = 16;
constexpr unsigned kNoIdx = 0x7fffffffu;
constexpr int kThreads = 1024;     // rerank: 32 warps, one candidate each per round
constexpr int kTopThreads = 256;   // top-K of whole rows: 8 warps

__device__ __forceinline__ bool better(float a, unsigned ai, float b, unsigned bi) {
  // NaN never wins: a comparison with NaN is false, and a NaN `b` loses to any real `a`
  if (a != a) return false;
  if (b != b) return true;
  return a > b || (a == b && ai < bi);
}

struct TopkParams {
  const float* logits;   // [rows][ld]; second stage: the warps' partial values, [rows][n]
  const unsigned* in_ids;   // second stage: the partial entries' indices (nullptr: the position is the index)
  int ld, n, used, k;
  int lists;             // first stage: warps (= partial lists of kTopMax pairs) per row
  const int* id_table;   // draft vocabulary: index -> real id (ascending), or nullptr
  float out_mult, softcap;
  unsigned* cand;        // [rows][k] real ids        (first stage: [rows][lists][kTopMax] indices)
  float* value;          // [rows][k]
};

// the partial lists of one launch pair: rows x lists x kTopMax pairs, part of the library's image so that a call
// allocates nothing (calls on one stream follow one another; two streams must not run the top-K at once)
constexpr int kPartRows = 64, kPartLists = 128;
__device__ float g_part_val[kPartRows * kPartLists * kTopMax];
__device__ unsigned g_part_id[kPartRows * kPartLists * kTopMax];

// A warp's running best-32 of the entries [lo, hi) it scans, kept sorted ACROSS the lanes (lane j holds rank j): a
// batch of 32 entries per load, a ballot of those that beat rank K - 1, and per survivor one ballot (its place), one
// shuffle-up (the ranks behind it move) -- about ten instructions, against the ~150 of a bubble through a private
// register list, and no block-wide round per output.  After warm-up a survivor is rare (K ln(n / K) in n entries).
// `x`/`xi` may point to global or shared memory; an entry whose index is kNoIdx is absent.
__device__ __forceinline__ void warp_topk_scan(const float* x, const unsigned* xi, int lo, int hi, int K, float& lv,
                                               unsigned& li) {
  const int lane = threadIdx.x & 31;
  lv = -INFINITY;
  li = kNoIdx;
  for (int i0 = lo; i0 < hi; i0 += 128) {
    float a4[4];
    unsigned i4[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = i0 + u * 32 + lane;
      a4[u] = i < hi ? x[i] : -INFINITY;
      i4[u] = i < hi ? (xi ? xi[i] : (unsigned)i) : kNoIdx;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float tv = __shfl_sync(0xffffffffu, lv, K - 1);
      const unsigned ti = __shfl_sync(0xffffffffu, li, K - 1);
      unsigned mask = __ballot_sync(0xffffffffu, i4[u] != kNoIdx && better(a4[u], i4[u], tv, ti));
      while (mask) {
        const int src = __ffs(mask) - 1;
        mask &= mask - 1;
        const float cv = __shfl_sync(0xffffffffu, a4[u], src);
        const unsigned ci = __shfl_sync(0xffffffffu, i4[u], src);
        const int pos = __popc(__ballot_sync(0xffffffffu, better(lv, li, cv, ci)));   // the ranks that stay ahead
        const float pv = __shfl_up_sync(0xffffffffu, lv, 1);
        const unsigned pi = __shfl_up_sync(0xffffffffu, li, 1);
        if (lane == pos) {
          lv = cv;
          li = ci;
        } else if (lane > pos) {
          lv = pv;
          li = pi;
        }
      }
    }
  }
}

// first stage: grid (ceil(lists / 4), rows), 128 threads; warp = one slice of the row -> its kTopMax best, raw
__global__ void __launch_bounds__(128) df_topk_part_kernel(const TopkParams p) {
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.y, lane = threadIdx.x & 31, list = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (list >= p.lists) return;
  const int lim = min(p.n, p.used);
  const int per = (lim + p.lists - 1) / p.lists;
  float lv;
  unsigned li;
  warp_topk_scan(p.logits + (size_t)row * p.ld, nullptr, list * per, min(lim, (list + 1) * per), kTopMax, lv, li);
  if (lane < kTopMax) {
    p.value[((size_t)row * p.lists + list) * kTopMax + lane] = lv;
    p.cand[((size_t)row * p.lists + list) * kTopMax + lane] = li;
  }
}

// whole rows (a short row, or the second stage over the partial lists): grid rows, 256 threads = 8 warps over
// eighths of the row, their lists through shared memory, warp 0 over those
__global__ void __launch_bounds__(kTopThreads) df_topk_kernel(const TopkParams p) {
  __shared__ float s_v[kTopThreads / 32 * kTopMax];
  __shared__ unsigned s_i[kTopThreads / 32 * kTopMax];
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned* xi = p.in_ids ? p.in_ids + (size_t)row * p.ld : nullptr;
  const int lim = xi ? p.n : min(p.n, p.used);
  constexpr int W = kTopThreads / 32;
  const int per = (lim + W - 1) / W;
  float lv;
  unsigned li;
  warp_topk_scan(p.logits + (size_t)row * p.ld, xi, warp * per, min(lim, (warp + 1) * per), kTopMax, lv, li);
  if (lane < kTopMax) {
    s_v[warp * kTopMax + lane] = lv;
    s_i[warp * kTopMax + lane] = li;
  }
  __syncthreads();
  if (warp != 0) return;
  warp_topk_scan(s_v, s_i, 0, W * kTopMax, p.k, lv, li);
  if (lane < p.k) {
    float out = lv;
    unsigned real = li;
    if (li == kNoIdx) {
      out = -INFINITY;
    } else {
      out *= p.out_mult;
      if (p.softcap > 0.f) out = p.softcap * tanhf(out / p.softcap);
      if (p.id_table) real = (unsigned)p.id_table[li];
    }
    p.cand[(size_t)row * p.k + lane] = real;
    p.value[(size_t)row * p.k + lane] = out;
  }
}

struct RerankParams {
  const __nv_bfloat16* head;   // [vocab][H] the target's lm_head
  const __nv_bfloat16* x;      // [rows][ldx] hidden rows (already normalised)
  long long ldx;
  int H, used, c, k;
  const unsigned* ids;         // [rows][c] candidates (real ids; kNoIdx: absent)
  unsigned* cand;              // [rows][k]
  float* value;                // [rows][k]
};

// grid rows, 1024 threads = 32 warps; warp w scores candidates w, w + 32, ...
__global__ void __launch_bounds__(kThreads) df_rerank_kernel(const RerankParams p) {
  extern __shared__ float s_x[];            // [H] the row as fp32
  __shared__ float s_score[256];
  __shared__ unsigned s_id[256];
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int i = tid; i < p.H; i += kThreads) s_x[i] = __bfloat162float(p.x[(size_t)row * p.ldx + i]);
  __syncthreads();
  for (int c = warp; c < p.c; c += 32) {
    const unsigned id = p.ids[(size_t)row * p.c + c];
    float a = 0.f;
    if (id < (unsigned)p.used) {
      const uint4* w = reinterpret_cast<const uint4*>(p.head + (size_t)id * p.H);
      for (int j = lane; j < p.H / 8; j += 32) {     // lane-strided 16-byte loads, ascending k per lane
        const uint4 q = w[j];
        const float* xs = s_x + 8 * j;
        a = fmaf(bf16_lo(q.x), xs[0], a); a = fmaf(bf16_hi(q.x), xs[1], a);
        a = fmaf(bf16_lo(q.y), xs[2], a); a = fmaf(bf16_hi(q.y), xs[3], a);
        a = fmaf(bf16_lo(q.z), xs[4], a); a = fmaf(bf16_hi(q.z), xs[5], a);
        a = fmaf(bf16_lo(q.w), xs[6], a); a = fmaf(bf16_hi(q.w), xs[7], a);
      }
      // fixed butterfly: the same bits on every replay
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) a += __shfl_xor_sync(0xffffffffu, a, d);
    } else {
      a = -INFINITY;
    }
    if (lane == 0) {
      s_score[c] = a;
      s_id[c] = id < (unsigned)p.used ? id : kNoIdx;
    }
  }
  __syncthreads();
  // the K best of at most 256 candidates: thread 0 walks them (a few hundred comparisons)
  if (tid == 0) {
    for (int r = 0; r < p.k; ++r) {
      float bv = -INFINITY;
      unsigned bi = kNoIdx;
      int at = -1;
      for (int c = 0; c < p.c; ++c)
        if (s_id[c] != kNoIdx && better(s_score[c], s_id[c], bv, bi)) {
          bv = s_score[c];
          bi = s_id[c];
          at = c;
        }
      p.cand[(size_t)row * p.k + r] = bi;
      p.value[(size_t)row * p.k + r] = bv;
      if (at >= 0) s_id[at] = kNoIdx;
    }
  }
}

// 32-bit finaliser of MurmurHash3 applied to the three key words in turn
__device__ __host__ __forceinline__ unsigned fmix32(unsigned h) {
  h ^= h >> 16;
  h *= 0x85ebca6bu;
  h ^= h >> 13;
  h *= 0xc2b2ae35u;
  h ^= h >> 16;
  return h;
}
__device__ __host__ __forceinline__ unsigned keyed_hash(unsigned seed, unsigned pos, unsigned id) {
  unsigned h = fmix32(seed ^ 0x9e3779b9u);
  h = fmix32(h ^ pos);
  h = fmix32(h ^ id);
  return h;
}

struct SelectParams {
  const unsigned* cand;   // [rows][k]
  const float* score;     // [rows][k]
  int k, rows;
  float temperature;
  unsigned seed;
  const int* ctrl;        // positions of the rows (CTRL_ROW_POS), or nullptr: pos0 + row
  int pos0;
  int* out_ids;           // [rows]
  int* out_chosen;        // [rows] index into the row's candidates
  int* ctrl_tokens;       // optional: ctrl.cur_token[1 + row] = the id (the verify list's draft rows)
};

constexpr int CTRL_ROW_POS = 80, CTRL_CUR_TOKEN = 144;
constexpr unsigned kDraftSalt = 1u << 30;   // keeps the draft noise apart from the target sampler's at the same position

// one warp per row
__global__ void df_select_kernel(const SelectParams p) {
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= p.rows) return;
  float s = -INFINITY;
  unsigned id = kNoIdx;
  if (lane < p.k) {
    id = p.cand[(size_t)row * p.k + lane];
    s = p.score[(size_t)row * p.k + lane];
    if (id == kNoIdx) s = -INFINITY;
    else if (p.temperature > 0.f) {
      const int pos = p.ctrl ? p.ctrl[CTRL_ROW_POS + row] : p.pos0 + row;
      const unsigned h = keyed_hash(p.seed, (unsigned)pos + kDraftSalt, id);
      const float u = ((float)(h >> 8) + 0.5f) * (1.0f / 16777216.0f);   // in (0, 1)
      s = s / p.temperature - logf(-log1pf(-u));
    }
  }
  // arg-max over the lanes; ties: the lower candidate index (the better-ranked candidate)
  float bv = s;
  int bc = lane < p.k && id != kNoIdx ? lane : 0x7fffffff;
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, d);
    const int oc = __shfl_xor_sync(0xffffffffu, bc, d);
    const bool take = (ov == ov) && (oc != 0x7fffffff) && (bc == 0x7fffffff || bv != bv || ov > bv || (ov == bv && oc < bc));
    if (take) {
      bv = ov;
      bc = oc;
    }
  }
  if (lane == 0) {
    const int chosen = bc == 0x7fffffff ? 0 : bc;
    const unsigned tok = p.cand[(size_t)row * p.k + chosen];
    p.out_ids[row] = tok == kNoIdx ? 0 : (int)tok;
    p.out_chosen[row] = chosen;
    if (p.ctrl_tokens) p.ctrl_tokens[CTRL_CUR_TOKEN + 1 + row] = tok == kNoIdx ? 0 : (int)tok;
  }
}

}  // namespace

extern "C" int b2_df_topk(const float* logits, int rows, int ld, int n, int used, int k, const int* id_table, float out_mult,
                          float softcap, unsigned* cand, float* value, void* stream) {
  if (rows < 1 || k < 1 || k > kTopMax || n < 1 || n > ld) return -1;
  TopkParams p;
  p.used = used; p.k = k; p.id_table = id_table; p.out_mult = out_mult; p.softcap = softcap; p.in_ids = nullptr;
  p.lists = 0;
  const int lim = n < used ? n : used;
  int lists = lim / 1024;   // a warp per ~1k entries and more: enough warps to fill the GPU from a handful of rows
  if (lists > kPartLists) lists = kPartLists;
  static float* pvs[64] = {};   // per device: each has its own copy of the arrays
  static unsigned* pis[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  float*& pv = pvs[dev & 63];
  unsigned*& pi = pis[dev & 63];
  if (lists >= 16 && (!pv || !pi)) {
    if (cudaGetSymbolAddress((void**)&pv, g_part_val) != cudaSuccess) return -3;
    if (cudaGetSymbolAddress((void**)&pi, g_part_id) != cudaSuccess) return -3;
  }
  for (int r0 = 0; r0 < rows; r0 += kPartRows) {
    const int nr = rows - r0 < kPartRows ? rows - r0 : kPartRows;
    p.logits = logits + (size_t)r0 * ld; p.ld = ld; p.n = n;
    p.cand = cand + (size_t)r0 * k; p.value = value + (size_t)r0 * k;
    if (lists < 16) {
      int rc = b2_launch(df_topk_kernel, dim3(nr), dim3(kTopThreads), 0, (cudaStream_t)stream, true, p);
      if (rc) return rc;
      continue;
    }
    TopkParams a = p;
    a.lists = lists; a.cand = pi; a.value = pv;
    int rc = b2_launch(df_topk_part_kernel, dim3((lists + 3) / 4, nr), dim3(128), 0, (cudaStream_t)stream, true, a);
    if (rc) return rc;
    TopkParams b = p;
    b.logits = pv; b.in_ids = pi; b.ld = lists * kTopMax; b.n = lists * kTopMax;
    rc = b2_launch(df_topk_kernel, dim3(nr), dim3(kTopThreads), 0, (cudaStream_t)stream, true, b);
    if (rc) return rc;
  }
  return 0;
}

extern "C" int b2_df_rerank(const void* head, const void* x, long long ldx, int rows, int H, int used, const unsigned* ids,
                            int c, int k, unsigned* cand, float* value, void* stream) {
  if (rows < 1 || H % 8 || c < 1 || c > 256 || k < 1 || k > c || k > kTopMax || ldx % 8) return -1;
  RerankParams p;
  p.head = (const __nv_bfloat16*)head; p.x = (const __nv_bfloat16*)x; p.ldx = ldx; p.H = H; p.used = used; p.c = c; p.k = k;
  p.ids = ids; p.cand = cand; p.value = value;
  const size_t smem = (size_t)H * 4;
  static bool configured = false;
  if (smem > 48 * 1024 && !configured) {
    cudaError_t e = cudaFuncSetAttribute(df_rerank_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  if (smem > 160 * 1024) return -2;
  return b2_launch(df_rerank_kernel, dim3(rows), dim3(kThreads), smem, (cudaStream_t)stream, true, p);
}

extern "C" int b2_df_select(const unsigned* cand, const float* score, int rows, int k, float temperature, unsigned seed,
                            const int* ctrl, int pos0, int* out_ids, int* out_chosen, int* ctrl_tokens, void* stream) {
  if (rows < 1 || k < 1 || k > 32) return -1;
  SelectParams p;
  p.cand = cand; p.score = score; p.k = k; p.rows = rows; p.temperature = temperature; p.seed = seed; p.ctrl = ctrl;
  p.pos0 = pos0; p.out_ids = out_ids; p.out_chosen = out_chosen; p.ctrl_tokens = ctrl_tokens;
  return b2_launch(df_select_kernel, dim3((rows + 3) / 4), dim3(128), 0, (cudaStream_t)stream, true, p);
}

// the hash the selector keys its noise with (host twin for tests and for the host sampler)
extern "C" unsigned b2_df_keyed_hash(unsigned seed, unsigned pos, unsigned id) { return keyed_hash(seed, pos, id); }

B2_DEFINE_STATUS(dflash)
