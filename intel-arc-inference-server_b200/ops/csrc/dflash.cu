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
// B200 form: a row of logits (up to ~250k floats = 1 MB) is L2-resident right after the head GEMV wrote it, so the
// top-K is one pass per row: 512 threads keep their own sorted K-lists over a strided slice (registers), then K
// rounds of a block-wide arg-max over the lists' heads (warp shuffles + one shared-memory step) pop the winners in
// order.  The rerank is one warp per candidate streaming that head row (bf16, 10 KB at hidden 5120) against the
// drafter's hidden row in shared memory.
#include "common.cuh"

using namespace b2;

namespace {

constexpr int kTopMax = 16;
constexpr unsigned kNoIdx = 0x7fffffffu;
constexpr int kThreads = 1024;     // rerank: 32 warps, one candidate each per round
constexpr int kTopThreads = 512;   // top-K: the private lists want 32 registers of a thread's 128

__device__ __forceinline__ bool better(float a, unsigned ai, float b, unsigned bi) {
  // NaN never wins: a comparison with NaN is false, and a NaN `b` loses to any real `a`
  if (a != a) return false;
  if (b != b) return true;
  return a > b || (a == b && ai < bi);
}

struct TopkParams {
  const float* logits;   // [rows][ld]
  int ld, n, used, k;
  const int* id_table;   // draft vocabulary: index -> real id (ascending), or nullptr
  float out_mult, softcap;
  unsigned* cand;        // [rows][k] real ids
  float* value;          // [rows][k]
};

// grid rows, 512 threads
__global__ void __launch_bounds__(kTopThreads) df_topk_kernel(const TopkParams p) {
  __shared__ float s_v[32];
  __shared__ unsigned s_i[32];
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* x = p.logits + (size_t)row * p.ld;
  float v[kTopMax];
  unsigned id[kTopMax];
#pragma unroll
  for (int i = 0; i < kTopMax; ++i) {
    v[i] = -INFINITY;
    id[i] = kNoIdx;
  }
  const int lim = min(p.n, p.used);
  for (int i = tid; i < lim; i += kTopThreads) {
    const float a = x[i];
    if (!better(a, (unsigned)i, v[kTopMax - 1], id[kTopMax - 1])) continue;
    // insertion into the sorted private list (K <= 16: a short unrolled bubble, all in registers)
    float cv = a;
    unsigned ci = (unsigned)i;
#pragma unroll
    for (int s = 0; s < kTopMax; ++s) {
      if (better(cv, ci, v[s], id[s])) {
        const float tv = v[s];
        const unsigned ti = id[s];
        v[s] = cv;
        id[s] = ci;
        cv = tv;
        ci = ti;
      }
    }
  }
  // K rounds: the block-wide best of the lists' heads; its owner pops
  for (int r = 0; r < p.k; ++r) {
    float bv = v[0];
    unsigned bi = id[0];
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, d);
      const unsigned oi = __shfl_xor_sync(0xffffffffu, bi, d);
      if (better(ov, oi, bv, bi)) {
        bv = ov;
        bi = oi;
      }
    }
    if (lane == 0) {
      s_v[warp] = bv;
      s_i[warp] = bi;
    }
    __syncthreads();
    if (warp == 0) {
      float wv = lane < kTopThreads / 32 ? s_v[lane] : -INFINITY;
      unsigned wi = lane < kTopThreads / 32 ? s_i[lane] : kNoIdx;
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, wv, d);
        const unsigned oi = __shfl_xor_sync(0xffffffffu, wi, d);
        if (better(ov, oi, wv, wi)) {
          wv = ov;
          wi = oi;
        }
      }
      if (lane == 0) {
        float out = wv;
        unsigned real = wi;
        if (wi != kNoIdx) {
          out *= p.out_mult;
          if (p.softcap > 0.f) out = p.softcap * tanhf(out / p.softcap);
          if (p.id_table) real = (unsigned)p.id_table[wi];
        } else {
          out = -INFINITY;
        }
        p.cand[(size_t)row * p.k + r] = real;
        p.value[(size_t)row * p.k + r] = out;
        s_i[0] = wi;   // the winner's index: its owner pops
      }
    }
    __syncthreads();
    const unsigned win = s_i[0];
    if (win != kNoIdx && id[0] == win) {
#pragma unroll
      for (int s = 0; s + 1 < kTopMax; ++s) {
        v[s] = v[s + 1];
        id[s] = id[s + 1];
      }
      v[kTopMax - 1] = -INFINITY;
      id[kTopMax - 1] = kNoIdx;
    }
    __syncthreads();
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
  p.logits = logits; p.ld = ld; p.n = n; p.used = used; p.k = k; p.id_table = id_table; p.out_mult = out_mult;
  p.softcap = softcap; p.cand = cand; p.value = value;
  return b2_launch(df_topk_kernel, dim3(rows), dim3(kTopThreads), 0, (cudaStream_t)stream, true, p);
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
