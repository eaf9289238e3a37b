// Token sampling on the device: repetition penalty, temperature, top-k, top-p and the draw for the rows of a
// step, without reading 600 KB of logits per row back to the host.
//
// The rule is the host sampler's (native/src/spec.h: filter_probs + draw, the role of the reference's
// src/server/spec_accept.cc:16-92 filter and of its host sampler): candidates in descending (logit, then
// ascending id) order, softmax over the top-k at the temperature in double precision, cut after the first
// prefix whose mass reaches top_p (not renormalised), one uniform u from mt19937_64(seed) as (x >> 11) * 2^-53,
// the first candidate whose cumulative mass exceeds u * mass.  A row therefore draws the same token on the
// device as on the host (up to the last bit of a double-precision exp at a boundary).
//
// One CTA of 1024 threads per row:
//   1. bitmap of the history ids (repetition penalty is applied on the fly, once per listed id);
//   2. maximum, and for an uncapped top-k the partition sum over the whole vocabulary (double accumulators,
//      fixed reduction tree);
//   3. radix select (11 + 11 + 10 bits over an order-preserving integer image of the logit) of the C-th
//      largest value, C = min(top_k, 1024);
//   4. compaction of everything >= that value into shared memory as 64-bit keys (value image, inverted id),
//      bitonic sort: the exact order, ties by id;
//   5. probabilities, prefix sums, the top-p cut and the draw.
// When the filtered set cannot be decided inside 1024 candidates (top_k above 1024 but below the vocabulary, a
// flat distribution whose top-p prefix is longer, or more than 2048 values tied at the cut), the row's status
// is 1 and the caller samples that row on the host.
#include "common.cuh"

using namespace b2;

namespace {

constexpr int kSampThreads = 1024;
constexpr int kCand = 1024;    // candidates the top-p cut may span
constexpr int kSort = 2048;    // keys sorted (candidates + ties at the cut)

struct SampleParams {
  const float* logits;   // [M][ld]
  int ld, n_valid;
  const float* temperature;   // [M]  <= 0: greedy
  const int* top_k;           // [M]  0: no cap
  const float* top_p;         // [M]
  const unsigned long long* seed;  // [M]
  const float* penalty;       // [M] or nullptr
  const int* hist;            // [M][hist_cap] ids the penalty applies to, or nullptr
  const int* hist_len;        // [M]
  int hist_cap;
  int* token;    // [M]
  int* status;   // [M] 0: sampled, 1: the host must sample this row
  int* kept;     // [M] size of the filtered set (or nullptr)
};

__device__ __forceinline__ uint32_t key_of(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float float_of(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k ^ 0x80000000u) : ~k);
}

// first output of std::mt19937_64 seeded with `seed` (it depends on words 0, 1 and 156 of the initial state)
__device__ unsigned long long mt64_first(unsigned long long seed) {
  unsigned long long x = seed, s0 = seed, s1 = 0, s156 = 0;
  for (int i = 1; i <= 156; ++i) {
    x = 6364136223846793005ull * (x ^ (x >> 62)) + (unsigned long long)i;
    if (i == 1) s1 = x;
    if (i == 156) s156 = x;
  }
  const unsigned long long y = (s0 & 0xFFFFFFFF80000000ull) | (s1 & 0x7FFFFFFFull);
  unsigned long long v = s156 ^ (y >> 1) ^ ((y & 1ull) ? 0xB5026F5AA96619E9ull : 0ull);
  v ^= (v >> 29) & 0x5555555555555555ull;
  v ^= (v << 17) & 0x71D67FFFEDA60000ull;
  v ^= (v << 37) & 0xFFF7EEE000000000ull;
  v ^= v >> 43;
  return v;
}

__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// block-wide sum of doubles over 1024 threads, fixed tree; `red` holds 32 doubles
__device__ double block_sum_d(double v, double* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum_d(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  double t = red[lane];
  t = warp_sum_d(t);
  return t;
}

}  // namespace

namespace {

__global__ void __launch_bounds__(kSampThreads) sample_rows_kernel(const SampleParams p) {
  extern __shared__ uint8_t sm_raw[];
  uint32_t* hist = reinterpret_cast<uint32_t*>(sm_raw);                                  // 2048 bins; later 1024 doubles
  unsigned long long* keys = reinterpret_cast<unsigned long long*>(sm_raw + 8192);       // kSort keys
  uint32_t* bitmap = reinterpret_cast<uint32_t*>(sm_raw + 8192 + kSort * 8);             // n_valid bits
  __shared__ double red[32];
  __shared__ float redf[32];
  __shared__ uint32_t s_prefix, s_mask, s_remaining, s_cnt;
  __shared__ int s_keep, s_tok;
  pdl_wait();
  pdl_launch_dependents();
  const int m = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* row = p.logits + (size_t)m * p.ld;
  const int V = p.n_valid;
  const float temp = p.temperature[m];
  const bool greedy = !(temp > 0.f);
  const double T = greedy ? 1.0 : (double)temp;
  const int topk = p.top_k[m];
  const int k_eff = (topk <= 0 || topk > V) ? V : topk;
  const bool full = k_eff == V;                 // softmax over the whole vocabulary
  const int C = greedy ? 1 : min(k_eff, kCand);
  const bool capped = !greedy && k_eff > kCand;
  if (capped && !full) {                        // the partition sum of a top-k beyond the candidates is not formed here
    if (tid == 0) {
      p.status[m] = 1;
      p.token[m] = -1;
    }
    return;
  }
  // ---- 1. history bitmap
  const float pen = p.penalty ? p.penalty[m] : 1.f;
  const bool use_pen = p.hist != nullptr && pen != 1.f;
  if (use_pen) {
    for (int i = tid; i < (V + 31) / 32; i += kSampThreads) bitmap[i] = 0u;
    __syncthreads();
    const int n = min(p.hist_len[m], p.hist_cap);
    for (int i = tid; i < n; i += kSampThreads) {
      const int id = p.hist[(size_t)m * p.hist_cap + i];
      if (id >= 0 && id < V) atomicOr(&bitmap[id >> 5], 1u << (id & 31));
    }
    __syncthreads();
  }
  auto lg = [&](int i) -> float {
    float l = row[i];
    if (use_pen && ((bitmap[i >> 5] >> (i & 31)) & 1u)) l = l < 0.f ? l * pen : l / pen;
    return l;
  };
  // ---- 2. maximum; partition sum over the vocabulary when top-k does not cap it
  float mx = -INFINITY;
  for (int i = tid; i < V; i += kSampThreads) mx = fmaxf(mx, lg(i));
  mx = warp_max(mx);
  if (lane == 0) redf[warp] = mx;
  __syncthreads();
  mx = warp_max(redf[lane]);
  double zfull = 0.0;
  if (full && !greedy) {
    double acc = 0.0;
    for (int i = tid; i < V; i += kSampThreads) acc += exp(((double)lg(i) - (double)mx) / T);
    zfull = block_sum_d(acc, red);
  }
  // ---- 3. radix select of the C-th largest value image
  if (tid == 0) {
    s_prefix = 0u;
    s_mask = 0u;
    s_remaining = (uint32_t)C;
  }
#pragma unroll 1
  for (int pass = 0; pass < 3; ++pass) {
    const int shift = pass == 0 ? 21 : (pass == 1 ? 10 : 0);
    const int bits = pass == 2 ? 10 : 11;
    const uint32_t dmask = (1u << bits) - 1u;
    for (int i = tid; i < 2048; i += kSampThreads) hist[i] = 0u;
    __syncthreads();
    const uint32_t prefix = s_prefix, pmask = s_mask;
    for (int i = tid; i < V; i += kSampThreads) {
      const uint32_t k = key_of(lg(i));
      if ((k & pmask) == prefix) atomicAdd(&hist[(k >> shift) & dmask], 1u);
    }
    __syncthreads();
    if (warp == 0) {
      // bins from the top: lane L owns the L-th run of nb / 32 bins below the top one
      const int nb = 1 << bits, per = nb / 32;
      const int hi = nb - 1 - lane * per;
      uint32_t mine = 0;
      for (int j = 0; j < per; ++j) mine += hist[hi - j];
      uint32_t incl = mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      const uint32_t before = incl - mine, need = s_remaining;
      __syncwarp();   // every lane has read the count before the crossing lane replaces it
      if (before < need && need <= incl) {   // the crossing is inside this lane's bins
        uint32_t cum = before;
        for (int j = 0; j < per; ++j) {
          const uint32_t h = hist[hi - j];
          if (cum + h >= need) {
            s_prefix = prefix | ((uint32_t)(hi - j) << shift);
            s_mask = pmask | (dmask << shift);
            s_remaining = need - cum;
            break;
          }
          cum += h;
        }
      }
    }
    __syncthreads();
  }
  const uint32_t tau = s_prefix;
  // ---- 4. everything >= tau as (value image, inverted id), sorted descending
  if (tid == 0) s_cnt = 0u;
  for (int i = tid; i < kSort; i += kSampThreads) keys[i] = 0ull;
  __syncthreads();
  for (int i = tid; i < V; i += kSampThreads) {
    const uint32_t k = key_of(lg(i));
    if (k >= tau) {
      const uint32_t pos = atomicAdd(&s_cnt, 1u);
      if (pos < (uint32_t)kSort) keys[pos] = ((unsigned long long)k << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)i);
    }
  }
  __syncthreads();
  if (s_cnt > (uint32_t)kSort || s_cnt < (uint32_t)C) {   // too many ties at the cut (or a NaN row): the host decides
    if (tid == 0) {
      p.status[m] = 1;
      p.token[m] = -1;
    }
    return;
  }
  for (int k = 2; k <= kSort; k <<= 1)
    for (int j = k >> 1; j > 0; j >>= 1) {
      const int i = 2 * tid - (tid & (j - 1));   // the lower index of this thread's pair
      const int q = i + j;
      const unsigned long long a = keys[i], b = keys[q];
      const bool desc = (i & k) == 0;
      if (desc ? a < b : a > b) {
        keys[i] = b;
        keys[q] = a;
      }
      __syncthreads();
    }
  if (greedy) {
    if (tid == 0) {
      p.token[m] = (int)(0xFFFFFFFFu - (uint32_t)(keys[0] & 0xFFFFFFFFull));
      p.status[m] = 0;
      if (p.kept) p.kept[m] = 1;
    }
    return;
  }
  // ---- 5. probabilities of the C candidates, prefix sums, the top-p cut, the draw
  const float l0 = float_of((uint32_t)(keys[0] >> 32));
  double pi = 0.0;
  if (tid < C) pi = exp(((double)float_of((uint32_t)(keys[tid] >> 32)) - (double)l0) / T);
  const double z = full ? zfull : block_sum_d(pi, red);
  const double qi = pi / z;
  // inclusive scan over the 1024 threads
  double incl = qi;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const double v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  __syncthreads();
  if (lane == 31) red[warp] = incl;
  __syncthreads();
  double wbase = 0.0;
  for (int w = 0; w < warp; ++w) wbase += red[w];
  incl += wbase;
  double* cum = reinterpret_cast<double*>(hist);   // 1024 doubles
  cum[tid] = incl;
  if (tid == 0) s_keep = 0;
  __syncthreads();
  const double tp = (double)p.top_p[m];
  if (tid < C && incl >= tp && (tid == 0 || cum[tid - 1] < tp)) s_keep = tid + 1;
  __syncthreads();
  int n_keep = s_keep;
  if (n_keep == 0) {
    if (capped) {   // the top-p prefix is longer than the candidates
      if (tid == 0) {
        p.status[m] = 1;
        p.token[m] = -1;
      }
      return;
    }
    n_keep = C;     // the top-k set's mass stays below top_p: all of it is kept
  }
  const double mass = cum[n_keep - 1];
  const double u = (double)(mt64_first(p.seed[m]) >> 11) * (1.0 / 9007199254740992.0) * mass;
  if (tid == 0) s_tok = n_keep - 1;
  __syncthreads();
  if (tid < n_keep && u < incl && (tid == 0 || !(u < cum[tid - 1]))) s_tok = tid;
  __syncthreads();
  if (tid == 0) {
    p.token[m] = (int)(0xFFFFFFFFu - (uint32_t)(keys[s_tok] & 0xFFFFFFFFull));
    p.status[m] = 0;
    if (p.kept) p.kept[m] = n_keep;
  }
}

}  // namespace

// Samples one token per row of ``logits`` [M][ld] (ids below n_valid).  hist / hist_len / penalty may be null
// (no repetition penalty).  status[m] = 1 marks a row the caller must sample on the host.
extern "C" int b2_sample_rows(const float* logits, int M, int ld, int n_valid, const float* temperature,
                              const int* top_k, const float* top_p, const unsigned long long* seed,
                              const float* penalty, const int* hist, const int* hist_len, int hist_cap, int* token,
                              int* status, int* kept, void* stream) {
  if (M < 1 || n_valid < 1 || n_valid > ld || n_valid > (1 << 20)) return -1;
  SampleParams p{logits, ld, n_valid, temperature, top_k, top_p, seed, penalty, hist, hist_len, hist_cap, token, status, kept};
  const int smem = 8192 + kSort * 8 + ((n_valid + 31) / 32) * 4 + 16;
  static int configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(sample_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         8192 + kSort * 8 + (1 << 20) / 8 + 16);
    if (e != cudaSuccess) return (int)e;
    configured[dev & 63] = 1;
  }
  return b2_launch(sample_rows_kernel, dim3(M), dim3(kSampThreads), smem, (cudaStream_t)stream, true, p);
}

B2_DEFINE_STATUS(sampler)
