// Mixture-of-experts glue kernels: routing, expert-major sorting with a device-side block table,
// gather, and the weighted combine.
//
//   moe_route     softmax over all experts -> top-k (ties to the lower id) -> renormalise
//   moe_count     per-expert histogram + the rank of every (token, slot) inside its expert
//   moe_plan      prefix over experts padded to 128-row blocks -> block table for the grouped GEMM
//   moe_scatter   (token, slot) -> sorted row; gather of the activation rows in sorted order
//   moe_combine   out = resid + sum_slot w * y[row(token, slot)] + sigmoid(gate) * shared   (fixed slot order)
//
// Same division of labour as the reference's pf_moe_sort_mw.cl / pf_moe.cl / moe.cl (moe_route):
// the host never reads a count; the tile table is padded and the grouped GEMM reads the block
// count on the device.  The rank inside an expert comes from an atomic counter, so the ORDER of
// rows inside an expert varies from run to run, but every row is computed independently of its
// neighbours and the combine adds a token's slots in slot order, so the output bits do not.
#include "common.cuh"

using namespace b2;

namespace {

// ---------------------------------------------------------------- route: one warp per token
// logits fp32 [T][ld], the first E columns are the experts (E <= 512).  topk_idx int32 [T][k], topk_w fp32 [T][k].
__global__ void __launch_bounds__(256) moe_route_kernel(const float* __restrict__ logits, int ld, int T, int E, int k,
                                                        int* __restrict__ topk_idx, float* __restrict__ topk_w) {
  pdl_wait();
  pdl_launch_dependents();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= T) return;
  constexpr int PER = 16;  // experts per lane (E <= 512)
  float v[PER];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < E ? logits[(size_t)warp * ld + e] : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
  mx = warp_max(mx);
  float z = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    v[i] = (lane + 32 * i) < E ? __expf(v[i] - mx) : -1.f;  // probabilities (unnormalised); -1 marks "taken / absent"
    if (v[i] > 0.f) z += v[i];
  }
  z = warp_sum(z);
  float wsum = 0.f;
  float myw = 0.f;
  int myid = 0;
  for (int r = 0; r < k; ++r) {
    // arg-max over the remaining experts; ties resolve to the lower id
    float bv = -1.f;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = lane + 32 * i;
      if (v[i] > bv) { bv = v[i]; bi = e; }  // e ascends with i inside a lane: the first maximum is the lowest id
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((bi & 31) == lane) v[bi >> 5] = -1.f;
    wsum += bv;
    if (lane == r) { myw = bv; myid = bi; }
  }
  if (lane < k) {
    topk_idx[(size_t)warp * k + lane] = myid;
    topk_w[(size_t)warp * k + lane] = myw / wsum;  // softmax normaliser cancels: p_i / sum p_topk
  }
  (void)z;
}

// ---------------------------------------------------------------- count + rank
__global__ void moe_count_kernel(const int* __restrict__ topk_idx, int n, int* __restrict__ counts,
                                 int* __restrict__ rank) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) rank[i] = atomicAdd(&counts[topk_idx[i]], 1);
}

// ---------------------------------------------------------------- plan: one CTA, E <= 1024
// expert_base[e] = first sorted row of expert e (a multiple of 128); block table of 128-row blocks.
__global__ void __launch_bounds__(1024) moe_plan_kernel(const int* __restrict__ counts, int E, int max_blk,
                                                        int* __restrict__ expert_base, int* __restrict__ blk_expert,
                                                        int* __restrict__ blk_row0, int* __restrict__ blk_rows,
                                                        int* __restrict__ n_blk, int* __restrict__ total_rows) {
  __shared__ int s_blocks[1024];
  __shared__ int s_scan[1024];
  const int e = threadIdx.x;
  const int c = e < E ? counts[e] : 0;
  const int nb = (c + 127) >> 7;
  s_blocks[e] = nb;
  s_scan[e] = nb;
  __syncthreads();
  for (int o = 1; o < 1024; o <<= 1) {  // inclusive scan (Hillis-Steele)
    const int v = e >= o ? s_scan[e - o] : 0;
    __syncthreads();
    s_scan[e] += v;
    __syncthreads();
  }
  const int first = s_scan[e] - nb;  // exclusive
  if (e < E) {
    expert_base[e] = first * 128;
    for (int j = 0; j < nb && first + j < max_blk; ++j) {
      blk_expert[first + j] = e;
      blk_row0[first + j] = (first + j) * 128;
      blk_rows[first + j] = min(128, c - j * 128);
    }
  }
  if (e == 1023) {
    *n_blk = min(s_scan[1023], max_blk);
    *total_rows = s_scan[1023] * 128;
  }
}

// ---------------------------------------------------------------- scatter + gather
// One CTA per (token, slot): writes the inverse map and copies the token's activation row to its
// sorted position.
__global__ void __launch_bounds__(256) moe_scatter_kernel(const int* __restrict__ topk_idx, const int* __restrict__ rank,
                                                          const int* __restrict__ expert_base, int k,
                                                          const __nv_bfloat16* __restrict__ x, int H,
                                                          int* __restrict__ row_of, __nv_bfloat16* __restrict__ xs) {
  const int i = blockIdx.x;  // token * k + slot
  const int token = i / k;
  const int pos = expert_base[topk_idx[i]] + rank[i];
  if (threadIdx.x == 0) row_of[i] = pos;
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)token * H);
  uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)pos * H);
  for (int j = threadIdx.x; j < H / 8; j += blockDim.x) dst[j] = src[j];
}

// ---------------------------------------------------------------- combine (prefill): one CTA per token
// out[token] = resid[token] + sum_slot w[slot] * y[row_of[token][slot]] + sigmoid(gate_logit[token]) * shared[token]
__global__ void __launch_bounds__(256) moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ row_of,
                                                          const float* __restrict__ topk_w, int k, int H,
                                                          const __nv_bfloat16* __restrict__ shared_y,
                                                          const float* __restrict__ gate_logit, int gate_ld,
                                                          const __nv_bfloat16* __restrict__ resid,
                                                          __nv_bfloat16* __restrict__ out) {
  const int token = blockIdx.x;
  float g = 0.f;
  if (shared_y) g = gate_logit ? 1.f / (1.f + __expf(-gate_logit[(size_t)token * gate_ld])) : 1.f;
  for (int j = threadIdx.x; j < H / 2; j += blockDim.x) {
    float2 acc = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(resid + (size_t)token * H)[j]);
    for (int s = 0; s < k; ++s) {
      const int row = row_of[token * k + s];
      const float w = topk_w[token * k + s];
      const float2 v = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(y + (size_t)row * H)[j]);
      acc.x = fmaf(w, v.x, acc.x);
      acc.y = fmaf(w, v.y, acc.y);
    }
    if (shared_y) {
      const float2 v = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(shared_y + (size_t)token * H)[j]);
      acc.x = fmaf(g, v.x, acc.x);
      acc.y = fmaf(g, v.y, acc.y);
    }
    reinterpret_cast<__nv_bfloat162*>(out + (size_t)token * H)[j] = __floats2bfloat162_rn(acc.x, acc.y);
  }
}

// ---------------------------------------------------------------- combine (decode rows): one CTA per row
// Folds the split-K slices of the batched expert GEMVs: part is [batch = M * k (+ M shared)][S][H] fp32,
// written as out[0][m][H] fp32 (one slice) for the next residual fold.
__global__ void __launch_bounds__(256) moe_combine_rows_kernel(const float* __restrict__ part, int S, int M, int k, int H,
                                                               const float* __restrict__ topk_w,
                                                               const float* __restrict__ shared_part, int S_sh,
                                                               const float* __restrict__ gate_logit, int gate_ld,
                                                               float* __restrict__ out) {
  pdl_wait();
  pdl_launch_dependents();
  const int m = blockIdx.x;
  float g = 0.f;
  if (shared_part) g = gate_logit ? 1.f / (1.f + __expf(-gate_logit[(size_t)m * gate_ld])) : 1.f;
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < k; ++s) {
      const float* p = part + ((size_t)(m * k + s) * S) * H + j;
      float v = 0.f;
      for (int q = 0; q < S; ++q) v += p[(size_t)q * H];
      acc = fmaf(topk_w[m * k + s], v, acc);
    }
    if (shared_part) {
      const float* p = shared_part + (size_t)m * H + j;  // shared expert: [S_sh][M][H]
      float v = 0.f;
      for (int q = 0; q < S_sh; ++q) v += p[(size_t)q * M * H];
      acc = fmaf(g, v, acc);
    }
    out[(size_t)m * H + j] = acc;
  }
}

}  // namespace

extern "C" int b2_moe_route(const float* logits, int ld, int T, int E, int k, int* topk_idx, float* topk_w,
                            void* stream) {
  if (E > 512 || k > 32 || k < 1) return -1;
  const int blocks = (T * 32 + 255) / 256;
  return b2_launch(moe_route_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, true, logits, ld, T, E, k,
                   topk_idx, topk_w);
}

// counts must hold E zeros on entry (the caller clears it on the stream).
extern "C" int b2_moe_sort(const int* topk_idx, int T, int k, int E, int max_blk, int* counts, int* rank,
                           int* expert_base, int* blk_expert, int* blk_row0, int* blk_rows, int* n_blk,
                           int* total_rows, void* stream) {
  if (E > 1024) return -1;
  cudaStream_t st = (cudaStream_t)stream;
  const int n = T * k;
  moe_count_kernel<<<(n + 255) / 256, 256, 0, st>>>(topk_idx, n, counts, rank);
  moe_plan_kernel<<<1, 1024, 0, st>>>(counts, E, max_blk, expert_base, blk_expert, blk_row0, blk_rows, n_blk, total_rows);
  return (int)cudaGetLastError();
}

// histogram + rank only (the expert-parallel plan needs every rank's counts before it can lay rows out)
extern "C" int b2_moe_count(const int* topk_idx, int n, int* counts, int* rank, void* stream) {
  moe_count_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(topk_idx, n, counts, rank);
  return (int)cudaGetLastError();
}

extern "C" int b2_moe_scatter(const int* topk_idx, const int* rank, const int* expert_base, int T, int k, const void* x,
                              int H, int* row_of, void* xs, void* stream) {
  if (H % 8) return -1;
  moe_scatter_kernel<<<T * k, 256, 0, (cudaStream_t)stream>>>(topk_idx, rank, expert_base, k, (const __nv_bfloat16*)x, H,
                                                                row_of, (__nv_bfloat16*)xs);
  return (int)cudaGetLastError();
}

extern "C" int b2_moe_combine(const void* y, const int* row_of, const float* topk_w, int T, int k, int H,
                              const void* shared_y, const float* gate_logit, int gate_ld, const void* resid, void* out,
                              void* stream) {
  if (H % 2) return -1;
  moe_combine_kernel<<<T, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)y, row_of, topk_w, k, H,
                                                           (const __nv_bfloat16*)shared_y, gate_logit, gate_ld,
                                                           (const __nv_bfloat16*)resid, (__nv_bfloat16*)out);
  return (int)cudaGetLastError();
}

extern "C" int b2_moe_combine_rows(const float* part, int S, int M, int k, int H, const float* topk_w,
                                   const float* shared_part, int S_sh, const float* gate_logit, int gate_ld, float* out,
                                   void* stream) {
  return b2_launch(moe_combine_rows_kernel, dim3(M), dim3(256), 0, (cudaStream_t)stream, true, part, S, M, k, H, topk_w,
                   shared_part, S_sh, gate_logit, gate_ld, out);
}

B2_DEFINE_STATUS(moe)
