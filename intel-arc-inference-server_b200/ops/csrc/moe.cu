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
// One row's routing by a whole warp: softmax over E logits, top-k by repeated arg-max (ties to the lower id), weights
// renormalised over the chosen k.  `stride` >= k entries per row in topk_idx / topk_w.
__device__ __forceinline__ void route_row(const float* __restrict__ lrow, int E, int k, int* __restrict__ idx_out,
                                          float* __restrict__ w_out, int lane) {
  constexpr int PER = 16;  // experts per lane (E <= 512)
  float v[PER];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < E ? __ldcg(lrow + e) : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
  mx = warp_max(mx);
#pragma unroll
  for (int i = 0; i < PER; ++i)
    v[i] = (lane + 32 * i) < E ? __expf(v[i] - mx) : -1.f;  // probabilities (unnormalised); -1 marks "taken / absent"
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
    idx_out[lane] = myid;
    w_out[lane] = myw / wsum;  // softmax normaliser cancels: p_i / sum p_topk
  }
}

__global__ void __launch_bounds__(256) moe_route_kernel(const float* __restrict__ logits, int ld, int T, int E, int k,
                                                        int* __restrict__ topk_idx, float* __restrict__ topk_w) {
  pdl_wait();
  pdl_launch_dependents();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= T) return;
  route_row(logits + (size_t)warp * ld, E, k, topk_idx + (size_t)warp * k, topk_w + (size_t)warp * k, lane);
}

// ---------------------------------------------------------------- decode rows: router logits + routing in one launch
// logits[m][r] = x[m] . W[r] for the R router rows (E experts, then the shared expert's gate row when there is one):
// a warp per router row, eight token rows per pass over the weights.  The CTA that finishes last (a ticket) then
// routes every token row.  With `shared_slot` each row gets one more slot: expert id E (the shared expert, see the
// batched GEMV's alt weights) with weight sigmoid(gate logit), or 1 without a gate row.
struct RouterRowsParams {
  const __nv_bfloat16* w;   // [R][H]
  const __nv_bfloat16* x;   // [M][H]
  float* logits;            // [M][ld]
  int M, R, H, ld, E, k;
  int shared_slot, has_gate;
  int* topk_idx;            // [M][k + shared_slot]
  float* topk_w;
  int* ticket;              // one zeroed word; left zero
};

__global__ void __launch_bounds__(256) moe_router_rows_kernel(const RouterRowsParams p) {
  __shared__ int s_last;
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x * 8 + warp;
  if (r < p.R) {
    const uint4* wr = reinterpret_cast<const uint4*>(p.w + (size_t)r * p.H);
    const int chunks = p.H / 8;                 // 16-byte pieces of a row; a lane takes every 32nd
    for (int m0 = 0; m0 < p.M; m0 += 8) {
      const int mt = min(8, p.M - m0);
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int c0 = lane; c0 < chunks; c0 += 32 * 8) {
        // eight pieces of the router row in flight, then the token rows against them
        uint4 wv[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int c = c0 + 32 * u;
          wv[u] = c < chunks ? __ldg(wr + c) : make_uint4(0, 0, 0, 0);
        }
        for (int mm = 0; mm < mt; ++mm) {
          const uint4* xr = reinterpret_cast<const uint4*>(p.x + (size_t)(m0 + mm) * p.H);
          uint4 xv[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int c = c0 + 32 * u;
            xv[u] = c < chunks ? __ldg(xr + c) : make_uint4(0, 0, 0, 0);
          }
          float a = 0.f, b = 0.f;
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const uint32_t ww[4] = {wv[u].x, wv[u].y, wv[u].z, wv[u].w}, xx[4] = {xv[u].x, xv[u].y, xv[u].z, xv[u].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              a = fmaf(bf16_lo(ww[j]), bf16_lo(xx[j]), a);
              b = fmaf(bf16_hi(ww[j]), bf16_hi(xx[j]), b);
            }
          }
          acc[mm] += a + b;
        }
      }
      for (int mm = 0; mm < mt; ++mm) {
        const float v = warp_sum(acc[mm]);
        if (lane == 0) p.logits[(size_t)(m0 + mm) * p.ld + r] = v;
      }
    }
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int t = atomicAdd(p.ticket, 1);
    s_last = t == (int)gridDim.x - 1;
    if (s_last) *p.ticket = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const int stride = p.k + p.shared_slot;
  for (int m = warp; m < p.M; m += 8) {
    const float* lrow = p.logits + (size_t)m * p.ld;
    route_row(lrow, p.E, p.k, p.topk_idx + (size_t)m * stride, p.topk_w + (size_t)m * stride, lane);
    if (p.shared_slot && lane == 0) {
      p.topk_idx[(size_t)m * stride + p.k] = p.E;
      p.topk_w[(size_t)m * stride + p.k] = p.has_gate ? 1.f / (1.f + __expf(-__ldcg(lrow + p.E))) : 1.f;
    }
  }
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

// ---------------------------------------------------------------- combine (decode rows): a thread per (row, column)
// Folds the split-K slices of the batched expert GEMVs: part is [batch = M * k (+ M shared)][S][H] fp32,
// written as out[0][m][H] fp32 (one slice) for the next residual fold.  Grid (M, H / 256): a thread's k * S loads
// are independent, so the kernel is one memory latency long (one CTA per row looping over the columns took 75 us
// for a 2048-wide row).
__global__ void __launch_bounds__(256) moe_combine_rows_kernel(const float* __restrict__ part, int S, int M, int k, int H,
                                                               const float* __restrict__ topk_w,
                                                               const float* __restrict__ shared_part, int S_sh,
                                                               const float* __restrict__ gate_logit, int gate_ld,
                                                               float* __restrict__ out, __nv_bfloat16* fold_resid,
                                                               float* __restrict__ fold_ssq) {
  __shared__ float s_ss[8];
  pdl_wait();
  pdl_launch_dependents();
  const int m = blockIdx.x;
  float g = 0.f;
  if (shared_part) g = gate_logit ? 1.f / (1.f + __expf(-gate_logit[(size_t)m * gate_ld])) : 1.f;
  const int j = blockIdx.y * blockDim.x + threadIdx.x;
  float acc = 0.f;
  if (j < H) {
    // every load of the row's slots goes out before the first is used (up to 12 slots x 4 slices a pass)
    for (int s0 = 0; s0 < k; s0 += 12) {
      float v[12][4], w[12];
#pragma unroll
      for (int u = 0; u < 12; ++u) {
        const int s = s0 + u;
        w[u] = s < k ? topk_w[m * k + s] : 0.f;
#pragma unroll
        for (int q = 0; q < 4; ++q)
          v[u][q] = (s < k && q < S) ? part[((size_t)(m * k + s) * S + q) * H + j] : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 12; ++u) {
        float t = v[u][0];
#pragma unroll
        for (int q = 1; q < 4; ++q) t += v[u][q];      // slices in order; absent ones add 0
        acc = fmaf(w[u], t, acc);
      }
    }
    if (S > 4) {   // more slices than a pass holds: the rest, slot by slot
      for (int s = 0; s < k; ++s) {
        float t = 0.f;
        for (int q = 4; q < S; ++q) t += part[((size_t)(m * k + s) * S + q) * H + j];
        acc = fmaf(topk_w[m * k + s], t, acc);
      }
    }
    if (shared_part) {
      const float* p = shared_part + (size_t)m * H + j;  // shared expert: [S_sh][M][H]
      float v = 0.f;
      for (int q = 0; q < S_sh; ++q) v += p[(size_t)q * M * H];
      acc = fmaf(g, v, acc);
    }
  }
  if (!fold_resid) {
    if (j < H) out[(size_t)m * H + j] = acc;
    return;
  }
  // Fold form: the row's residual stream takes the sum in place (bf16) and every 128-column block's sum of squares
  // of the ROUNDED values is left for the next layer's fused RMSNorm -- the arithmetic and the order of the four
  // 32-column partial sums are those of the GEMV's fold epilogue.
  float rf = 0.f;
  if (j < H) {
    const __nv_bfloat16 rb = __float2bfloat16(__bfloat162float(fold_resid[(size_t)m * H + j]) + acc);
    fold_resid[(size_t)m * H + j] = rb;
    rf = __bfloat162float(rb);
  }
  const float ss = warp_sum(rf * rf);
  if ((threadIdx.x & 31) == 0) s_ss[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 2) {
    const int nb = blockIdx.y * 2 + threadIdx.x;
    if (nb * 128 < H) {
      const float* q = s_ss + 4 * threadIdx.x;
      fold_ssq[(size_t)m * ((H + 127) / 128) + nb] = ((q[0] + q[1]) + q[2]) + q[3];
    }
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

extern "C" int b2_moe_router_rows(const void* w, const void* x, float* logits, int M, int R, int H, int ld, int E, int k,
                                  int shared_slot, int has_gate, int* topk_idx, float* topk_w, int* ticket,
                                  void* stream) {
  if (E > 512 || k > 32 || k < 1 || H % 8 || M < 1 || R < E + (has_gate ? 1 : 0) || ld < R) return -1;
  RouterRowsParams p{(const __nv_bfloat16*)w, (const __nv_bfloat16*)x, logits, M, R, H, ld, E, k, shared_slot, has_gate,
                     topk_idx, topk_w, ticket};
  return b2_launch(moe_router_rows_kernel, dim3((R + 7) / 8), dim3(256), 0, (cudaStream_t)stream, true, p);
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
                                   void* fold_resid, float* fold_ssq, void* stream) {
  if (fold_resid && (!fold_ssq || H % 128)) return -1;
  return b2_launch(moe_combine_rows_kernel, dim3(M, (H + 255) / 256), dim3(256), 0, (cudaStream_t)stream, true, part, S, M,
                   k, H, topk_w, shared_part, S_sh, gate_logit, gate_ld, out, (__nv_bfloat16*)fold_resid, fold_ssq);
}

B2_DEFINE_STATUS(moe)
