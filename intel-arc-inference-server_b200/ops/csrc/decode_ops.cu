// Element-wise and reduction kernels of the decode / verify step.
//
//   resid_norm      split-K fold + residual add + RMSNorm (or embedding gather + RMSNorm)
//   rope_append     split-K fold of qkv + rotate-half RoPE + paged KV append (bf16 or int8)
//   attn_decode     paged split-KV flash-decode for M rows (GQA packed per KV head)
//   attn_merge      merge of the split partials -> bf16 attention output
//   gemv_bf16       bf16 weight GEMV (lm_head, router), logits + per-CTA arg-max candidates
//   gemv_i8         int8 weight GEMV with one fp32 scale per row (int8 lm_head)
//   argmax_finish   deterministic arg-max (ties -> lower id) + control-block advance
//
// They stand where the reference has prep.cl, embed_gather.cl, attn.cl (attn_prep),
// attn_v2.cl, gemv_bf16.cl, gemv_i8w.cl and argmax.cl.  All of them read the row
// table of the device-resident control block, so a captured CUDA graph replays
// without host writes (the reference's central idea: docs/04-architecture.md:214-228).
#include "common.cuh"

using namespace b2;

namespace {

// Control block (int32 words), shared by host and device.
constexpr int CTRL_N_ROWS = 0;
constexpr int CTRL_ROW_REQ = 16;     // [64] request slot of each row
constexpr int CTRL_ROW_POS = 80;     // [64] absolute position of each row
constexpr int CTRL_CUR_TOKEN = 144;  // [64] input token of each row
constexpr int CTRL_OUT_TOKEN = 208;  // [64] arg-max of each row
constexpr int CTRL_OUT_VALUE = 272;  // [64] its logit (float bits)
constexpr int CTRL_WORDS = 512;

// ------------------------------------------------------------------ resid_norm
// One CTA per row.  mode 0: r = embed[cur_token[m]];  mode 1: r = resid_in + sum_s part[s].
// resid_out = bf16(r);  x_out = bf16(resid_out * rsqrt(mean(resid_out^2) + eps) * w).
struct ResidNormParams {
  const __nv_bfloat16* embed;
  const int* ctrl;
  const __nv_bfloat16* resid_in;
  const float* part;
  long long part_slice;
  int S, H, mode, vocab;
  const float* w;
  float eps;
  __nv_bfloat16* resid_out;
  __nv_bfloat16* x_out;
  int* flag;
};

// blockDim = H/8 rounded up to a warp (at most 1024): each thread owns 8 consecutive elements per
// pass, and the S slice loads of a pass are independent, so they are all in flight together.
__global__ void __launch_bounds__(1024) resid_norm_kernel(const ResidNormParams p) {
  extern __shared__ float vals[];
  __shared__ float red[32];
  pdl_wait();
  pdl_launch_dependents();
  const int m = blockIdx.x, tid = threadIdx.x, nthr = blockDim.x;
  const int H8 = p.H >> 3;
  float ss = 0.f;
  const uint4* src;
  if (p.mode == 0) {
    int tok = p.ctrl[CTRL_CUR_TOKEN + m];
    if (tok < 0 || tok >= p.vocab) {  // out-of-vocabulary id: flag it, read row 0
      if (tid == 0 && p.flag) atomicExch(p.flag, 0xDEAD0001);
      tok = 0;
    }
    src = reinterpret_cast<const uint4*>(p.embed + (size_t)tok * p.H);
  } else {
    src = reinterpret_cast<const uint4*>(p.resid_in + (size_t)m * p.H);
  }
  for (int i = tid; i < H8; i += nthr) {
    const uint4 rv = src[i];
    float v[8] = {bf16_lo(rv.x), bf16_hi(rv.x), bf16_lo(rv.y), bf16_hi(rv.y),
                  bf16_lo(rv.z), bf16_hi(rv.z), bf16_lo(rv.w), bf16_hi(rv.w)};
    if (p.mode == 1) {
      const float* pp = p.part + (size_t)m * p.H + 8 * i;
#pragma unroll 4
      for (int s = 0; s < p.S; ++s) {
        const float4 a0 = *reinterpret_cast<const float4*>(pp + (size_t)s * p.part_slice);
        const float4 a1 = *reinterpret_cast<const float4*>(pp + (size_t)s * p.part_slice + 4);
        v[0] += a0.x; v[1] += a0.y; v[2] += a0.z; v[3] += a0.w;
        v[4] += a1.x; v[5] += a1.y; v[6] += a1.z; v[7] += a1.w;
      }
    }
    uint4 o;
    o.x = pack_bf16(v[0], v[1]); o.y = pack_bf16(v[2], v[3]); o.z = pack_bf16(v[4], v[5]); o.w = pack_bf16(v[6], v[7]);
    reinterpret_cast<uint4*>(p.resid_out + (size_t)m * p.H)[i] = o;
    const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float f0 = bf16_lo(ow[j]), f1 = bf16_hi(ow[j]);
      vals[8 * i + 2 * j] = f0;
      vals[8 * i + 2 * j + 1] = f1;
      ss += f0 * f0 + f1 * f1;
    }
  }
  ss = warp_sum(ss);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < (nthr >> 5); ++i) tot += red[i];
  const float rinv = rsqrtf(tot / (float)p.H + p.eps);
  if (p.x_out) {
    for (int i = tid; i < H8; i += nthr) {
      const float4 w0 = *reinterpret_cast<const float4*>(p.w + 8 * i), w1 = *reinterpret_cast<const float4*>(p.w + 8 * i + 4);
      const float* vv = vals + 8 * i;
      uint4 o;
      o.x = pack_bf16(vv[0] * rinv * w0.x, vv[1] * rinv * w0.y);
      o.y = pack_bf16(vv[2] * rinv * w0.z, vv[3] * rinv * w0.w);
      o.z = pack_bf16(vv[4] * rinv * w1.x, vv[5] * rinv * w1.y);
      o.w = pack_bf16(vv[6] * rinv * w1.z, vv[7] * rinv * w1.w);
      reinterpret_cast<uint4*>(p.x_out + (size_t)m * p.H)[i] = o;
    }
  }
}

// ------------------------------------------------------------------ draft-head front
// One CTA per row: xcat[m] = [ RMSNorm(embed[cur_token[m]]) * w_e  |  RMSNorm(hidden[m]) * w_h ]  (bf16, 2 H wide),
// the input of a draft head's fc projection (the reference's pf_mtp_front: src/kernels/prefill/pf_mtp_front.cl).
// The token comes from the control block, so a captured draft step chains on the token the step before it left there.
__global__ void __launch_bounds__(1024) draft_front_kernel(const __nv_bfloat16* embed, const int* ctrl, int vocab,
                                                           const __nv_bfloat16* hidden, long long hidden_ld,
                                                           const float* w_e, const float* w_h, float eps, int H,
                                                           __nv_bfloat16* xcat, int* flag) {
  extern __shared__ float vals[];   // [2][H]
  __shared__ float red[2][32];
  pdl_wait();
  pdl_launch_dependents();
  const int m = blockIdx.x, tid = threadIdx.x, nthr = blockDim.x, H8 = H >> 3;
  int tok = ctrl[CTRL_CUR_TOKEN + m];
  if (tok < 0 || tok >= vocab) {
    if (tid == 0 && flag) atomicExch(flag, 0xDEAD0001);
    tok = 0;
  }
  const uint4* src[2] = {reinterpret_cast<const uint4*>(embed + (size_t)tok * H),
                         reinterpret_cast<const uint4*>(hidden + (size_t)m * hidden_ld)};
  float ss[2] = {0.f, 0.f};
  for (int i = tid; i < H8; i += nthr)
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      const uint4 rv = src[which][i];
      const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float f0 = bf16_lo(rw[j]), f1 = bf16_hi(rw[j]);
        vals[which * H + 8 * i + 2 * j] = f0;
        vals[which * H + 8 * i + 2 * j + 1] = f1;
        ss[which] += f0 * f0 + f1 * f1;
      }
    }
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    ss[which] = warp_sum(ss[which]);
    if ((tid & 31) == 0) red[which][tid >> 5] = ss[which];
  }
  __syncthreads();
  float rinv[2];
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    float tot = 0.f;
    for (int i = 0; i < (nthr >> 5); ++i) tot += red[which][i];
    rinv[which] = rsqrtf(tot / (float)H + eps);
  }
  for (int i = tid; i < H8; i += nthr)
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      const float* w = (which ? w_h : w_e) + 8 * i;
      const float* vv = vals + which * H + 8 * i;
      uint4 o;
      o.x = pack_bf16(vv[0] * rinv[which] * w[0], vv[1] * rinv[which] * w[1]);
      o.y = pack_bf16(vv[2] * rinv[which] * w[2], vv[3] * rinv[which] * w[3]);
      o.z = pack_bf16(vv[4] * rinv[which] * w[4], vv[5] * rinv[which] * w[5]);
      o.w = pack_bf16(vv[6] * rinv[which] * w[6], vv[7] * rinv[which] * w[7]);
      reinterpret_cast<uint4*>(xcat + (size_t)m * 2 * H + (size_t)which * H)[i] = o;
    }
}

// ------------------------------------------------------------------ rope_append
// One CTA per row.  Folds the qkv split-K slices, applies rotate-half RoPE to q and k,
// writes q (bf16 [M][q_dim]) and appends k, v to the paged cache at the row's position.
// Cache layout per layer: [page][kv_head][16][D] (bf16), or int8 with one fp32 scale
// per (page, kv_head, slot) stored in a side array [page][kv_head][16].
struct RopeParams {
  const float* qkv;
  long long slice;
  int S;
  const int* ctrl;
  const int* block_table;
  int max_blocks;
  const float* cos_t;  // [max_pos][D/2]
  const float* sin_t;
  int n_q, n_kv, D;
  __nv_bfloat16* q_out;
  void* k_cache;
  void* v_cache;
  float* k_scale;
  float* v_scale;
  int kv_int8;
  int req, pos0;  // used when ctrl == nullptr: row m of request `req` sits at position pos0 + m
};

__global__ void __launch_bounds__(256) rope_append_kernel(const RopeParams p) {
  pdl_wait();
  pdl_launch_dependents();
  const int m = blockIdx.x;
  const int req = p.ctrl ? p.ctrl[CTRL_ROW_REQ + m] : p.req, pos = p.ctrl ? p.ctrl[CTRL_ROW_POS + m] : p.pos0 + m;
  const int D = p.D, Dh = D >> 1;
  const int q_dim = p.n_q * D, kv_dim = p.n_kv * D, ld = q_dim + 2 * kv_dim;
  const float* row = p.qkv + (size_t)m * ld;
  const int page = p.block_table[(size_t)req * p.max_blocks + (pos >> 4)], slot = pos & 15;
  const int n_pairs = (p.n_q + p.n_kv) * Dh;
  if (!p.kv_int8) {
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < n_pairs + kv_dim / 2; i += gridDim.y * blockDim.x) {
      if (i < n_pairs) {
        const int head = i / Dh, j = i % Dh;
        const int c0 = head * D + j;
        float x1 = 0.f, x2 = 0.f;
        _Pragma("unroll 4") for (int s = 0; s < p.S; ++s) {
          x1 += row[(size_t)s * p.slice + c0];
          x2 += row[(size_t)s * p.slice + c0 + Dh];
        }
        const float c = p.cos_t[(size_t)pos * Dh + j], sn = p.sin_t[(size_t)pos * Dh + j];
        const float y1 = x1 * c - x2 * sn, y2 = x2 * c + x1 * sn;
        if (head < p.n_q) {
          p.q_out[(size_t)m * q_dim + c0] = __float2bfloat16(y1);
          p.q_out[(size_t)m * q_dim + c0 + Dh] = __float2bfloat16(y2);
        } else {
          const int kh = head - p.n_q;
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.k_cache) + (((size_t)page * p.n_kv + kh) * 16 + slot) * D;
          dst[j] = __float2bfloat16(y1);
          dst[j + Dh] = __float2bfloat16(y2);
        }
      } else {
        const int e = (i - n_pairs) * 2;  // v element pair
        const int kh = e / D, j = e % D;
        float v0 = 0.f, v1 = 0.f;
        _Pragma("unroll 4") for (int s = 0; s < p.S; ++s) {
          v0 += row[(size_t)s * p.slice + q_dim + kv_dim + e];
          v1 += row[(size_t)s * p.slice + q_dim + kv_dim + e + 1];
        }
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.v_cache) + (((size_t)page * p.n_kv + kh) * 16 + slot) * D;
        *reinterpret_cast<__nv_bfloat162*>(dst + j) = __floats2bfloat162_rn(v0, v1);
      }
    }
  } else {
    // int8 KV: one warp per (k|v, kv head); per-(token, head) scale = max|x| / 127.
    // q is written first by all threads.
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < p.n_q * Dh; i += gridDim.y * blockDim.x) {
      const int head = i / Dh, j = i % Dh, c0 = head * D + j;
      float x1 = 0.f, x2 = 0.f;
      _Pragma("unroll 4") for (int s = 0; s < p.S; ++s) {
        x1 += row[(size_t)s * p.slice + c0];
        x2 += row[(size_t)s * p.slice + c0 + Dh];
      }
      const float c = p.cos_t[(size_t)pos * Dh + j], sn = p.sin_t[(size_t)pos * Dh + j];
      p.q_out[(size_t)m * q_dim + c0] = __float2bfloat16(x1 * c - x2 * sn);
      p.q_out[(size_t)m * q_dim + c0 + Dh] = __float2bfloat16(x2 * c + x1 * sn);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int job = blockIdx.y * nw + warp; job < 2 * p.n_kv; job += gridDim.y * nw) {
      const bool is_v = job >= p.n_kv;
      const int kh = is_v ? job - p.n_kv : job;
      // each lane holds D/32 elements (pairs j and j + D/2 for k so the rotation stays in-lane)
      float vals[8];
      const int per = D / 32;  // 2 or 4 (D = 64 / 128); up to 8 for D = 256
      float amax = 0.f;
      if (!is_v) {
        for (int u = 0; u < per / 2; ++u) {
          const int j = lane * (per / 2) + u;
          const int c0 = q_dim + kh * D + j;
          float x1 = 0.f, x2 = 0.f;
          _Pragma("unroll 4") for (int s = 0; s < p.S; ++s) {
            x1 += row[(size_t)s * p.slice + c0];
            x2 += row[(size_t)s * p.slice + c0 + Dh];
          }
          const float c = p.cos_t[(size_t)pos * Dh + j], sn = p.sin_t[(size_t)pos * Dh + j];
          vals[2 * u] = x1 * c - x2 * sn;
          vals[2 * u + 1] = x2 * c + x1 * sn;
        }
      } else {
        for (int u = 0; u < per; ++u) {
          const int e = q_dim + kv_dim + kh * D + lane * per + u;
          float v = 0.f;
          _Pragma("unroll 4") for (int s = 0; s < p.S; ++s) v += row[(size_t)s * p.slice + e];
          vals[u] = v;
        }
      }
      for (int u = 0; u < per; ++u) amax = fmaxf(amax, fabsf(vals[u]));
      amax = warp_max(amax);
      const float sc = amax > 0.f ? amax / 127.f : 1.f, inv = 1.f / sc;
      int8_t* base = reinterpret_cast<int8_t*>(is_v ? p.v_cache : p.k_cache) + (((size_t)page * p.n_kv + kh) * 16 + slot) * D;
      if (!is_v) {
        for (int u = 0; u < per / 2; ++u) {
          const int j = lane * (per / 2) + u;
          base[j] = (int8_t)__float2int_rn(vals[2 * u] * inv);
          base[j + Dh] = (int8_t)__float2int_rn(vals[2 * u + 1] * inv);
        }
      } else {
        for (int u = 0; u < per; ++u) base[lane * per + u] = (int8_t)__float2int_rn(vals[u] * inv);
      }
      if (lane == 0) (is_v ? p.v_scale : p.k_scale)[((size_t)page * p.n_kv + kh) * 16 + slot] = sc;
    }
  }
}

// ------------------------------------------------------------------ attn_decode
// grid (n_kv, nsplit, M), 256 threads.  Each warp takes keys strided by 8 inside the
// CTA's page range, four keys per iteration; each lane owns D/32 dims of q, k, v for
// all GQA query heads of the KV head, so K and V rows are read once per group of heads.
struct AttnDecParams {
  const __nv_bfloat16* q;  // [M][n_q*D]
  const void* k_cache;
  const void* v_cache;
  const float* k_scale;
  const float* v_scale;
  const int* block_table;
  const int* ctrl;
  float* o_part;   // [M][n_q][nsplit][D]
  float* ml_part;  // [M][n_q][nsplit][2]
  int n_q, n_kv, nsplit, max_blocks;
  float scale_log2;  // softmax scale * log2(e)
  int kv_int8;
  int* tickets;          // [M][n_kv] zeroed counters: the last split CTA of a (row, KV head) merges in-kernel
  __nv_bfloat16* out;    // [M][n_q*D], written by the merging CTA when tickets != nullptr
};

template <int D, int GQA>
__global__ void __launch_bounds__(256) attn_decode_kernel(const AttnDecParams p) {
  constexpr int DL = D / 32;
  constexpr int KPI = 4;  // keys per iteration per warp (8 row loads per lane in flight; more costs a resident CTA)
  __shared__ int sm_last;
  __shared__ float sm_o[8][GQA][D];
  __shared__ float sm_ml[8][GQA][2];
  pdl_wait();
  pdl_launch_dependents();
  const int kh = blockIdx.x, split = blockIdx.y, m = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int req = p.ctrl[CTRL_ROW_REQ + m], ctx = p.ctrl[CTRL_ROW_POS + m] + 1;
  const int total_pages = (ctx + 15) >> 4;
  const int pps = (total_pages + p.nsplit - 1) / p.nsplit;
  const int key0 = split * pps * 16, key1 = min(ctx, (split + 1) * pps * 16);

  float qv[GQA][DL];
#pragma unroll
  for (int h = 0; h < GQA; ++h) {
    const __nv_bfloat16* qp = p.q + (size_t)m * p.n_q * D + (size_t)(kh * GQA + h) * D + lane * DL;
#pragma unroll
    for (int d = 0; d < DL; ++d) qv[h][d] = __bfloat162float(qp[d]) * p.scale_log2;
  }
  float mx[GQA], l[GQA], acc[GQA][DL];
#pragma unroll
  for (int h = 0; h < GQA; ++h) {
    mx[h] = -INFINITY;
    l[h] = 0.f;
#pragma unroll
    for (int d = 0; d < DL; ++d) acc[h][d] = 0.f;
  }
  const int* bt = p.block_table + (size_t)req * p.max_blocks;

  for (int kb = key0 + warp * KPI; kb < key1; kb += 8 * KPI) {
    float kf[KPI][DL], vf[KPI][DL];
    bool valid[KPI];
#pragma unroll
    for (int u = 0; u < KPI; ++u) {
      const int key = kb + u;
      valid[u] = key < key1;
      const int kk = valid[u] ? key : key0;
      const int page = bt[kk >> 4], slot = kk & 15;
      const size_t off = (((size_t)page * p.n_kv + kh) * 16 + slot);
      if (!p.kv_int8) {
        const __nv_bfloat16* kp = reinterpret_cast<const __nv_bfloat16*>(p.k_cache) + off * D + lane * DL;
        const __nv_bfloat16* vp = reinterpret_cast<const __nv_bfloat16*>(p.v_cache) + off * D + lane * DL;
        if constexpr (DL == 4) {
          const uint2 kr = *reinterpret_cast<const uint2*>(kp), vr = *reinterpret_cast<const uint2*>(vp);
          kf[u][0] = bf16_lo(kr.x); kf[u][1] = bf16_hi(kr.x); kf[u][2] = bf16_lo(kr.y); kf[u][3] = bf16_hi(kr.y);
          vf[u][0] = bf16_lo(vr.x); vf[u][1] = bf16_hi(vr.x); vf[u][2] = bf16_lo(vr.y); vf[u][3] = bf16_hi(vr.y);
        } else {
#pragma unroll
          for (int d = 0; d < DL; ++d) {
            kf[u][d] = __bfloat162float(kp[d]);
            vf[u][d] = __bfloat162float(vp[d]);
          }
        }
      } else {
        const int8_t* kp = reinterpret_cast<const int8_t*>(p.k_cache) + off * D + lane * DL;
        const int8_t* vp = reinterpret_cast<const int8_t*>(p.v_cache) + off * D + lane * DL;
        const float ks = p.k_scale[off], vs = p.v_scale[off];
#pragma unroll
        for (int d = 0; d < DL; ++d) {
          kf[u][d] = (float)kp[d] * ks;
          vf[u][d] = (float)vp[d] * vs;
        }
      }
    }
    float s[GQA][KPI];
#pragma unroll
    for (int h = 0; h < GQA; ++h)
#pragma unroll
      for (int u = 0; u < KPI; ++u) {
        float d0 = 0.f;
#pragma unroll
        for (int d = 0; d < DL; ++d) d0 = fmaf(qv[h][d], kf[u][d], d0);
        d0 = warp_sum(d0);
        s[h][u] = valid[u] ? d0 : -INFINITY;
      }
#pragma unroll
    for (int h = 0; h < GQA; ++h) {
      float mn = mx[h];
#pragma unroll
      for (int u = 0; u < KPI; ++u) mn = fmaxf(mn, s[h][u]);
      const float corr = exp2f(mx[h] - mn);  // mx = -inf on first pass -> 0
      l[h] *= corr;
#pragma unroll
      for (int d = 0; d < DL; ++d) acc[h][d] *= corr;
#pragma unroll
      for (int u = 0; u < KPI; ++u) {
        const float pe = exp2f(s[h][u] - mn);
        l[h] += pe;
#pragma unroll
        for (int d = 0; d < DL; ++d) acc[h][d] = fmaf(pe, vf[u][d], acc[h][d]);
      }
      mx[h] = mn;
    }
  }
  // ---- merge the 8 warps in a fixed order
#pragma unroll
  for (int h = 0; h < GQA; ++h) {
#pragma unroll
    for (int d = 0; d < DL; ++d) sm_o[warp][h][lane * DL + d] = acc[h][d];
    if (lane == 0) {
      sm_ml[warp][h][0] = mx[h];
      sm_ml[warp][h][1] = l[h];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < GQA * D; i += 256) {
    const int h = i / D, d = i % D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 8; ++w) mm = fmaxf(mm, sm_ml[w][h][0]);
    float lt = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const float mw = sm_ml[w][h][0];
      const float c = (mw == -INFINITY) ? 0.f : exp2f(mw - mm);
      lt += sm_ml[w][h][1] * c;
      o += sm_o[w][h][d] * c;
    }
    const size_t base = ((size_t)m * p.n_q + kh * GQA + h) * p.nsplit + split;
    p.o_part[base * D + d] = o;
    if (d == 0) {
      p.ml_part[base * 2] = mm;
      p.ml_part[base * 2 + 1] = lt;
    }
  }
  if (p.tickets == nullptr) return;
  // ---- fused merge: the CTA that finishes last for this (row, KV head) folds all splits, in split
  // order, so the result does not depend on which CTA that is.  The counter returns to zero for
  // the next launch (graph replays need no host reset).
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int t = atomicAdd(&p.tickets[m * p.n_kv + kh], 1);
    sm_last = (t == p.nsplit - 1);
    if (sm_last) p.tickets[m * p.n_kv + kh] = 0;
  }
  __syncthreads();
  if (!sm_last) return;
  __threadfence();
  // weights of the splits first (one thread per (head, split)), then every (head, dim) output with its
  // split loads issued together; the sums run in split order
  float* cw = &sm_o[0][0][0];  // [GQA][nsplit] reuses the warp-merge buffer (8 * D >= nsplit for nsplit <= 64)
  for (int i = threadIdx.x; i < GQA * p.nsplit; i += 256) {
    const int h = i / p.nsplit, sp = i % p.nsplit;
    const size_t base = ((size_t)m * p.n_q + kh * GQA + h) * p.nsplit;
    cw[i] = __ldcg(p.ml_part + (base + sp) * 2);
    sm_o[4][0][i] = __ldcg(p.ml_part + (base + sp) * 2 + 1);
  }
  __syncthreads();
  if (threadIdx.x < GQA) {
    const int h = threadIdx.x;
    float mm = -INFINITY;
    for (int sp = 0; sp < p.nsplit; ++sp) mm = fmaxf(mm, cw[h * p.nsplit + sp]);
    float lt = 0.f;
    for (int sp = 0; sp < p.nsplit; ++sp) {
      const float ms = cw[h * p.nsplit + sp];
      const float c = (ms == -INFINITY) ? 0.f : exp2f(ms - mm);
      lt += sm_o[4][0][h * p.nsplit + sp] * c;
      cw[h * p.nsplit + sp] = c;
    }
    const float inv = lt > 0.f ? 1.f / lt : 0.f;
    for (int sp = 0; sp < p.nsplit; ++sp) cw[h * p.nsplit + sp] *= inv;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < GQA * D; i += 256) {
    const int h = i / D, d = i % D;
    const float* src = p.o_part + (((size_t)m * p.n_q + kh * GQA + h) * p.nsplit) * D + d;
    float o = 0.f;
    for (int s0 = 0; s0 < p.nsplit; s0 += 8) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = (s0 + u < p.nsplit) ? __ldcg(src + (size_t)(s0 + u) * D) : 0.f;
#pragma unroll
      for (int u = 0; u < 8; ++u) o = fmaf(v[u], (s0 + u < p.nsplit) ? cw[h * p.nsplit + s0 + u] : 0.f, o);
    }
    p.out[((size_t)m * p.n_q + kh * GQA + h) * D + d] = __float2bfloat16(o);
  }
}

// grid (n_q, M), D threads.  xq != nullptr (D = 128): the head's 128 outputs, as rounded to bf16, also leave as the two
// quantised 64-k groups the o projection's integer GEMV reads (the work of quant_x_kernel on this row slice, same
// bits), which saves that launch in a step of several rows.
__global__ void attn_merge_kernel(const float* o_part, const float* ml_part, __nv_bfloat16* out, int n_q, int nsplit,
                                  int D, uint8_t* xq, uint32_t* xq_gs, int gs_rows) {
  __shared__ float cw[64];
  __shared__ __align__(16) __nv_bfloat16 srow[128];
  pdl_wait();
  pdl_launch_dependents();
  const int h = blockIdx.x, m = blockIdx.y, d = threadIdx.x;
  const size_t base = ((size_t)m * n_q + h) * nsplit;
  float merged;
  if (nsplit <= 64) {
    // weights of the splits once per CTA (one lane per split), then every thread's loads are independent
    if (d < 32) {
      float m0 = d < nsplit ? ml_part[(base + d) * 2] : -INFINITY, m1 = d + 32 < nsplit ? ml_part[(base + d + 32) * 2] : -INFINITY;
      const float mm = warp_max(fmaxf(m0, m1));
      const float c0 = m0 == -INFINITY ? 0.f : exp2f(m0 - mm), c1 = m1 == -INFINITY ? 0.f : exp2f(m1 - mm);
      float l = (d < nsplit ? ml_part[(base + d) * 2 + 1] * c0 : 0.f) + (d + 32 < nsplit ? ml_part[(base + d + 32) * 2 + 1] * c1 : 0.f);
      // a fixed-shape tree over the lanes: the same bits on every run
      l = warp_sum(l);
      const float inv = l > 0.f ? 1.f / l : 0.f;
      cw[d] = c0 * inv;
      cw[d + 32] = c1 * inv;
    }
    // the first 32 splits' values are requested before the weights are known: one round trip for both
    float v0[32];
#pragma unroll
    for (int u = 0; u < 32; ++u) v0[u] = u < nsplit ? o_part[(base + u) * D + d] : 0.f;
    __syncthreads();
    float o = 0.f;
#pragma unroll
    for (int u = 0; u < 32; ++u) o = fmaf(v0[u], u < nsplit ? cw[u] : 0.f, o);
    if (nsplit > 32) {
#pragma unroll
      for (int u = 0; u < 32; ++u) v0[u] = 32 + u < nsplit ? o_part[(base + 32 + u) * D + d] : 0.f;
#pragma unroll
      for (int u = 0; u < 32; ++u) o = fmaf(v0[u], 32 + u < nsplit ? cw[32 + u] : 0.f, o);
    }
    merged = o;
  } else {
  float mm = -INFINITY;
  for (int s = 0; s < nsplit; ++s) mm = fmaxf(mm, ml_part[(base + s) * 2]);
  float lt = 0.f, o = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float ms = ml_part[(base + s) * 2];
    const float c = (ms == -INFINITY) ? 0.f : exp2f(ms - mm);
    lt += ml_part[(base + s) * 2 + 1] * c;
    o += o_part[(base + s) * D + d] * c;
  }
  merged = lt > 0.f ? o / lt : 0.f;
  }
  const __nv_bfloat16 ob = __float2bfloat16(merged);
  out[((size_t)m * n_q + h) * D + d] = ob;
  if (xq) {
    srow[d] = ob;
    __syncthreads();
    if (d < 32) {   // lanes 0..15 hold the head's sixteen 16-byte vectors; every lane of the warp calls the quantiser
      const uint4 val = d < 16 ? reinterpret_cast<const uint4*>(srow)[d] : make_uint4(0, 0, 0, 0);
      const StagedVec sv = stage_quant(val);
      if (d < 16) {
        const int KG = n_q * 2, group = h * 2 + (d >> 3), vq = d & 7;
        uint32_t* dst = reinterpret_cast<uint32_t*>(xq + ((size_t)m * KG + group) * 128) + stage_word(vq);
        dst[0] = sv.w[0];
        dst[4] = sv.w[1];
        dst[8] = sv.w[2];
        dst[12] = sv.w[3];
        if (vq == 0) {
          xq_gs[((size_t)group * gs_rows + m) * 2] = __float_as_uint(sv.scale);
          xq_gs[((size_t)group * gs_rows + m) * 2 + 1] = (uint32_t)sv.m8sum;
        }
      }
    }
  }
}

// ------------------------------------------------------------------ gemv_bf16 / gemv_i8 (lm_head, router)
// 256 threads = 8 warps, each warp owns RW rows; lanes stride K in 16-byte vectors.
// Writes logits fp32 [M][ldo] and, when cand_val != nullptr, the CTA's best (value, id) per row m.
template <typename WT>
struct HeadParams {
  const WT* w;          // [N][K]
  const float* wscale;  // int8: [N]
  const __nv_bfloat16* x;  // [M][K]
  float* out;
  int M, N, K, ldo;
  float* cand_val;  // [M][gridDim.x]
  int* cand_idx;
  int n_valid;      // ids >= n_valid never win the arg-max
};

template <typename WT, int MT>
__global__ void __launch_bounds__(256) head_gemv_kernel(const HeadParams<WT> p, int m0) {
  constexpr int RW = 8;                       // rows per warp
  constexpr int VE = 16 / sizeof(WT);         // weights per 16-byte vector
  __shared__ float sv[8][MT];
  __shared__ int si[8][MT];
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = (blockIdx.x * 8 + warp) * RW;
  float best[MT];
  int besti[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) { best[m] = -INFINITY; besti[m] = 0x7fffffff; }
  for (int rr = 0; rr < RW; rr += 4) {
    float acc[4][MT];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int m = 0; m < MT; ++m) acc[r][m] = 0.f;
    for (int k = lane * VE; k < p.K; k += 32 * VE) {
      uint4 wv[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int n = min(row0 + rr + r, p.N - 1);
        wv[r] = __ldcs(reinterpret_cast<const uint4*>(p.w + (size_t)n * p.K + k));
      }
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const int mm = min(m0 + m, p.M - 1);
        float xf[VE];
        const uint4* xp = reinterpret_cast<const uint4*>(p.x + (size_t)mm * p.K + k);
#pragma unroll
        for (int v = 0; v < VE / 8; ++v) {
          const uint4 xv = __ldg(xp + v);
          xf[8 * v + 0] = bf16_lo(xv.x); xf[8 * v + 1] = bf16_hi(xv.x);
          xf[8 * v + 2] = bf16_lo(xv.y); xf[8 * v + 3] = bf16_hi(xv.y);
          xf[8 * v + 4] = bf16_lo(xv.z); xf[8 * v + 5] = bf16_hi(xv.z);
          xf[8 * v + 6] = bf16_lo(xv.w); xf[8 * v + 7] = bf16_hi(xv.w);
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const uint32_t ww[4] = {wv[r].x, wv[r].y, wv[r].z, wv[r].w};
          float a = acc[r][m];
          if constexpr (sizeof(WT) == 2) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              a = fmaf(bf16_lo(ww[j]), xf[2 * j], a);
              a = fmaf(bf16_hi(ww[j]), xf[2 * j + 1], a);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              // int8 -> fp32 by a byte permute into the mantissa of 2^23 and one subtraction (exact; the integer
              // conversion unit is a quarter-rate pipe and capped this loop below the memory rate)
              const uint32_t u = ww[j] ^ 0x80808080u;
              a = fmaf(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7540)) - 8388736.f, xf[4 * j], a);
              a = fmaf(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7541)) - 8388736.f, xf[4 * j + 1], a);
              a = fmaf(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7542)) - 8388736.f, xf[4 * j + 2], a);
              a = fmaf(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7543)) - 8388736.f, xf[4 * j + 3], a);
            }
          }
          acc[r][m] = a;
        }
      }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int n = row0 + rr + r;
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        float v = warp_sum(acc[r][m]);
        if constexpr (sizeof(WT) == 1) v *= (n < p.N ? p.wscale[n] : 0.f);
        if (n < p.N && m0 + m < p.M) {
          if (lane == 0) p.out[(size_t)(m0 + m) * p.ldo + n] = v;
          if (n < p.n_valid && (v > best[m])) { best[m] = v; besti[m] = n; }  // rows ascend: ties keep the lower id
        }
      }
    }
  }
  if (p.cand_val) {
    if (lane == 0) {
#pragma unroll
      for (int m = 0; m < MT; ++m) { sv[warp][m] = best[m]; si[warp][m] = besti[m]; }
    }
    __syncthreads();
    if (threadIdx.x < MT && m0 + threadIdx.x < p.M) {
      const int m = threadIdx.x;
      float b = -INFINITY;
      int bi = 0x7fffffff;
      for (int w = 0; w < 8; ++w)
        if (sv[w][m] > b) { b = sv[w][m]; bi = si[w][m]; }
      p.cand_val[(size_t)(m0 + m) * gridDim.x + blockIdx.x] = b;
      p.cand_idx[(size_t)(m0 + m) * gridDim.x + blockIdx.x] = bi;
    }
  }
}

// The bf16 head on the tensor cores, up to 16 activation rows per pass over the weights: the FMA form above is bound
// by fp32 issue from 5 rows up (8 rows take twice the time the bytes need), and a 16-row verify step read the head
// twice.  64 threads = 2 warps, 32 weight rows per warp, 64 per CTA (the arg-max candidate count stays
// ceil(N / 64)).  mma.m16n8k16 with the activations as A and the weight rows as B; a dot product does not care in
// which order its k terms are taken, so a lane loads 8 consecutive k of its weight row (and of its two activation
// rows) as one 16-byte vector and feeds the words to two MMAs in matching slots -- no transposes.
// With the vectors of a step held in registers (92 per thread) 16 warps fit an SM and the kernel waits on memory
// latency; so the loads are cp.async into a ring of six stages in shared memory in which every lane owns its slots
// (it reads back only what it copied: no barrier, no bank conflict) and five stages per warp are in flight: 72 KB per
// CTA, three CTAs per SM, 120 KB of weights on their way per SM.
// Every row count runs this kernel, so a row's logits do not depend on how many rows share the step.
constexpr int kHeadStages = 6, kHeadVecs = 12;   // per stage and lane: 2 x 4 weight vectors, 2 x 2 activation vectors
constexpr int kHeadSmem = 2 * kHeadStages * kHeadVecs * 512;

__global__ void __launch_bounds__(64) head_gemv_mma_kernel(const HeadParams<__nv_bfloat16> p, int m0) {
  constexpr int NG = 4, KU = 2, NW = 2;
  extern __shared__ __align__(16) unsigned char head_smem[];
  __shared__ float sv[NW][16];
  __shared__ int si[NW][16];
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int row0 = blockIdx.x * 64 + warp * 8 * NG;
  const __nv_bfloat16* wp[NG];
#pragma unroll
  for (int i = 0; i < NG; ++i) wp[i] = p.w + (size_t)min(row0 + 8 * i + g, p.N - 1) * p.K + t * 8;
  const __nv_bfloat16* xa = p.x + (size_t)min(m0 + g, p.M - 1) * p.K + t * 8;
  const __nv_bfloat16* xb = p.x + (size_t)min(m0 + 8 + g, p.M - 1) * p.K + t * 8;
  // this lane's slots: stage s, vector v at ring + ((s * kHeadVecs + v) * 32 + lane) * 16
  unsigned char* ring = head_smem + (size_t)warp * kHeadStages * kHeadVecs * 512 + lane * 16;
  const uint32_t ring_s = (uint32_t)__cvta_generic_to_shared(ring);
  const int steps = p.K / (32 * KU);
  auto issue = [&](int step) {
    if (step < steps) {
      const int k = step * 32 * KU;
      const uint32_t dst = ring_s + (step % kHeadStages) * kHeadVecs * 512;
#pragma unroll
      for (int u = 0; u < KU; ++u) {
#pragma unroll
        for (int i = 0; i < NG; ++i)
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + (u * NG + i) * 512), "l"(wp[i] + k + 32 * u)
                       : "memory");
        asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst + (KU * NG + 2 * u) * 512), "l"(xa + k + 32 * u)
                     : "memory");
        asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst + (KU * NG + 2 * u + 1) * 512),
                     "l"(xb + k + 32 * u)
                     : "memory");
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");   // an empty group past the end keeps the count uniform
  };
  float acc[NG][4];
#pragma unroll
  for (int i = 0; i < NG; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
#pragma unroll
  for (int s0 = 0; s0 < kHeadStages; ++s0) issue(s0);
  for (int step = 0; step < steps; ++step) {
    asm volatile("cp.async.wait_group %0;" ::"n"(kHeadStages - 1) : "memory");
    const uint4* st = reinterpret_cast<const uint4*>(ring + (size_t)(step % kHeadStages) * kHeadVecs * 512);
#pragma unroll
    for (int u = 0; u < KU; ++u) {
      const uint4 av = st[(KU * NG + 2 * u) * 32], bv = st[(KU * NG + 2 * u + 1) * 32];
#pragma unroll
      for (int i = 0; i < NG; ++i) {
        const uint4 wv = st[(u * NG + i) * 32];
        mma_bf16_16816(acc[i], av.x, bv.x, av.y, bv.y, wv.x, wv.y);
        mma_bf16_16816(acc[i], av.z, bv.z, av.w, bv.w, wv.z, wv.w);
      }
    }
    issue(step + kHeadStages);   // into the stage just read: its values sit in MMA operands by now
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  // c[0], c[1]: activation row g, weight rows 2t, 2t + 1 of the group; c[2], c[3]: activation row g + 8
  float best[2] = {-INFINITY, -INFINITY};
  int besti[2] = {0x7fffffff, 0x7fffffff};
#pragma unroll
  for (int grp = 0; grp < NG; ++grp) {
    const float* c = acc[grp];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int n = row0 + grp * 8 + 2 * t + j;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int m = m0 + g + 8 * h;
        const float v = c[2 * h + j];
        if (n < p.N && m < p.M) {
          p.out[(size_t)m * p.ldo + n] = v;
          if (n < p.n_valid && v > best[h]) { best[h] = v; besti[h] = n; }   // n ascends: ties keep the lower id
        }
      }
    }
  }
  if (!p.cand_val) return;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
#pragma unroll
    for (int d = 1; d <= 2; d <<= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best[h], d);
      const int oi = __shfl_xor_sync(0xffffffffu, besti[h], d);
      if (ov > best[h] || (ov == best[h] && oi < besti[h])) { best[h] = ov; besti[h] = oi; }
    }
    if (t == 0) { sv[warp][g + 8 * h] = best[h]; si[warp][g + 8 * h] = besti[h]; }
  }
  __syncthreads();
  if (threadIdx.x < 16 && m0 + threadIdx.x < p.M) {
    const int m = threadIdx.x;
    float b = -INFINITY;
    int bi = 0x7fffffff;
    for (int w = 0; w < NW; ++w)
      if (sv[w][m] > b) { b = sv[w][m]; bi = si[w][m]; }   // warps ascend in n
    p.cand_val[(size_t)(m0 + m) * gridDim.x + blockIdx.x] = b;
    p.cand_idx[(size_t)(m0 + m) * gridDim.x + blockIdx.x] = bi;
  }
}

// grid M, 256 threads: reduce the candidates; ties -> lower id; write control block.
__global__ void __launch_bounds__(256) argmax_finish_kernel(const float* cand_val, const int* cand_idx, int ncand,
                                                            int* ctrl, int advance) {
  __shared__ float sv[256];
  __shared__ int si[256];
  pdl_wait();
  pdl_launch_dependents();
  const int m = blockIdx.x, tid = threadIdx.x;
  float b = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = tid; i < ncand; i += 256) {
    const float v = cand_val[(size_t)m * ncand + i];
    const int id = cand_idx[(size_t)m * ncand + i];
    if (v > b || (v == b && id < bi)) { b = v; bi = id; }
  }
  sv[tid] = b;
  si[tid] = bi;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (tid < o) {
      const float v = sv[tid + o];
      const int id = si[tid + o];
      if (v > sv[tid] || (v == sv[tid] && id < si[tid])) { sv[tid] = v; si[tid] = id; }
    }
    __syncthreads();
  }
  if (tid == 0) {
    ctrl[CTRL_OUT_TOKEN + m] = si[0];
    ctrl[CTRL_OUT_VALUE + m] = __float_as_int(sv[0]);
    if (advance) {
      ctrl[CTRL_CUR_TOKEN + m] = si[0];
      ctrl[CTRL_ROW_POS + m] += 1;
    }
  }
}

// ------------------------------------------------------------------ KV form conversion (int8 cache <-> bf16 scratch)
// grid (tokens, n_kv), one warp: the row of one (position, KV head), D values.  The int8 cache keeps one fp32
// scale per row (max |x| / 127), the scheme of rope_append's int8 path (the reference's per-head per-token
// scale: src/common/kv8.h:1-157).  to_int8 = 1: rows of the bf16 pages (table a) -> int8 pages (table b);
// 0: the other way.  Positions pos0 .. pos0 + tokens - 1.
__global__ void __launch_bounds__(32) kv_convert_kernel(__nv_bfloat16* k16, __nv_bfloat16* v16, const int* table16,
                                                        int8_t* k8, int8_t* v8, float* ks, float* vs, const int* table8,
                                                        int pos0, int n_kv, int D, int to_int8) {
  const int pos = pos0 + blockIdx.x, kh = blockIdx.y, lane = threadIdx.x;
  const size_t r16 = (((size_t)table16[pos >> 4] * n_kv + kh) * 16 + (pos & 15));
  const size_t r8 = (((size_t)table8[pos >> 4] * n_kv + kh) * 16 + (pos & 15));
  for (int which = 0; which < 2; ++which) {
    __nv_bfloat16* p16 = (which ? v16 : k16) + r16 * D;
    int8_t* p8 = (which ? v8 : k8) + r8 * D;
    float* sc = (which ? vs : ks) + r8;
    if (to_int8) {
      float x[8];
      float amax = 0.f;
      const int per = D / 32;
      for (int u = 0; u < per; ++u) {
        x[u] = __bfloat162float(p16[lane * per + u]);
        amax = fmaxf(amax, fabsf(x[u]));
      }
      amax = warp_max(amax);
      const float s = amax > 0.f ? amax / 127.f : 1.f, inv = 1.f / s;
      for (int u = 0; u < per; ++u) p8[lane * per + u] = (int8_t)__float2int_rn(x[u] * inv);
      if (lane == 0) *sc = s;
    } else {
      const float s = *sc;
      const int per = D / 32;
      for (int u = 0; u < per; ++u) p16[lane * per + u] = __float2bfloat16((float)p8[lane * per + u] * s);
    }
  }
}

}  // namespace

// =================================================================== C entry points
extern "C" int b2_resid_norm(const void* embed, const int* ctrl, const void* resid_in, const float* part,
                             long long part_slice, int S, int M, int H, int mode, int vocab, const float* w, float eps,
                             void* resid_out, void* x_out, int* flag, void* stream) {
  ResidNormParams p;
  p.embed = (const __nv_bfloat16*)embed; p.ctrl = ctrl; p.resid_in = (const __nv_bfloat16*)resid_in;
  p.part = part; p.part_slice = part_slice; p.S = S; p.H = H; p.mode = mode; p.vocab = vocab; p.w = w; p.eps = eps;
  p.resid_out = (__nv_bfloat16*)resid_out; p.x_out = (__nv_bfloat16*)x_out; p.flag = flag;
  if (H % 8) return -1;
  int threads = ((H / 8 + 31) / 32) * 32;
  if (threads > 1024) threads = 1024;
  return b2_launch(resid_norm_kernel, dim3(M), dim3(threads), (size_t)H * 4, (cudaStream_t)stream, true, p);
}

extern "C" int b2_draft_front(const void* embed, const int* ctrl, int vocab, const void* hidden, long long hidden_ld,
                              const float* w_e, const float* w_h, float eps, int M, int H, void* xcat, int* flag,
                              void* stream) {
  if (H % 8 || hidden_ld % 8) return -1;
  int threads = ((H / 8 + 31) / 32) * 32;
  if (threads > 1024) threads = 1024;
  return b2_launch(draft_front_kernel, dim3(M), dim3(threads), (size_t)H * 8, (cudaStream_t)stream, true,
                   (const __nv_bfloat16*)embed, ctrl, vocab, (const __nv_bfloat16*)hidden, hidden_ld, w_e, w_h, eps, H,
                   (__nv_bfloat16*)xcat, flag);
}

extern "C" int b2_rope_append(const float* qkv, long long slice, int S, int M, const int* ctrl, const int* block_table,
                              int max_blocks, const float* cos_t, const float* sin_t, int n_q, int n_kv, int D,
                              void* q_out, void* k_cache, void* v_cache, float* k_scale, float* v_scale, int kv_int8,
                              int req, int pos0, void* stream) {
  RopeParams p;
  p.qkv = qkv; p.slice = slice; p.S = S; p.ctrl = ctrl; p.block_table = block_table; p.max_blocks = max_blocks;
  p.cos_t = cos_t; p.sin_t = sin_t; p.n_q = n_q; p.n_kv = n_kv; p.D = D; p.q_out = (__nv_bfloat16*)q_out;
  p.k_cache = k_cache; p.v_cache = v_cache; p.k_scale = k_scale; p.v_scale = v_scale; p.kv_int8 = kv_int8; p.req = req; p.pos0 = pos0;
  if (D % 64 || D > 256) return -1;
  const int items = (n_q + n_kv) * (D / 2) + n_kv * D / 2;
  int gy = kv_int8 ? max((n_q * D / 2 + 255) / 256, (2 * n_kv + 7) / 8) : (items + 255) / 256;
  return b2_launch(rope_append_kernel, dim3(M, gy), dim3(256), 0, (cudaStream_t)stream, true, p);
}

template <int D>
static int attn_decode_dispatch(int gqa, const AttnDecParams& p, dim3 grid, cudaStream_t st) {
  switch (gqa) {
    case 1: return b2_launch(attn_decode_kernel<D, 1>, grid, dim3(256), 0, st, true, p);
    case 2: return b2_launch(attn_decode_kernel<D, 2>, grid, dim3(256), 0, st, true, p);
    case 4: return b2_launch(attn_decode_kernel<D, 4>, grid, dim3(256), 0, st, true, p);
    case 5: return b2_launch(attn_decode_kernel<D, 5>, grid, dim3(256), 0, st, true, p);
    case 8: return b2_launch(attn_decode_kernel<D, 8>, grid, dim3(256), 0, st, true, p);
  }
  return -3;
}

extern "C" int b2_attn_decode(const void* q, const void* k_cache, const void* v_cache, const float* k_scale,
                              const float* v_scale, const int* block_table, const int* ctrl, float* o_part,
                              float* ml_part, void* out, int M, int n_q, int n_kv, int D, int nsplit, int max_blocks,
                              float scale, int kv_int8, int* tickets, void* stream) {
  AttnDecParams p;
  p.tickets = tickets; p.out = (__nv_bfloat16*)out;
  p.q = (const __nv_bfloat16*)q; p.k_cache = k_cache; p.v_cache = v_cache; p.k_scale = k_scale; p.v_scale = v_scale;
  p.block_table = block_table; p.ctrl = ctrl; p.o_part = o_part; p.ml_part = ml_part;
  p.n_q = n_q; p.n_kv = n_kv; p.nsplit = nsplit; p.max_blocks = max_blocks;
  p.scale_log2 = scale * 1.4426950408889634f; p.kv_int8 = kv_int8;
  dim3 grid(n_kv, nsplit, M);
  cudaStream_t st = (cudaStream_t)stream;
  int rc;
  if (D == 128) rc = attn_decode_dispatch<128>(n_q / n_kv, p, grid, st);
  else if (D == 64) rc = attn_decode_dispatch<64>(n_q / n_kv, p, grid, st);
  else return -2;
  if (rc || tickets) return rc;
  return b2_launch(attn_merge_kernel, dim3(n_q, M), dim3(D), 0, st, true, (const float*)o_part, (const float*)ml_part,
                   (__nv_bfloat16*)out, n_q, nsplit, D, (uint8_t*)nullptr, (uint32_t*)nullptr, 0);
}

extern "C" int b2_kv_convert(void* k16, void* v16, const int* table16, void* k8, void* v8, float* ks, float* vs,
                             const int* table8, int pos0, int tokens, int n_kv, int D, int to_int8, void* stream) {
  if (tokens < 1) return 0;
  if (D % 32 || D > 256) return -1;
  kv_convert_kernel<<<dim3(tokens, n_kv), 32, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)k16, (__nv_bfloat16*)v16, table16,
                                                                        (int8_t*)k8, (int8_t*)v8, ks, vs, table8, pos0, n_kv,
                                                                        D, to_int8);
  return (int)cudaGetLastError();
}

// Merge of split-KV partials as its own launch (one CTA per row and query head).
extern "C" int b2_attn_merge(const float* o_part, const float* ml_part, void* out, int M, int n_q, int nsplit, int D,
                             void* stream) {
  return b2_launch(attn_merge_kernel, dim3(n_q, M), dim3(D), 0, (cudaStream_t)stream, true, o_part, ml_part,
                   (__nv_bfloat16*)out, n_q, nsplit, D, (uint8_t*)nullptr, (uint32_t*)nullptr, 0);
}

// The merge that also writes the rows' quantised form for the o projection (head size 128; xq [M][n_q * 2][128 B],
// xq_gs [n_q * 2][gs_rows] {scale, -8 sum}: the layout of b2_quant_x for K = n_q * 128).
extern "C" int b2_attn_merge_quant(const float* o_part, const float* ml_part, void* out, int M, int n_q, int nsplit, int D,
                                   void* xq, void* xq_gs, int gs_rows, void* stream) {
  if (D != 128 || !xq || !xq_gs || gs_rows < M) return -1;
  return b2_launch(attn_merge_kernel, dim3(n_q, M), dim3(D), 0, (cudaStream_t)stream, true, o_part, ml_part,
                   (__nv_bfloat16*)out, n_q, nsplit, D, (uint8_t*)xq, (uint32_t*)xq_gs, gs_rows);
}

template <typename WT>
static int head_launch(const HeadParams<WT>& p, cudaStream_t st) {
  const int rows_per_cta = 64;
  dim3 grid((p.N + rows_per_cta - 1) / rows_per_cta);
  if constexpr (sizeof(WT) == 2) {
    if (p.K % 64 == 0) {
      static bool configured[64] = {};   // per device: the attribute belongs to the device's copy of the kernel
      int dev = 0;
      cudaGetDevice(&dev);
      if (!configured[dev & 63]) {
        cudaError_t e = cudaFuncSetAttribute(head_gemv_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kHeadSmem);
        if (e != cudaSuccess) return (int)e;
        configured[dev & 63] = true;
      }
      for (int m0 = 0; m0 < p.M; m0 += 16) {
        int rc = b2_launch(head_gemv_mma_kernel, grid, dim3(64), kHeadSmem, st, true, p, m0);
        if (rc) return rc;
      }
      return 0;
    }
  }
  // up to 8 rows per pass over the weights (the rows share every weight vector a lane loads)
  for (int m0 = 0; m0 < p.M; m0 += 8) {
    const int mt = min(8, p.M - m0);
    int rc;
    if (mt == 1) rc = b2_launch(head_gemv_kernel<WT, 1>, grid, dim3(256), 0, st, true, p, m0);
    else if (mt == 2) rc = b2_launch(head_gemv_kernel<WT, 2>, grid, dim3(256), 0, st, true, p, m0);
    else if (mt <= 4) rc = b2_launch(head_gemv_kernel<WT, 4>, grid, dim3(256), 0, st, true, p, m0);
    else rc = b2_launch(head_gemv_kernel<WT, 8>, grid, dim3(256), 0, st, true, p, m0);
    if (rc) return rc;
  }
  return 0;
}

// Number of arg-max candidates per row that b2_head_gemv writes (= its grid size).
extern "C" int b2_head_ncand(int N) { return (N + 63) / 64; }

extern "C" int b2_head_gemv(const void* w, const float* wscale, int w_int8, const void* x, float* out, int M, int N,
                            int K, int ldo, float* cand_val, int* cand_idx, int n_valid, void* stream) {
  if (K % (w_int8 ? 16 : 8) != 0) return -1;
  if (w_int8) {
    HeadParams<int8_t> p{(const int8_t*)w, wscale, (const __nv_bfloat16*)x, out, M, N, K, ldo, cand_val, cand_idx, n_valid};
    return head_launch(p, (cudaStream_t)stream);
  }
  HeadParams<__nv_bfloat16> p{(const __nv_bfloat16*)w, nullptr, (const __nv_bfloat16*)x, out, M, N, K, ldo, cand_val, cand_idx, n_valid};
  return head_launch(p, (cudaStream_t)stream);
}

extern "C" int b2_argmax_finish(const float* cand_val, const int* cand_idx, int ncand, int M, int* ctrl, int advance,
                                void* stream) {
  return b2_launch(argmax_finish_kernel, dim3(M), dim3(256), 0, (cudaStream_t)stream, true, cand_val, cand_idx, ncand,
                   ctrl, advance);
}

// ------------------------------------------------------------------ allocation-free decode attention
// b2_attn_decode_static: the same two kernels as b2_attn_decode, with the split-KV partials kept in a
// fixed device array that is part of this library's image instead of a buffer the caller allocates.
// See b200serve_noalloc.h for who needs this and for the limits.
namespace {
constexpr int kStaticMaxRows = 4, kStaticMaxHeads = 64, kStaticMaxSplit = 16, kStaticMaxD = 128;
constexpr size_t kStaticOFloats = (size_t)kStaticMaxRows * kStaticMaxHeads * kStaticMaxSplit * kStaticMaxD;
constexpr size_t kStaticMlFloats = (size_t)kStaticMaxRows * kStaticMaxHeads * kStaticMaxSplit * 2;
// 2 MiB + 32 KiB, resident on every GPU that loads the library until the process exits
static __device__ __align__(256) float g_static_attn_scratch[kStaticOFloats + kStaticMlFloats];
static float* g_static_attn_ptr[64] = {};  // per device: the array's DEVICE address (the symbol itself is a host-side stand-in)
}  // namespace

extern "C" int b2_attn_decode_static(const void* q, const void* k_cache, const void* v_cache, const float* k_scale,
                                     const float* v_scale, const int* block_table, const int* ctrl, void* out, int M,
                                     int n_q, int n_kv, int D, int nsplit, int max_blocks, float scale, int kv_int8,
                                     void* stream) {
  if (M < 1 || M > kStaticMaxRows || n_q < 1 || n_q > kStaticMaxHeads || nsplit < 1 || nsplit > kStaticMaxSplit ||
      (D != 64 && D != 128) || n_kv < 1 || n_q % n_kv != 0)
    return -10;  // beyond the fixed scratch: use b2_attn_decode with caller-owned buffers
  {
    const int gqa = n_q / n_kv;   // the head groupings the kernel is built for
    if (gqa != 1 && gqa != 2 && gqa != 4 && gqa != 5 && gqa != 8) return -10;
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return -10;   // the per-device address table holds 64 devices
  if (!g_static_attn_ptr[dev]) {
    // first call on this device: resolve the array's device address (no allocation takes place)
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_attn_scratch);
    if (e != cudaSuccess) return (int)e;
    g_static_attn_ptr[dev] = static_cast<float*>(ptr);
  }
  float* o_part = g_static_attn_ptr[dev];
  float* ml_part = o_part + kStaticOFloats;
  // Nothing has to start at zero: every (row, head, split) entry that the merge reads is written by
  // the split kernel of the same call, empty splits included (they write m = -inf, l = 0).
  AttnDecParams p;
  p.tickets = nullptr; p.out = nullptr;
  p.q = (const __nv_bfloat16*)q; p.k_cache = k_cache; p.v_cache = v_cache; p.k_scale = k_scale; p.v_scale = v_scale;
  p.block_table = block_table; p.ctrl = ctrl; p.o_part = o_part; p.ml_part = ml_part;
  p.n_q = n_q; p.n_kv = n_kv; p.nsplit = nsplit; p.max_blocks = max_blocks;
  p.scale_log2 = scale * 1.4426950408889634f; p.kv_int8 = kv_int8;
  dim3 grid(n_kv, nsplit, M);
  cudaStream_t st = (cudaStream_t)stream;
  int rc;
  if (D == 128) rc = attn_decode_dispatch<128>(n_q / n_kv, p, grid, st);
  else rc = attn_decode_dispatch<64>(n_q / n_kv, p, grid, st);
  if (rc) return rc;
  return b2_launch(attn_merge_kernel, dim3(n_q, M), dim3(D), 0, st, true, (const float*)o_part, (const float*)ml_part,
                   (__nv_bfloat16*)out, n_q, nsplit, D, (uint8_t*)nullptr, (uint32_t*)nullptr, 0);
}

B2_DEFINE_STATUS(decode)
