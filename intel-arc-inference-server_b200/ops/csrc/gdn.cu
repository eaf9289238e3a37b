// Gated delta-net (linear attention) layers: the per-token recurrent step of the hybrid model family.
//
// The role of the reference's GDN decode kernels (src/kernels/gdn_step.cl and the gated head of
// src/kernels/prep.cl: prep_gated_head).  A layer projects the normalised hidden row to
// [ q | k | v | z | b | a ]  (q, k: n_k heads x 128; v, z: n_v heads x 128; b, a: n_v scalars), passes q, k, v through
// a depthwise causal convolution of 4 taps + SiLU, and updates one 128 x 128 fp32 state per value head:
//     S <- S * exp(g);   delta = (v - S^T k) * beta;   S <- S + k delta^T;   o = S^T q
// with  g = -exp(A_log) * softplus(a + dt_bias),  beta = sigmoid(b),  q and k L2-normalised (q also scaled by
// 128^-1/2).  The output is RMS-normalised per head, scaled by a learned weight and gated by SiLU(z).
//
// Two kernels per layer and step:
//   gdn_conv_kernel  one thread per projected column: folds the GEMV's split-K partials, and for the q / k / v
//                    columns applies the convolution over the slot's last three inputs (kept per slot) + SiLU;
//   gdn_step_kernel  one CTA per value head, thread j owns column j of the state (128 fp32 registers): decay,
//                    delta rule, read-out, gated norm; q and k are shared through shared memory.
// Rows of a step are walked in order inside each thread, so several rows of one slot (a prompt chunk, verify
// rows) see each other's state; a thread keeps the state in registers while consecutive rows stay on one slot.
#include "common.cuh"

using namespace b2;

namespace {

constexpr int CTRL_ROW_REQ = 16;
constexpr int DH = 128;      // head size of q, k, v
constexpr int TAPS = 4;

struct GdnConvParams {
  const float* part;   // [splits][M][N] fp32 partial sums of the input projection
  int splits, M, N, conv_ch;
  const int* ctrl;       // row -> slot; nullptr: every row belongs to `slot` (a prompt chunk)
  int slot;
  const float* conv_w;   // [conv_ch][TAPS], tap TAPS-1 multiplies the newest input
  float* conv_state;     // [slots][conv_ch][TAPS-1], oldest first
  float* act;            // [M][N]: convolved + SiLU for the first conv_ch columns, plain sums for the rest
};

__global__ void __launch_bounds__(256) gdn_conv_kernel(const GdnConvParams p) {
  pdl_wait();
  pdl_launch_dependents();
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= p.N) return;
  const bool conv = n < p.conv_ch;
  float w[TAPS] = {0.f, 0.f, 0.f, 0.f}, st[TAPS - 1] = {0.f, 0.f, 0.f};
  if (conv) {
#pragma unroll
    for (int t = 0; t < TAPS; ++t) w[t] = p.conv_w[(size_t)n * TAPS + t];
  }
  int cur = -1;
  for (int m = 0; m < p.M; ++m) {
    float x = 0.f;
    for (int s = 0; s < p.splits; ++s) x += p.part[((size_t)s * p.M + m) * p.N + n];
    if (conv) {
      const int slot = p.ctrl ? p.ctrl[CTRL_ROW_REQ + m] : p.slot;
      if (slot != cur) {
        if (cur >= 0) {
#pragma unroll
          for (int t = 0; t < TAPS - 1; ++t) p.conv_state[((size_t)cur * p.conv_ch + n) * (TAPS - 1) + t] = st[t];
        }
        cur = slot;
#pragma unroll
        for (int t = 0; t < TAPS - 1; ++t) st[t] = p.conv_state[((size_t)cur * p.conv_ch + n) * (TAPS - 1) + t];
      }
      const float y = w[0] * st[0] + w[1] * st[1] + w[2] * st[2] + w[3] * x;
      st[0] = st[1]; st[1] = st[2]; st[2] = x;
      x = y / (1.f + __expf(-y));
    }
    p.act[(size_t)m * p.N + n] = x;
  }
  if (conv && cur >= 0) {
#pragma unroll
    for (int t = 0; t < TAPS - 1; ++t) p.conv_state[((size_t)cur * p.conv_ch + n) * (TAPS - 1) + t] = st[t];
  }
}

struct GdnStepParams {
  const float* act;    // [M][N]
  int M, N, n_k, n_v;
  const int* ctrl;       // row -> slot; nullptr: every row belongs to `slot`
  int slot;
  const float* a_log;    // [n_v]
  const float* dt_bias;  // [n_v]
  const float* norm_w;   // [DH]
  float eps;
  float* state;          // [slots][n_v][DH][DH] fp32, element (i, j) = key dim i, value dim j
  __nv_bfloat16* out;    // [M][n_v * DH]
};

__device__ __forceinline__ float block_sum_128(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  return red[0] + red[1] + red[2] + red[3];
}

__global__ void __launch_bounds__(DH) gdn_step_kernel(const GdnStepParams p) {
  __shared__ float qs[DH], ks[DH], red[4];
  pdl_wait();
  pdl_launch_dependents();
  const int h = blockIdx.x, j = threadIdx.x;
  const int hk = h / (p.n_v / p.n_k);
  const int kd = p.n_k * DH, vd = p.n_v * DH;
  const float a_neg = -__expf(p.a_log[h]), dtb = p.dt_bias[h], nw = p.norm_w[j];
  float S[DH];
  int cur = -1;
  for (int m = 0; m < p.M; ++m) {
    const int slot = p.ctrl ? p.ctrl[CTRL_ROW_REQ + m] : p.slot;
    if (slot != cur) {
      if (cur >= 0) {
        float* sp = p.state + ((size_t)cur * p.n_v + h) * DH * DH + j;
#pragma unroll
        for (int i = 0; i < DH; ++i) sp[(size_t)i * DH] = S[i];
      }
      cur = slot;
      const float* sp = p.state + ((size_t)cur * p.n_v + h) * DH * DH + j;
#pragma unroll
      for (int i = 0; i < DH; ++i) S[i] = sp[(size_t)i * DH];
    }
    const float* a = p.act + (size_t)m * p.N;
    const float qv = a[hk * DH + j], kv = a[kd + hk * DH + j];
    const float vj = a[2 * kd + h * DH + j], zj = a[2 * kd + vd + h * DH + j];
    const float bb = a[2 * kd + 2 * vd + h], aa = a[2 * kd + 2 * vd + p.n_v + h];
    const float qn = block_sum_128(qv * qv, red), kn = block_sum_128(kv * kv, red);
    __syncthreads();   // the previous row's readers of qs / ks are done (block_sum_128 synchronised after them)
    qs[j] = qv * rsqrtf(qn + 1e-6f) * 0.08838834764831845f;   // 128^-1/2
    ks[j] = kv * rsqrtf(kn + 1e-6f);
    __syncthreads();
    const float beta = 1.f / (1.f + __expf(-bb));
    const float sp_in = aa + dtb;
    const float softplus = sp_in > 20.f ? sp_in : log1pf(__expf(sp_in));
    const float decay = __expf(a_neg * softplus);
    float mem = 0.f;
#pragma unroll
    for (int i = 0; i < DH; ++i) {
      S[i] *= decay;
      mem = fmaf(S[i], ks[i], mem);
    }
    const float delta = (vj - mem) * beta;
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < DH; ++i) {
      S[i] = fmaf(ks[i], delta, S[i]);
      o = fmaf(S[i], qs[i], o);
    }
    const float ms = block_sum_128(o * o, red) * (1.f / DH);
    const float y = o * rsqrtf(ms + p.eps) * nw * (zj / (1.f + __expf(-zj)));
    p.out[(size_t)m * vd + h * DH + j] = __float2bfloat16(y);
  }
  if (cur >= 0) {
    float* sp = p.state + ((size_t)cur * p.n_v + h) * DH * DH + j;
#pragma unroll
    for (int i = 0; i < DH; ++i) sp[(size_t)i * DH] = S[i];
  }
}

// ---- prompt chunks: the same layer as three kernels, so that everything that does not depend on the state runs
// in parallel over the chunk's rows and the sequential scan is left with two 128-long loops per row.
//   gdn_prep_kernel  grid (rows, n_k + 1): L2-normalises q and k of a key head in place (q also scaled); the last
//                    block of a row turns b, a into beta and the decay factor in place;
//   gdn_scan_kernel  grid (n_v): walks the rows in order; thread j owns state column j; the row's q / k reach the
//                    threads through a double-buffered shared-memory copy (one barrier per row), the next row's
//                    operands are fetched while this row's loops run; the raw read-out replaces v in place;
//   gdn_gate_kernel  grid (rows, n_v): RMS norm of the read-out, weight, SiLU(z) gate, bf16 store.
struct GdnChunkParams {
  float* act;   // [M][N]
  int M, N, n_k, n_v;
  int slot;
  const float* a_log;
  const float* dt_bias;
  const float* norm_w;
  float eps;
  float* state;
  __nv_bfloat16* out;
};

__global__ void __launch_bounds__(DH) gdn_prep_kernel(const GdnChunkParams p) {
  __shared__ float red[4];
  pdl_wait();
  pdl_launch_dependents();
  const int m = blockIdx.x, y = blockIdx.y, j = threadIdx.x;
  const int kd = p.n_k * DH, vd = p.n_v * DH;
  float* a = p.act + (size_t)m * p.N;
  if (y < p.n_k) {
    const float qv = a[y * DH + j], kv = a[kd + y * DH + j];
    const float qn = block_sum_128(qv * qv, red), kn = block_sum_128(kv * kv, red);
    a[y * DH + j] = qv * rsqrtf(qn + 1e-6f) * 0.08838834764831845f;
    a[kd + y * DH + j] = kv * rsqrtf(kn + 1e-6f);
  } else {
    for (int h = j; h < p.n_v; h += DH) {
      const float bb = a[2 * kd + 2 * vd + h], sp_in = a[2 * kd + 2 * vd + p.n_v + h] + p.dt_bias[h];
      const float softplus = sp_in > 20.f ? sp_in : log1pf(__expf(sp_in));
      a[2 * kd + 2 * vd + h] = 1.f / (1.f + __expf(-bb));
      a[2 * kd + 2 * vd + p.n_v + h] = __expf(-__expf(p.a_log[h]) * softplus);
    }
  }
}

__global__ void __launch_bounds__(DH) gdn_scan_kernel(const GdnChunkParams p) {
  __shared__ float qk[2][2 * DH];
  pdl_wait();
  pdl_launch_dependents();
  const int h = blockIdx.x, j = threadIdx.x;
  const int hk = h / (p.n_v / p.n_k);
  const int kd = p.n_k * DH, vd = p.n_v * DH;
  const int oq = hk * DH + j, ok = kd + hk * DH + j, ov = 2 * kd + h * DH + j, ob = 2 * kd + 2 * vd + h, od = ob + p.n_v;
  float S[DH];
  float* sp = p.state + ((size_t)p.slot * p.n_v + h) * DH * DH + j;
#pragma unroll
  for (int i = 0; i < DH; ++i) S[i] = sp[(size_t)i * DH];
  float* a = p.act;
  qk[0][j] = a[oq];
  qk[0][DH + j] = a[ok];
  float vj = a[ov], beta = a[ob], decay = a[od];
  __syncthreads();
  for (int m = 0; m < p.M; ++m) {
    const int buf = m & 1;
    float nq = 0.f, nk = 0.f, nv = 0.f, nb = 0.f, nd = 0.f;
    if (m + 1 < p.M) {   // the next row's operands travel while this row's loops run
      const float* an = a + p.N;
      nq = an[oq]; nk = an[ok]; nv = an[ov]; nb = an[ob]; nd = an[od];
    }
    float mem = 0.f;
#pragma unroll
    for (int i = 0; i < DH; ++i) {
      S[i] *= decay;
      mem = fmaf(S[i], qk[buf][DH + i], mem);
    }
    const float delta = (vj - mem) * beta;
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < DH; ++i) {
      S[i] = fmaf(qk[buf][DH + i], delta, S[i]);
      o = fmaf(S[i], qk[buf][i], o);
    }
    a[ov] = o;   // the raw read-out takes v's place (this thread alone reads and writes the element)
    qk[buf ^ 1][j] = nq;
    qk[buf ^ 1][DH + j] = nk;
    vj = nv; beta = nb; decay = nd;
    a += p.N;
    __syncthreads();   // the other buffer is complete; nobody still reads the one that row m + 1 will refill
  }
#pragma unroll
  for (int i = 0; i < DH; ++i) sp[(size_t)i * DH] = S[i];
}

__global__ void __launch_bounds__(DH) gdn_gate_kernel(const GdnChunkParams p) {
  __shared__ float red[4];
  pdl_wait();
  pdl_launch_dependents();
  const int m = blockIdx.x, h = blockIdx.y, j = threadIdx.x;
  const int kd = p.n_k * DH, vd = p.n_v * DH;
  const float* a = p.act + (size_t)m * p.N;
  const float o = a[2 * kd + h * DH + j], zj = a[2 * kd + vd + h * DH + j];
  const float ms = block_sum_128(o * o, red) * (1.f / DH);
  p.out[(size_t)m * vd + h * DH + j] = __float2bfloat16(o * rsqrtf(ms + p.eps) * p.norm_w[j] * (zj / (1.f + __expf(-zj))));
}

}  // namespace

// A prompt chunk of one slot through a gated delta-net layer's recurrence: act [M][N] (after b2_gdn_conv) is
// overwritten with intermediate values; out [M][n_v * 128] bf16.
extern "C" int b2_gdn_chunk(float* act, int M, int N, int n_k, int n_v, int head_dim, int slot, const float* a_log,
                            const float* dt_bias, const float* norm_w, float eps, float* state, void* out, void* stream) {
  if (head_dim != DH || M < 1 || slot < 0 || n_k < 1 || n_v % n_k != 0 || N != 2 * n_k * DH + 2 * n_v * DH + 2 * n_v) return -1;
  GdnChunkParams p{act, M, N, n_k, n_v, slot, a_log, dt_bias, norm_w, eps, state, (__nv_bfloat16*)out};
  cudaStream_t st = (cudaStream_t)stream;
  int rc = b2_launch(gdn_prep_kernel, dim3(M, n_k + 1), dim3(DH), 0, st, true, p);
  if (rc) return rc;
  rc = b2_launch(gdn_scan_kernel, dim3(n_v), dim3(DH), 0, st, true, p);
  if (rc) return rc;
  return b2_launch(gdn_gate_kernel, dim3(M, n_v), dim3(DH), 0, st, true, p);
}

// act [M][N] from the projection's split-K partials; the first conv_ch columns go through the 4-tap causal
// convolution over the row's slot (ctrl row -> slot, at most 64 rows; or ctrl = nullptr and one slot for all rows of a
// prompt chunk) and SiLU.
extern "C" int b2_gdn_conv(const float* part, int splits, int M, int N, int conv_ch, const int* ctrl, int slot,
                           const float* conv_w, float* conv_state, float* act, void* stream) {
  if (M < 1 || (ctrl && M > 64) || (!ctrl && slot < 0) || splits < 1 || conv_ch > N) return -1;
  GdnConvParams p{part, splits, M, N, conv_ch, ctrl, slot, conv_w, conv_state, act};
  return b2_launch(gdn_conv_kernel, dim3((N + 255) / 256), dim3(256), 0, (cudaStream_t)stream, true, p);
}

// One recurrent step per row and value head; out [M][n_v * 128] bf16 is the layer's gated, normalised read-out.
extern "C" int b2_gdn_step(const float* act, int M, int N, int n_k, int n_v, int head_dim, const int* ctrl, int slot,
                           const float* a_log, const float* dt_bias, const float* norm_w, float eps, float* state,
                           void* out, void* stream) {
  if (head_dim != DH || M < 1 || (ctrl && M > 64) || (!ctrl && slot < 0) || n_k < 1 || n_v % n_k != 0 || N != 2 * n_k * DH + 2 * n_v * DH + 2 * n_v) return -1;
  GdnStepParams p{act, M, N, n_k, n_v, ctrl, slot, a_log, dt_bias, norm_w, eps, state, (__nv_bfloat16*)out};
  return b2_launch(gdn_step_kernel, dim3(n_v), dim3(DH), 0, (cudaStream_t)stream, true, p);
}

B2_DEFINE_STATUS(gdn)
