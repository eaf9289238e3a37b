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
  const int* ctrl;
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
      const int slot = p.ctrl[CTRL_ROW_REQ + m];
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
  const int* ctrl;
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
    const int slot = p.ctrl[CTRL_ROW_REQ + m];
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

}  // namespace

// act [M][N] from the projection's split-K partials; the first conv_ch columns go through the 4-tap causal
// convolution over the row's slot (ctrl row -> slot) and SiLU.
extern "C" int b2_gdn_conv(const float* part, int splits, int M, int N, int conv_ch, const int* ctrl, const float* conv_w,
                           float* conv_state, float* act, void* stream) {
  if (M < 1 || M > 64 || splits < 1 || conv_ch > N) return -1;
  GdnConvParams p{part, splits, M, N, conv_ch, ctrl, conv_w, conv_state, act};
  return b2_launch(gdn_conv_kernel, dim3((N + 255) / 256), dim3(256), 0, (cudaStream_t)stream, true, p);
}

// One recurrent step per row and value head; out [M][n_v * 128] bf16 is the layer's gated, normalised read-out.
extern "C" int b2_gdn_step(const float* act, int M, int N, int n_k, int n_v, int head_dim, const int* ctrl,
                           const float* a_log, const float* dt_bias, const float* norm_w, float eps, float* state,
                           void* out, void* stream) {
  if (head_dim != DH || M < 1 || M > 64 || n_k < 1 || n_v % n_k != 0 || N != 2 * n_k * DH + 2 * n_v * DH + 2 * n_v) return -1;
  GdnStepParams p{act, M, N, n_k, n_v, ctrl, a_log, dt_bias, norm_w, eps, state, (__nv_bfloat16*)out};
  return b2_launch(gdn_step_kernel, dim3(n_v), dim3(DH), 0, (cudaStream_t)stream, true, p);
}

B2_DEFINE_STATUS(gdn)
