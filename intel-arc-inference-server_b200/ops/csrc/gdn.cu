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
//   gdn_prep_kernel  a warp per (row, key head): L2-normalises q and k of a key head in place (q also scaled); the last
//                    warp of a row turns b, a into beta and the decay factor in place;
//   gdn_scan_kernel  grid (n_v): walks the rows in order; thread j owns state column j; the row's q / k reach the
//                    threads through a double-buffered shared-memory copy (one barrier per row), the next row's
//                    operands are fetched while this row's loops run; the raw read-out replaces v in place;
//   gdn_gate_kernel  a warp per (row, value head): RMS norm of the read-out, weight, SiLU(z) gate, bf16 store.
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

// one warp per (row, key head) -- or per row for the gates; lanes hold four consecutive elements
__global__ void __launch_bounds__(256) gdn_prep_kernel(const GdnChunkParams p) {
  pdl_wait();
  pdl_launch_dependents();
  const int wid = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  const int m = wid / (p.n_k + 1), y = wid % (p.n_k + 1);
  if (m >= p.M) return;
  const int kd = p.n_k * DH, vd = p.n_v * DH;
  float* a = p.act + (size_t)m * p.N;
  if (y < p.n_k) {
    float4* qp = reinterpret_cast<float4*>(a + y * DH) + lane;
    float4* kp = reinterpret_cast<float4*>(a + kd + y * DH) + lane;
    float4 q = *qp, k = *kp;
    const float qn = warp_sum(q.x * q.x + q.y * q.y + q.z * q.z + q.w * q.w);
    const float kn = warp_sum(k.x * k.x + k.y * k.y + k.z * k.z + k.w * k.w);
    const float qs = rsqrtf(qn + 1e-6f) * 0.08838834764831845f, ks = rsqrtf(kn + 1e-6f);
    *qp = make_float4(q.x * qs, q.y * qs, q.z * qs, q.w * qs);
    *kp = make_float4(k.x * ks, k.y * ks, k.z * ks, k.w * ks);
  } else {
    for (int h = lane; h < p.n_v; h += 32) {
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

// one warp per (row, value head)
__global__ void __launch_bounds__(256) gdn_gate_kernel(const GdnChunkParams p) {
  pdl_wait();
  pdl_launch_dependents();
  const int wid = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  const int m = wid / p.n_v, h = wid % p.n_v;
  if (m >= p.M) return;
  const int kd = p.n_k * DH, vd = p.n_v * DH;
  const float* a = p.act + (size_t)m * p.N;
  const float4 o = reinterpret_cast<const float4*>(a + 2 * kd + h * DH)[lane];
  const float4 z = reinterpret_cast<const float4*>(a + 2 * kd + vd + h * DH)[lane];
  const float4 w = reinterpret_cast<const float4*>(p.norm_w)[lane];
  const float r = rsqrtf(warp_sum(o.x * o.x + o.y * o.y + o.z * o.z + o.w * o.w) * (1.f / DH) + p.eps);
  uint2 packed;
  packed.x = pack_bf16(o.x * r * w.x * silu(z.x), o.y * r * w.y * silu(z.y));
  packed.y = pack_bf16(o.z * r * w.z * silu(z.z), o.w * r * w.w * silu(z.w));
  reinterpret_cast<uint2*>(p.out + (size_t)m * vd + h * DH)[lane] = packed;
}

// ---------------------------------------------------------------------------------------------------------------
// Chunked form of the same recurrence on the tensor cores (the role of the reference's
// src/kernels/prefill/pf_gdn_wy.cl, pf_gdn_intra.cl, pf_gdn_scan.cl).  Rows are taken in chunks of 64.  With
// gamma_s the product of the decay factors of the chunk's rows up to s, the rows' deltas U (one per row, [64][128])
// solve a unit lower-triangular system that involves the state S0 at the chunk's start only through one product:
//     (I + A) U = diag(beta) V - diag(beta gamma) K S0,     A[s][r] = beta_s (gamma_s / gamma_r) (k_s . k_r), r < s
//     U = Wv - Wk S0,   Wv = (I + A)^-1 diag(beta) V,   Wk = (I + A)^-1 diag(beta gamma) K
//     O = diag(gamma) Q S0 + P U,   P[t][s] = (gamma_t / gamma_s) (q_t . k_s), s <= t
//     S  <- gamma_63 S0 + (diag(gamma_63 / gamma) K)^T U
// gdn_wy_prep_kernel  grid (chunks, n_v), all chunks at once: the products K K^T and Q K^T (bf16 split in two
//                     limbs where the triangular solve amplifies errors), the solve by forward substitution in
//                     fp32 (thread = one column of [Wk | Wv], its 64 values in registers), and the operand images
//                     of the scan, padded for conflict-free ldmatrix, in a workspace block per (chunk, head);
// gdn_wy_scan_kernel  grid (n_v, 2), four warps: walks the chunks; a warp owns 16 value columns of the state, S^T[16][128] fp32 in
//                     MMA accumulator registers for the whole walk.  Every product is written with the value
//                     dimension as M, so accumulators turn into the next product's A operand in registers
//                     (S^T -> A of S^T Wk^T and S^T Qg^T; U^T -> A of U^T P^T and U^T Kg) and the warps never
//                     exchange anything; the chunk's block arrives by one bulk copy, two chunks in flight.
constexpr int WY_C = 64;
constexpr int WY_LDK = 136;                       // bf16 per row of a [64][128] image
constexpr int WY_LDP = 72;                        // bf16 per row of a [..][64] image
constexpr int WY_LDV = 68;                        // fp32 per row of Wv^T [128][64]
constexpr int WY_OFF_WK = 0;                      // Wk   [64][136] bf16  (row s, column dk)
constexpr int WY_OFF_QG = WY_OFF_WK + WY_C * WY_LDK * 2;     // Qg   [64][136] bf16  gamma_s q_s
constexpr int WY_OFF_KGT = WY_OFF_QG + WY_C * WY_LDK * 2;    // Kg^T [128][72] bf16  (row dk, column s) (gamma_63 / gamma_s) k_s
constexpr int WY_OFF_P = WY_OFF_KGT + DH * WY_LDP * 2;       // P    [64][72]  bf16  (row t, column s)
constexpr int WY_OFF_WVT = WY_OFF_P + WY_C * WY_LDP * 2;     // Wv^T [128][68] fp32  (row dv, column s)
constexpr int WY_OFF_GC = WY_OFF_WVT + DH * WY_LDV * 4;      // gamma_63 (fp32) + padding
constexpr int WY_BLOCK = WY_OFF_GC + 16;
static_assert(WY_BLOCK % 16 == 0 && WY_OFF_WVT % 16 == 0, "bulk copies move multiples of 16 bytes");

struct GdnWyParams {
  float* act;      // [M][N] after gdn_prep_kernel: q, k normalised; beta and the decay factor in place of b, a
  int M, N, n_k, n_v, slot, chunks;
  uint8_t* ws;     // [chunks][n_v][WY_BLOCK]
  float* state;    // [slots][n_v][128 dk][128 dv]
};

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
// A operand tile (16 rows x 16 k) of a row-major bf16 image: rows m0.., columns k0..
__device__ __forceinline__ uint32_t ldsm_a_addr(uint32_t base, int ld, int m0, int k0, int lane) {
  return base + (uint32_t)(((m0 + (lane & 15)) * ld + k0 + ((lane >> 4) << 3)) * 2);
}
// B operand, two n-tiles (16 n x 16 k) of an image stored [n][k] (k contiguous): r0, r1 = tile n0; r2, r3 = tile n0 + 8
__device__ __forceinline__ uint32_t ldsm_b_addr(uint32_t base, int ld, int n0, int k0, int lane) {
  return base + (uint32_t)(((n0 + (lane & 7) + ((lane >> 4) << 3)) * ld + k0 + (((lane >> 3) & 1) << 3)) * 2);
}

constexpr int WYA_SMEM = 3 * WY_C * WY_LDK * 2 + WY_C * WY_LDV * 4 + 2 * WY_C * 4;

__global__ void __launch_bounds__(256, 2) gdn_wy_prep_kernel(const GdnWyParams p) {
  extern __shared__ __align__(16) uint8_t wy_smem[];
  __nv_bfloat16* Khi = reinterpret_cast<__nv_bfloat16*>(wy_smem);
  __nv_bfloat16* Klo = Khi + WY_C * WY_LDK;
  __nv_bfloat16* Qhi = Klo + WY_C * WY_LDK;
  float* As = reinterpret_cast<float*>(Qhi + WY_C * WY_LDK);      // [64][68]
  float* lg = As + WY_C * WY_LDV;                                 // log gamma_s
  float* bet = lg + WY_C;
  pdl_wait();
  pdl_launch_dependents();
  const int c = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int hk = h / (p.n_v / p.n_k);
  const int kd = p.n_k * DH, vd = p.n_v * DH;
  const int row0 = c * WY_C, valid = min(WY_C, p.M - row0);
  const float* a0 = p.act + (size_t)row0 * p.N;
  uint8_t* blk = p.ws + ((size_t)c * p.n_v + h) * WY_BLOCK;
  if (warp == 0) {   // beta and the running log of the decay, rows 2 * lane and 2 * lane + 1
    float b0 = 0.f, b1 = 0.f, l0 = 0.f, l1 = 0.f;
    const int s0 = 2 * lane, s1 = s0 + 1;
    if (s0 < valid) {
      b0 = a0[(size_t)s0 * p.N + 2 * kd + 2 * vd + h];
      l0 = fmaxf(__logf(a0[(size_t)s0 * p.N + 2 * kd + 2 * vd + p.n_v + h]), -80.f);
    }
    if (s1 < valid) {
      b1 = a0[(size_t)s1 * p.N + 2 * kd + 2 * vd + h];
      l1 = fmaxf(__logf(a0[(size_t)s1 * p.N + 2 * kd + 2 * vd + p.n_v + h]), -80.f);
    }
    float run = l0 + l1;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float v = __shfl_up_sync(0xffffffffu, run, o);
      if (lane >= o) run += v;
    }
    lg[s1] = run;
    lg[s0] = run - l1;
    bet[s0] = b0;
    bet[s1] = b1;
  }
  // rows of K and Q into shared memory as bf16 limbs; 16 rows' loads are in flight per thread at a time
  {
    const int col = tid & 127, sh = tid >> 7;      // this thread: column col of rows sh, sh + 2, ...
#pragma unroll
    for (int s0 = 0; s0 < WY_C; s0 += 32) {
      float kv[16], qv[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        const int s = s0 + 2 * u + sh;
        kv[u] = s < valid ? a0[(size_t)s * p.N + kd + hk * DH + col] : 0.f;
        qv[u] = s < valid ? a0[(size_t)s * p.N + hk * DH + col] : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        const int s = s0 + 2 * u + sh;
        const __nv_bfloat16 kh = __float2bfloat16(kv[u]);
        Khi[s * WY_LDK + col] = kh;
        Klo[s * WY_LDK + col] = __float2bfloat16(kv[u] - __bfloat162float(kh));
        Qhi[s * WY_LDK + col] = __float2bfloat16(qv[u]);
      }
    }
  }
  __syncthreads();
  // ---- K K^T (three limb products) and Q K^T (two): warp = (16-row tile, half of the columns)
  {
    const int mt = warp & 3, nt0 = (warp >> 2) * 4;
    const uint32_t kh_b = smem_u32(Khi), kl_b = smem_u32(Klo), qh_b = smem_u32(Qhi);
    float gacc[4][4] = {}, pacc[4][4] = {};
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      uint32_t ah[4], al[4], aq[4];
      ldsm_x4(ldsm_a_addr(kh_b, WY_LDK, 16 * mt, 16 * kk, lane), ah[0], ah[1], ah[2], ah[3]);
      ldsm_x4(ldsm_a_addr(kl_b, WY_LDK, 16 * mt, 16 * kk, lane), al[0], al[1], al[2], al[3]);
      ldsm_x4(ldsm_a_addr(qh_b, WY_LDK, 16 * mt, 16 * kk, lane), aq[0], aq[1], aq[2], aq[3]);
#pragma unroll
      for (int jj = 0; jj < 2; ++jj) {
        uint32_t bh[4], bl[4];
        ldsm_x4(ldsm_b_addr(kh_b, WY_LDK, 8 * (nt0 + 2 * jj), 16 * kk, lane), bh[0], bh[1], bh[2], bh[3]);
        ldsm_x4(ldsm_b_addr(kl_b, WY_LDK, 8 * (nt0 + 2 * jj), 16 * kk, lane), bl[0], bl[1], bl[2], bl[3]);
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          mma_bf16_16816(gacc[2 * jj + u], ah[0], ah[1], ah[2], ah[3], bh[2 * u], bh[2 * u + 1]);
          mma_bf16_16816(gacc[2 * jj + u], ah[0], ah[1], ah[2], ah[3], bl[2 * u], bl[2 * u + 1]);
          mma_bf16_16816(gacc[2 * jj + u], al[0], al[1], al[2], al[3], bh[2 * u], bh[2 * u + 1]);
          mma_bf16_16816(pacc[2 * jj + u], aq[0], aq[1], aq[2], aq[3], bh[2 * u], bh[2 * u + 1]);
          mma_bf16_16816(pacc[2 * jj + u], aq[0], aq[1], aq[2], aq[3], bl[2 * u], bl[2 * u + 1]);
        }
      }
    }
    const int g = lane >> 2, t = lane & 3;
    uint32_t* Pw = reinterpret_cast<uint32_t*>(blk + WY_OFF_P);
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int s = 16 * mt + g + 8 * hf, r = 8 * (nt0 + j) + 2 * t;
        const float ls = lg[s], bs = bet[s];
        const float e0 = __expf(ls - lg[r]), e1 = __expf(ls - lg[r + 1]);
        As[s * WY_LDV + r] = r < s ? bs * e0 * gacc[j][2 * hf] : 0.f;
        As[s * WY_LDV + r + 1] = r + 1 < s ? bs * e1 * gacc[j][2 * hf + 1] : 0.f;
        Pw[(s * WY_LDP + r) >> 1] = pack_bf16(r <= s ? e0 * pacc[j][2 * hf] : 0.f, r + 1 <= s ? e1 * pacc[j][2 * hf + 1] : 0.f);
      }
  }
  // ---- this thread's column of the right-hand side [diag(beta gamma) K | diag(beta) V], then the substitution
  float w[WY_C];
  {
    const float* src = tid < DH ? a0 + kd + hk * DH + tid : a0 + 2 * kd + h * DH + (tid - DH);
#pragma unroll
    for (int s = 0; s < WY_C; ++s) w[s] = s < valid ? src[(size_t)s * p.N] : 0.f;
#pragma unroll
    for (int s = 0; s < WY_C; ++s) w[s] *= tid < DH ? bet[s] * __expf(lg[s]) : bet[s];
  }
  __syncthreads();
#pragma unroll
  for (int s = 1; s < WY_C; ++s) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < s; r += 4) {      // A[s][r] is zero from r = s on: whole float4 groups
      const float4 a4 = *reinterpret_cast<const float4*>(As + s * WY_LDV + r);
      acc[0] = fmaf(a4.x, w[r], acc[0]);
      if (r + 1 < s) acc[1] = fmaf(a4.y, w[r + 1], acc[1]);
      if (r + 2 < s) acc[2] = fmaf(a4.z, w[r + 2], acc[2]);
      if (r + 3 < s) acc[3] = fmaf(a4.w, w[r + 3], acc[3]);
    }
    w[s] -= (acc[0] + acc[1]) + (acc[2] + acc[3]);
  }
  if (tid < DH) {
    __nv_bfloat16* Wk = reinterpret_cast<__nv_bfloat16*>(blk + WY_OFF_WK);
#pragma unroll
    for (int s = 0; s < WY_C; ++s) Wk[s * WY_LDK + tid] = __float2bfloat16(w[s]);
    // Kg^T row dk = tid: (gamma_63 / gamma_s) k_s[dk]
    uint32_t* Kg = reinterpret_cast<uint32_t*>(blk + WY_OFF_KGT) + tid * (WY_LDP / 2);
    const float l63 = lg[WY_C - 1];
#pragma unroll
    for (int s = 0; s < WY_C; s += 2) {
      const float k0 = __bfloat162float(Khi[s * WY_LDK + tid]) + __bfloat162float(Klo[s * WY_LDK + tid]);
      const float k1 = __bfloat162float(Khi[(s + 1) * WY_LDK + tid]) + __bfloat162float(Klo[(s + 1) * WY_LDK + tid]);
      Kg[s >> 1] = pack_bf16(k0 * __expf(l63 - lg[s]), k1 * __expf(l63 - lg[s + 1]));
    }
  } else {
    float4* Wv = reinterpret_cast<float4*>(blk + WY_OFF_WVT) + (tid - DH) * (WY_LDV / 4);
#pragma unroll
    for (int s = 0; s < WY_C; s += 4) Wv[s >> 2] = make_float4(w[s], w[s + 1], w[s + 2], w[s + 3]);
  }
  // Qg = gamma_s q_s (from the fp32 rows)
  __nv_bfloat16* Qg = reinterpret_cast<__nv_bfloat16*>(blk + WY_OFF_QG);
  {
    const int col = tid & 127, sh = tid >> 7;
#pragma unroll
    for (int s0 = 0; s0 < WY_C; s0 += 32) {
      float qv[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        const int s = s0 + 2 * u + sh;
        qv[u] = s < valid ? a0[(size_t)s * p.N + hk * DH + col] : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        const int s = s0 + 2 * u + sh;
        Qg[s * WY_LDK + col] = __float2bfloat16(qv[u] * __expf(lg[s]));
      }
    }
  }
  if (tid == 0) *reinterpret_cast<float*>(blk + WY_OFF_GC) = __expf(lg[WY_C - 1]);
}

// the scan's stage: the block's images up to Wv^T, this CTA's half of Wv^T (64 value columns), gamma_63
constexpr int WYB_WV_HALF = (DH / 2) * WY_LDV * 4;
constexpr int WYB_STAGE = WY_OFF_WVT + WYB_WV_HALF + 16;
constexpr int WYB_SMEM = 2 * WYB_STAGE + 64;
static_assert(WYB_STAGE % 128 == 0 || WYB_STAGE % 16 == 0, "stages start on 16-byte boundaries");

// hi and lo bf16 limbs of a pair of fp32 values (x = hi + lo to about 16 bits)
__device__ __forceinline__ void split2(float x, float y, uint32_t& hi, uint32_t& lo) {
  hi = pack_bf16(x, y);
  lo = pack_bf16(x - bf16_lo(hi), y - bf16_hi(hi));
}

__global__ void __launch_bounds__(128, 1) gdn_wy_scan_kernel(const GdnWyParams p) {
  extern __shared__ __align__(128) uint8_t wy_smem[];
  const uint32_t stage0 = smem_u32(wy_smem);
  const uint32_t bar0 = stage0 + 2 * WYB_STAGE;
  const int h = blockIdx.x, half = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int kd = p.n_k * DH;
  const uint8_t* ws = p.ws + (size_t)h * WY_BLOCK;
  const size_t ws_step = (size_t)p.n_v * WY_BLOCK;
  if (tid == 0) {
    mbar_init(bar0, 1);
    mbar_init(bar0 + 8, 1);
    mbar_fence_init();
  }
  __syncthreads();
  pdl_wait();             // the workspace is the previous kernel's output
  pdl_launch_dependents();
  auto fetch = [&](int c, int b) {   // three pieces of chunk c's block into stage b
    const uint32_t dst = stage0 + b * WYB_STAGE, bar = bar0 + 8 * b;
    const uint8_t* src = ws + (size_t)c * ws_step;
    mbar_expect_tx(bar, WYB_STAGE);
    bulk_g2s(dst, src, WY_OFF_WVT, bar);
    bulk_g2s(dst + WY_OFF_WVT, src + WY_OFF_WVT + half * WYB_WV_HALF, WYB_WV_HALF, bar);
    bulk_g2s(dst + WY_OFF_WVT + WYB_WV_HALF, src + WY_OFF_GC, 16, bar);
  };
  if (tid == 0)
    for (int c = 0; c < min(2, p.chunks); ++c) fetch(c, c);
  // ---- S^T[dv][dk] of this warp's 16 value columns as accumulator tiles: st[j] covers dk 8j .. 8j+7;
  // [0], [1]: row dv0 = 16 warp + g, columns 8j + 2t, +1;  [2], [3]: row dv0 + 8
  float st[16][4];
  float* sp = p.state + ((size_t)p.slot * p.n_v + h) * DH * DH;
  const int dvl = 16 * warp + g, dv0 = 64 * half + dvl;     // row within this CTA's half, and within the head
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const int dk = 8 * j + 2 * t;
    st[j][0] = sp[(size_t)dk * DH + dv0];
    st[j][1] = sp[(size_t)(dk + 1) * DH + dv0];
    st[j][2] = sp[(size_t)dk * DH + dv0 + 8];
    st[j][3] = sp[(size_t)(dk + 1) * DH + dv0 + 8];
  }
  bool ok = true;
  for (int c = 0; c < p.chunks; ++c) {
    const int b = c & 1;
    const uint32_t sb = stage0 + b * WYB_STAGE;
    ok = mbar_wait(bar0 + 8 * b, (c >> 1) & 1, ERR_GDN_WAIT);
    if (!__syncthreads_and(ok)) {
      // a copy gave up: wait (bounded) for the other stage's copy, which may still be in flight, and leave the
      // state as it was
      if (tid == 0 && c + 1 < p.chunks) mbar_wait(bar0 + 8 * (b ^ 1), ((c + 1) >> 1) & 1, ERR_GDN_WAIT);
      ok = false;
      break;
    }
    // ---- R1^T = S^T Wk^T and R2^T = S^T Qg^T ([16 dv][64 rows] each), S^T as two bf16 limbs
    float r1[8][4] = {}, r2[8][4] = {};
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      uint32_t ah[4], al[4];
      split2(st[2 * kk][0], st[2 * kk][1], ah[0], al[0]);
      split2(st[2 * kk][2], st[2 * kk][3], ah[1], al[1]);
      split2(st[2 * kk + 1][0], st[2 * kk + 1][1], ah[2], al[2]);
      split2(st[2 * kk + 1][2], st[2 * kk + 1][3], ah[3], al[3]);
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        uint32_t bw[4], bq[4];
        ldsm_x4(ldsm_b_addr(sb + WY_OFF_WK, WY_LDK, 16 * jj, 16 * kk, lane), bw[0], bw[1], bw[2], bw[3]);
        ldsm_x4(ldsm_b_addr(sb + WY_OFF_QG, WY_LDK, 16 * jj, 16 * kk, lane), bq[0], bq[1], bq[2], bq[3]);
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          mma_bf16_16816(r1[2 * jj + u], ah[0], ah[1], ah[2], ah[3], bw[2 * u], bw[2 * u + 1]);
          mma_bf16_16816(r1[2 * jj + u], al[0], al[1], al[2], al[3], bw[2 * u], bw[2 * u + 1]);
          mma_bf16_16816(r2[2 * jj + u], ah[0], ah[1], ah[2], ah[3], bq[2 * u], bq[2 * u + 1]);   // read-out only: one limb
        }
      }
    }
    // ---- U^T = Wv^T - R1^T, as A operand limbs over the chunk's rows (4 k-steps of 16)
    uint32_t uh[4][4], ul[4][4];
    {
      const float* wv = reinterpret_cast<const float*>(wy_smem + b * WYB_STAGE + WY_OFF_WVT);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float2 v0 = *reinterpret_cast<const float2*>(wv + dvl * WY_LDV + 8 * j + 2 * t);
        const float2 v1 = *reinterpret_cast<const float2*>(wv + (dvl + 8) * WY_LDV + 8 * j + 2 * t);
        const float u0 = v0.x - r1[j][0], u1 = v0.y - r1[j][1], u2 = v1.x - r1[j][2], u3 = v1.y - r1[j][3];
        // tile j is the k-half (j & 1) of k-step j >> 1: regs 0, 1 (rows g, g + 8) or 2, 3
        split2(u0, u1, uh[j >> 1][2 * (j & 1)], ul[j >> 1][2 * (j & 1)]);
        split2(u2, u3, uh[j >> 1][2 * (j & 1) + 1], ul[j >> 1][2 * (j & 1) + 1]);
      }
    }
    // ---- O^T = R2^T + U^T P^T  ([16 dv][64 rows])
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        uint32_t bp[4];
        ldsm_x4(ldsm_b_addr(sb + WY_OFF_P, WY_LDP, 16 * jj, 16 * kk, lane), bp[0], bp[1], bp[2], bp[3]);
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          mma_bf16_16816(r2[2 * jj + u], uh[kk][0], uh[kk][1], uh[kk][2], uh[kk][3], bp[2 * u], bp[2 * u + 1]);
        }
      }
    {   // the raw read-out takes v's place in the rows (as the sequential scan leaves it)
      const int row0 = c * WY_C;
      float* ov = p.act + (size_t)row0 * p.N + 2 * kd + h * DH;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int r = 8 * j + 2 * t;
        if (row0 + r < p.M) {
          ov[(size_t)r * p.N + dv0] = r2[j][0];
          ov[(size_t)r * p.N + dv0 + 8] = r2[j][2];
        }
        if (row0 + r + 1 < p.M) {
          ov[(size_t)(r + 1) * p.N + dv0] = r2[j][1];
          ov[(size_t)(r + 1) * p.N + dv0 + 8] = r2[j][3];
        }
      }
    }
    // ---- S^T <- gamma_63 S^T + U^T Kg  (B[k = row s][n = dk] from Kg^T [dk][s])
    {
      const float gc = *reinterpret_cast<const float*>(wy_smem + b * WYB_STAGE + WY_OFF_WVT + WYB_WV_HALF);
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        st[j][0] *= gc; st[j][1] *= gc; st[j][2] *= gc; st[j][3] *= gc;
      }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          uint32_t bk[4];
          ldsm_x4(ldsm_b_addr(sb + WY_OFF_KGT, WY_LDP, 16 * jj, 16 * kk, lane), bk[0], bk[1], bk[2], bk[3]);
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            mma_bf16_16816(st[2 * jj + u], uh[kk][0], uh[kk][1], uh[kk][2], uh[kk][3], bk[2 * u], bk[2 * u + 1]);
            mma_bf16_16816(st[2 * jj + u], ul[kk][0], ul[kk][1], ul[kk][2], ul[kk][3], bk[2 * u], bk[2 * u + 1]);
          }
        }
    }
    __syncthreads();     // every warp is done with this stage: the chunk after the next one may land in it
    if (tid == 0 && c + 2 < p.chunks) fetch(c + 2, b);
  }
  if (!ok) {
    // a copy gave up: wait (bounded) for what may still be in flight, leave the state as it was
    return;
  }
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const int dk = 8 * j + 2 * t;
    sp[(size_t)dk * DH + dv0] = st[j][0];
    sp[(size_t)(dk + 1) * DH + dv0] = st[j][1];
    sp[(size_t)dk * DH + dv0 + 8] = st[j][2];
    sp[(size_t)(dk + 1) * DH + dv0 + 8] = st[j][3];
  }
}

}  // namespace

// A prompt chunk of one slot through a gated delta-net layer's recurrence: act [M][N] (after b2_gdn_conv) is
// overwritten with intermediate values; out [M][n_v * 128] bf16.
extern "C" int b2_gdn_chunk(float* act, int M, int N, int n_k, int n_v, int head_dim, int slot, const float* a_log,
                            const float* dt_bias, const float* norm_w, float eps, float* state, void* out, void* stream) {
  if (head_dim != DH || M < 1 || slot < 0 || n_k < 1 || n_v % n_k != 0 || N != 2 * n_k * DH + 2 * n_v * DH + 2 * n_v) return -1;
  if (N % 4) return -1;   // rows are read in 16-byte pieces
  GdnChunkParams p{act, M, N, n_k, n_v, slot, a_log, dt_bias, norm_w, eps, state, (__nv_bfloat16*)out};
  cudaStream_t st = (cudaStream_t)stream;
  int rc = b2_launch(gdn_prep_kernel, dim3((M * (n_k + 1) + 7) / 8), dim3(256), 0, st, true, p);
  if (rc) return rc;
  rc = b2_launch(gdn_scan_kernel, dim3(n_v), dim3(DH), 0, st, true, p);
  if (rc) return rc;
  return b2_launch(gdn_gate_kernel, dim3((M * n_v + 7) / 8), dim3(256), 0, st, true, p);
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

// The same on the tensor cores, rows in chunks of 64: `ws` holds chunks x n_v blocks of b2_gdn_wy_block_bytes().
extern "C" int b2_gdn_wy_block_bytes() { return WY_BLOCK; }

extern "C" int b2_gdn_chunk_wy(float* act, int M, int N, int n_k, int n_v, int head_dim, int slot, const float* a_log,
                               const float* dt_bias, const float* norm_w, float eps, float* state, void* out, void* ws,
                               long long ws_bytes, void* stream) {
  if (head_dim != DH || M < 1 || slot < 0 || n_k < 1 || n_v % n_k != 0 || N != 2 * n_k * DH + 2 * n_v * DH + 2 * n_v) return -1;
  if (N % 4) return -1;   // rows are read in 16-byte pieces
  const int chunks = (M + WY_C - 1) / WY_C;
  if (!ws || ((uintptr_t)ws & 15) || (long long)chunks * n_v * WY_BLOCK > ws_bytes) return -2;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gdn_wy_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, WYA_SMEM);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gdn_wy_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, WYB_SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  GdnChunkParams p{act, M, N, n_k, n_v, slot, a_log, dt_bias, norm_w, eps, state, (__nv_bfloat16*)out};
  GdnWyParams w{act, M, N, n_k, n_v, slot, chunks, (uint8_t*)ws, state};
  cudaStream_t st = (cudaStream_t)stream;
  int rc = b2_launch(gdn_prep_kernel, dim3((M * (n_k + 1) + 7) / 8), dim3(256), 0, st, true, p);
  if (rc) return rc;
  rc = b2_launch(gdn_wy_prep_kernel, dim3(chunks, n_v), dim3(256), WYA_SMEM, st, true, w);
  if (rc) return rc;
  rc = b2_launch(gdn_wy_scan_kernel, dim3(n_v, 2), dim3(128), WYB_SMEM, st, true, w);
  if (rc) return rc;
  return b2_launch(gdn_gate_kernel, dim3((M * n_v + 7) / 8), dim3(256), 0, st, true, p);
}

B2_DEFINE_STATUS(gdn)
