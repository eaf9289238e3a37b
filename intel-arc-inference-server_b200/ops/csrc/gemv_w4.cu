// W4A16 weight-streaming kernel for decode and verify rows (M = 1..64).
//
//   out[s][m][n] = sum over the k range of split s of  x[m][k] * (q[n][k] - 8) * scale[n][k/64]
//
// Replaces the reference's decode GEMV (src/kernels/gemv.cl) and its small-M
// weight-stationary GEMMs (src/kernels/gemm_sm.cl, gemm_sm_wide.cl).  Design for
// B200: the step is bound by HBM bandwidth, so the kernel is organised around the
// weight stream.  One producer lane issues 1-D TMA bulk copies of whole W4B
// blocks (4352 B = 128 rows x 64 k of nibbles plus their 128 scales) into an
// 8-stage shared-memory ring guarded by mbarriers; the copies are issued BEFORE
// griddepcontrol.wait, so under programmatic dependent launch the weights of this
// linear are already in flight while the previous kernel finishes.  Eight
// consumer warps each own 16 output rows.  The inner loop of such a kernel is
// bound by instruction issue (expanding nibbles to a floating-point operand costs
// more integer instructions than the copy engine leaves time for), so the
// contraction runs on the integer tensor path instead: the nibbles q = 0..15 are
// used AS unsigned 8-bit operands (a 32-bit word of eight nibbles becomes two
// operand registers with three logic instructions), and each token's activations
// are quantised per 64-k group, while they are staged, to 15-bit integers with one
// fp32 scale, X = 128 X_hi + X_lo, two signed 8-bit limbs.  mma.m16n8k32.u8.s8 takes
// the weights as the 16-row operand and up to 8 tokens as the 8-column operand
// (tokens beyond 8 reuse the weight registers: weight-stationary for any M); four
// MMAs per group and token tile give exact integer sums, the zero point is folded by
// starting the low-limb accumulator at -8 sum(X), and the group's weight scale times
// the token's activation scale is applied in fp32.  The activation grid is 2^-14 of
// the group's largest value: finer than the bf16 the activations arrive in.
// Split-K slices are written separately and summed by the consumer kernel in a
// fixed order: no atomics, bitwise reproducible, and a row's result does not
// depend on M (the split count is a function of N and K only) -- the
// reference's "property R" (src/kernels/gemm_sm.cl:44-50).
#include "common.cuh"
#include "wire.cuh"

using namespace b2;

namespace {

constexpr int kBlockBytes = 4352;
constexpr int CTRL_ROW_REQ = 16, CTRL_ROW_POS = 80;   // control block words (ops/lib.py)
constexpr int kG = 4;  // quantisation groups (W4B blocks) per ring stage: per-stage waits and hand-backs are paid per 17 KB
constexpr int kStages = 4;
constexpr int kStageBytes = kG * kBlockBytes;
constexpr int kRingBytes = kStages * kStageBytes;
constexpr int kConsumerThreads = 256;
constexpr int kThreads = kConsumerThreads + 32;
constexpr int kXBudget = 36 * 1024;  // bytes of staged activations per chunk

struct GemvParams {
  const uint8_t* w;  // [nb][KG][4352]
  const void* x;     // x_mode 0: bf16 [M][ldx];  x_mode 1: fp32 [s_in][M][ldx] (gate/up interleave16)
  float* out;        // [S][M][ldo]
  int M, N, KG, S, gps;
  int ldx, ldo;
  int x_mode, s_in;
  long long x_slice;  // elements between input slices (x_mode 1)
  int rows;           // staged token rows (M rounded up to 1, 2, 4, 8, 16, 32, 64)
  int xcg;            // groups of x staged at a time
  int batches;        // grid.z
  // batched form (MoE decode): blockIdx.z = b selects an expert's weights and that batch's one row
  const int* expert_ids;     // [batches] or nullptr
  int skip_negative;         // batched form: a batch whose expert id is negative does nothing (its CTAs leave at once)
  long long expert_bytes;    // bytes between experts' W4B tensors
  const uint8_t* alt_w;      // batched form: a batch whose expert id is alt_id reads these weights instead of the stack's
  int alt_id;                //   (the shared expert as one more slot of a row: same shapes, its own tensor)
  int x_div;                 // batch b reads activations of batch b / x_div
  long long x_batch_bytes;   // bytes between activation batches
  long long out_batch;       // floats between output batches
  // fused residual fold (producer side): the last split CTA of an n-block adds the slices to the
  // residual stream, writes it back as bf16 and leaves the block's sum of squares for the next norm
  int* fold_tickets;                     // [nb] zeroed counters, or nullptr
  const __nv_bfloat16* fold_resid_in;    // [M][N]
  __nv_bfloat16* fold_resid_out;         // [M][N] (may alias fold_resid_in)
  float* fold_ssq;                       // [M][nb]
  // fused RoPE + KV append (the qkv projection, head size 128, bf16 cache): the last split CTA of an n-block (= one
  // head) sums the slices in split order, rotates q / k heads and writes q rows or the row's slot of the paged cache
  __nv_bfloat16* rope_q;                 // [M][n_q * 128], or nullptr: no such fold
  const float* rope_cos;                 // [position][64]
  const float* rope_sin;
  const int* rope_ctrl;                  // control block: request and position of every row
  const int* rope_block_table;
  int rope_max_blocks, rope_n_q, rope_n_kv;
  __nv_bfloat16* rope_k;                 // the layer's planes [page][n_kv][16][128]
  __nv_bfloat16* rope_v;
  // fused RMSNorm (consumer side, x_mode 2): x = bf16(resid * rsqrt(sum(ssq) / K + eps) * norm_w)
  const float* norm_w;                   // [K]
  const float* norm_ssq;                 // [M][norm_nb]
  int norm_nb;
  float norm_eps;
  // x_mode 3: x is the output of quant_x_kernel, [M][KG][128 B] limbs in operand order; xq_gs [M][KG] {scale, -8 sum X}
  const uint32_t* xq_gs;
  // tensor-parallel fold (row-parallel linear): the n-block's partial sums are pushed into every rank's
  // landing buffer [2 slots][world][tp_mcap][N], flagged per (slot, source rank, n-block), and the fold
  // adds the ranks' parts in rank order.  tp.world <= 1: single GPU.
  Wire tp;
  int tp_mcap;
};

__host__ __device__ inline int stride_words(int xcg) { return xcg * 32 + 4; }  // +4 words: conflict-free B reads

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
__device__ __forceinline__ int consumers_any(uint32_t scratch, bool pred, int tid) {
  // OR of `pred` over the 256 consumer threads (named barrier 1); `scratch` is one shared word
  if (tid == 0) asm volatile("st.shared.u32 [%0], %1;" ::"r"(scratch), "r"(0) : "memory");
  consumer_sync();
  if (pred) asm volatile("st.shared.u32 [%0], %1;" ::"r"(scratch), "r"(1) : "memory");
  consumer_sync();
  int v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(scratch));
  return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ float2 lds64f(uint32_t a) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a));
  return v;
}
__device__ __forceinline__ void sts32(uint32_t a, uint32_t v) {
  asm volatile("st.shared.u32 [%0], %1;" ::"r"(a), "r"(v) : "memory");
}

// One warp-level integer MMA: D (16 x 8, s32) += A (16 x 32, u8, rows) x B (32 x 8, s8, columns).
__device__ __forceinline__ void mma_u8s8_16832(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NG quantisation groups (64 k each, consecutive blocks of one ring stage) of one 16-row tile against
// T token tiles.  A group's activations are 15-bit integers X = 128 X_hi + X_lo with one fp32 scale;
// the nibbles q (0..15) are the unsigned operand as they are, so a 32-bit word of eight nibbles
// becomes two operand registers with three integer instructions.  The low-limb accumulator starts
// at -8 sum(X), which folds the zero point.  2 NG T independent MMA chains are in flight.
template <int T, int NG>
__device__ __forceinline__ void group_mma(float (&acc)[T][4], uint32_t blk_addr, uint32_t w_off, uint32_t sc_off,
                                          const uint32_t (&x_addr)[T], uint32_t gs_addr) {
  constexpr uint32_t kMask = 0x0F0F0F0Fu;
  uint4 wv[NG];
  uint32_t sc2[NG];
#pragma unroll
  for (int q = 0; q < NG; ++q) {
    wv[q] = lds128(blk_addr + q * kBlockBytes + w_off);
    sc2[q] = lds32(blk_addr + q * kBlockBytes + sc_off);  // scales of rows g and g + 8 (stored as a pair)
  }
#pragma unroll
  for (int q = 0; q < NG; ++q) {
    // words 0, 1: k 0..31 of rows g, g + 8;  words 2, 3: k 32..63.  Low nibbles are k 4t + b, high
    // nibbles k 16 + 4t + b of the 32-k step: exactly the a0/a1 and a2/a3 registers of the MMA.
    const uint32_t l0 = wv[q].x & kMask, l1 = wv[q].y & kMask, l2 = wv[q].z & kMask, l3 = wv[q].w & kMask;
    const uint32_t h0 = (wv[q].x >> 4) & kMask, h1 = (wv[q].y >> 4) & kMask;
    const uint32_t h2 = (wv[q].z >> 4) & kMask, h3 = (wv[q].w >> 4) & kMask;
    const __half2 sh = *reinterpret_cast<const __half2*>(&sc2[q]);
    const float s_lo = __low2float(sh), s_hi = __high2float(sh);
#pragma unroll
    for (int tt = 0; tt < T; ++tt) {
      const uint4 xh = lds128(x_addr[tt] + q * 128);       // high limbs: step 0 (b0, b1), step 1 (b0, b1)
      const uint4 xl = lds128(x_addr[tt] + q * 128 + 16);  // low limbs
      // (scale, -8 sum X) of tokens 8 tt + 2t and + 1
      const uint4 gs = lds128(gs_addr + (q * 8 * T + tt * 8) * 8);
      int ih[4] = {0, 0, 0, 0};
      int il[4] = {(int)gs.y, (int)gs.w, (int)gs.y, (int)gs.w};
      mma_u8s8_16832(ih, l0, l1, h0, h1, xh.x, xh.y);
      mma_u8s8_16832(il, l0, l1, h0, h1, xl.x, xl.y);
      mma_u8s8_16832(ih, l2, l3, h2, h3, xh.z, xh.w);
      mma_u8s8_16832(il, l2, l3, h2, h3, xl.z, xl.w);
      const float sx0 = __uint_as_float(gs.x), sx1 = __uint_as_float(gs.z);
      acc[tt][0] = fmaf(s_lo * sx0, (float)(ih[0] * 128 + il[0]), acc[tt][0]);
      acc[tt][1] = fmaf(s_lo * sx1, (float)(ih[1] * 128 + il[1]), acc[tt][1]);
      acc[tt][2] = fmaf(s_hi * sx0, (float)(ih[2] * 128 + il[2]), acc[tt][2]);
      acc[tt][3] = fmaf(s_hi * sx1, (float)(ih[3] * 128 + il[3]), acc[tt][3]);
    }
  }
}

// ---- activation staging, shared by the GEMV's own prologue and the stand-alone quantiser
// Eight activations (one 16-byte vector of a row, k .. k + 7) as packed bf16, by input mode.
__device__ __forceinline__ uint4 stage_load(const GemvParams& p, const uint8_t* xbase, int row, int k, float rinv) {
  uint4 val;
  if (p.x_mode == 0) {
    val = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(xbase) + (size_t)row * p.ldx + k);
  } else if (p.x_mode == 2) {
    const uint4 rv = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(xbase) + (size_t)row * p.ldx + k);
    const float4 w0 = *reinterpret_cast<const float4*>(p.norm_w + k), w1 = *reinterpret_cast<const float4*>(p.norm_w + k + 4);
    val.x = pack_bf16(bf16_lo(rv.x) * rinv * w0.x, bf16_hi(rv.x) * rinv * w0.y);
    val.y = pack_bf16(bf16_lo(rv.y) * rinv * w0.z, bf16_hi(rv.y) * rinv * w0.w);
    val.z = pack_bf16(bf16_lo(rv.z) * rinv * w1.x, bf16_hi(rv.z) * rinv * w1.y);
    val.w = pack_bf16(bf16_lo(rv.w) * rinv * w1.z, bf16_hi(rv.w) * rinv * w1.w);
  } else {
    // SiLU(gate) * up over summed fp32 slices; gate/up alternate in runs of 16
    const float* base = reinterpret_cast<const float*>(xbase) + (size_t)row * p.ldx + (k >> 4) * 32 + (k & 15);
    float gsum[8], usum[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) gsum[i] = usum[i] = 0.f;
#pragma unroll 4
    for (int s = 0; s < p.s_in; ++s) {
      const float4* gp = reinterpret_cast<const float4*>(base + (size_t)s * p.x_slice);
      const float4 g0 = gp[0], g1 = gp[1], u0 = gp[4], u1 = gp[5];
      gsum[0] += g0.x; gsum[1] += g0.y; gsum[2] += g0.z; gsum[3] += g0.w;
      gsum[4] += g1.x; gsum[5] += g1.y; gsum[6] += g1.z; gsum[7] += g1.w;
      usum[0] += u0.x; usum[1] += u0.y; usum[2] += u0.z; usum[3] += u0.w;
      usum[4] += u1.x; usum[5] += u1.y; usum[6] += u1.z; usum[7] += u1.w;
    }
    val.x = pack_bf16(silu(gsum[0]) * usum[0], silu(gsum[1]) * usum[1]);
    val.y = pack_bf16(silu(gsum[2]) * usum[2], silu(gsum[3]) * usum[3]);
    val.z = pack_bf16(silu(gsum[4]) * usum[4], silu(gsum[5]) * usum[5]);
    val.w = pack_bf16(silu(gsum[6]) * usum[6], silu(gsum[7]) * usum[7]);
  }
  return val;
}

// StagedVec / stage_quant / stage_word (the quantiser of one 16-byte vector and its place in a group) live in
// common.cuh: the attention merge uses them too.


template <int T>
__global__ void __launch_bounds__(kThreads, (T <= 2 ? 2 : 1)) gemv_w4_kernel(const GemvParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem0 = (smem_u32(smem_raw) + 127u) & ~127u;
  const uint32_t ring = smem0;
  const uint32_t bars = smem0 + kRingBytes;               // 16 mbarriers
  const uint32_t rinv0 = bars + 128;                      // float [64] per-row 1/rms (x_mode 2)
  const uint32_t gs0 = rinv0 + 256;                       // {float scale, int -8 sum X} [xcg][8 T]
  const uint32_t xs0 = gs0 + ((p.xcg * 8 * T * 8 + 127) & ~127) * (p.x_mode == 3 ? 2 : 1);  // int8 limbs of the rows, in operand order
  const uint32_t full0 = bars, empty0 = bars + 8 * kStages;
  const int strideB = stride_words(p.xcg) * 4;
  // x_mode 3: two activation buffers filled by the producer (barriers live in the unused 1/rms slots)
  const uint32_t xfull0 = rinv0, xempty0 = rinv0 + 16;
  const uint32_t gsB = (p.xcg * 8 * T * 8 + 127) & ~127;   // bytes of one buffer's group scales
  const uint32_t xsB = (uint32_t)p.rows * strideB;          // bytes of one buffer's rows

  // One token tile (M <= 8): the eight consumer warps form two groups of four that take alternate ring stages, a warp
  // owning 32 rows of the block as two 16-row tiles.  Two stages of a CTA (four of an SM) are then in work at a time
  // and a warp has twice the independent MMA chains per wait; with all eight warps on every stage the loop was bound
  // by the latency of one stage's wait -> load -> MMA -> hand-back chain, not by HBM.
  constexpr bool kSplit = T == 1;
  constexpr int RT = kSplit ? 2 : 1;   // row tiles per warp
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nblk = blockIdx.x, split = blockIdx.y;
  if (p.skip_negative) {   // the ids are the previous kernel's output
    pdl_wait();
    if (p.expert_ids[blockIdx.z] < 0) return;
  }
  const int gbeg = split * p.gps;
  const int gend = min(p.KG, gbeg + p.gps);
  const int ngroups = max(0, gend - gbeg);
  const int nstage = (ngroups + kG - 1) / kG;

  if (tid == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(full0 + 8 * i, 1);
      mbar_init(empty0 + 8 * i, kSplit ? 4 : 8);   // warps that hand a stage back
    }
    if (p.x_mode == 3) {
      for (int i = 0; i < 2; ++i) {
        mbar_init(xfull0 + 8 * i, 1);
        mbar_init(xempty0 + 8 * i, 8);
      }
    }
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == 8) {
    // ---------------- producer: stream this CTA's blocks; weights do not depend on the previous kernel
    if (lane == 0) {
      // the expert ids come from the routing kernel before this one: in the batched form the producer
      // has to wait for it too (the dense form streams weights that depend on nothing)
      if (p.expert_ids) pdl_wait();
      const uint8_t* wbase = p.w;
      if (p.expert_ids) {
        const int eid = p.expert_ids[blockIdx.z];
        wbase = (p.alt_w && eid == p.alt_id) ? p.alt_w : p.w + (size_t)eid * p.expert_bytes;
      }
      const uint8_t* src = wbase + ((size_t)nblk * p.KG + gbeg) * kBlockBytes;
      bool ok = true;
      int issued = 0;
      auto issue_w = [&](int i) {
        const int s = i % kStages;
        const int ng = min(kG, ngroups - i * kG);
        const uint32_t bytes = ng * kBlockBytes;
        mbar_expect_tx(full0 + 8 * s, bytes);
        bulk_g2s(ring + s * kStageBytes, src + (size_t)i * kStageBytes, bytes, full0 + 8 * s);
        issued = i + 1;
      };
      if (p.x_mode == 3) {
        // Pre-quantised activations come in by bulk copy too, chunk by chunk into two buffers, so the consumer
        // warps never stage anything.  The first ring stages go out before griddepcontrol.wait (weights depend
        // on nothing); the activations are the previous kernel's output.
        const int first = min(nstage, kStages);
        for (int i = 0; i < first; ++i) issue_w(i);
        pdl_wait();
        const uint8_t* xq = reinterpret_cast<const uint8_t*>(p.x);
        int next_chunk = 0;
        for (int i = 0; i < nstage && ok; ++i) {
          while (ok && next_chunk * p.xcg <= i * kG && next_chunk * p.xcg < ngroups) {   // the chunk this stage reads
            const int c = next_chunk, b = c & 1;
            if (c >= 2) ok = mbar_wait(xempty0 + 8 * b, ((c >> 1) - 1) & 1, ERR_GEMV_EMPTY_WAIT);
            if (!ok) break;
            const int c0 = c * p.xcg, cg = min(p.xcg, ngroups - c0);
            const uint32_t gbytes = (uint32_t)cg * 8 * T * 8, rbytes = (uint32_t)cg * 128;
            mbar_expect_tx(xfull0 + 8 * b, gbytes + rbytes * p.M);
            bulk_g2s(gs0 + b * gsB, reinterpret_cast<const uint8_t*>(p.xq_gs) + (size_t)(gbeg + c0) * 8 * T * 8, gbytes,
                     xfull0 + 8 * b);
            for (int r = 0; r < p.M; ++r)
              bulk_g2s(xs0 + b * xsB + r * strideB, xq + ((size_t)r * p.KG + gbeg + c0) * 128, rbytes, xfull0 + 8 * b);
            ++next_chunk;
          }
          if (!ok) break;
          if (i >= kStages) {
            ok = mbar_wait(empty0 + 8 * (i % kStages), ((i / kStages) - 1) & 1, ERR_GEMV_EMPTY_WAIT);
            if (!ok) break;
            issue_w(i);
          }
        }
        if (!ok)   // wait (bounded) for the activation copies that may still be in flight
          for (int c = max(0, next_chunk - 2); c < next_chunk; ++c) mbar_wait(xfull0 + 8 * (c & 1), (c >> 1) & 1, ERR_GEMV_FULL_WAIT);
      } else {
        for (int i = 0; i < nstage && ok; ++i) {
          if (i >= kStages) ok = mbar_wait(empty0 + 8 * (i % kStages), ((i / kStages) - 1) & 1, ERR_GEMV_EMPTY_WAIT);
          if (!ok) break;
          issue_w(i);
        }
      }
      if (!ok) {
        // drain: wait (bounded) for the copies that were issued and possibly never consumed
        for (int i = max(0, issued - kStages); i < issued; ++i)
          mbar_wait(full0 + 8 * (i % kStages), (i / kStages) & 1, ERR_GEMV_FULL_WAIT);
      }
    }
    pdl_launch_dependents();
    return;
  }

  // ---------------- consumers
  pdl_wait();  // activations come from the previous kernel
  pdl_launch_dependents();

  const uint8_t* xbase = reinterpret_cast<const uint8_t*>(p.x) + (size_t)(blockIdx.z / p.x_div) * p.x_batch_bytes;
  const int g = lane >> 2, t = lane & 3;
  float acc[T * RT][4];
#pragma unroll
  for (int i = 0; i < T * RT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  bool ok = true;
  const int wgrp = kSplit ? (warp >> 2) : 0;            // stage parity this warp serves
  const int row16 = kSplit ? (warp & 3) * 2 : warp;     // first 16-row tile of the warp

  // per-thread constant offsets.  A token row beyond the staged rows aliases the last staged row:
  // column j of the MMA result depends on token j alone, and columns of absent tokens are not stored.
  const uint32_t w_off = row16 * 512 + lane * 16;
  const uint32_t sc_off = 4096 + (row16 * 16 + 2 * g) * 2;
  uint32_t x_row[T];
#pragma unroll
  for (int tt = 0; tt < T; ++tt) x_row[tt] = xs0 + min(tt * 8 + g, p.rows - 1) * strideB + t * 32;
  const uint32_t gs_t = gs0 + 2 * t * 8;

  if (p.x_mode == 2) {
    // 1 / rms of each row from the per-block sums the producing kernel left (summed in block order)
    if (tid < p.M) {
      float ss = 0.f;
      for (int j = 0; j < p.norm_nb; ++j) ss += p.norm_ssq[(size_t)tid * p.norm_nb + j];
      asm volatile("st.shared.f32 [%0], %1;" ::"r"(rinv0 + tid * 4), "f"(rsqrtf(ss / (float)(p.KG * 64) + p.norm_eps)) : "memory");
    }
  }
  const int xvec = p.xcg * 8;  // 16-byte vectors per staged row
  const bool fed = p.x_mode == 3;   // the producer fills the activation buffers: no staging, no CTA barriers
  for (int c0 = 0, chunk = 0; c0 < ngroups; c0 += p.xcg, ++chunk) {
    const int cg = min(p.xcg, ngroups - c0);  // groups in this chunk
    const int xb = fed ? (chunk & 1) : 0;
    if (fed) {
      if (ok) ok = mbar_wait(xfull0 + 8 * xb, (chunk >> 1) & 1, ERR_GEMV_FULL_WAIT);
    } else {
      consumer_sync();
    }
    // ---- stage x[:, k0 : k0 + 64 cg] as bf16, permuted inside each group
    if (!fed) {
      const int k0 = (gbeg + c0) * 64;
      const int nvec = cg * 8;
      const int total = p.rows * xvec;  // a multiple of 8; lanes of a warp stay together in groups of 8
      {
      for (int v0 = 0; v0 < total; v0 += kConsumerThreads) {
        const int v = v0 + tid;
        const int row = v / xvec, col = v - row * xvec;
        uint4 val = make_uint4(0, 0, 0, 0);
        if (v < total && row < p.M && col < nvec) {
          float ri = 1.f;
          if (p.x_mode == 2) asm volatile("ld.shared.f32 %0, [%1];" : "=f"(ri) : "r"(rinv0 + row * 4));
          val = stage_load(p, xbase, row, k0 + col * 8, ri);
        }
        const StagedVec sv = stage_quant(val);
        if (v < total) {
          const int vq = col & 7;
          const uint32_t dst = xs0 + row * strideB + ((col >> 3) * 32 + stage_word(vq)) * 4;
          sts32(dst, sv.w[0]);
          sts32(dst + 16, sv.w[1]);
          sts32(dst + 32, sv.w[2]);
          sts32(dst + 48, sv.w[3]);
          if (vq == 0) {
            const uint32_t ga = gs0 + ((col >> 3) * 8 * T + row) * 8;
            asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(ga), "r"(__float_as_uint(sv.scale)), "r"((uint32_t)sv.m8sum) : "memory");
          }
        }
      }
      }
    }
    if (!fed) consumer_sync();

    // ---- consume the ring stages that cover this chunk.  After a failed wait the warp skips the rest
    // of its work but still meets the others at the named barrier, so a lost copy costs one bounded
    // wait and never a deadlock.
    for (int gi = 0; gi < cg; gi += kG) {
      const int i = (c0 + gi) / kG;  // stage index since kernel start
      if (kSplit && (i & 1) != wgrp) continue;   // the other group's stage
      const int s = i % kStages;
      if (ok) ok = mbar_wait(full0 + 8 * s, (i / kStages) & 1, ERR_GEMV_FULL_WAIT);
      if (!ok) continue;
      const uint32_t st = ring + s * kStageBytes;
      uint32_t xa[T];
#pragma unroll
      for (int tt = 0; tt < T; ++tt) xa[tt] = x_row[tt] + xb * xsB + gi * 128;
      const uint32_t gsa = gs_t + xb * gsB;
      const int ng = min(kG, cg - gi);   // groups of this stage
      constexpr int NGq = T <= 2 ? 2 : 1;   // groups whose MMA chains are interleaved
#pragma unroll 1
      for (int q0 = 0; q0 < ng; q0 += NGq) {
        if (kSplit) {
          float (&a0)[1][4] = *reinterpret_cast<float (*)[1][4]>(&acc[0]);
          float (&a1)[1][4] = *reinterpret_cast<float (*)[1][4]>(&acc[T]);
          const uint32_t (&xa1)[1] = *reinterpret_cast<const uint32_t (*)[1]>(&xa[0]);
          if (q0 + 1 < ng) {
            group_mma<1, 2>(a0, st + q0 * kBlockBytes, w_off, sc_off, xa1, gsa + (gi + q0) * 8 * T * 8);
            group_mma<1, 2>(a1, st + q0 * kBlockBytes, w_off + 512, sc_off + 32, xa1, gsa + (gi + q0) * 8 * T * 8);
          } else {
            group_mma<1, 1>(a0, st + q0 * kBlockBytes, w_off, sc_off, xa1, gsa + (gi + q0) * 8 * T * 8);
            group_mma<1, 1>(a1, st + q0 * kBlockBytes, w_off + 512, sc_off + 32, xa1, gsa + (gi + q0) * 8 * T * 8);
          }
        } else if (NGq == 2 && q0 + 1 < ng) group_mma<T, NGq>(*reinterpret_cast<float (*)[T][4]>(&acc[0]), st + q0 * kBlockBytes, w_off, sc_off, xa, gsa + (gi + q0) * 8 * T * 8);
        else group_mma<T, 1>(*reinterpret_cast<float (*)[T][4]>(&acc[0]), st + q0 * kBlockBytes, w_off, sc_off, xa, gsa + (gi + q0) * 8 * T * 8);
#pragma unroll
        for (int tt = 0; tt < T; ++tt) xa[tt] += 128 * NGq;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + 8 * s);
    }
    if (fed) {
      __syncwarp();
      if (lane == 0) mbar_arrive(xempty0 + 8 * xb);   // this warp is done with the buffer
    }
  }

  // ---- write this split's partial sums
  float* outp = p.out + (size_t)blockIdx.z * p.out_batch + (size_t)split * p.M * p.ldo;
  if (kSplit) {
    // the two groups hold the sums of alternate stages of the same rows: they meet in shared memory (the ring is
    // free now: every stage has been waited for and consumed), group 0 first, so the order of the sum is fixed
    consumer_sync();
    const uint32_t scr = ring + ((warp & 3) * 32 + lane) * 32;   // 8 floats per thread of a group
    if (wgrp == 1) {
#pragma unroll
      for (int h = 0; h < RT; ++h)
        asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(scr + 16 * h), "f"(acc[h][0]), "f"(acc[h][1]), "f"(acc[h][2]), "f"(acc[h][3]) : "memory");
    }
    consumer_sync();
    if (wgrp == 0) {
#pragma unroll
      for (int h = 0; h < RT; ++h) {
        float4 o;
        asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(o.x), "=f"(o.y), "=f"(o.z), "=f"(o.w) : "r"(scr + 16 * h));
        acc[h][0] += o.x; acc[h][1] += o.y; acc[h][2] += o.z; acc[h][3] += o.w;
      }
    }
  }
#pragma unroll
  for (int h = 0; h < RT; ++h) {
    if (kSplit && wgrp != 0) break;
    const int n_lo = nblk * 128 + (row16 + h) * 16 + g, n_hi = n_lo + 8;
#pragma unroll
    for (int tt = 0; tt < T; ++tt) {
      const int m0 = tt * 8 + 2 * t, m1 = m0 + 1;
      const float (&a)[4] = acc[kSplit ? h : tt];
      if (m0 < p.M) {
        if (n_lo < p.N) outp[(size_t)m0 * p.ldo + n_lo] = a[0];
        if (n_hi < p.N) outp[(size_t)m0 * p.ldo + n_hi] = a[2];
      }
      if (m1 < p.M) {
        if (n_lo < p.N) outp[(size_t)m1 * p.ldo + n_lo] = a[1];
        if (n_hi < p.N) outp[(size_t)m1 * p.ldo + n_hi] = a[3];
      }
    }
  }
  if (p.fold_tickets == nullptr) return;
  // ---- fused fold: whichever split CTA of this n-block finishes last sums the slices in split order
  // (so the bits do not depend on which one it is), adds the residual, rounds to bf16 and leaves
  // the sum of squares of its 128 columns.  The counter returns to zero for the next launch.
  __threadfence();
  consumer_sync();
  if (tid == 0) {
    const int tk = atomicAdd(&p.fold_tickets[nblk], 1);
    const int last = tk == p.S - 1;
    if (last) p.fold_tickets[nblk] = 0;
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(rinv0 + 252), "r"(last) : "memory");
  }
  consumer_sync();
  uint32_t is_last;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(is_last) : "r"(rinv0 + 252));
  if (!is_last) return;
  __threadfence();
  const int nb_total = (p.N + 127) / 128;
  const int items = p.M * 128;
  if (p.rope_q != nullptr) {
    // the head's 128 columns of every row, summed in split order, meet in shared memory (the ring is free) so that
    // column d finds its rotate-half partner d +- 64
    for (int idx0 = 0; idx0 < items; idx0 += kConsumerThreads) {
      const int idx = idx0 + tid;
      if (idx < items) {
        const int m = idx >> 7, c = idx & 127, n = nblk * 128 + c;
        float v[16];
#pragma unroll
        for (int sp = 0; sp < 16; ++sp) v[sp] = sp < p.S ? __ldcg(p.out + ((size_t)sp * p.M + m) * p.ldo + n) : 0.f;
        float x = 0.f;
#pragma unroll
        for (int sp = 0; sp < 16; ++sp) x += v[sp];
        asm volatile("st.shared.f32 [%0], %1;" ::"r"(ring + idx * 4), "f"(x) : "memory");
      }
    }
    consumer_sync();
    const int head = nblk;
    for (int idx0 = 0; idx0 < items; idx0 += kConsumerThreads) {
      const int idx = idx0 + tid;
      if (idx >= items) continue;
      const int m = idx >> 7, c = idx & 127, j = c & 63;
      float x1, x2;
      asm volatile("ld.shared.f32 %0, [%1];" : "=f"(x1) : "r"(ring + (m * 128 + j) * 4));
      asm volatile("ld.shared.f32 %0, [%1];" : "=f"(x2) : "r"(ring + (m * 128 + j + 64) * 4));
      const int req = p.rope_ctrl[CTRL_ROW_REQ + m], pos = p.rope_ctrl[CTRL_ROW_POS + m];
      float y;
      if (head < p.rope_n_q + p.rope_n_kv) {
        const float cs = p.rope_cos[(size_t)pos * 64 + j], sn = p.rope_sin[(size_t)pos * 64 + j];
        y = c < 64 ? x1 * cs - x2 * sn : x2 * cs + x1 * sn;
      } else {
        y = c < 64 ? x1 : x2;
      }
      if (head < p.rope_n_q) {
        p.rope_q[(size_t)m * p.rope_n_q * 128 + (size_t)head * 128 + c] = __float2bfloat16(y);
      } else {
        const bool is_v = head >= p.rope_n_q + p.rope_n_kv;
        const int kh = head - p.rope_n_q - (is_v ? p.rope_n_kv : 0);
        const int page = p.rope_block_table[(size_t)req * p.rope_max_blocks + (pos >> 4)];
        __nv_bfloat16* dst = (is_v ? p.rope_v : p.rope_k) + (((size_t)page * p.rope_n_kv + kh) * 16 + (pos & 15)) * 128;
        dst[c] = __float2bfloat16(y);
      }
    }
    return;
  }
  const bool tp = p.tp.world > 1;
  const float* land_me = nullptr;
  if (tp) {
    // ---- all-reduce over NVLink inside the fold.  Step 1: sum the split slices (split order) and store
    // this rank's part of the n-block into every rank's landing buffer, its own included.
    if (tid == 0) {
      const int e = p.tp.epoch[nblk] + 1;   // call number of this n-block: the same on every rank
      p.tp.epoch[nblk] = e;
      asm volatile("st.shared.u32 [%0], %1;" ::"r"(rinv0 + 248), "r"(e) : "memory");
    }
    consumer_sync();
    int epoch;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(epoch) : "r"(rinv0 + 248));
    const int slot = epoch & 1, W = p.tp.world, me = p.tp.rank;
    const size_t src_stride = (size_t)p.tp_mcap * p.N;
    for (int idx0 = 0; idx0 < items; idx0 += kConsumerThreads) {
      const int idx = idx0 + tid;
      const int m = idx >> 7, c = idx & 127, n = nblk * 128 + c;
      if (idx < items && n < p.N) {
        float v[16];
#pragma unroll
        for (int sp = 0; sp < 16; ++sp) v[sp] = sp < p.S ? __ldcg(p.out + ((size_t)sp * p.M + m) * p.ldo + n) : 0.f;
        float part = 0.f;
#pragma unroll
        for (int sp = 0; sp < 16; ++sp) part += v[sp];
        const size_t off = ((size_t)slot * W + me) * src_stride + (size_t)m * p.N + n;
        for (int r = 0; r < W; ++r) wire_land(p.tp, r)[off] = part;
      }
    }
    __threadfence_system();
    consumer_sync();
    // Step 2: flag every peer, then wait (bounded) for every peer's flag in this rank's own memory.
    bool got = true;
    if (tid < W && tid != me) {
      st_release_sys(wire_flags(p.tp, tid) + ((size_t)slot * W + me) * nb_total + nblk, epoch);
      got = wire_wait(wire_flags(p.tp, me) + ((size_t)slot * W + tid) * nb_total + nblk, epoch, (unsigned)(tid << 16 | nblk));
    }
    const int all = consumers_any(rinv0 + 244, !got, tid);
    if (all) return;  // a peer never arrived: status is set, the residual stream is left as it was
    land_me = wire_land(p.tp, me) + (size_t)slot * W * src_stride;
  }
  // one (row, column) per thread; the parts of an element are loaded together and added in a fixed order
  for (int idx0 = 0; idx0 < items; idx0 += kConsumerThreads) {
    const int idx = idx0 + tid;
    const int m = idx >> 7, c = idx & 127, n = nblk * 128 + c;
    float rf = 0.f;
    if (idx < items && n < p.N) {
      float v[16];
      if (tp) {
#pragma unroll
        for (int sp = 0; sp < 16; ++sp)
          v[sp] = sp < p.tp.world ? ld_sys_f32(land_me + (size_t)sp * p.tp_mcap * p.N + (size_t)m * p.N + n) : 0.f;
      } else {
#pragma unroll
        for (int sp = 0; sp < 16; ++sp) v[sp] = sp < p.S ? __ldcg(p.out + ((size_t)sp * p.M + m) * p.ldo + n) : 0.f;
      }
      float r = __bfloat162float(p.fold_resid_in[(size_t)m * p.N + n]);
#pragma unroll
      for (int sp = 0; sp < 16; ++sp) r += v[sp];
      const __nv_bfloat16 rb = __float2bfloat16(r);
      p.fold_resid_out[(size_t)m * p.N + n] = rb;
      rf = __bfloat162float(rb);
    }
    const float ss = warp_sum(rf * rf);  // a warp's 32 columns belong to one row
    if (lane == 0 && idx < items) asm volatile("st.shared.f32 [%0], %1;" ::"r"(ring + (m * 4 + (c >> 5)) * 4), "f"(ss) : "memory");
  }
  consumer_sync();
  if (tid < p.M) {
    float4 q4;
    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(q4.x), "=f"(q4.y), "=f"(q4.z), "=f"(q4.w) : "r"(ring + tid * 16));
    p.fold_ssq[(size_t)tid * nb_total + nblk] = ((q4.x + q4.y) + q4.z) + q4.w;
  }
}


// Stand-alone activation quantiser: what the GEMV's prologue does, once per row instead of once per CTA.
// Worth its launch from a few rows up, where every CTA of the GEMV would otherwise repeat M rows of work.
// grid (ceil(KG / 32), M), 256 threads: one 16-byte vector per thread.
__global__ void __launch_bounds__(256) quant_x_kernel(const GemvParams p, uint8_t* xq, uint32_t* xq_gs) {
  __shared__ float s_rinv;
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.y, tid = threadIdx.x;
  if (p.x_mode == 2) {
    if (tid < 32) {
      float ss = 0.f;
      for (int j = tid; j < p.norm_nb; j += 32) ss += p.norm_ssq[(size_t)row * p.norm_nb + j];
      ss = warp_sum(ss);
      if (tid == 0) s_rinv = rsqrtf(ss / (float)(p.KG * 64) + p.norm_eps);
    }
    __syncthreads();
  }
  const int v = blockIdx.x * 256 + tid;      // vector of the row
  const int group = v >> 3, vq = v & 7;
  uint4 val = make_uint4(0, 0, 0, 0);
  if (group < p.KG) val = stage_load(p, reinterpret_cast<const uint8_t*>(p.x), row, v * 8, p.x_mode == 2 ? s_rinv : 1.f);
  const StagedVec sv = stage_quant(val);
  if (group < p.KG) {
    uint32_t* dst = reinterpret_cast<uint32_t*>(xq + ((size_t)row * p.KG + group) * 128) + stage_word(vq);
    dst[0] = sv.w[0];
    dst[4] = sv.w[1];
    dst[8] = sv.w[2];
    dst[12] = sv.w[3];
    if (vq == 0) {   // [group][8 T token slots]: a chunk of groups is one contiguous block for the GEMV's bulk copy
      xq_gs[((size_t)group * p.rows + row) * 2] = __float_as_uint(sv.scale);
      xq_gs[((size_t)group * p.rows + row) * 2 + 1] = (uint32_t)sv.m8sum;
    }
  }
}

template <int T>
int launch_t(GemvParams& p, cudaStream_t stream) {
  // staged rows and chunk length: as much of the split's k range as fits the activation budget
  int rows = 1;
  while (rows < p.M) rows *= 2;
  p.rows = rows;
  int xcg = (kXBudget / (rows * 2) - 8) / 64;
  xcg &= ~(kG - 1);
  if (xcg > 160) xcg = 160;   // keeps two CTAs per SM at one staged row
  if (p.x_mode == 3) xcg = (xcg / 2) & ~(kG - 1);   // two buffers
  if (xcg > p.gps) xcg = p.gps;
  if (xcg < kG) xcg = kG;
  p.xcg = xcg;
  const int nbuf = p.x_mode == 3 ? 2 : 1;
  const int smem = 128 + kRingBytes + 128 + 256 + nbuf * (((xcg * 8 * T * 8 + 127) & ~127) + rows * stride_words(xcg) * 4);
  static int configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured[dev & 63] < smem) {
    int want = 128 + kRingBytes + 128 + 256 + 16384 + kXBudget + 4096;
    if (want < smem) want = smem;   // many rows with two activation buffers of at least one stage's groups each
    if (want > 232448) return -7;
    cudaError_t e = cudaFuncSetAttribute(gemv_w4_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, want);
    if (e != cudaSuccess) return (int)e;
    configured[dev & 63] = want;
  }
  dim3 grid((p.N + 127) / 128, p.S, p.batches);
  return b2_launch(gemv_w4_kernel<T>, grid, dim3(kThreads), smem, stream, true, p);
}

}  // namespace

// Number of k splits: a function of (N, K) only, so that a row's bits do not depend on M.
// The grid (N/128 x splits) is sized to one wave of 296 CTA slots (148 SMs x 2 resident CTAs):
// a second, partly filled wave would cost a full stream latency for a fraction of the work.
extern "C" int b2_gemv_w4_splits(int N, int K) {
  const int nb = (N + 127) / 128, kg = K / 64;
  int s = 296 / nb;
  int smax = kg / 4;  // at least 4 groups (256 k, two ring stages) per split
  if (smax < 1) smax = 1;
  if (s > smax) s = smax;
  if (s > 16) s = 16;
  if (s < 1) s = 1;
  return s;
}

extern "C" int b2_gemv_w4(const void* w4b, const void* x, float* out, int M, int N, int K, int S, int ldx, int ldo,
                          int x_mode, int s_in, long long x_slice, void* stream) {
  if (M < 1 || M > 64 || K % 64 != 0 || S < 1) return -1;
  if (x_mode == 0 && (ldx % 8 != 0)) return -2;
  if (x_mode == 1 && (ldx % 4 != 0 || x_slice % 4 != 0)) return -2;
  GemvParams p;
  p.w = reinterpret_cast<const uint8_t*>(w4b);
  p.x = x;
  p.out = out;
  p.batches = 1; p.expert_ids = nullptr; p.skip_negative = 0; p.expert_bytes = 0; p.x_div = 1; p.x_batch_bytes = 0; p.out_batch = 0;
  p.fold_tickets = nullptr; p.fold_resid_in = nullptr; p.fold_resid_out = nullptr; p.fold_ssq = nullptr; p.rope_q = nullptr;
  p.norm_w = nullptr; p.norm_ssq = nullptr; p.norm_nb = 0; p.norm_eps = 0.f;
  p.tp.table = nullptr; p.tp.epoch = nullptr; p.tp.world = 0; p.tp.rank = 0; p.tp_mcap = 0; p.xq_gs = nullptr;
  p.M = M; p.N = N; p.KG = K / 64; p.S = S;
  p.gps = (p.KG + S - 1) / S;
  if (p.gps % kG != 0) p.gps += kG - p.gps % kG;   // splits start on a stage boundary
  p.ldx = ldx; p.ldo = ldo; p.x_mode = x_mode; p.s_in = s_in; p.x_slice = x_slice;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (M <= 8) return launch_t<1>(p, st);
  if (M <= 16) return launch_t<2>(p, st);
  if (M <= 32) return launch_t<4>(p, st);
  return launch_t<8>(p, st);
}

// Fused form for the dense decode layers.  x_mode 2 normalises the residual stream while staging it
// (norm_w, norm_ssq [M][K/128], eps); fold_* make the kernel's last split CTA per n-block add the
// slices to the residual (N must be the residual width) and leave the per-block sums of squares.
extern "C" int b2_gemv_w4_fused(const void* w4b, const void* x, float* out, int M, int N, int K, int S, int ldx,
                                int x_mode, int s_in, long long x_slice, const float* norm_w, const float* norm_ssq,
                                float norm_eps, int* fold_tickets, const void* fold_resid_in, void* fold_resid_out,
                                float* fold_ssq, const void* tp_table, int* tp_epoch, int tp_world, int tp_rank,
                                int tp_mcap, void* stream) {
  if (M < 1 || M > 64 || K % 64 != 0 || S < 1) return -1;
  if (x_mode == 2 && (K % 128 != 0 || !norm_w || !norm_ssq)) return -2;
  if (x_mode == 3 && !norm_ssq) return -2;
  if (tp_world > 1 && (tp_world > kMaxRanks || tp_rank < 0 || tp_rank >= tp_world || !tp_table || !tp_epoch ||
                       !fold_tickets || M > tp_mcap))
    return -3;
  GemvParams p;
  p.w = reinterpret_cast<const uint8_t*>(w4b);
  p.x = x;
  p.out = out;
  p.M = M; p.N = N; p.KG = K / 64; p.S = S;
  p.gps = (p.KG + S - 1) / S;
  if (p.gps % kG != 0) p.gps += kG - p.gps % kG;
  p.ldx = ldx; p.ldo = N; p.x_mode = x_mode; p.s_in = s_in; p.x_slice = x_slice;
  p.batches = 1; p.expert_ids = nullptr; p.skip_negative = 0; p.expert_bytes = 0; p.x_div = 1; p.x_batch_bytes = 0; p.out_batch = 0;
  p.rope_q = nullptr;
  p.fold_tickets = fold_tickets; p.fold_resid_in = (const __nv_bfloat16*)fold_resid_in;
  p.fold_resid_out = (__nv_bfloat16*)fold_resid_out; p.fold_ssq = fold_ssq;
  p.norm_w = norm_w; p.norm_ssq = norm_ssq; p.norm_nb = K / 128; p.norm_eps = norm_eps;
  p.tp.table = (const unsigned long long*)tp_table; p.tp.epoch = tp_epoch; p.tp.world = tp_world; p.tp.rank = tp_rank;
  p.tp_mcap = tp_mcap;
  p.xq_gs = reinterpret_cast<const uint32_t*>(norm_ssq);   // x_mode 3: the group scales ride in the norm_ssq slot
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (M <= 8) return launch_t<1>(p, st);
  if (M <= 16) return launch_t<2>(p, st);
  if (M <= 32) return launch_t<4>(p, st);
  return launch_t<8>(p, st);
}

// The qkv projection with the RoPE / KV-append fold: heads of 128 dims, bf16 cache planes of the layer.  x_mode 0
// (normalised rows), 2 (residual rows + RMSNorm) or 3 (pre-quantised rows, group scales in norm_ssq).
extern "C" int b2_gemv_w4_qkv_rope(const void* w4b, const void* x, float* out, int M, int K, int S, int ldx, int x_mode,
                                   const float* norm_w, const float* norm_ssq, float norm_eps, int* tickets, void* q_out,
                                   const float* cos_t, const float* sin_t, const int* ctrl, const int* block_table,
                                   int max_blocks, int n_q, int n_kv, void* k_plane, void* v_plane, void* stream) {
  if (M < 1 || M > 64 || K % 64 != 0 || S < 1 || S > 16 || !tickets || !q_out || n_q < 1 || n_kv < 1) return -1;
  if (x_mode == 2 && (K % 128 != 0 || !norm_w || !norm_ssq)) return -2;
  if (x_mode == 3 && !norm_ssq) return -2;
  GemvParams p;
  p.w = reinterpret_cast<const uint8_t*>(w4b);
  p.x = x;
  p.out = out;
  p.M = M; p.N = (n_q + 2 * n_kv) * 128; p.KG = K / 64; p.S = S;
  p.gps = (p.KG + S - 1) / S;
  if (p.gps % kG != 0) p.gps += kG - p.gps % kG;
  p.ldx = ldx; p.ldo = p.N; p.x_mode = x_mode; p.s_in = 1; p.x_slice = 0;
  p.batches = 1; p.expert_ids = nullptr; p.skip_negative = 0; p.expert_bytes = 0; p.x_div = 1; p.x_batch_bytes = 0; p.out_batch = 0;
  p.fold_tickets = tickets; p.fold_resid_in = nullptr; p.fold_resid_out = nullptr; p.fold_ssq = nullptr;
  p.norm_w = norm_w; p.norm_ssq = norm_ssq; p.norm_nb = K / 128; p.norm_eps = norm_eps;
  p.tp.table = nullptr; p.tp.epoch = nullptr; p.tp.world = 0; p.tp.rank = 0; p.tp_mcap = 0;
  p.xq_gs = reinterpret_cast<const uint32_t*>(norm_ssq);
  p.rope_q = (__nv_bfloat16*)q_out; p.rope_cos = cos_t; p.rope_sin = sin_t; p.rope_ctrl = ctrl;
  p.rope_block_table = block_table; p.rope_max_blocks = max_blocks; p.rope_n_q = n_q; p.rope_n_kv = n_kv;
  p.rope_k = (__nv_bfloat16*)k_plane; p.rope_v = (__nv_bfloat16*)v_plane;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (M <= 8) return launch_t<1>(p, st);
  if (M <= 16) return launch_t<2>(p, st);
  if (M <= 32) return launch_t<4>(p, st);
  return launch_t<8>(p, st);
}

// Batched form for MoE decode: batch b (one row) uses the weights of expert expert_ids[b] out of a stack of
// equally shaped W4B tensors, reads the activations of batch b / x_div and writes out[b][S][N].
static int gemv_w4_experts_impl(const void* w4b_stack, long long expert_bytes, const int* expert_ids, int batches,
                                const void* x, int x_div, long long x_batch_bytes, float* out, int N, int K, int S,
                                int ldx, int x_mode, int s_in, long long x_slice, int skip_negative, void* stream,
                                const void* alt_w = nullptr, int alt_id = -1) {
  if (batches < 1 || batches > 65535 || K % 64 != 0 || S < 1 || x_div < 1) return -1;
  GemvParams p;
  p.alt_w = reinterpret_cast<const uint8_t*>(alt_w);
  p.alt_id = alt_id;
  p.w = reinterpret_cast<const uint8_t*>(w4b_stack);
  p.x = x;
  p.out = out;
  p.M = 1; p.N = N; p.KG = K / 64; p.S = S;
  p.gps = (p.KG + S - 1) / S;
  if (p.gps % kG != 0) p.gps += kG - p.gps % kG;
  p.ldx = ldx; p.ldo = N; p.x_mode = x_mode; p.s_in = s_in; p.x_slice = x_slice;
  p.batches = batches; p.expert_ids = expert_ids; p.expert_bytes = expert_bytes; p.x_div = x_div; p.skip_negative = skip_negative;
  p.x_batch_bytes = x_batch_bytes; p.out_batch = (long long)S * N;
  p.fold_tickets = nullptr; p.fold_resid_in = nullptr; p.fold_resid_out = nullptr; p.fold_ssq = nullptr; p.rope_q = nullptr;
  p.norm_w = nullptr; p.norm_ssq = nullptr; p.norm_nb = 0; p.norm_eps = 0.f;
  p.tp.table = nullptr; p.tp.epoch = nullptr; p.tp.world = 0; p.tp.rank = 0; p.tp_mcap = 0; p.xq_gs = nullptr;
  return launch_t<1>(p, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int b2_gemv_w4_experts(const void* w4b_stack, long long expert_bytes, const int* expert_ids, int batches,
                                  const void* x, int x_div, long long x_batch_bytes, float* out, int N, int K, int S,
                                  int ldx, int x_mode, int s_in, long long x_slice, void* stream) {
  return gemv_w4_experts_impl(w4b_stack, expert_bytes, expert_ids, batches, x, x_div, x_batch_bytes, out, N, K, S, ldx, x_mode,
                              s_in, x_slice, 0, stream);
}
// The same with batches whose expert id is negative skipped (an owner's receive buffer is sized for the worst case).
extern "C" int b2_gemv_w4_experts_sparse(const void* w4b_stack, long long expert_bytes, const int* expert_ids, int batches,
                                         const void* x, int x_div, long long x_batch_bytes, float* out, int N, int K, int S,
                                         int ldx, int x_mode, int s_in, long long x_slice, void* stream) {
  return gemv_w4_experts_impl(w4b_stack, expert_bytes, expert_ids, batches, x, x_div, x_batch_bytes, out, N, K, S, ldx, x_mode,
                              s_in, x_slice, 1, stream);
}

// The same with one more weight tensor outside the stack: batches whose id is alt_id read alt_w (the shared expert
// as slot k of every row).
extern "C" int b2_gemv_w4_experts_alt(const void* w4b_stack, long long expert_bytes, const int* expert_ids, int batches,
                                      const void* x, int x_div, long long x_batch_bytes, float* out, int N, int K, int S,
                                      int ldx, int x_mode, int s_in, long long x_slice, const void* alt_w, int alt_id,
                                      void* stream) {
  return gemv_w4_experts_impl(w4b_stack, expert_bytes, expert_ids, batches, x, x_div, x_batch_bytes, out, N, K, S, ldx, x_mode,
                              s_in, x_slice, 0, stream, alt_w, alt_id);
}

// Quantise activation rows for x_mode 3.  Input modes as the GEMV's (0 bf16 rows, 1 SiLU*up of fp32 slices,
// 2 residual rows with RMSNorm); xq is [M][K / 64][128] bytes, xq_gs [K / 64][8, 16, 32 or 64 token slots][2] words.
extern "C" int b2_quant_x(const void* x, int M, int K, int ldx, int x_mode, int s_in, long long x_slice,
                          const float* norm_w, const float* norm_ssq, float norm_eps, void* xq, void* xq_gs, void* stream) {
  if (M < 1 || K % 64 != 0 || x_mode < 0 || x_mode > 2) return -1;
  if (x_mode == 2 && (K % 128 != 0 || !norm_w || !norm_ssq)) return -2;
  GemvParams p = {};
  p.x = x; p.M = M; p.KG = K / 64; p.ldx = ldx; p.x_mode = x_mode; p.s_in = s_in; p.x_slice = x_slice;
  p.norm_w = norm_w; p.norm_ssq = norm_ssq; p.norm_nb = K / 128; p.norm_eps = norm_eps;
  p.rows = M <= 8 ? 8 : (M <= 16 ? 16 : (M <= 32 ? 32 : 64));   // token slots per group in xq_gs (8 x the GEMV's tile count)
  dim3 grid((p.KG * 8 + 255) / 256, M);
  return b2_launch(quant_x_kernel, grid, dim3(256), 0, (cudaStream_t)stream, true, p, (uint8_t*)xq, (uint32_t*)xq_gs);
}

B2_DEFINE_STATUS(gemv)
