// Causal flash attention for prompt chunks over the paged KV cache, on tcgen05 / TMEM (head_dim 128).
//
//   O[r] = softmax( q[r] . K[0 .. pos(r)]^T / sqrt(D) ) V[0 .. pos(r)]      pos(r) = pos0 + r
//
// Stands where the reference has pf_flash_attn / pf_flash_merge (src/kernels/prefill/pf_flash_attn.cl; its pair form
// shares K / V between two query tiles the same way).  One CTA owns TWO query tiles (256 rows) of one query head and
// walks the keys in tiles of 64 (4 pages of 16 tokens); the K and V tiles of the head's KV group are fetched page by
// page with 2-D TMA (box = 16 keys x 64 dims, 128-byte swizzle) straight from the page pool through the sequence's
// block table, double buffered.  Scores S = Q K^T (M 128, N 64) and the output O += P V (M 128, N 128; V is an
// MN-major operand: the cache keeps keys as rows, which is what P V needs along K) live in tensor memory; the
// softmax runs in fp32 with exp2 against a lazily updated reference maximum (a row's accumulator is rescaled in
// place in TMEM only when its maximum moved by more than 2^6); P goes through shared memory as bf16 in the swizzled
// K-major layout.  The roles, the buffers and what was measured to set their numbers are described at the kernel.
// All mbarrier waits are bounded (common.cuh); on a failed wait every role leaves its loop and the CTA still meets
// at the final barrier and frees its tensor memory.
#include "common.cuh"

using namespace b2;

namespace {

constexpr int D = 128;
constexpr int BQ = 128;   // rows of a query tile

struct AttnPfParams {
  const int* block_table;  // this sequence's page table
  int n_q, n_kv;
  int C;        // rows in the chunk
  int pos0;     // absolute position of row 0
  int max_blocks;  // entries in block_table
  int window;      // > 0: a row attends to its last `window` positions only; key tiles before the CTA's first window are skipped
  float scale_log2;
  __nv_bfloat16* out;  // [C][n_q * D]
};

#ifdef B2_ATTN_PROF
// measurement build: cycles per phase, summed over tiles and CTAs by one softmax thread and the MMA thread
__device__ unsigned long long g_attn_prof[16];
#define APROF_T(x) const long long x = clock64()
#define APROF_ADD(i, a, b) atomicAdd(&g_attn_prof[i], (unsigned long long)((b) - (a)))
#else
#define APROF_T(x)
#define APROF_ADD(i, a, b)
#endif

// ---------------------------------------------------------------------------------------------------------------
// One CTA owns TWO query tiles of one head (rows row0 .. row0 + 255) and walks the keys in tiles of 64.
// The two tiles share every K / V tile that comes in (half the L2 traffic per score), and each has its own softmax
// threads -- two per query row, a row's scores read from tensor memory ONCE into registers -- so while one group works
// on its scores the tensor pipe runs the other tile's products:
//     S0(i+1) = Q0 K(i+1)^T   after  O0 += P0(i) V(i),      S1(i+1) = Q1 K(i+1)^T   after  O1 += P1(i) V(i)
// Score buffers are double buffered per tile and handed back as soon as they are in registers, so the tensor pipe
// never waits for a softmax to END before it starts the next scores.  Tensor memory: 4 x 64 score columns + 2 x 128
// accumulator columns = 512.  Shared memory: Q 64 KB, K and V 2 x 16 KB each, P 2 x 2 x 16 KB.
//   warp 0      TMA producer (Q once, then K / V tiles, 4 pages of 16 keys each)
//   warp 1, 18  MMA issuers, one thread per query tile
//   warps 2-9   softmax of tile 0: two threads per query row (32 of the 64 key columns each; TMEM lane quarter =
//               warp & 3), warps 10-17 softmax of tile 1
// The second tile reaches two key tiles further than the first (causal); the first tile's group then leaves early.
constexpr int BK2 = 64;
constexpr int kThreads2 = 608;    // TMA warp, MMA warp of tile 0, 2 tiles x 2 column halves x 4 softmax warps, MMA warp of tile 1
constexpr int kMmaWarp1 = 18;
constexpr int Q2_BYTES = 2 * BQ * D * 2;          // two query tiles, each [2 d-blocks][128 rows][64]
constexpr int KV2_BYTES = BK2 * D * 2;            // 16 KB per K or V tile: [2 d-blocks][64 keys][64]
constexpr int KVS = 4;                            // K / V ring depth (tiles in flight)
constexpr int SMEM2 = Q2_BYTES + 2 * KVS * KV2_BYTES + 1024 + 256 + 2 * 2 * 2 * 128 * 4;   // + alignment, barriers, exchange slots

// smem descriptor for the MN-major V operand: rows are keys (128 B = 64 dims, 128-byte swizzle), 8-key groups are
// 1024 B apart (stride byte offset); the next block of 64 dims is a whole tile half away (leading byte offset).
__device__ __forceinline__ uint64_t make_desc_v2(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)((BK2 * 128) >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

__global__ void __launch_bounds__(kThreads2, 1)
attn_prefill_pair_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, const AttnPfParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_s = base, k_s0 = base + Q2_BYTES, v_s0 = k_s0 + KVS * KV2_BYTES, bars = v_s0 + KVS * KV2_BYTES;
  // barriers (8 bytes each): q_full; k_full, k_empty, v_full, v_empty [KVS each]; per tile w: s_full[w][2],
  // p_full[w], o_done[w][2]
  const uint32_t b_qfull = bars, b_kfull = bars + 8, b_kempty = b_kfull + 8 * KVS, b_vfull = b_kempty + 8 * KVS,
                 b_vempty = b_vfull + 8 * KVS;
  auto b_sfull = [&](int w, int b) { return bars + 136 + (w * 2 + b) * 8; };
  auto b_pfull = [&](int w) { return bars + 168 + w * 8; };
  auto b_odone = [&](int w, int b) { return bars + 184 + (w * 2 + b) * 8; };
  static_assert(8 + 4 * 8 * KVS <= 136, "the ring's barriers end where the tiles' begin");
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_raw + (bars + 224 - smem_u32(smem_raw)));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;   // heavy (late) pairs first
  const int head = blockIdx.y, kh = head / (p.n_q / p.n_kv);
  const int row0 = qt * 2 * BQ;
  // key tiles each query tile needs, counted from the first tile any of the CTA's rows needs
  const int t0 = p.window > 0 ? max(0, p.pos0 + row0 - p.window + 1) / BK2 : 0;
  int n_w[2];
  n_w[0] = (p.pos0 + min(row0 + BQ, p.C) - 1) / BK2 + 1 - t0;
  n_w[1] = row0 + BQ < p.C ? (p.pos0 + min(row0 + 2 * BQ, p.C) - 1) / BK2 + 1 - t0 : 0;
  const int n_all = max(n_w[0], n_w[1]);

  if (threadIdx.x == 0) {
    mbar_init(b_qfull, 1);
    for (int i = 0; i < KVS; ++i) {
      mbar_init(b_kfull + 8 * i, 1);
      mbar_init(b_kempty + 8 * i, 2);     // one arrival per issuing thread
      mbar_init(b_vfull + 8 * i, 1);
      mbar_init(b_vempty + 8 * i, 2);
    }
    for (int w = 0; w < 2; ++w) {
      for (int b = 0; b < 2; ++b) {
        mbar_init(b_sfull(w, b), 1);
        mbar_init(b_odone(w, b), 1);
      }
      mbar_init(b_pfull(w), 256);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  auto t_s = [&](int w, int b) { return tmem_base + (uint32_t)(w * 2 + b) * BK2; };
  auto t_o = [&](int w) { return tmem_base + 256 + (uint32_t)w * D; };

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tmap(&map_q);
      prefetch_tmap(&map_k);
      prefetch_tmap(&map_v);
      const int nq = n_w[1] > 0 ? 2 : 1;
      mbar_expect_tx(b_qfull, nq * BQ * D * 2);
      for (int w = 0; w < nq; ++w) {
        tma_load_2d(q_s + w * (BQ * D * 2), &map_q, head * D, row0 + w * BQ, b_qfull);
        tma_load_2d(q_s + w * (BQ * D * 2) + BQ * 128, &map_q, head * D + 64, row0 + w * BQ, b_qfull);
      }
      bool ok = true;
      int issued = 0;
      for (int i = 0; i < n_all && ok; ++i) {
        const int s = i % KVS, ph = (i / KVS) & 1;
        const uint32_t k_s = k_s0 + s * KV2_BYTES, v_s = v_s0 + s * KV2_BYTES;
        // Always 4 pages: table entries past the sequence point at pages that hold finite data (page 0 is the
        // never-allocated zero page) and those keys are masked out; an unfilled part of a tile could hold NaN bit
        // patterns, and 0 * NaN in P V would poison the row.
        constexpr int n_pages = BK2 / 16;
        int rowc[n_pages];
#pragma unroll
        for (int pg = 0; pg < n_pages; ++pg) {
          const int pi = (t0 + i) * n_pages + pg;
          const int page = pi < p.max_blocks ? __ldg(p.block_table + pi) : 0;
          rowc[pg] = (page * p.n_kv + kh) * 16;
        }
        if (i >= KVS) ok = mbar_wait(b_kempty + 8 * s, ph ^ 1, ERR_ATTN_WAIT);
        if (!ok) break;
        mbar_expect_tx(b_kfull + 8 * s, KV2_BYTES);
#pragma unroll
        for (int pg = 0; pg < n_pages; ++pg) {
          tma_load_2d(k_s + pg * 2048, &map_k, 0, rowc[pg], b_kfull + 8 * s);
          tma_load_2d(k_s + BK2 * 128 + pg * 2048, &map_k, 64, rowc[pg], b_kfull + 8 * s);
        }
        if (i >= KVS) ok = mbar_wait(b_vempty + 8 * s, ph ^ 1, ERR_ATTN_WAIT);
        if (!ok) {
          mbar_wait(b_kfull + 8 * s, ph, ERR_ATTN_WAIT);  // drain the K copies just issued
          break;
        }
        mbar_expect_tx(b_vfull + 8 * s, KV2_BYTES);
#pragma unroll
        for (int pg = 0; pg < n_pages; ++pg) {
          tma_load_2d(v_s + pg * 2048, &map_v, 0, rowc[pg], b_vfull + 8 * s);
          tma_load_2d(v_s + BK2 * 128 + pg * 2048, &map_v, 64, rowc[pg], b_vfull + 8 * s);
        }
        issued = i + 1;
      }
      if (!ok) {
        for (int i = max(0, issued - KVS); i < issued; ++i) {
          mbar_wait(b_kfull + 8 * (i % KVS), (i / KVS) & 1, ERR_ATTN_WAIT);
          mbar_wait(b_vfull + 8 * (i % KVS), (i / KVS) & 1, ERR_ATTN_WAIT);
        }
      }
    }
  } else if (warp == 1 || warp == kMmaWarp1) {
    // One issuing thread per query tile: a lone thread retires a dependent instruction only every ~10 cycles, and
    // with one thread for both tiles the MMA issue (not the tensor pipe, not the softmax) set the pace.  Each thread
    // hands the K / V buffers back for itself, so their "empty" barriers count two arrivals per tile.
    if (lane == 0) {
      const int w = warp == 1 ? 0 : 1;
      const int nt = n_w[w];
      constexpr uint32_t idesc_qk = make_idesc(1, 1, BQ, BK2);
      constexpr uint32_t idesc_pv = make_idesc(1, 1, BQ, D) | (1u << 16);  // B (V) is MN-major
      bool ok = mbar_wait(b_qfull, 0, ERR_ATTN_WAIT);
      // Descriptor words: every 128-byte-swizzled K-major operand shares one high word, V (MN-major) has its own; the
      // low word is (address >> 4) plus the leading-offset field, so an operand piece is one integer add away.
      const uint32_t hi_k = (uint32_t)(make_desc_sw128(0) >> 32), hi_v = (uint32_t)(make_desc_v2(0) >> 32);
      const uint32_t ql = (uint32_t)make_desc_sw128(q_s + w * (BQ * D * 2));
      const uint32_t k_lo0 = (uint32_t)make_desc_sw128(k_s0), v_lo0 = (uint32_t)make_desc_v2(v_s0);   // ring stage 0; a stage is KV2_BYTES >> 4 further
      const uint32_t to = t_o(w);
      auto issue_qk = [&](int j) -> bool {
        const int s = j & 1, ks = j % KVS;
        if (!mbar_wait(b_kfull + 8 * ks, (j / KVS) & 1, ERR_ATTN_WAIT)) return false;
        // the buffer's first 32 columns hold P(j - 2) until that tile's P V product has read them
        if (j >= 2 && !mbar_wait(b_odone(w, s), ((j >> 1) - 1) & 1, ERR_ATTN_WAIT)) return false;
        tc_fence_after();
        const uint32_t kl = k_lo0 + ks * (KV2_BYTES >> 4), ts = t_s(w, s);
#pragma unroll
        for (int k = 0; k < 8; ++k)   // 8 x 16 dims; dims 64.. live in the operands' second block
          umma_f16_w(ts, ql + (((k >> 2) * (BQ * 128) + (k & 3) * 32) >> 4), hi_k,
                     kl + (((k >> 2) * (BK2 * 128) + (k & 3) * 32) >> 4), hi_k, idesc_qk, k != 0);
        tc_commit(b_sfull(w, s));
        tc_commit(b_kempty + 8 * ks);
        return true;
      };
      if (ok && nt > 0) ok = issue_qk(0);
      for (int i = 0; i < n_all && ok; ++i) {
        const int s = i & 1, ks = i % KVS, kph = (i / KVS) & 1;
        if (i >= nt) {
          // the other tile still has key tiles: hand this thread's share of their buffers back as they arrive
          ok = mbar_wait(b_kfull + 8 * ks, kph, ERR_ATTN_WAIT);
          if (ok) mbar_arrive(b_kempty + 8 * ks);
          if (ok) ok = mbar_wait(b_vfull + 8 * ks, kph, ERR_ATTN_WAIT);
          if (ok) mbar_arrive(b_vempty + 8 * ks);
          continue;
        }
        // the tile's NEXT scores first (their buffer was handed back when the tile's threads had tile i - 1 in
        // registers), so that they are ready when its softmax threads finish tile i
        APROF_T(m0);
        if (i + 1 < nt) ok = issue_qk(i + 1);
        if (!ok) break;
        APROF_T(m1);
        // O_w += P_w(i) V(i) once the tile's softmax threads have written P (and rescaled O where a maximum moved)
        ok = mbar_wait(b_pfull(w), i & 1, ERR_ATTN_WAIT);
        APROF_T(m2);
        if (ok) ok = mbar_wait(b_vfull + 8 * ks, kph, ERR_ATTN_WAIT);
        if (!ok) break;
        APROF_T(m3);
        APROF_ADD(8, m0, m1); APROF_ADD(9, m1, m2); APROF_ADD(10, m2, m3); APROF_ADD(11, m0, m0 + 1);
        tc_fence_after();
        const uint32_t vl = v_lo0 + ks * (KV2_BYTES >> 4), tp = t_s(w, s);
#pragma unroll
        for (int k = 0; k < 4; ++k)   // 4 x 16 keys: P comes from tensor memory, 8 columns (16 bf16) per step
          umma_f16_ts_w(to, tp + 8 * k, vl + ((k * 16 * 128) >> 4), hi_v, idesc_pv, (i | k) != 0);
        tc_commit(b_odone(w, s));
        tc_commit(b_vempty + 8 * ks);
      }
    }
  } else {
    // ---------------------------------------------------------- softmax: two threads per query row of tile w
    // (32 of the tile's 64 key columns each; sixteen softmax warps give every scheduler four warps to pick from --
    // with one thread per row the kernel was bound by instruction issue at two warps per scheduler)
    constexpr float kLazy = 6.f;
    const int sw = warp - 2;
    const int w = sw >> 3;                // which query tile
    const int half = (sw >> 2) & 1;       // which 32 of the 64 key columns
    const int quarter = warp & 3;         // TMEM lane quarter this warp may touch
    const int r = quarter * 32 + lane;    // row inside the tile
    const int rowg = row0 + w * BQ + r;   // row inside the chunk
    const int qpos = p.pos0 + rowg;
    const int qlo = p.window > 0 ? qpos - p.window + 1 : 0;   // the row's keys: qlo <= key <= qpos
    const bool row_ok = rowg < p.C;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const int first_pos = p.pos0 + row0 + w * BQ;             // position of the tile's first row
    const int nt = n_w[w];
    // float [tile w][tile parity][half][128 rows]: the halves of a row exchange their maxima (and, at the end, sums)
    const uint32_t xch = bars + 256 + (uint32_t)w * (2 * 2 * 128 * 4);
    float mref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int i = 0; i < nt; ++i) {
      const int sb = i & 1;
      APROF_T(t0_);
      if (ok) ok = mbar_wait(b_sfull(w, sb), (i >> 1) & 1, ERR_ATTN_WAIT);
      tc_fence_after();
      APROF_T(t1_);
      const int key0 = (t0 + i) * BK2 + half * 32;
      // this thread's 32 scores, once: the score buffer goes back to the tensor pipe as soon as they are in registers
      uint32_t v[32];
      if (ok) {
        B2_TMEM_LD_32(t_s(w, sb) + lane_addr + half * 32, v);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = 0xff800000u;
      }
      // only tiles that reach past the tile's first row, or below the window of its last row, need the mask; a
      // masked score becomes -inf and drops out of the maximum and (2^-inf = 0) of the sums below
      if (key0 + 31 > first_pos || (p.window > 0 && key0 < first_pos + BQ - p.window)) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int kj = key0 + j;
          if (kj > qpos || kj < qlo) v[j] = 0xff800000u;
        }
      }
      APROF_T(t2_);
      float ma = __uint_as_float(v[0]), mb = __uint_as_float(v[1]);
#pragma unroll
      for (int j = 2; j < 32; j += 4) {   // three-input maxima, two chains
        asm("max.f32 %0, %0, %1, %2;" : "+f"(ma) : "f"(__uint_as_float(v[j])), "f"(__uint_as_float(v[j + 1])));
        if (j + 3 < 32)
          asm("max.f32 %0, %0, %1, %2;" : "+f"(mb) : "f"(__uint_as_float(v[j + 2])), "f"(__uint_as_float(v[j + 3])));
      }
      float tmax = fmaxf(ma, mb);
      const uint32_t slot = xch + (uint32_t)((sb * 2 + half) * 128 + r) * 4;
      asm volatile("st.shared.f32 [%0], %1;" ::"r"(slot), "f"(tmax) : "memory");
      asm volatile("bar.sync %0, 256;" ::"r"(2 + w) : "memory");
      float other;
      asm volatile("ld.shared.f32 %0, [%1];" : "=f"(other) : "r"(xch + (uint32_t)((sb * 2 + (half ^ 1)) * 128 + r) * 4));
      tmax = fmaxf(tmax, other) * p.scale_log2;
      APROF_T(t3_);
      float alpha = 1.f;
      if (tmax > mref + kLazy || (mref == -INFINITY && tmax > -INFINITY)) {
        alpha = exp2f(mref - tmax);  // 0 when this is the row's first finite maximum
        mref = tmax;
      }
      const float nmref = (mref == -INFINITY) ? 0.f : -mref;
      // P is double buffered: P(i - 2) V(i - 2) must be done before its buffer is overwritten (long done in steady
      // state); only a row whose reference moved must also wait for P(i - 1) V(i - 1) before it rescales the accumulator
      if (i > 0) {
        const bool resc = __any_sync(0xffffffffu, alpha != 1.f);
        if (ok && resc) ok = mbar_wait(b_odone(w, sb ^ 1), ((i - 1) >> 1) & 1, ERR_ATTN_WAIT);
        tc_fence_after();
        if (ok && resc) {
#pragma unroll 1
          for (int c = 2 * half; c < 2 * half + 2; ++c) {   // this thread's half of the row's accumulator
            uint32_t o[32];
            B2_TMEM_LD_32(t_o(w) + lane_addr + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
            B2_TMEM_ST_32(t_o(w) + lane_addr + c * 32, o);
          }
          tmem_st_wait();
        }
      }
      APROF_T(t4_);
      // P = 2^(s * scale - m) as bf16 into shared memory (one 128-byte swizzled row per query row), row sum in fp32;
      // scale-and-shift and the sums run as packed pairs (fma.f32x2 / add.f32x2)
      unsigned long long sc2, nm2, acc0 = 0ull, acc1 = 0ull;
      asm("mov.b64 %0, {%1, %1};" : "=l"(sc2) : "f"(p.scale_log2));
      asm("mov.b64 %0, {%1, %1};" : "=l"(nm2) : "f"(nmref));
      uint32_t pk[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        unsigned long long xy;
        asm("mov.b64 %0, {%1, %2};" : "=l"(xy) : "r"(v[2 * j]), "r"(v[2 * j + 1]));
        asm("fma.rn.f32x2 %0, %0, %1, %2;" : "+l"(xy) : "l"(sc2), "l"(nm2));
        float x0, x1, e0, e1;
        asm("mov.b64 {%0, %1}, %2;" : "=f"(x0), "=f"(x1) : "l"(xy));
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e0) : "f"(x0));
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e1) : "f"(x1));
        unsigned long long ee;
        asm("mov.b64 %0, {%1, %2};" : "=l"(ee) : "f"(e0), "f"(e1));
        if (j & 1)
          asm("add.rn.f32x2 %0, %0, %1;" : "+l"(acc1) : "l"(ee));
        else
          asm("add.rn.f32x2 %0, %0, %1;" : "+l"(acc0) : "l"(ee));
        pk[j] = pack_bf16(e0, e1);
      }
      if (ok) {
        // P goes back into tensor memory, over the first 32 columns of the score buffer it came from (both halves
        // of the row have their scores in registers: they met at the barrier above): 16 packed columns per thread,
        // the A operand of P V without a trip through shared memory
        asm volatile(
            "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15};" ::"r"(pk[0]),
            "r"(pk[1]), "r"(pk[2]), "r"(pk[3]), "r"(pk[4]), "r"(pk[5]), "r"(pk[6]), "r"(pk[7]), "r"(pk[8]), "r"(pk[9]),
            "r"(pk[10]), "r"(pk[11]), "r"(pk[12]), "r"(pk[13]), "r"(pk[14]), "r"(pk[15]),
            "r"(t_s(w, sb) + lane_addr + half * 16)
            : "memory");
        tmem_st_wait();
      }
      {
        float a0, a1, a2, a3;
        asm("mov.b64 {%0, %1}, %2;" : "=f"(a0), "=f"(a1) : "l"(acc0));
        asm("mov.b64 {%0, %1}, %2;" : "=f"(a2), "=f"(a3) : "l"(acc1));
        l = l * alpha + (a0 + a1) + (a2 + a3);   // this half's share of the row sum; the halves are added at the end
      }
      APROF_T(t5_);
      if (ok) {
        tc_fence_before();
        mbar_arrive(b_pfull(w));
      }
#ifdef B2_ATTN_PROF
      if (warp == 2 && lane == 0) {
        APROF_T(t6_);
        APROF_ADD(0, t0_, t1_); APROF_ADD(1, t1_, t2_); APROF_ADD(2, t2_, t3_); APROF_ADD(3, t3_, t4_);
        APROF_ADD(4, t4_, t5_); APROF_ADD(5, t5_, t6_); APROF_ADD(6, t0_, t0_ + 1);
      }
#endif
    }
    // the row sum: both halves (the slot of the parity the last tile did not use)
    if (nt > 0) {
      const int sb = nt & 1;
      asm volatile("st.shared.f32 [%0], %1;" ::"r"(xch + (uint32_t)((sb * 2 + half) * 128 + r) * 4), "f"(l) : "memory");
      asm volatile("bar.sync %0, 256;" ::"r"(2 + w) : "memory");
      float lo;
      asm volatile("ld.shared.f32 %0, [%1];" : "=f"(lo) : "r"(xch + (uint32_t)((sb * 2 + (half ^ 1)) * 128 + r) * 4));
      l += lo;
    }
    // the last product (and, accumulating in issue order, every product before it)
    if (ok && nt > 0) ok = mbar_wait(b_odone(w, (nt - 1) & 1), ((nt - 1) >> 1) & 1, ERR_ATTN_WAIT);
    if (ok && nt > 0) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = p.out + (size_t)rowg * (p.n_q * D) + head * D;
#pragma unroll 1
      for (int c = 2 * half; c < 2 * half + 2; ++c) {
        uint32_t o[32];
        B2_TMEM_LD_32(t_o(w) + lane_addr + c * 32, o);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            *reinterpret_cast<uint4*>(dst + c * 32 + 8 * j) = make_uint4(
                pack_bf16(__uint_as_float(o[8 * j]) * inv, __uint_as_float(o[8 * j + 1]) * inv),
                pack_bf16(__uint_as_float(o[8 * j + 2]) * inv, __uint_as_float(o[8 * j + 3]) * inv),
                pack_bf16(__uint_as_float(o[8 * j + 4]) * inv, __uint_as_float(o[8 * j + 5]) * inv),
                pack_bf16(__uint_as_float(o[8 * j + 6]) * inv, __uint_as_float(o[8 * j + 7]) * inv));
        }
      }
      tc_fence_before();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}
int make_map_bf16(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -100;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -101 - (int)r;
}

}  // namespace

// q: bf16 [C][n_q*128]; k_cache / v_cache: bf16 [num_pages][n_kv][16][128]; block_table: the sequence's
// page ids (device); rows of the chunk sit at positions pos0 .. pos0 + C - 1 and their K / V must
// already be in the cache.
#ifdef B2_ATTN_PROF
extern "C" int b2_attn_prof_read(unsigned long long* out16, int clear) {
  cudaError_t e = cudaMemcpyFromSymbol(out16, g_attn_prof, sizeof(unsigned long long) * 16);
  if (e == cudaSuccess && clear) {
    unsigned long long z[16] = {};
    e = cudaMemcpyToSymbol(g_attn_prof, z, sizeof(z));
  }
  return (int)e;
}
#endif

extern "C" int b2_attn_prefill(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                               void* out, int C, int pos0, int n_q, int n_kv, int head_dim, int num_pages,
                               int max_blocks, float scale, int window, void* stream) {
  if (head_dim != D || n_q % n_kv != 0 || C < 1) return -1;
  CUtensorMap mq, mk, mv;
  int rc = make_map_bf16(&mq, q, (uint64_t)C, (uint64_t)n_q * D, BQ);
  if (rc) return rc;
  rc = make_map_bf16(&mk, k_cache, (uint64_t)num_pages * n_kv * 16, D, 16);
  if (rc) return rc;
  rc = make_map_bf16(&mv, v_cache, (uint64_t)num_pages * n_kv * 16, D, 16);
  if (rc) return rc;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM2);
    if (e != cudaSuccess) return (int)e;
    configured[dev & 63] = true;
  }
  AttnPfParams p;
  p.block_table = block_table; p.n_q = n_q; p.n_kv = n_kv; p.C = C; p.pos0 = pos0; p.max_blocks = max_blocks;
  p.scale_log2 = scale * 1.4426950408889634f; p.out = (__nv_bfloat16*)out;
  p.window = window > 0 ? window : 0;
  dim3 grid((C + 2 * BQ - 1) / (2 * BQ), n_q);
  attn_prefill_pair_kernel<<<grid, kThreads2, SMEM2, (cudaStream_t)stream>>>(mq, mk, mv, p);
  return (int)cudaGetLastError();
}

B2_DEFINE_STATUS(attn)
