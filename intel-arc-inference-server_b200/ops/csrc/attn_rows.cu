// Paged decode / verify attention for groups of rows that share a KV cache, on the tensor cores.
//
// Rows of one request (the pending token and its draft rows, or a short prompt chunk) read the same
// keys and values; the per-row kernel (decode_ops.cu: attn_decode_kernel) re-reads them for every row and
// its per-lane loads keep only a few KB in flight.  Here one CTA serves up to 8 rows x GQA query heads
// of one KV head and one KV split:
//   * K and V of up to 128 keys are fetched page by page with tiled TMA copies (16 keys x 64 dims = 2 KB per
//     copy, 128-byte swizzle, all of a batch in flight on one mbarrier): one copy instruction per 2 KB keeps the
//     copy engine fed where one bulk copy per 256-byte row did not (measured: 6 us per 64 KB batch), and the
//     swizzle gives conflict-free ldmatrix without padded rows;
//   * S = Q K^T and O += P V run on mma.m16n8k16 (bf16, fp32 accumulate): warp w owns query rows
//     16 w .. 16 w + 15 (row = token row x GQA + head), K through ldmatrix, V through ldmatrix.trans, P stays
//     in registers (the accumulator layout of S is the A-operand layout of the next MMA);
//   * every row masks the keys beyond its own position (causal inside the group);
//   * a group of at most 16 (32) query rows leaves three (two) of the four warps without rows: those warps
//     then take a quarter (half) of every batch's keys with their own running maximum and sum, and the
//     slices are merged in slice order through shared memory before the split's partial is written;
//   * split-KV partials and the in-kernel merge by the last CTA ("ticket") have the layout and the fixed
//     split order of the per-row kernel, so either kernel can serve a row.
// An int8 cache (one fp32 scale per row) is staged as int8 and expanded to bf16 in shared memory by the thread
// that owns the key, then takes the same path.
// The role of the reference's verify attention (src/kernels/attn_verify_dpas.cl) and of its decode
// attention's GQA packing (src/kernels/attn_v2.cl).
#include "common.cuh"

#include <cstdlib>
#include <mutex>
#include <unordered_map>

using namespace b2;

namespace {

constexpr int CTRL_ROW_REQ = 16, CTRL_ROW_POS = 80, CTRL_ROW_BLOCK = 336;
constexpr int D = 128;
constexpr int KB = 128;          // keys per batch
constexpr int HALFB = KB * 128;  // one tile half: 128 keys x 64 dims (128-byte rows, TMA 128-byte swizzle)
constexpr int TILEB = 2 * HALFB; // a K or V tile: dims 0..63, then dims 64..127
constexpr int kMaxRows = 8;      // token rows per CTA
constexpr int kThreads = 128;    // 4 warps = up to 64 query rows
constexpr int kBtSmem = 256;     // page ids of a split kept in shared memory
constexpr int kPassKeys = 64;    // S of one pass lives in registers: 64 keys = 32 registers

struct AttnRowsParams {
  const __nv_bfloat16* q;  // [M][n_q * D]
  CUtensorMap k_map, v_map;  // the caches [page][n_kv][16][D] as 2-D tensors of rows x D: boxes of 16 rows x 128 bytes
  const float* k_scale;    // int8 form: [page][n_kv][16]
  const float* v_scale;
  const int* block_table;
  const int* ctrl;
  float* o_part;   // [M][n_q][nsplit][D]
  float* ml_part;  // [M][n_q][nsplit][2]
  __nv_bfloat16* out;  // [M][n_q * D]
  int* tickets;        // [M][n_kv]
  int M, n_q, n_kv, gqa, nsplit, max_blocks;
  int nbuf;        // 1: one K / V tile pair; 2: the next batch of keys is fetched while this one is multiplied
  int window;      // > 0: a row attends to its last `window` positions only (sliding-window layers)
  int one_group;   // 1: the host knows that all rows belong to one request at consecutive positions: grid.z counts
                   //    groups of rmax rows, not rows (no CTAs that only find out they are not a group's leader)
  int block;       // 1: a row whose CTRL_ROW_BLOCK word is set attends to ALL positions of its group, those after it
                   //    too (a block drafter's rows see one another: no causal mask inside the block); the group's
                   //    other rows stay causal
  int one_slice;   // 1: never cut a batch's keys over idle warps (a row's bits then do not depend on the group's size)
  int span_pages;  // > 0: every split covers this many pages whatever the context (a row's bits then do not depend
                   // on which rows share its CTA); 0: the group's context is cut into nsplit equal parts
  float scale_log2;
};

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

// byte offset of (key row, dim d) inside a swizzled tile; d a multiple of 8
__device__ __forceinline__ uint32_t tile_off(int row, int d) {
  return (uint32_t)((d >> 6) * HALFB + row * 128 + ((((d & 63) >> 3) ^ (row & 7)) << 4));
}

// NKS: key slices per batch (1, 2 or 4); the four warps are NKS slices x (4 / NKS) groups of 16 query rows.
template <bool I8, int NKS>
__device__ __forceinline__ void attn_rows_body(const AttnRowsParams& p, uint8_t* smem_raw, const int* s_pos, int* s_last_p, int* s_bt,
                                               const int req, const int rows, const int QR, const int ctx_max, const int z) {
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;   // the swizzle pattern repeats every 1024 bytes
  // bf16 form: nbuf pairs of operand tiles.  int8 form: one pair of operand tiles, nbuf pairs of staged int8 rows.
  const int ntile = I8 ? 1 : p.nbuf;
  const uint32_t ks0 = base, vs0 = base + TILEB, tileB = 2 * TILEB;
  const uint32_t k8s0 = base + ntile * tileB, v8s0 = k8s0 + KB * D, stageB = 2 * KB * D;   // int8 rows (128 B each, swizzled)
  const uint32_t bar0 = k8s0 + (I8 ? p.nbuf * stageB : 0);
  float* scratch = reinterpret_cast<float*>(smem_raw + (base - smem_u32(smem_raw)));  // merges reuse the K / V tiles
  int& s_last = *s_last_p;
  constexpr int NRG = 4 / NKS;    // groups of 16 query rows
  constexpr int KW = KB / NKS;              // keys per warp and batch
  constexpr int KS = KW > kPassKeys ? kPassKeys : KW;   // keys per pass over the warp's slice
  constexpr int NJ = KS / 8;                // n8 tiles of keys per pass
  const int kh = blockIdx.x, split = blockIdx.y;   // z: the group's first row
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int rg = warp % NRG, ksl = warp / NRG;
  const int total_pages = (ctx_max + 15) >> 4;
  // sliding window: pages before the first row's window are never read
  const int page0 = p.window > 0 ? max(0, s_pos[z] + 1 - p.window) >> 4 : 0;
  int pps, key0, key1;
  if (p.span_pages > 0) {   // fixed spans of absolute pages, cut at the window
    pps = p.span_pages;
    key0 = max(split * pps, page0) * 16;
    key1 = min(ctx_max, (split + 1) * pps * 16);
  } else {                  // the pages from the window's first one on, in nsplit equal parts
    pps = (total_pages - page0 + p.nsplit - 1) / p.nsplit;
    key0 = (page0 + split * pps) * 16;
    key1 = min(ctx_max, key0 + pps * 16);
  }
  const int* btg = p.block_table + (size_t)req * p.max_blocks + (key0 >> 4);
  // the split's page ids once, so that a batch's copies do not wait for a table load
  const int npg = max(key1 - key0 + 15, 0) >> 4;
  const bool bt_smem = npg <= kBtSmem;
  if (bt_smem)
    for (int i = tid; i < npg; i += kThreads) s_bt[i] = btg[i];
  const int* bt = bt_smem ? s_bt : btg;

  if (tid == 0) {
    mbar_init(bar0, 1);
    mbar_init(bar0 + 8, 1);
    mbar_fence_init();
  }
  __syncthreads();

  // ---- this warp's 16 query rows: (token row, head) of rows g and g + 8, their contexts, Q fragments
  const bool active = rg * 16 < QR;
  int ctx[2] = {0, 0}, wlo[2] = {0, 0};   // a row's keys: wlo <= key < ctx
  uint32_t qa[8][4];
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    const int qr = rg * 16 + g + 8 * hf;
    const bool ok = qr < QR;
    const int m = z + (ok ? qr / p.gqa : 0), h = ok ? qr % p.gqa : 0;
    ctx[hf] = ok ? (s_pos[m] < 0 ? ctx_max : s_pos[m] + 1) : 0;
    wlo[hf] = p.window > 0 ? ctx[hf] - p.window : 0;
    const __nv_bfloat16* qp = p.q + (size_t)m * p.n_q * D + (size_t)(kh * p.gqa + h) * D;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      qa[kk][hf] = ok ? *reinterpret_cast<const uint32_t*>(qp + 16 * kk + 2 * t) : 0u;          // k = 2t, 2t + 1
      qa[kk][2 + hf] = ok ? *reinterpret_cast<const uint32_t*>(qp + 16 * kk + 8 + 2 * t) : 0u;  // k + 8
    }
  }
  float o[16][4];
#pragma unroll
  for (int j = 0; j < 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float mx[2] = {-INFINITY, -INFINITY}, lsum[2] = {0.f, 0.f};

  bool okw = true;
  const int nbatch = (max(key1 - key0, 0) + KB - 1) / KB;
  float ksc[2] = {0.f, 0.f}, vsc[2] = {0.f, 0.f};
  // The pages of batch b into buffer b % nbuf: lanes of warp 0 issue one tiled copy each (page, K or V, half).
  auto issue = [&](int b) {
    const int kb0 = key0 + b * KB, nk = min(KB, key1 - kb0), buf = b % p.nbuf;
    const int npages = (nk + 15) >> 4;
    const uint32_t bar = bar0 + 8 * buf;
    if (tid == 0) mbar_expect_tx(bar, (uint32_t)npages * (I8 ? 4096u : 8192u));
    __syncthreads();
    const uint32_t kt = ks0 + (I8 ? 0 : buf) * tileB, vt = vs0 + (I8 ? 0 : buf) * tileB;
    if (tid < 32) {
      const int pi = tid >> 2, which = tid & 3;   // which: 0 K low dims, 1 K high dims, 2 V low, 3 V high
      if (pi < npages && (!I8 || !(which & 1))) {
        const int page = bt[((kb0 - key0) >> 4) + pi];
        const int row = (page * p.n_kv + kh) * 16;
        const CUtensorMap* map = (which & 2) ? &p.v_map : &p.k_map;
        if (I8)
          tma_load_2d(((which & 2) ? v8s0 : k8s0) + buf * stageB + pi * 2048, map, 0, row, bar);
        else
          tma_load_2d(((which & 2) ? vt : kt) + (which & 1) * HALFB + pi * 2048, map, (which & 1) * 64, row, bar);
      }
    }
    if (I8) {
      if (tid < nk) {
        const int key = kb0 + tid;
        const size_t row = ((size_t)bt[(key - key0) >> 4] * p.n_kv + kh) * 16 + (key & 15);
        ksc[buf] = p.k_scale[row];
        vsc[buf] = p.v_scale[row];
      }
    } else if (tid >= npages * 16) {
      // rows of pages that are not fetched: V must be finite (its products are multiplied by P = 0)
#pragma unroll
      for (int i = 0; i < 16; ++i)
        asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(vt + (i >> 3) * HALFB + tid * 128 + 16 * (i & 7)), "r"(0) : "memory");
    }
  };
  if (p.nbuf == 2 && nbatch > 0) issue(0);
  for (int batch = 0; batch < nbatch; ++batch) {
    const int kb0 = key0 + batch * KB;
    const int nk = min(KB, key1 - kb0);
    const int buf = batch % p.nbuf;
    const uint32_t ks = ks0 + (I8 ? 0 : buf) * tileB, vs = vs0 + (I8 ? 0 : buf) * tileB;
    const uint32_t k8s = k8s0 + buf * stageB, v8s = v8s0 + buf * stageB, bar = bar0 + 8 * buf;
    __syncthreads();  // the previous batch is consumed: its buffer may be refilled
    if (p.nbuf == 2) {
      if (batch + 1 < nbatch) issue(batch + 1);
    } else {
      issue(batch);
    }
    if (okw) okw = mbar_wait(bar, (batch / p.nbuf) & 1, ERR_ATTN_WAIT);
    if (I8) {
      // every thread expands its own key's row: int8 x per-row scale -> bf16 into the operand tiles
      if (tid >= nk) {   // rows without a key: V must be finite (its products are multiplied by P = 0)
#pragma unroll
        for (int i = 0; i < 16; ++i)
          asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(vs + (i >> 3) * HALFB + tid * 128 + 16 * (i & 7)), "r"(0) : "memory");
      }
      if (okw && tid < nk) {
#pragma unroll
        for (int which = 0; which < 2; ++which) {
          const uint32_t src = (which ? v8s : k8s) + tid * D, dst = which ? vs : ks;
          const float sc = which ? vsc[buf] : ksc[buf];
#pragma unroll
          for (int i = 0; i < D / 16; ++i) {
            uint32_t w0, w1, w2, w3;
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w0), "=r"(w1), "=r"(w2), "=r"(w3) : "r"(src + ((i ^ (tid & 7)) << 4)));
            const uint32_t ww[4] = {w0, w1, w2, w3};
            uint32_t o[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              // int8 -> fp32 without the conversion unit (a quarter-rate pipe that capped this loop): the byte, biased
              // to 0..255, dropped into the mantissa of 2^23 is 8388608 + u, and subtracting 8388736 leaves the signed
              // value exactly -- the same floats as (float)(int8_t), so the same products
              const uint32_t u = ww[j] ^ 0x80808080u;
              const float f0 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7540)) - 8388736.f;
              const float f1 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7541)) - 8388736.f;
              const float f2 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7542)) - 8388736.f;
              const float f3 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7543)) - 8388736.f;
              o[2 * j] = pack_bf16(f0 * sc, f1 * sc);
              o[2 * j + 1] = pack_bf16(f2 * sc, f3 * sc);
            }
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst + tile_off(tid, 16 * i)), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]) : "memory");
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst + tile_off(tid, 16 * i + 8)), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7]) : "memory");
          }
        }
      }
    }
    __syncthreads();
    if (!okw || !active) continue;
#pragma unroll 1
    for (int sub = 0; sub < KW / KS; ++sub) {
    const int kofs = ksl * KW + sub * KS;   // this warp's slice of the batch, this pass
    if (kofs >= nk) break;

    // ---- S = Q K^T for this pass's keys: NJ n8 tiles x 8 k16 steps
    float s[NJ][4];
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
      s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < 8; kk += 2) {
        uint32_t b0, b1, b2, b3;
        // matrices: (keys 8j.., d 16kk..), (d 16kk + 8..), (d 16(kk+1)..), (d 16(kk+1) + 8..)
        ldsm_x4(ks + tile_off(kofs + 8 * j + (lane & 7), 16 * kk + 8 * (lane >> 3)), b0, b1, b2, b3);
        mma_bf16_16816(s[j], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], b0, b1);
        mma_bf16_16816(s[j], qa[kk + 1][0], qa[kk + 1][1], qa[kk + 1][2], qa[kk + 1][3], b2, b3);
      }
    }
    // ---- scale, causal mask per row, online softmax (rows g and g + 8 of the tile)
    float mnew[2] = {mx[0], mx[1]};
#pragma unroll
    for (int j = 0; j < NJ; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = kb0 + kofs + 8 * j + 2 * t + (e & 1);
        const int hf = e >> 1;
        const float v = key < ctx[hf] && key < key1 && key >= wlo[hf] ? s[j][e] * p.scale_log2 : -INFINITY;
        s[j][e] = v;
        mnew[hf] = fmaxf(mnew[hf], v);
      }
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      mnew[hf] = fmaxf(mnew[hf], __shfl_xor_sync(0xffffffffu, mnew[hf], 1));
      mnew[hf] = fmaxf(mnew[hf], __shfl_xor_sync(0xffffffffu, mnew[hf], 2));
    }
    float corr[2];
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      corr[hf] = mnew[hf] == -INFINITY ? 1.f : exp2f(mx[hf] - mnew[hf]);   // mx = -inf on the first keys -> 0
      lsum[hf] *= corr[hf];
      mx[hf] = mnew[hf];
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      o[j][0] *= corr[0]; o[j][1] *= corr[0]; o[j][2] *= corr[1]; o[j][3] *= corr[1];
    }
#pragma unroll
    for (int j = 0; j < NJ; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int hf = e >> 1;
        const float pe = mnew[hf] == -INFINITY ? 0.f : exp2f(s[j][e] - mnew[hf]);
        s[j][e] = pe;
        lsum[hf] += pe;
      }
    // ---- O += P V: NJ / 2 k16 steps over this warp's keys, 16 n8 tiles over d
#pragma unroll
    for (int kk = 0; kk < NJ / 2; ++kk) {
      const uint32_t pa0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]), pa1 = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      const uint32_t pa2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]), pa3 = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int jd = 0; jd < 16; jd += 2) {
        uint32_t b0, b1, b2, b3;
        // matrices: (keys 16kk.., d 8jd..), (keys 16kk + 8.., d 8jd..), (keys 16kk.., d 8(jd+1)..), (keys + 8, d 8(jd+1)..)
        const int mi = lane >> 3;
        ldsm_x4_trans(vs + tile_off(kofs + 16 * kk + 8 * (mi & 1) + (lane & 7), 8 * (jd + (mi >> 1))), b0, b1, b2, b3);
        mma_bf16_16816(o[jd], pa0, pa1, pa2, pa3, b0, b1);
        mma_bf16_16816(o[jd + 1], pa0, pa1, pa2, pa3, b2, b3);
      }
    }
    }  // pass
  }

  // ---- this split's partials: unnormalised O against the running maximum, (max, sum)
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    lsum[hf] += __shfl_xor_sync(0xffffffffu, lsum[hf], 1);
    lsum[hf] += __shfl_xor_sync(0xffffffffu, lsum[hf], 2);
  }
  if (NKS > 1) {
    // ---- the slices of a query row meet in shared memory (slice order), then one partial per row is written
    constexpr int SROW = D + 4;   // O, maximum, sum, pad
    __syncthreads();              // every warp is done with the K / V tiles
    if (active) {
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        float* dst = scratch + (size_t)(ksl * (NRG * 16) + rg * 16 + g + 8 * hf) * SROW;
#pragma unroll
        for (int j = 0; j < 16; ++j) *reinterpret_cast<float2*>(dst + 8 * j + 2 * t) = make_float2(o[j][2 * hf], o[j][2 * hf + 1]);
        if (t == 0) {
          dst[D] = mx[hf];
          dst[D + 1] = lsum[hf];
        }
      }
    }
    __syncthreads();
    for (int i = tid; i < QR * (D / 4); i += kThreads) {
      const int qr = i / (D / 4), d4 = (i % (D / 4)) * 4;
      const float* src = scratch + (size_t)qr * SROW;
      float mm = -INFINITY;
#pragma unroll
      for (int sl = 0; sl < NKS; ++sl) mm = fmaxf(mm, src[(size_t)sl * (NRG * 16) * SROW + D]);
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      float lt = 0.f;
#pragma unroll
      for (int sl = 0; sl < NKS; ++sl) {
        const float* ss = src + (size_t)sl * (NRG * 16) * SROW;
        const float ms = ss[D];
        const float c = ms == -INFINITY ? 0.f : exp2f(ms - mm);
        const float4 v = *reinterpret_cast<const float4*>(ss + d4);
        lt = fmaf(ss[D + 1], c, lt);
        acc.x = fmaf(v.x, c, acc.x); acc.y = fmaf(v.y, c, acc.y);
        acc.z = fmaf(v.z, c, acc.z); acc.w = fmaf(v.w, c, acc.w);
      }
      const int m = z + qr / p.gqa, h = qr % p.gqa;
      const size_t pb = ((size_t)m * p.n_q + kh * p.gqa + h) * p.nsplit + split;
      *reinterpret_cast<float4*>(p.o_part + pb * D + d4) = acc;
      if (d4 == 0) {
        p.ml_part[pb * 2] = mm;
        p.ml_part[pb * 2 + 1] = lt;
      }
    }
  } else if (active) {
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int qr = rg * 16 + g + 8 * hf;
      if (qr < QR) {
        const int m = z + qr / p.gqa, h = qr % p.gqa;
        const size_t pb = ((size_t)m * p.n_q + kh * p.gqa + h) * p.nsplit + split;
#pragma unroll
        for (int j = 0; j < 16; ++j)
          *reinterpret_cast<float2*>(p.o_part + pb * D + 8 * j + 2 * t) = make_float2(o[j][2 * hf], o[j][2 * hf + 1]);
        if (t == 0) {
          p.ml_part[pb * 2] = mx[hf];
          p.ml_part[pb * 2 + 1] = lsum[hf];
        }
      }
    }
  }
  if (p.tickets == nullptr) return;   // the caller merges with its own kernel (many rows: more CTAs than one per KV head)
  // ---- the last split CTA of this (group, KV head) merges all splits in split order
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int tk = atomicAdd(&p.tickets[z * p.n_kv + kh], 1);
    s_last = (tk == p.nsplit - 1);
    if (s_last) p.tickets[z * p.n_kv + kh] = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  float* cw = scratch;  // [QR][nsplit] weights of the splits
  for (int i = tid; i < QR; i += kThreads) {
    const int m = z + i / p.gqa, h = i % p.gqa;
    const size_t pb = ((size_t)m * p.n_q + kh * p.gqa + h) * p.nsplit;
    float mm = -INFINITY;
    for (int sp = 0; sp < p.nsplit; ++sp) mm = fmaxf(mm, __ldcg(p.ml_part + (pb + sp) * 2));
    float lt = 0.f;
    for (int sp = 0; sp < p.nsplit; ++sp) {
      const float ms = __ldcg(p.ml_part + (pb + sp) * 2);
      const float c = (ms == -INFINITY) ? 0.f : exp2f(ms - mm);
      lt += __ldcg(p.ml_part + (pb + sp) * 2 + 1) * c;
      cw[i * p.nsplit + sp] = c;
    }
    const float inv = lt > 0.f ? 1.f / lt : 0.f;
    for (int sp = 0; sp < p.nsplit; ++sp) cw[i * p.nsplit + sp] *= inv;
  }
  __syncthreads();
  for (int i = tid; i < QR * (D / 4); i += kThreads) {
    const int qr = i / (D / 4), d4 = (i % (D / 4)) * 4;
    const int m = z + qr / p.gqa, h = qr % p.gqa;
    const float* src = p.o_part + (((size_t)m * p.n_q + kh * p.gqa + h) * p.nsplit) * D + d4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < p.nsplit; s0 += 4) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        v[u] = (s0 + u < p.nsplit) ? __ldcg(reinterpret_cast<const float4*>(src + (size_t)(s0 + u) * D)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float c = (s0 + u < p.nsplit) ? cw[qr * p.nsplit + s0 + u] : 0.f;
        acc.x = fmaf(v[u].x, c, acc.x); acc.y = fmaf(v[u].y, c, acc.y);
        acc.z = fmaf(v[u].z, c, acc.z); acc.w = fmaf(v[u].w, c, acc.w);
      }
    }
    uint2 ob;
    ob.x = pack_bf16(acc.x, acc.y);
    ob.y = pack_bf16(acc.z, acc.w);
    *reinterpret_cast<uint2*>(p.out + ((size_t)m * p.n_q + kh * p.gqa + h) * D + d4) = ob;
  }
}

template <bool I8>
__global__ void __launch_bounds__(kThreads, 2) attn_rows_kernel(const __grid_constant__ AttnRowsParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_last;
  const int z = p.one_group ? blockIdx.z * min(kMaxRows, 64 / p.gqa) : blockIdx.z, tid = threadIdx.x;
  if (tid == 0) {   // the descriptors are launch parameters: their fetch overlaps the wait for the previous kernel
    prefetch_tmap(&p.k_map);
    prefetch_tmap(&p.v_map);
  }
  pdl_wait();
  pdl_launch_dependents();
  // ---- the group: consecutive rows of one request; this CTA is its leader or leaves.  The rows' request
  // ids and positions are read once, in parallel, into shared memory.
  __shared__ int s_req[64], s_pos[64], s_bt[kBtSmem];
  if (tid < 64) {
    s_req[tid] = tid < p.M ? p.ctrl[CTRL_ROW_REQ + tid] : -1;
    s_pos[tid] = tid < p.M ? p.ctrl[CTRL_ROW_POS + tid] : 0;
  }
  const bool blk = p.block && tid < p.M && p.ctrl[CTRL_ROW_BLOCK + tid] != 0;
  __syncthreads();
  const int req = s_req[z];
  int gs = z;
  while (gs > 0 && s_req[gs - 1] == req) --gs;
  const int rmax = min(kMaxRows, 64 / p.gqa);
  if ((z - gs) % rmax != 0) return;
  int rows = 1;
  while (rows < rmax && z + rows < p.M && s_req[z + rows] == req) ++rows;
  const int QR = rows * p.gqa;
  int ctx_max = 0;
  for (int r = 0; r < rows; ++r) ctx_max = max(ctx_max, s_pos[z + r] + 1);
  if (p.block) {           // a block row sees every position of its REQUEST's rows in this step, also those a
                           // sibling CTA serves; its position becomes -1: "all of these keys" for the body
    for (int r = gs; r < p.M && s_req[r] == req; ++r) ctx_max = max(ctx_max, s_pos[r] + 1);
    __syncthreads();
    if (blk) s_pos[tid] = -1;
    __syncthreads();
  }
  if (QR <= 16 && !p.one_slice)
    attn_rows_body<I8, 4>(p, smem_raw, s_pos, &s_last, s_bt, req, rows, QR, ctx_max, z);
  else if (QR <= 32 && !p.one_slice)
    attn_rows_body<I8, 2>(p, smem_raw, s_pos, &s_last, s_bt, req, rows, QR, ctx_max, z);
  else
    attn_rows_body<I8, 1>(p, smem_raw, s_pos, &s_last, s_bt, req, rows, QR, ctx_max, z);
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

// A cache [rows][128 elements] as a 2-D tensor with boxes of 16 rows x 128 bytes (64 bf16 or 128 int8), 128-byte
// swizzle.  The maps of a KV pool never change, so they are kept per (pointer, rows, form).
struct MapKey {
  const void* ptr; uint64_t rows; int i8;
  bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && i8 == o.i8; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const { return std::hash<const void*>()(k.ptr) ^ (size_t)(k.rows * 0x9E3779B97F4A7C15ull) ^ (size_t)k.i8; }
};
int cache_map(CUtensorMap* out, const void* ptr, uint64_t rows, int i8) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> maps;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  const MapKey key{ptr, rows, i8};
  auto it = maps.find(key);
  if (it != maps.end()) {
    *out = it->second;
    return 0;
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -100;
  const cuuint64_t esz = i8 ? 1 : 2;
  cuuint64_t dims[2] = {(cuuint64_t)D, rows};
  cuuint64_t strides[1] = {(cuuint64_t)D * esz};
  cuuint32_t box[2] = {(cuuint32_t)(128 / esz), 16};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  CUresult r = fn(&m, i8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr),
                  dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -101;
  if (maps.size() > 8192) maps.clear();
  maps.emplace(key, m);
  *out = m;
  return 0;
}

}  // namespace

// Rows of a request that follow one another in the control block are served together.  bf16 or int8 KV, head size 128,
// nsplit <= 64, GQA <= 16.  tickets [M][n_kv] (zeroed once; the kernel leaves them zero): the last split CTA of a
// group merges in the kernel; nullptr: the partials are left for b2_attn_merge.
extern "C" int b2_attn_rows(const void* q, const void* k_cache, const void* v_cache, const float* k_scale,
                            const float* v_scale, int kv_int8, const int* block_table,
                            const int* ctrl, float* o_part, float* ml_part, void* out, int* tickets, int M, int n_q,
                            int n_kv, int D_, int nsplit, int max_blocks, float scale, int span_pages, int num_pages,
                            int window, int one_group, void* stream) {
  if (D_ != D || nsplit < 1 || nsplit > 64 || n_q % n_kv != 0 || n_q / n_kv > 16 || M > 64 || num_pages < 1) return -1;
  if (((uintptr_t)k_cache | (uintptr_t)v_cache) & 15) return -4;
  AttnRowsParams p;
  p.q = (const __nv_bfloat16*)q; p.k_scale = k_scale; p.v_scale = v_scale;
  const uint64_t cache_rows = (uint64_t)num_pages * n_kv * 16;
  int mrc = cache_map(&p.k_map, k_cache, cache_rows, kv_int8 ? 1 : 0);
  if (mrc == 0) mrc = cache_map(&p.v_map, v_cache, cache_rows, kv_int8 ? 1 : 0);
  if (mrc) return mrc;
  if (kv_int8 && (!k_scale || !v_scale)) return -3;
  p.block_table = block_table; p.ctrl = ctrl; p.o_part = o_part; p.ml_part = ml_part; p.out = (__nv_bfloat16*)out;
  p.tickets = tickets; p.M = M; p.n_q = n_q; p.n_kv = n_kv; p.gqa = n_q / n_kv; p.nsplit = nsplit; p.max_blocks = max_blocks;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.span_pages = span_pages;
  p.window = window > 0 ? window : 0;
  p.block = window == -1 ? 1 : 0;          // window -1: rows flagged in the control block are non-causal block rows
  p.one_slice = span_pages > 0 ? 1 : 0;   // fixed spans promise bits that do not depend on the group
  if (span_pages > 0 && (long)span_pages * nsplit < max_blocks) return -2;  // fixed spans must cover the longest sequence
  // Two CTAs per SM, each with one batch in flight, hide the copies as well as one CTA that prefetches (measured
  // at depth 32768: 1.10 against 1.12 ms for 8 layers); the second tile pair pays only when the grid leaves SMs
  // with a single CTA and a split holds several batches.  B2_ATTN_NBUF=1|2 overrides.
  const int pages_per_split = span_pages > 0 ? span_pages : (max_blocks + nsplit - 1) / nsplit;
  const int rmax = min(kMaxRows, 64 / (n_q / n_kv));
  const int gz = one_group ? (M + rmax - 1) / rmax : M;     // grid.z: groups, or rows that find their group themselves
  p.one_group = one_group ? 1 : 0;
  p.nbuf = (pages_per_split * 16 > 2 * KB && n_kv * nsplit * gz <= 148) ? 2 : 1;
  static const int nbuf_env = [] { const char* e = getenv("B2_ATTN_NBUF"); return e ? atoi(e) : 0; }();
  if (nbuf_env == 1 || nbuf_env == 2) p.nbuf = nbuf_env;
  const int smem = 1024 + (kv_int8 ? 1 : p.nbuf) * 2 * TILEB + 64 + (kv_int8 ? p.nbuf * 2 * KB * D : 0);
  static int configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    const int most = 1024 + 2 * 2 * TILEB + 64;
    cudaError_t e = cudaFuncSetAttribute(attn_rows_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_rows_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
    if (e != cudaSuccess) return (int)e;
    configured[dev & 63] = 1;
  }
  if (kv_int8)
    return b2_launch(attn_rows_kernel<true>, dim3(n_kv, nsplit, gz), dim3(kThreads), smem, (cudaStream_t)stream, true, p);
  return b2_launch(attn_rows_kernel<false>, dim3(n_kv, nsplit, gz), dim3(kThreads), smem, (cudaStream_t)stream, true, p);
}

B2_DEFINE_STATUS(attnrows)
