// Paged decode / verify attention for groups of rows that share a KV cache, on the tensor cores.
//
// Rows of one request (the pending token and its draft rows, or a short prompt chunk) read the same
// keys and values; the per-row kernel (decode_ops.cu: attn_decode_kernel) re-reads them for every row and
// its per-lane loads keep only a few KB in flight.  Here one CTA serves up to 8 rows x GQA query heads
// of one KV head and one KV split:
//   * K and V rows of up to 128 keys are fetched with one bulk copy each (cp.async.bulk, 256 B per row, all
//     in flight at once, one mbarrier) into padded shared-memory rows (272 B: conflict-free ldmatrix);
//   * S = Q K^T and O += P V run on mma.m16n8k16 (bf16, fp32 accumulate): warp w owns query rows
//     16 w .. 16 w + 15 (row = token row x GQA + head), K through ldmatrix, V through ldmatrix.trans, P stays
//     in registers (the accumulator layout of S is the A-operand layout of the next MMA);
//   * every row masks the keys beyond its own position (causal inside the group);
//   * split-KV partials and the in-kernel merge by the last CTA ("ticket") have the layout and the fixed
//     split order of the per-row kernel, so either kernel can serve a row.
// An int8 cache (one fp32 scale per row) is staged as int8 and expanded to bf16 in shared memory by the thread
// that owns the key, then takes the same path.
// The role of the reference's verify attention (src/kernels/attn_verify_dpas.cl) and of its decode
// attention's GQA packing (src/kernels/attn_v2.cl).
#include "common.cuh"

using namespace b2;

namespace {

constexpr int CTRL_ROW_REQ = 16, CTRL_ROW_POS = 80;
constexpr int D = 128;
constexpr int KB = 128;          // keys per batch
constexpr int ROWB = 272;        // bytes per staged K / V row (256 + 16 pad)
constexpr int kMaxRows = 8;      // token rows per CTA
constexpr int kThreads = 128;    // 4 warps = up to 64 query rows

struct AttnRowsParams {
  const __nv_bfloat16* q;  // [M][n_q * D]
  const void* k_cache;     // bf16 or int8 [page][n_kv][16][D]
  const void* v_cache;
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

template <bool I8>
__global__ void __launch_bounds__(kThreads) attn_rows_kernel(const AttnRowsParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 127u) & ~127u;
  // bf16 form: nbuf pairs of operand tiles.  int8 form: one pair of operand tiles, nbuf pairs of staged int8 rows.
  const int ntile = I8 ? 1 : p.nbuf;
  const uint32_t ks0 = base, vs0 = base + KB * ROWB, tileB = 2 * KB * ROWB;
  const uint32_t bar0 = base + ntile * tileB;
  const uint32_t k8s0 = bar0 + 64, v8s0 = k8s0 + KB * D, stageB = 2 * KB * D;   // int8 rows before expansion (128 B each)
  float* scratch = reinterpret_cast<float*>(smem_raw + (base - smem_u32(smem_raw)));  // merge reuses the K / V tiles
  __shared__ int s_last;
  pdl_wait();
  pdl_launch_dependents();
  const int kh = blockIdx.x, split = blockIdx.y, z = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  // ---- the group: consecutive rows of one request; this CTA is its leader or leaves.  The rows' request
  // ids and positions are read once, in parallel, into shared memory.
  __shared__ int s_req[64], s_pos[64];
  if (tid < 64) {
    s_req[tid] = tid < p.M ? p.ctrl[CTRL_ROW_REQ + tid] : -1;
    s_pos[tid] = tid < p.M ? p.ctrl[CTRL_ROW_POS + tid] : 0;
  }
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
  const int total_pages = (ctx_max + 15) >> 4;
  const int pps = p.span_pages > 0 ? p.span_pages : (total_pages + p.nsplit - 1) / p.nsplit;
  const int key0 = split * pps * 16, key1 = min(ctx_max, (split + 1) * pps * 16);
  const int* bt = p.block_table + (size_t)req * p.max_blocks;

  if (tid == 0) {
    mbar_init(bar0, 1);
    mbar_init(bar0 + 8, 1);
    mbar_fence_init();
  }
  __syncthreads();

  // ---- this warp's 16 query rows: (token row, head) of rows g and g + 8, their contexts, Q fragments
  const bool active = warp * 16 < QR;
  int ctx[2] = {0, 0};
  uint32_t qa[8][4];
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    const int qr = warp * 16 + g + 8 * hf;
    const bool ok = qr < QR;
    const int m = z + (ok ? qr / p.gqa : 0), h = ok ? qr % p.gqa : 0;
    ctx[hf] = ok ? s_pos[m] + 1 : 0;
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
  // One bulk copy per key row into buffer b % nbuf (every thread fetches the row of its own key).
  auto issue = [&](int b) {
    const int kb0 = key0 + b * KB, nk = min(KB, key1 - kb0), buf = b % p.nbuf;
    const uint32_t bar = bar0 + 8 * buf;
    if (tid == 0) mbar_expect_tx(bar, (uint32_t)nk * (I8 ? 256u : 512u));
    __syncthreads();
    const uint32_t vt = vs0 + (I8 ? 0 : buf) * tileB;
    if (tid < nk) {
      const int key = kb0 + tid;
      const int page = bt[key >> 4], slot = key & 15;
      const size_t row = ((size_t)page * p.n_kv + kh) * 16 + slot;
      if (I8) {
        bulk_g2s(k8s0 + buf * stageB + tid * D, reinterpret_cast<const int8_t*>(p.k_cache) + row * D, D, bar);
        bulk_g2s(v8s0 + buf * stageB + tid * D, reinterpret_cast<const int8_t*>(p.v_cache) + row * D, D, bar);
        ksc[buf] = p.k_scale[row];
        vsc[buf] = p.v_scale[row];
      } else {
        bulk_g2s(ks0 + buf * tileB + tid * ROWB, reinterpret_cast<const __nv_bfloat16*>(p.k_cache) + row * D, 256, bar);
        bulk_g2s(vt + tid * ROWB, reinterpret_cast<const __nv_bfloat16*>(p.v_cache) + row * D, 256, bar);
      }
    } else if (!I8) {
      // rows without a key: V must be finite (its products are multiplied by P = 0)
#pragma unroll
      for (int i = 0; i < 16; ++i)
        asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(vt + tid * ROWB + 16 * i), "r"(0) : "memory");
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
          asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(vs + tid * ROWB + 16 * i), "r"(0) : "memory");
      }
      if (okw && tid < nk) {
#pragma unroll
        for (int which = 0; which < 2; ++which) {
          const uint32_t src = (which ? v8s : k8s) + tid * D, dst = (which ? vs : ks) + tid * ROWB;
          const float sc = which ? vsc[buf] : ksc[buf];
#pragma unroll
          for (int i = 0; i < D / 16; ++i) {
            uint32_t w0, w1, w2, w3;
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w0), "=r"(w1), "=r"(w2), "=r"(w3) : "r"(src + 16 * i));
            const uint32_t ww[4] = {w0, w1, w2, w3};
            uint32_t o[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              o[2 * j] = pack_bf16((float)(int8_t)(ww[j] & 0xff) * sc, (float)(int8_t)((ww[j] >> 8) & 0xff) * sc);
              o[2 * j + 1] = pack_bf16((float)(int8_t)((ww[j] >> 16) & 0xff) * sc, (float)(int8_t)(ww[j] >> 24) * sc);
            }
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst + 32 * i), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]) : "memory");
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst + 32 * i + 16), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7]) : "memory");
          }
        }
      }
    }
    __syncthreads();
    if (!okw || !active) continue;

    // ---- S = Q K^T for 128 keys: 16 n8 tiles x 8 k16 steps
    float s[16][4];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < 8; kk += 2) {
        uint32_t b0, b1, b2, b3;
        // matrices: (keys 8j.., d 16kk..), (d 16kk + 8..), (d 16(kk+1)..), (d 16(kk+1) + 8..)
        ldsm_x4(ks + (8 * j + (lane & 7)) * ROWB + (16 * kk + 8 * (lane >> 3)) * 2, b0, b1, b2, b3);
        mma_bf16_16816(s[j], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], b0, b1);
        mma_bf16_16816(s[j], qa[kk + 1][0], qa[kk + 1][1], qa[kk + 1][2], qa[kk + 1][3], b2, b3);
      }
    }
    // ---- scale, causal mask per row, online softmax (rows g and g + 8 of the tile)
    float mnew[2] = {mx[0], mx[1]};
#pragma unroll
    for (int j = 0; j < 16; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = kb0 + 8 * j + 2 * t + (e & 1);
        const int hf = e >> 1;
        const float v = key < ctx[hf] && key < key1 ? s[j][e] * p.scale_log2 : -INFINITY;
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
    for (int j = 0; j < 16; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int hf = e >> 1;
        const float pe = mnew[hf] == -INFINITY ? 0.f : exp2f(s[j][e] - mnew[hf]);
        s[j][e] = pe;
        lsum[hf] += pe;
      }
    // ---- O += P V: 8 k16 steps over the keys, 16 n8 tiles over d
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const uint32_t pa0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]), pa1 = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      const uint32_t pa2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]), pa3 = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int jd = 0; jd < 16; jd += 2) {
        uint32_t b0, b1, b2, b3;
        // matrices: (keys 16kk.., d 8jd..), (keys 16kk + 8.., d 8jd..), (keys 16kk.., d 8(jd+1)..), (keys + 8, d 8(jd+1)..)
        const int mi = lane >> 3;
        ldsm_x4_trans(vs + (16 * kk + 8 * (mi & 1) + (lane & 7)) * ROWB + (8 * (jd + (mi >> 1))) * 2, b0, b1, b2, b3);
        mma_bf16_16816(o[jd], pa0, pa1, pa2, pa3, b0, b1);
        mma_bf16_16816(o[jd + 1], pa0, pa1, pa2, pa3, b2, b3);
      }
    }
  }

  // ---- this split's partials: unnormalised O against the running maximum, (max, sum)
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    lsum[hf] += __shfl_xor_sync(0xffffffffu, lsum[hf], 1);
    lsum[hf] += __shfl_xor_sync(0xffffffffu, lsum[hf], 2);
  }
  if (active) {
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int qr = warp * 16 + g + 8 * hf;
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

}  // namespace

// Rows of a request that follow one another in the control block are served together.  bf16 KV, head size 128,
// nsplit <= 64, GQA <= 16.  tickets [M][n_kv] (zeroed once; the kernel leaves them zero): the last split CTA of a
// group merges in the kernel; nullptr: the partials are left for b2_attn_merge.
extern "C" int b2_attn_rows(const void* q, const void* k_cache, const void* v_cache, const float* k_scale,
                            const float* v_scale, int kv_int8, const int* block_table,
                            const int* ctrl, float* o_part, float* ml_part, void* out, int* tickets, int M, int n_q,
                            int n_kv, int D_, int nsplit, int max_blocks, float scale, int span_pages, void* stream) {
  if (D_ != D || nsplit < 1 || nsplit > 64 || n_q % n_kv != 0 || n_q / n_kv > 16 || M > 64) return -1;
  AttnRowsParams p;
  p.q = (const __nv_bfloat16*)q; p.k_cache = k_cache; p.v_cache = v_cache; p.k_scale = k_scale; p.v_scale = v_scale;
  if (kv_int8 && (!k_scale || !v_scale)) return -3;
  p.block_table = block_table; p.ctrl = ctrl; p.o_part = o_part; p.ml_part = ml_part; p.out = (__nv_bfloat16*)out;
  p.tickets = tickets; p.M = M; p.n_q = n_q; p.n_kv = n_kv; p.gqa = n_q / n_kv; p.nsplit = nsplit; p.max_blocks = max_blocks;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.span_pages = span_pages;
  if (span_pages > 0 && (long)span_pages * nsplit < max_blocks) return -2;  // fixed spans must cover the longest sequence
  // prefetch the next batch when a split holds more than two batches of keys (long contexts); short ones
  // keep the small footprint that lets two CTAs share an SM
  const int pages_per_split = span_pages > 0 ? span_pages : (max_blocks + nsplit - 1) / nsplit;
  p.nbuf = pages_per_split * 16 > 2 * KB ? 2 : 1;
  const int smem = 128 + (kv_int8 ? 1 : p.nbuf) * 2 * KB * ROWB + 64 + (kv_int8 ? p.nbuf * 2 * KB * D : 0);
  static int configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    const int most = 128 + 2 * 2 * KB * ROWB + 64 + 2 * 2 * KB * D;
    cudaError_t e = cudaFuncSetAttribute(attn_rows_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_rows_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
    if (e != cudaSuccess) return (int)e;
    configured[dev & 63] = 1;
  }
  if (kv_int8)
    return b2_launch(attn_rows_kernel<true>, dim3(n_kv, nsplit, M), dim3(kThreads), smem, (cudaStream_t)stream, true, p);
  return b2_launch(attn_rows_kernel<false>, dim3(n_kv, nsplit, M), dim3(kThreads), smem, (cudaStream_t)stream, true, p);
}

B2_DEFINE_STATUS(attnrows)
