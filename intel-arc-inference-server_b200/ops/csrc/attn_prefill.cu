// Causal flash attention for prompt chunks over the paged KV cache, on tcgen05 / TMEM (head_dim 128).
//
//   O[r] = softmax( q[r] . K[0 .. pos(r)]^T / sqrt(D) ) V[0 .. pos(r)]      pos(r) = pos0 + r
//
// Stands where the reference has pf_flash_attn / pf_flash_merge (src/kernels/prefill/
// pf_flash_attn.cl).  One CTA owns 128 query rows of one query head and walks the keys in tiles
// of 128 (8 pages of 16 tokens); the K and V tiles of the head's KV group are fetched page by page
// with 2-D TMA (box = 16 keys x 64 dims, 128-byte swizzle) straight from the page pool through the
// sequence's block table, double buffered.
//   warp 0     TMA producer (Q once, then K / V tiles)
//   warp 1     MMA issuer: S = Q K^T (M 128, N 128, K 16 x 8) into TMEM, then O_tile = P V with V as
//              an MN-major operand (the cache keeps keys as rows, which is what P V needs along K)
//   warps 2-5  one thread per query row: tcgen05.ld of the S row, causal mask, online softmax in
//              fp32 with exp2, P written to shared memory as bf16 in the swizzled K-major layout,
//              then O_tile read back and folded into register accumulators with the running rescale
// All mbarrier waits are bounded (common.cuh); on a failed wait every role leaves its loop and the
// CTA still meets at the final barrier and frees its tensor memory.
#include "common.cuh"

using namespace b2;

namespace {

constexpr int D = 128;
constexpr int BQ = 128;   // query rows per CTA
constexpr int BK = 128;   // keys per tile
constexpr int kThreads = 192;
constexpr int Q_BYTES = BQ * D * 2;       // 32 KB: [2 d-blocks][128 rows][64]
constexpr int KV_BYTES = BK * D * 2;      // 32 KB each for K and V
constexpr int P_BYTES = BQ * BK * 2;      // 32 KB: [2 key-blocks][128 rows][64]
constexpr int SMEM = Q_BYTES + 2 * 2 * KV_BYTES + P_BYTES + 1024 + 256;

struct AttnPfParams {
  const int* block_table;  // this sequence's page table
  int n_q, n_kv;
  int C;        // rows in the chunk
  int pos0;     // absolute position of row 0
  int max_blocks;  // entries in block_table
  float scale_log2;
  __nv_bfloat16* out;  // [C][n_q * D]
};

// smem descriptor for the MN-major V operand: rows are keys (128 B = 64 dims, 128-byte swizzle),
// 8-key groups are 1024 B apart (stride byte offset); the next block of 64 dims is a whole tile
// half away (leading byte offset).
__device__ __forceinline__ uint64_t make_desc_v(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)((BK * 128) >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

__global__ void __launch_bounds__(kThreads, 1)
attn_prefill_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const AttnPfParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_s = base, kv_s = base + Q_BYTES, p_s = kv_s + 4 * KV_BYTES, bars = p_s + P_BYTES;
  // barriers: q_full, k_full[2], v_full[2], kv_empty[2], s_full, p_full, o_full
  const uint32_t b_qfull = bars, b_kfull = bars + 8, b_vfull = bars + 24, b_empty = bars + 40, b_sfull = bars + 56,
                 b_pfull = bars + 64, b_ofull = bars + 72;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_raw + (bars + 80 - smem_u32(smem_raw)));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;  // heavy (late) tiles first
  const int head = blockIdx.y, kh = head / (p.n_q / p.n_kv);
  const int row0 = qt * BQ;
  const int last_pos = p.pos0 + min(row0 + BQ, p.C) - 1;
  const int n_tiles = last_pos / BK + 1;

  if (threadIdx.x == 0) {
    mbar_init(b_qfull, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(b_kfull + 8 * i, 1);
      mbar_init(b_vfull + 8 * i, 1);
      mbar_init(b_empty + 8 * i, 1);
    }
    mbar_init(b_sfull, 1);
    mbar_init(b_pfull, 128);
    mbar_init(b_ofull, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_s = tmem_base, t_o = tmem_base + 128;

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tmap(&map_q);
      prefetch_tmap(&map_k);
      prefetch_tmap(&map_v);
      mbar_expect_tx(b_qfull, Q_BYTES);
      tma_load_2d(q_s, &map_q, head * D, row0, b_qfull);
      tma_load_2d(q_s + BQ * 128, &map_q, head * D + 64, row0, b_qfull);
      bool ok = true;
      int issued = 0;
      for (int i = 0; i < n_tiles && ok; ++i) {
        const int s = i & 1;
        if (i >= 2) ok = mbar_wait(b_empty + 8 * s, ((i >> 1) - 1) & 1, ERR_ATTN_WAIT);
        if (!ok) break;
        const uint32_t k_s = kv_s + s * 2 * KV_BYTES, v_s = k_s + KV_BYTES;
        // Always 8 pages: table entries past the sequence point at pages that hold finite data (page 0
        // is the never-allocated zero page), and those keys are masked out; an unfilled tile half
        // could hold NaN bit patterns, and 0 * NaN in P V would poison the row.
        constexpr int n_pages = 8;
        mbar_expect_tx(b_kfull + 8 * s, n_pages * 4096);
        mbar_expect_tx(b_vfull + 8 * s, n_pages * 4096);
        for (int pg = 0; pg < n_pages; ++pg) {
          const int page = (i * 8 + pg < p.max_blocks) ? p.block_table[i * 8 + pg] : 0;
          const int r = (page * p.n_kv + kh) * 16;
          tma_load_2d(k_s + pg * 2048, &map_k, 0, r, b_kfull + 8 * s);
          tma_load_2d(k_s + BK * 128 + pg * 2048, &map_k, 64, r, b_kfull + 8 * s);
        }
        for (int pg = 0; pg < n_pages; ++pg) {
          const int page = (i * 8 + pg < p.max_blocks) ? p.block_table[i * 8 + pg] : 0;
          const int r = (page * p.n_kv + kh) * 16;
          tma_load_2d(v_s + pg * 2048, &map_v, 0, r, b_vfull + 8 * s);
          tma_load_2d(v_s + BK * 128 + pg * 2048, &map_v, 64, r, b_vfull + 8 * s);
        }
        issued = i + 1;
      }
      if (!ok) {
        for (int i = max(0, issued - 2); i < issued; ++i) {
          mbar_wait(b_kfull + 8 * (i & 1), (i >> 1) & 1, ERR_ATTN_WAIT);
          mbar_wait(b_vfull + 8 * (i & 1), (i >> 1) & 1, ERR_ATTN_WAIT);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc(1, 1, BQ, BK);
      constexpr uint32_t idesc_pv = make_idesc(1, 1, BQ, D) | (1u << 16);  // B (V) is MN-major
      bool ok = mbar_wait(b_qfull, 0, ERR_ATTN_WAIT);
      for (int i = 0; i < n_tiles && ok; ++i) {
        const int s = i & 1;
        const uint32_t k_s = kv_s + s * 2 * KV_BYTES, v_s = k_s + KV_BYTES;
        // S = Q K^T.  The S buffer is free: the softmax threads arrived on p_full(i-1) after reading it.
        ok = mbar_wait(b_kfull + 8 * s, (i >> 1) & 1, ERR_ATTN_WAIT);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) {  // 8 x 16 dims; dims 64.. live in the second 16 KB block
          const uint32_t off = (k >> 2) * (BQ * 128) + (k & 3) * 32;
          umma_f16(t_s, make_desc_sw128(q_s + off), make_desc_sw128(k_s + off), idesc_qk, k != 0);
        }
        tc_commit(b_sfull);
        // O_tile = P V once the softmax threads have written P (and read the previous O_tile)
        ok = mbar_wait(b_pfull, i & 1, ERR_ATTN_WAIT);
        if (ok) ok = mbar_wait(b_vfull + 8 * s, (i >> 1) & 1, ERR_ATTN_WAIT);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) {  // 8 x 16 keys; keys 64.. of P live in its second 16 KB block
          const uint32_t p_off = (k >> 2) * (BQ * 128) + (k & 3) * 32;
          umma_f16(t_o, make_desc_sw128(p_s + p_off), make_desc_v(v_s + k * 16 * 128), idesc_pv, k != 0);
        }
        tc_commit(b_ofull);
        tc_commit(b_empty + 8 * s);
      }
    }
  } else {
    // ---------------------------------------------------------- softmax + accumulate: one thread per query row
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int qpos = p.pos0 + row0 + r;
    const bool row_ok = row0 + r < p.C;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    float o[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o[i] = 0.f;
    float mx = -INFINITY, l = 0.f;
    bool ok = true;
    for (int i = 0; i < n_tiles && ok; ++i) {
      ok = mbar_wait(b_sfull, i & 1, ERR_ATTN_WAIT);
      if (!ok) break;
      tc_fence_after();
      // pass 1: row maximum
      float tmax = -INFINITY;
      const int key0 = i * BK;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        B2_TMEM_LD_32(t_s + lane_addr + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float sv = (key0 + c * 32 + j <= qpos) ? __uint_as_float(v[j]) : -INFINITY;
          tmax = fmaxf(tmax, sv);
        }
      }
      const float mnew = fmaxf(mx, tmax * p.scale_log2);
      const float msafe = (mnew == -INFINITY) ? 0.f : mnew;
      const float alpha = exp2f(mx - msafe);  // 0 on the first tile (mx = -inf)
      // pass 2: P = exp2(s * scale - m), row sum, bf16 to shared memory (swizzled, K-major over keys)
      float lsum = 0.f;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        B2_TMEM_LD_32(t_s + lane_addr + c * 32, v);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int k0 = key0 + c * 32 + 2 * j;
          const float p0 = (k0 <= qpos) ? exp2f(fmaf(__uint_as_float(v[2 * j]), p.scale_log2, -msafe)) : 0.f;
          const float p1 = (k0 + 1 <= qpos) ? exp2f(fmaf(__uint_as_float(v[2 * j + 1]), p.scale_log2, -msafe)) : 0.f;
          pk[j] = pack_bf16(p0, p1);
          // the row sum uses the rounded values, i.e. exactly what the tensor core multiplies with V
          lsum += bf16_lo(pk[j]) + bf16_hi(pk[j]);
        }
        const uint32_t rowb = p_s + (c >> 1) * (BQ * 128) + r * 128;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int chunk = ((c & 1) * 4 + q) ^ (r & 7);
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(rowb + chunk * 16), "r"(pk[4 * q]),
                       "r"(pk[4 * q + 1]), "r"(pk[4 * q + 2]), "r"(pk[4 * q + 3])
                       : "memory");
        }
      }
      l = l * alpha + lsum;
      mx = mnew;
      tc_fence_before();
      fence_proxy_async_smem();  // P was written with generic stores, the MMA reads it through the async proxy
      mbar_arrive(b_pfull);
      // fold O_tile into the accumulators
      ok = mbar_wait(b_ofull, i & 1, ERR_ATTN_WAIT);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        B2_TMEM_LD_32(t_o + lane_addr + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) o[c * 32 + j] = fmaf(o[c * 32 + j], alpha, __uint_as_float(v[j]));
      }
      tc_fence_before();
    }
    if (ok && row_ok) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = p.out + (size_t)(row0 + r) * (p.n_q * D) + head * D;
#pragma unroll
      for (int j = 0; j < D / 8; ++j)
        *reinterpret_cast<uint4*>(dst + 8 * j) =
            make_uint4(pack_bf16(o[8 * j] * inv, o[8 * j + 1] * inv), pack_bf16(o[8 * j + 2] * inv, o[8 * j + 3] * inv),
                       pack_bf16(o[8 * j + 4] * inv, o[8 * j + 5] * inv), pack_bf16(o[8 * j + 6] * inv, o[8 * j + 7] * inv));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
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
extern "C" int b2_attn_prefill(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                               void* out, int C, int pos0, int n_q, int n_kv, int head_dim, int num_pages,
                               int max_blocks, float scale, void* stream) {
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
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return (int)e;
    configured[dev & 63] = true;
  }
  AttnPfParams p;
  p.block_table = block_table; p.n_q = n_q; p.n_kv = n_kv; p.C = C; p.pos0 = pos0; p.max_blocks = max_blocks;
  p.scale_log2 = scale * 1.4426950408889634f; p.out = (__nv_bfloat16*)out;
  dim3 grid((C + BQ - 1) / BQ, n_q);
  attn_prefill_kernel<<<grid, kThreads, SMEM, (cudaStream_t)stream>>>(mq, mk, mv, p);
  return (int)cudaGetLastError();
}

B2_DEFINE_STATUS(attn)
