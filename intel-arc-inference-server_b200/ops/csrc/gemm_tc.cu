// Prefill GEMMs on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a only.
//
//   C[M][N] = A[M][K] * B[N][K]^T        A, B K-major (row-major activations, row-major weights)
//
//   * bf16 x bf16 -> fp32 (kind::f16)            prefill linears on dequantised weights
//   * int8 x int8 -> int32 (kind::i8)            the int8 prompt pass: per-token activation scales and
//                                                per-row weight scales applied in the epilogue
//   * grouped form (MoE): the M dimension is a device-side table of expert row blocks, B is a
//     3-D tensor [E][N][K]; tile counts are read on the device so the host never syncs
//
// They replace the reference's pf_gemm / pf_gemm_small (src/kernels/prefill/pf_gemm.cl), its int8
// GEMM (pf_int8.cl: pf_gemm_i8) and the grouped expert GEMM (pf_moe_gemm.cl).
//
// Structure: one persistent CTA per SM, 192 threads, warp-specialised.
//   warp 0   TMA producer: cp.async.bulk.tensor 2-D/3-D tiles (128-byte swizzle) into a smem ring
//   warp 1   MMA issuer: one elected lane issues tcgen05.mma (M = 128, N = BN, K = 16 / 32) and
//            commits stage-free and accumulator-full mbarriers; owns the TMEM allocation
//   warps 2-5 epilogue: tcgen05.ld of the accumulator (two TMEM buffers, so the epilogue of tile i
//            overlaps the main loop of tile i + 1), scale / SiLU*up / residual add, global stores
// Tiles are walked M-fastest so CTAs that run together share one weight tile in L2.
//
// W4 form (template parameter W4): B is never materialised in global memory.  The producer fetches the W4B blocks of
// a stage (4352 bytes per 128 rows x 64 k: nibbles + fp16 group scales) with bulk copies; eight more warps expand them
// to bf16 -- bf16_rne((q - 8) * scale), the same rounding as the dequantising pass -- straight into the stage's
// B tile in the 128-byte-swizzled K-major layout the MMA descriptors expect, fence the generic stores against the
// async proxy and complete the stage's barrier.  The weights cross HBM as int4 (a quarter of the bf16 bytes) and
// no bf16 copy of the model is resident.  The role of the reference's direct-int4 GEMMs
// (src/kernels/prefill/pf_gemm_q4.cl, src/kernels/prefill/pf_moe_q4gemm.cl:1-40).
#include "common.cuh"
#include "wire.cuh"

#include <map>
#include <mutex>
#include <tuple>

using namespace b2;

namespace {

constexpr int BM = 128;
constexpr int BKB = 128;  // bytes of K per stage row (64 bf16 or 128 int8)
constexpr int kThreads = 192;

enum Epi : int { EPI_BF16 = 0, EPI_F32 = 1, EPI_SILU_MUL = 2, EPI_RESID_ADD = 3, EPI_RS_PUSH = 4, EPI_EP_RETURN = 5 };

struct GemmParams {
  int M, N, K;       // K in elements
  int ldc;           // leading dimension of C (elements)
  void* C;
  const __nv_bfloat16* resid;  // EPI_RESID_ADD: [M][ldc]
  const float* a_scale;        // int8: per row of A
  const float* b_scale;        // int8: per row of B ([E][N] in the grouped form)
  int epi;
  // grouped form
  const int* blk_expert;  // [n_blk]
  const int* blk_row0;    // [n_blk] first row of the block in A / C
  const int* blk_rows;    // [n_blk] valid rows (<= 128)
  const int* n_blk;       // device scalar
  int max_blk;
  // ---- tensor-parallel forms (see wire.cuh for the protocol)
  // EPI_RS_PUSH (row-parallel GEMM -> reduce-scatter): the bf16 tile of m-tile mt is stored into the
  // landing buffer of the rank that owns those rows, [source rank][rows_cap][N], and the owner's counter
  // [source rank][m-tile of the owner] gets one increment per epilogue warp and n-tile.
  const unsigned long long* rs_table;  // [2][kMaxRanks]: landing, counters of every rank
  int rs_rank, rs_world;
  int rs_tpr;       // m-tiles per owner (rows_cap = 128 rs_tpr)
  int mt_rot;       // m-tile walk starts here, so ranks do not all push to one owner at a time
  // all-gather -> GEMM: the producer waits until m-tile mt of A (pushed into this GPU's memory by the
  // owners of those rows) has ag_expect arrivals
  const int* ag_cnt;
  int ag_expect;
  // ---- expert-parallel forms (grouped mode)
  // dispatch -> grouped GEMM: block i of the expert-sorted rows is loaded once blk_wait[i] (arrivals counted
  // by the source ranks' dispatch kernels) has reached the block's row count.
  const int* blk_wait;
  // EPI_EP_RETURN (grouped GEMM -> combine): row r of the sorted buffer belongs to slot (row_src[r] & 0xffffff)
  // of source rank (row_src[r] >> 24); its bf16 result row is stored into that rank's return buffer
  // ret_table[rank][slot][N] over NVLink, where the source adds its tokens' slots in slot order.
  const int* row_src;
  const unsigned long long* ret_table;
  // ---- W4 form: B as W4B blocks [expert][ceil(N / 128)][K / 64][4352 bytes]
  const uint8_t* w4;
  long long w4_expert_bytes;
};

constexpr int kW4Block = 4352;     // one W4B block: 128 rows x 64 k of nibbles (4096 B) + 128 fp16 scales
constexpr int kDequantWarps = 16;  // W4 form: warps that expand the blocks into the B tile (one 16-byte vector per thread and
                                   // stage at BN = 256: eight warps left a third of the issue slots empty on dependent chains)

template <int BN, bool W4 = false>
struct Cfg {
  static constexpr int A_BYTES = BM * BKB;
  static constexpr int B_BYTES = BN * BKB;
  static constexpr int STAGE = A_BYTES + B_BYTES;
  static constexpr int RAW = W4 ? (BN / 128) * kW4Block : 0;   // the stage's W4B blocks, kept apart so that tiles stay 1024-aligned
  static constexpr int STAGES = W4 ? ((BN == 256) ? 3 : 5) : ((BN == 256) ? 4 : 6);
  static constexpr int PUSH_STAGE = 4 * 32 * 144;  // per epilogue warp: 32 rows x (128 B + 16 B pad) for coalesced peer stores
  static constexpr int BARS = 384;
  static constexpr int SMEM = STAGES * STAGE + 1024 /*align*/ + BARS + PUSH_STAGE + STAGES * RAW;
  static constexpr int TMEM_COLS = 2 * BN;  // two accumulators
  static constexpr int THREADS = kThreads + (W4 ? kDequantWarps * 32 : 0);
};

template <int BN, bool I8, bool W4 = false>
__global__ void __launch_bounds__(Cfg<BN, W4>::THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const GemmParams p) {
  using C = Cfg<BN, W4>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE);
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + C::STAGES);
  const uint32_t tfull0 = smem_u32(bars + 2 * C::STAGES), tempty0 = smem_u32(bars + 2 * C::STAGES + 2);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::STAGES + 4);
  const uint32_t rawfull0 = smem_u32(bars + 2 * C::STAGES + 6);   // W4 form: a stage's W4B blocks have landed
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t push_base = smem_base + C::STAGES * C::STAGE + C::BARS;
  const uint32_t raw_base = push_base + C::PUSH_STAGE;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool grouped = p.blk_expert != nullptr;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int tiles_m = grouped ? min(*p.n_blk, p.max_blk) : (p.M + BM - 1) / BM;
  const int n_tiles = tiles_m * tiles_n;
  const int KB = (p.K * (I8 ? 1 : 2) + BKB - 1) / BKB;  // k blocks

  if (threadIdx.x == 0) {
    for (int i = 0; i < C::STAGES; ++i) {
      mbar_init(full0 + 8 * i, W4 ? 1 + kDequantWarps : 1);   // W4: the A tile's copy and every expanding warp
      mbar_init(empty0 + 8 * i, 1);
      if (W4) mbar_init(rawfull0 + 8 * i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(tfull0 + 8 * i, 1);
      mbar_init(tempty0 + 8 * i, 4);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tmap(&map_a);
      prefetch_tmap(&map_b);
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
        const int mt = (t % tiles_m + p.mt_rot) % tiles_m, nt = t / tiles_m;
        int row0 = mt * BM, expert = 0;
        if (grouped) {
          row0 = p.blk_row0[mt];
          expert = p.blk_expert[mt];
        }
        if (p.ag_cnt) {
          // rows of this m-tile arrive from their owner rank: bounded wait on the tile's counter in this
          // GPU's own memory, then order the generic-proxy acquire before the async-proxy (TMA) reads
          ok = wire_wait(p.ag_cnt + mt, p.ag_expect, (unsigned)(0x20000000u | mt));
          if (!ok) break;
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        if (p.blk_wait) {
          ok = wire_wait(p.blk_wait + mt, p.blk_rows[mt], (unsigned)(0x28000000u | mt));
          if (!ok) break;
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % C::STAGES;
          if (it >= C::STAGES) ok = mbar_wait(empty0 + 8 * s, ((it / C::STAGES) - 1) & 1, ERR_GEMM_EMPTY_WAIT);
          if (!ok) break;
          const uint32_t sa = smem_base + s * C::STAGE, sb = sa + C::A_BYTES;
          const int kx = kb * (I8 ? BKB : BKB / 2);
          if (W4) {
            // A by TMA; B as the W4B blocks of this 64-k group (one block per 128 rows), expanded by the other warps
            mbar_expect_tx(full0 + 8 * s, C::A_BYTES);
            tma_load_2d(sa, &map_a, kx, row0, full0 + 8 * s);
            const int nb_total = (p.N + 127) / 128, nb0 = nt * (BN / 128);
            const int nblk = min(BN / 128, nb_total - nb0);
            const uint8_t* wsrc = p.w4 + (size_t)expert * p.w4_expert_bytes + ((size_t)nb0 * KB + kb) * kW4Block;
            mbar_expect_tx(rawfull0 + 8 * s, (uint32_t)nblk * kW4Block);
            for (int b = 0; b < nblk; ++b)
              bulk_g2s(raw_base + s * C::RAW + b * kW4Block, wsrc + (size_t)b * KB * kW4Block, kW4Block, rawfull0 + 8 * s);
          } else {
            mbar_expect_tx(full0 + 8 * s, C::STAGE);
            tma_load_2d(sa, &map_a, kx, row0, full0 + 8 * s);
            if (grouped) tma_load_3d(sb, &map_b, kx, nt * BN, expert, full0 + 8 * s);
            else tma_load_2d(sb, &map_b, kx, nt * BN, full0 + 8 * s);
          }
        }
      }
      if (!ok) {  // drain what was issued and may never be consumed
        for (int i = max(0, it - C::STAGES); i < it; ++i) {
          if (W4) mbar_wait(rawfull0 + 8 * (i % C::STAGES), (i / C::STAGES) & 1, ERR_GEMM_FULL_WAIT);
          else mbar_wait(full0 + 8 * (i % C::STAGES), (i / C::STAGES) & 1, ERR_GEMM_FULL_WAIT);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = I8 ? make_idesc(2, 1, BM, BN) : make_idesc(1, 1, BM, BN);
      int it = 0, lt = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++lt) {
        const int a = lt & 1;
        if (lt >= 2) ok = mbar_wait(tempty0 + 8 * a, ((lt >> 1) - 1) & 1, ERR_GEMM_TMEM_EMPTY_WAIT);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + a * BN;
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % C::STAGES;
          ok = mbar_wait(full0 + 8 * s, (it / C::STAGES) & 1, ERR_GEMM_FULL_WAIT);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_base + s * C::STAGE, sb = sa + C::A_BYTES;
#pragma unroll
          for (int k = 0; k < 4; ++k) {  // 4 x 32 bytes of K per stage
            const uint64_t da = make_desc_sw128(sa + k * 32), db = make_desc_sw128(sb + k * 32);
            if (I8) umma_i8(d_tmem, da, db, idesc, (kb | k) != 0);
            else umma_f16(d_tmem, da, db, idesc, (kb | k) != 0);
          }
          tc_commit(empty0 + 8 * s);  // stage is free once these MMAs have read it
        }
        if (ok) tc_commit(tfull0 + 8 * a);
      }
    }
  } else if (W4 && warp >= 6) {
    // ------------------------------------------------------------ W4 expansion (warps 6 .. 6 + kDequantWarps - 1)
    // One 16-byte vector of a W4B block holds rows g and g + 8 of a 16-row tile, 64 k: low nibbles are k 4t..4t+3 of a
    // 32-k step, high nibbles k + 16 (the operand order of the decode GEMV).  Each vector becomes sixteen 8-byte
    // pieces of the B tile: row r at r * 128 bytes, 16-byte chunk (k / 8) XOR (r mod 8) -- the 128-byte swizzle.
    const int dt = threadIdx.x - 6 * 32;   // 0 .. 32 * kDequantWarps - 1
    int it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
      const int nt = t / tiles_m;
      const int nb_total = (p.N + 127) / 128, nb0 = nt * (BN / 128);
      const int nblk = min(BN / 128, nb_total - nb0);
      for (int kb = 0; kb < KB; ++kb, ++it) {
        const int s = it % C::STAGES;
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(rawfull0 + 8 * s, (it / C::STAGES) & 1, ERR_GEMM_FULL_WAIT));
        if (!ok) break;
        const uint32_t sb = smem_base + s * C::STAGE + C::A_BYTES, raw = raw_base + s * C::RAW;
        for (int u = dt; u < nblk * 256; u += kDequantWarps * 32) {
          const int b = u >> 8, v = u & 255, j = v >> 5, l = v & 31, g = l >> 2, tq = l & 3;
          uint4 wv;
          asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(wv.x), "=r"(wv.y), "=r"(wv.z), "=r"(wv.w)
                       : "r"(raw + b * kW4Block + v * 16));
          uint32_t sc2;
          asm volatile("ld.shared.u32 %0, [%1];" : "=r"(sc2) : "r"(raw + b * kW4Block + 4096 + (j * 16 + 2 * g) * 2));
          const __half2 sh = *reinterpret_cast<const __half2*>(&sc2);
          const float s_lo = __low2float(sh), s_hi = __high2float(sh);
          const uint32_t wa[4] = {wv.x, wv.y, wv.z, wv.w};
          uint64_t sc2x[2], off2;
          asm("mov.b64 %0, {%1, %1};" : "=l"(sc2x[0]) : "f"(s_lo));
          asm("mov.b64 %0, {%1, %1};" : "=l"(sc2x[1]) : "f"(s_hi));
          asm("mov.b64 %0, {%1, %1};" : "=l"(off2) : "f"(-8388616.f));
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int row = b * 128 + j * 16 + g + 8 * (c & 1);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const uint32_t x = (wa[c] >> (4 * e)) & 0x0F0F0F0Fu;
              // bytes -> floats through the 2^23 trick: 0x4B0000qq is 8388608 + q; q - 8 (exact) and the product with
              // the scale run as packed pairs (add.f32x2 / mul.f32x2), the same floats as the scalar form
              uint64_t f01, f23;
              asm("mov.b64 %0, {%1, %2};" : "=l"(f01) : "r"(__byte_perm(x, 0x4B000000u, 0x7440)), "r"(__byte_perm(x, 0x4B000000u, 0x7441)));
              asm("mov.b64 %0, {%1, %2};" : "=l"(f23) : "r"(__byte_perm(x, 0x4B000000u, 0x7442)), "r"(__byte_perm(x, 0x4B000000u, 0x7443)));
              asm("add.rn.f32x2 %0, %0, %1;" : "+l"(f01) : "l"(off2));
              asm("add.rn.f32x2 %0, %0, %1;" : "+l"(f23) : "l"(off2));
              asm("mul.rn.f32x2 %0, %0, %1;" : "+l"(f01) : "l"(sc2x[c & 1]));
              asm("mul.rn.f32x2 %0, %0, %1;" : "+l"(f23) : "l"(sc2x[c & 1]));
              float g0, g1, g2, g3;
              asm("mov.b64 {%0, %1}, %2;" : "=f"(g0), "=f"(g1) : "l"(f01));
              asm("mov.b64 {%0, %1}, %2;" : "=f"(g2), "=f"(g3) : "l"(f23));
              const uint32_t p01 = pack_bf16(g0, g1);
              const uint32_t p23 = pack_bf16(g2, g3);
              const int k0 = 32 * (c >> 1) + 16 * e + 4 * tq;
              const uint32_t dst = sb + row * 128 + ((((uint32_t)k0 >> 3) ^ ((uint32_t)row & 7u)) << 4) + (k0 & 7) * 2;
              asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(dst), "r"(p01), "r"(p23) : "memory");
            }
          }
        }
        fence_proxy_async_smem();   // the MMA reads the tile through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(full0 + 8 * s);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;  // TMEM lane quarter this warp may read
    int lt = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++lt) {
      const int a = lt & 1;
      const int mt = (t % tiles_m + p.mt_rot) % tiles_m, nt = t / tiles_m;
      int row0 = mt * BM, rows = min(BM, p.M - row0), expert = 0;
      if (grouped) {
        row0 = p.blk_row0[mt];
        rows = p.blk_rows[mt];
        expert = p.blk_expert[mt];
      }
      ok = mbar_wait(tfull0 + 8 * a, (lt >> 1) & 1, ERR_GEMM_TMEM_FULL_WAIT);
      if (!ok) break;
      tc_fence_after();
      const int r = quarter * 32 + lane;  // row inside the tile
      const int grow = row0 + r;
      const bool row_ok = r < rows;
      float asc = 1.f;
      if (I8 && row_ok) asc = p.a_scale[grow];
      const float* bsc = I8 ? p.b_scale + (size_t)expert * p.N : nullptr;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        const uint32_t taddr = tmem_base + a * BN + c * 32 + ((uint32_t)(quarter * 32) << 16);
        B2_TMEM_LD_32(taddr, v);
        tmem_ld_wait();
        const int n0 = nt * BN + c * 32;
        if (I8) {  // integer accumulators -> scaled floats, once, for every epilogue form
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __float_as_uint((float)(int)v[j] * asc * bsc[min(n0 + j, p.N - 1)]);
        }
        if (p.epi == EPI_RS_PUSH || p.epi == EPI_EP_RETURN) {
          // bf16 row piece -> this warp's staging tile; every second chunk the warp copies 32 rows x 128 B
          // to the owner's landing buffer as whole 128-byte lines (coalesced stores cross NVLink far better
          // than one row per thread)
          const uint32_t stg = push_base + (uint32_t)quarter * (32 * 144);
          const uint32_t mine = stg + lane * 144 + (c & 1) * 64;
#pragma unroll
          for (int j = 0; j < 4; ++j)
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(mine + 16 * j),
                         "r"(pack_bf16(__uint_as_float(v[8 * j]), __uint_as_float(v[8 * j + 1]))),
                         "r"(pack_bf16(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]))),
                         "r"(pack_bf16(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]))),
                         "r"(pack_bf16(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7])))
                         : "memory");
          if ((c & 1) && p.epi == EPI_EP_RETURN) {
            __syncwarp();
            if (n0 - 32 < p.N) {
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int rw = i * 4 + (lane >> 3), piece = lane & 7;
                uint4 q;
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w)
                             : "r"(stg + rw * 144 + piece * 16));
                if (quarter * 32 + rw < rows) {
                  const int meta = p.row_src[row0 + quarter * 32 + rw];
                  __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.ret_table[meta >> 24]) +
                                       (size_t)(meta & 0xffffff) * p.N + (n0 - 32) + piece * 8;
                  *reinterpret_cast<uint4*>(dst) = q;
                }
              }
            }
            __syncwarp();
          } else if (c & 1) {
            __syncwarp();
            const int owner = mt / p.rs_tpr, mtl = mt - owner * p.rs_tpr;
            __nv_bfloat16* land = reinterpret_cast<__nv_bfloat16*>(p.rs_table[owner]) +
                                  ((size_t)p.rs_rank * p.rs_tpr * BM + (size_t)mtl * BM + quarter * 32) * p.N + (n0 - 32);
            if (n0 - 32 < p.N) {
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int rw = i * 4 + (lane >> 3), piece = lane & 7;
                uint4 q;
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w)
                             : "r"(stg + rw * 144 + piece * 16));
                if (quarter * 32 + rw < rows) *reinterpret_cast<uint4*>(land + (size_t)rw * p.N + piece * 8) = q;
              }
            }
            __syncwarp();
          }
        } else if (row_ok && n0 < p.N) {
          float f[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
          if (p.epi == EPI_SILU_MUL) {
            // columns alternate 16 gate, 16 up: 16 outputs per 32 accumulator columns
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)grow * p.ldc + (n0 >> 1);
            uint32_t o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
              o[j] = pack_bf16(silu(f[2 * j]) * f[16 + 2 * j], silu(f[2 * j + 1]) * f[17 + 2 * j]);
            *reinterpret_cast<uint4*>(dst) = make_uint4(o[0], o[1], o[2], o[3]);
            *reinterpret_cast<uint4*>(dst + 8) = make_uint4(o[4], o[5], o[6], o[7]);
          } else if (p.epi == EPI_F32) {
            float* dst = reinterpret_cast<float*>(p.C) + (size_t)grow * p.ldc + n0;
            if (n0 + 32 <= p.N) {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                *reinterpret_cast<float4*>(dst + 4 * j) = make_float4(f[4 * j], f[4 * j + 1], f[4 * j + 2], f[4 * j + 3]);
            } else {
              for (int j = 0; j < 32 && n0 + j < p.N; ++j) dst[j] = f[j];
            }
          } else {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)grow * p.ldc + n0;
            if (p.epi == EPI_RESID_ADD) {
              const __nv_bfloat16* rs = p.resid + (size_t)grow * p.ldc + n0;
              if (n0 + 32 <= p.N) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const uint4 rv = *reinterpret_cast<const uint4*>(rs + 8 * j);
                  const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                  for (int q = 0; q < 4; ++q) {
                    f[8 * j + 2 * q] += bf16_lo(rw[q]);
                    f[8 * j + 2 * q + 1] += bf16_hi(rw[q]);
                  }
                }
              } else {
                for (int j = 0; j < 32 && n0 + j < p.N; ++j) f[j] += __bfloat162float(rs[j]);
              }
            }
            if (n0 + 32 <= p.N) {
#pragma unroll
              for (int j = 0; j < 4; ++j)
                *reinterpret_cast<uint4*>(dst + 8 * j) =
                    make_uint4(pack_bf16(f[8 * j], f[8 * j + 1]), pack_bf16(f[8 * j + 2], f[8 * j + 3]),
                               pack_bf16(f[8 * j + 4], f[8 * j + 5]), pack_bf16(f[8 * j + 6], f[8 * j + 7]));
            } else {
              for (int j = 0; j < 32 && n0 + j < p.N; ++j) dst[j] = __float2bfloat16(f[j]);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty0 + 8 * a);
      if (p.epi == EPI_RS_PUSH) {
        // this warp's part of the tile is on its way: make it visible system-wide, then count one arrival
        // at the owner (4 epilogue warps x tiles_n arrivals complete an m-tile of one source rank)
        __syncwarp();   // the warp's stores are ordered before lane 0's fence and release
        if (lane == 0) {
          const int owner = mt / p.rs_tpr, mtl = mt - owner * p.rs_tpr;
          int* cnt = reinterpret_cast<int*>(p.rs_table[kMaxRanks + owner]) + p.rs_rank * p.rs_tpr + mtl;
          __threadfence_system();
          asm volatile("red.release.sys.global.add.s32 [%0], 1;" ::"l"(cnt) : "memory");
        }
      }
    }
  }

  // ---- teardown: every thread arrives here on every path, then the owner frees the TMEM
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// ------------------------------------------------------------------ W4B -> bf16 [N][K] (two-pass prefill path)
// grid (K/64, N/128), 256 threads: thread (tile j = warp, lane) expands its 16 bytes, the tile is
// staged in shared memory and written as 128-byte row segments.
__global__ void __launch_bounds__(256) dequant_w4b_kernel(const uint8_t* __restrict__ w, __nv_bfloat16* __restrict__ out,
                                                          int N, int K) {
  __shared__ __align__(16) uint32_t tile[128][33];  // [row][k pairs] (+1 pad)
  const int kg = blockIdx.x, nb = blockIdx.y, KG = K / 64;
  const uint8_t* blk = w + ((size_t)nb * KG + kg) * 4352;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const uint4 wv = *reinterpret_cast<const uint4*>(blk + warp * 512 + lane * 16);
  const __half* sc = reinterpret_cast<const __half*>(blk + 4096) + warp * 16;
  const float s_lo = __half2float(sc[2 * g]), s_hi = __half2float(sc[2 * g + 1]);  // scales are stored as (g, g + 8) pairs
  const uint32_t wa[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int row = warp * 16 + g + 8 * (c & 1);
    const float s = (c & 1) ? s_hi : s_lo;
#pragma unroll
    for (int e = 0; e < 2; ++e) {  // e = 0: low nibbles (k = 4t + b of the 32-k step), 1: high nibbles (+ 16)
      const uint32_t x = (wa[c] >> (4 * e)) & 0x0F0F0F0Fu;
      const float f0 = (float)((int)(x & 0xFF) - 8) * s, f1 = (float)((int)((x >> 8) & 0xFF) - 8) * s;
      const float f2 = (float)((int)((x >> 16) & 0xFF) - 8) * s, f3 = (float)((int)(x >> 24) - 8) * s;
      const int kpair = (32 * (c >> 1) + 16 * e + 4 * t) >> 1;
      tile[row][kpair] = pack_bf16(f0, f1);
      tile[row][kpair + 1] = pack_bf16(f2, f3);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 128 * 32; i += 256) {
    const int row = i >> 5, kp = i & 31;
    const int n = nb * 128 + row;
    if (n < N) reinterpret_cast<uint32_t*>(out + (size_t)n * K + kg * 64)[kp] = tile[row][kp];
  }
}

// ------------------------------------------------------------------ per-token int8 activation quant
// one CTA per row: scale = max|x| / 127
__global__ void __launch_bounds__(256) quant_rows_i8_kernel(const __nv_bfloat16* __restrict__ x, int8_t* __restrict__ q,
                                                            float* __restrict__ scale, int K) {
  __shared__ float red[8];
  const int m = blockIdx.x;
  const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(x + (size_t)m * K);
  float amax = 0.f;
  for (int i = threadIdx.x; i < K / 2; i += 256) {
    const float2 v = __bfloat1622float2(xp[i]);
    amax = fmaxf(amax, fmaxf(fabsf(v.x), fabsf(v.y)));
  }
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, red[i]);
  const float sc = amax > 0.f ? amax / 127.f : 1.f, inv = 1.f / sc;
  for (int i = threadIdx.x; i < K / 2; i += 256) {
    const float2 v = __bfloat1622float2(xp[i]);
    char2 o;
    o.x = (signed char)__float2int_rn(v.x * inv);
    o.y = (signed char)__float2int_rn(v.y * inv);
    reinterpret_cast<char2*>(q + (size_t)m * K)[i] = o;
  }
  if (threadIdx.x == 0) scale[m] = sc;
}

// ------------------------------------------------------------------ host side: tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// rows x cols (cols contiguous) matrix, optionally a stack of `batch` of them; box = box_rows x 128 bytes
int make_map(CUtensorMap* map, const void* ptr, bool i8, uint64_t rows, uint64_t cols, uint64_t batch,
             uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -100;
  const uint64_t esz = i8 ? 1 : 2;
  cuuint64_t dims[3] = {cols, rows, batch};
  cuuint64_t strides[2] = {cols * esz, rows * cols * esz};
  cuuint32_t box[3] = {(cuuint32_t)(BKB / esz), box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const int rank = batch > 1 ? 3 : 2;
  CUresult r = fn(map, i8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank,
                  const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -101 - (int)r;
}

int sm_count() {
  static int n[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!n[dev & 63]) cudaDeviceGetAttribute(&n[dev & 63], cudaDevAttrMultiProcessorCount, dev);
  return n[dev & 63];
}

template <int BN, bool I8>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, int n_tiles_max, cudaStream_t st) {
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, I8>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<BN>::SMEM);
    if (e != cudaSuccess) return (int)e;
    configured[dev & 63] = true;
  }
  const int grid = min(n_tiles_max, sm_count());
  gemm_tc_kernel<BN, I8><<<grid, kThreads, Cfg<BN>::SMEM, st>>>(ma, mb, p);
  return (int)cudaGetLastError();
}

template <int BN>
int launch_w4(const CUtensorMap& ma, const GemmParams& p, int n_tiles_max, cudaStream_t st) {
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg<BN, true>::SMEM);
    if (e != cudaSuccess) return (int)e;
    configured[dev & 63] = true;
  }
  const int grid = min(n_tiles_max, sm_count());
  gemm_tc_kernel<BN, false, true><<<grid, Cfg<BN, true>::THREADS, Cfg<BN, true>::SMEM, st>>>(ma, ma, p);
  return (int)cudaGetLastError();
}

}  // namespace

// C = A * W^T with W read as int4: a [M][K] bf16, w4b the W4B blocks [E][ceil(N / 128)][K / 64][4352] (E = 1 unless the
// blk_* tables of the grouped form are given).  Epilogues 0..3 as b2_gemm_tc.
extern "C" int b2_gemm_w4(const void* a, const void* w4b, void* c, int M, int N, int K, int ldc, int epi, const void* resid,
                          const int* blk_expert, const int* blk_row0, const int* blk_rows, const int* n_blk, int max_blk,
                          int n_experts, int bn, void* stream) {
  if (K % 64 != 0 || M < 1 || N % 8 != 0 || epi < EPI_BF16 || epi > EPI_RESID_ADD) return -1;
  if (epi == EPI_SILU_MUL && N % 32 != 0) return -2;
  if (((uintptr_t)w4b) & 15) return -3;
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.C = c; p.resid = (const __nv_bfloat16*)resid; p.epi = epi;
  p.blk_expert = blk_expert; p.blk_row0 = blk_row0; p.blk_rows = blk_rows; p.n_blk = n_blk; p.max_blk = max_blk;
  p.rs_world = 1; p.rs_tpr = 1;
  p.w4 = (const uint8_t*)w4b;
  p.w4_expert_bytes = (long long)((N + 127) / 128) * (K / 64) * kW4Block;
  if (bn != 128 && bn != 256) bn = (N >= 256 && (N % 256 == 0 || N > 2048)) ? 256 : 128;
  CUtensorMap ma;
  int rc = make_map(&ma, a, false, (uint64_t)M, (uint64_t)K, 1, BM);
  if (rc) return rc;
  const int tiles_m = blk_expert ? max_blk : (M + BM - 1) / BM;
  const int n_tiles = tiles_m * ((N + bn - 1) / bn);
  (void)n_experts;
  cudaStream_t st = (cudaStream_t)stream;
  return bn == 256 ? launch_w4<256>(ma, p, n_tiles, st) : launch_w4<128>(ma, p, n_tiles, st);
}

// C = A * B^T.  a: [M][K], b: [N][K] (or [E][N][K] when blk_* are given), both bf16 (i8 = 0) or int8 (i8 = 1).
static int gemm_tc_impl(const void* a, const void* b, void* c, int M, int N, int K, int ldc, int i8, int epi,
                        const void* resid, const float* a_scale, const float* b_scale, const int* blk_expert,
                        const int* blk_row0, const int* blk_rows, const int* n_blk, int max_blk, int n_experts,
                        int bn, const void* rs_table, int rs_rank, int rs_world, int rs_tpr, const int* ag_cnt,
                        int ag_expect, const int* blk_wait, const int* row_src, const void* ret_table, void* stream) {
  if (K % (i8 ? 128 : 64) != 0 || M < 1 || N % 8 != 0) return -1;
  if (epi == EPI_SILU_MUL && N % 32 != 0) return -2;
  if (epi == EPI_RS_PUSH && (!rs_table || rs_world < 1 || rs_world > kMaxRanks || rs_rank < 0 || rs_rank >= rs_world ||
                             rs_tpr < 1 || N % 64 != 0 || blk_expert || (M + BM - 1) / BM > rs_tpr * rs_world))
    return -3;
  GemmParams p;
  p.rs_table = (const unsigned long long*)rs_table; p.rs_rank = rs_rank; p.rs_world = rs_world; p.rs_tpr = rs_tpr;
  p.ag_cnt = ag_cnt; p.ag_expect = ag_expect;
  p.blk_wait = blk_wait; p.row_src = row_src; p.ret_table = (const unsigned long long*)ret_table;
  if (epi == EPI_EP_RETURN && (!row_src || !ret_table || !blk_expert || N % 64 != 0)) return -4;
  p.mt_rot = (epi == EPI_RS_PUSH) ? (rs_rank * rs_tpr) % ((M + BM - 1) / BM) : 0;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.C = c; p.resid = (const __nv_bfloat16*)resid;
  p.a_scale = a_scale; p.b_scale = b_scale; p.epi = epi;
  p.blk_expert = blk_expert; p.blk_row0 = blk_row0; p.blk_rows = blk_rows; p.n_blk = n_blk; p.max_blk = max_blk;
  if (bn != 128 && bn != 256) bn = (N >= 256 && (N % 256 == 0 || N > 2048)) ? 256 : 128;
  CUtensorMap ma, mb;
  int rc = make_map(&ma, a, i8 != 0, (uint64_t)M, (uint64_t)K, 1, BM);
  if (rc) return rc;
  rc = make_map(&mb, b, i8 != 0, (uint64_t)N, (uint64_t)K, blk_expert ? (uint64_t)n_experts : 1, (uint32_t)bn);
  if (rc) return rc;
  const int tiles_m = blk_expert ? max_blk : (M + BM - 1) / BM;
  const int n_tiles = tiles_m * ((N + bn - 1) / bn);
  cudaStream_t st = (cudaStream_t)stream;
  if (bn == 256) return i8 ? launch<256, true>(ma, mb, p, n_tiles, st) : launch<256, false>(ma, mb, p, n_tiles, st);
  return i8 ? launch<128, true>(ma, mb, p, n_tiles, st) : launch<128, false>(ma, mb, p, n_tiles, st);
}

extern "C" int b2_gemm_tc(const void* a, const void* b, void* c, int M, int N, int K, int ldc, int i8, int epi,
                          const void* resid, const float* a_scale, const float* b_scale, const int* blk_expert,
                          const int* blk_row0, const int* blk_rows, const int* n_blk, int max_blk, int n_experts,
                          int bn, void* stream) {
  return gemm_tc_impl(a, b, c, M, N, K, ldc, i8, epi, resid, a_scale, b_scale, blk_expert, blk_row0, blk_rows, n_blk,
                      max_blk, n_experts, bn, nullptr, 0, 1, 1, nullptr, 0, nullptr, nullptr, nullptr, stream);
}

// Tensor-parallel forms of the same kernel.  epi = 4 (row-parallel GEMM -> reduce-scatter): c is unused, the
// bf16 tiles go to the row owners' landing buffers of rs_table (rs_tpr m-tiles per owner) and arrivals are
// counted at the owners.  ag_cnt (all-gather -> GEMM): the rows of a arrive from their owners in this GPU's
// memory; m-tile i is loaded once ag_cnt[i] has reached ag_expect.
extern "C" int b2_gemm_tc_tp(const void* a, const void* b, void* c, int M, int N, int K, int ldc, int i8, int epi,
                             const void* resid, const float* a_scale, const float* b_scale, int bn,
                             const void* rs_table, int rs_rank, int rs_world, int rs_tpr, const int* ag_cnt,
                             int ag_expect, void* stream) {
  return gemm_tc_impl(a, b, c, M, N, K, ldc, i8, epi, resid, a_scale, b_scale, nullptr, nullptr, nullptr, nullptr, 0, 1,
                      bn, rs_table, rs_rank, rs_world, rs_tpr, ag_cnt, ag_expect, nullptr, nullptr, nullptr, stream);
}

// Expert-parallel forms of the grouped GEMM.  blk_wait: the rows of a block arrive from the source ranks'
// dispatch kernels; block i is loaded once blk_wait[i] >= blk_rows[i].  epi = 5: every result row is stored
// into the return buffer of the rank its token came from (row_src, ret_table).
extern "C" int b2_gemm_tc_ep(const void* a, const void* b, void* c, int M, int N, int K, int ldc, int epi,
                             const int* blk_expert, const int* blk_row0, const int* blk_rows, const int* n_blk,
                             int max_blk, int n_experts, int bn, const int* blk_wait, const int* row_src,
                             const void* ret_table, void* stream) {
  return gemm_tc_impl(a, b, c, M, N, K, ldc, 0, epi, nullptr, nullptr, nullptr, blk_expert, blk_row0, blk_rows, n_blk,
                      max_blk, n_experts, bn, nullptr, 0, 1, 1, nullptr, 0, blk_wait, row_src, ret_table, stream);
}

extern "C" int b2_dequant_w4b(const void* w4b, void* out_bf16, int N, int K, void* stream) {
  if (K % 64) return -1;
  dim3 grid(K / 64, (N + 127) / 128);
  dequant_w4b_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)w4b, (__nv_bfloat16*)out_bf16, N, K);
  return (int)cudaGetLastError();
}

extern "C" int b2_quant_rows_i8(const void* x, void* q, float* scale, int M, int K, void* stream) {
  if (K % 2) return -1;
  quant_rows_i8_kernel<<<M, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, (int8_t*)q, scale, K);
  return (int)cudaGetLastError();
}

B2_DEFINE_STATUS(gemm)
