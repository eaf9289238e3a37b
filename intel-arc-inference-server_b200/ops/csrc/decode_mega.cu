// Whole-step decode kernel: embedding and every dense layer of one decode / verify step (M <= 8 rows of one
// request) in ONE cooperative launch, with the int4 weight stream never draining between linears.
//
// The launch-per-linear form (gemv_w4.cu) pays a ramp at both ends of every kernel: the ring of the next linear
// cannot fill while the CTAs of the previous one hold the SM's shared memory, so a 27B step spends more time in
// ramps and tails than a layer's weights take to stream.  Here one CTA per SM stays resident for the whole step:
//
//   * warp 16 (one lane) is the weight producer.  It walks a static schedule -- for every layer qkv, o, gate||up,
//     down; for every linear this CTA's contiguous run of ring stages ("stream-K": the linear's stages, two
//     4352-byte W4B blocks each, are dealt to the CTAs in equal contiguous runs, so every SM streams the same
//     number of bytes whatever N and K are) -- and issues one bulk copy per stage as soon as a ring slot is free.
//     Weights depend on nothing, so it never looks at the grid barrier: while the CTAs meet there, or run the
//     attention phase, the ring (about 145 KB per SM) keeps filling from HBM.
//   * warp 17 is the activation producer.  The activations of a stage (the two 64-k groups of every row, already
//     quantised to the two-limb 15-bit form of gemv_w4.cu by whoever produced them) ride in the same ring slot on
//     a second mbarrier; this warp issues the copy once the grid barrier before the phase has been passed, so it
//     is the only party that polls the barrier during the linears.
//   * 16 consumer warps in two groups of 8 take alternate stages (warp w of a group owns rows 16w..16w+15 of the
//     128-row block, mma.m16n8k32.u8.s8 on raw nibbles exactly as gemv_w4.cu).  They wait on nothing but their
//     stage's two mbarriers.  At the end of an n-block's run the accumulators go to a shared-memory hand-off buffer
//     and the warps carry on with the next stage at once.
//   * warp 18 is the epilogue warp.  It takes each hand-off, adds the two groups' sums, stores them in a slot of
//     that n-block and takes a ticket; the last CTA to finish an n-block sums the slots in slot order and does the
//     linear's epilogue:
//        qkv      RoPE, q -> bf16 rows, k / v -> the paged cache at the rows' positions
//        o, down  residual add -> bf16 stream, per-block sums of squares, next RMSNorm weight, quantised rows
//        gate||up SiLU(gate) * up -> quantised rows for down
//     and after the CTA's last run of a phase it makes the CTA's arrival at the grid barrier.  The fences, the
//     ticket's round trip and the fold (microseconds of latency in all) are off the consumers' path this way.
//     RMSNorm's 1/rms is a per-row scalar, so it is applied to the partial sums of the NEXT linear when they
//     are written, not to its input.
//   * attention is its own phase: CTA (KV head, KV split) serves all rows x GQA heads on mma.m16n8k16 over
//     pages fetched with tiled TMA copies (128-byte swizzle, two 64-key buffers), the last CTA of a KV head
//     merges the splits in split order and quantises the o-proj input.
//
// Phases are separated by a grid barrier (one arrival per CTA on a monotonic counter; only the activation producer
// and, for the attention phase, one consumer thread poll it).  Every wait is bounded; a wait that runs out sets the
// status word and a CTA-wide flag that makes all later waits fail at once, the CTA still walks to its exit.
// All sums run in a fixed order (stage order inside a run, slot order across runs, split order in attention):
// bitwise reproducible, and a row's bits do not depend on M.
//
// Replaces, for the dense one-request step, the reference's closed command list of ~774 launches per token
// (src/runtime/capture.cc:1332-1510, src/runtime/capture.h:157-163) by a single launch.
#include "common.cuh"

using namespace b2;

namespace {

constexpr int CTRL_ROW_REQ = 16, CTRL_ROW_POS = 80, CTRL_CUR_TOKEN = 144;
constexpr int kBlockBytes = 4352;
constexpr int kSB = 4;                     // 64-k groups (W4B blocks) of one 128-row block per ring stage; an n-block's last stage may hold 2
constexpr int kWStage = kSB * kBlockBytes;  // weight bytes of a full stage
constexpr int kXRow = 144;                 // one (group, row) of activation limbs: 128 bytes + 16 (conflict-free reads)
constexpr int kConsWarps = 16, kCons = kConsWarps * 32;
constexpr int kGroups = 4, kGroupWarps = kConsWarps / kGroups;   // consumer groups take stages round-robin
constexpr int kThreads = kCons + 96;   // + weight producer, activation producer, epilogue warp
constexpr int kMaxNS = 18;
constexpr int kMaxRows = 8;
constexpr int D = 128;
constexpr int KB = 64;                     // keys per attention batch
constexpr int HALFB = KB * 128;            // half a K / V tile: 64 keys x 64 dims, 128-byte rows, TMA 128-byte swizzle
constexpr int TILEB = 2 * HALFB;
constexpr int KVBUF = 2 * TILEB;           // K tile + V tile of one batch
constexpr int kAttnBytes = 2 * KVBUF;      // two batches in flight
constexpr int kMaxSplit = 64;
constexpr unsigned ERR_MEGA_RING = 0xA01, ERR_MEGA_GRID = 0xA02, ERR_MEGA_KV = 0xA03, ERR_MEGA_PRODUCER = 0xA04;

struct MegaLayer {   // 64 bytes, array in device memory
  const uint8_t* w[4];        // qkv, o, gate||up, down (W4B)
  const float* input_norm;
  const float* post_norm;
  long long kv_plane;         // plane of the KV cache that belongs to this layer
  long long pad;
};

struct MegaParams {
  CUtensorMap k_map, v_map;   // the whole cache [plane][page][kv head][16] rows x 128 dims, boxes of 16 rows x 64 dims
  const MegaLayer* layers;
  int n_layers, M, rows, nCTA, NS;
  int H, n_q, n_kv, gqa, nbH;
  int nb[4], SG[4], T[4], maxseg[4];     // per linear: n-blocks, stages per n-block, stages, most runs per n-block
  int KG[4];                             // per linear: 64-k groups per row (K / 64)
  const int* ctrl;
  const int* block_table;
  int max_blocks, num_pages;
  const __nv_bfloat16* embed;
  int vocab;
  int* flag;
  const float* cos_t;
  const float* sin_t;
  __nv_bfloat16* k_cache;
  __nv_bfloat16* v_cache;
  __nv_bfloat16* resid;       // [M][H]
  float* ssq;                 // [M][nbH]
  uint8_t* xq[3];             // quantised rows [K/64][rows][144]: 0 hidden-wide (qkv, gate||up), 1 o input, 2 down input
  uint32_t* gs[3];            // {scale, -8 sum X} [K/64][8 token slots][2]
  float* part;                // partial sums [2][n-block][2 * maxseg][M][128]: consecutive linears alternate halves
  long long part_half;        // floats per half
  int* tickets;               // [max n-blocks], zero between phases
  __nv_bfloat16* q;           // [M][n_q * 128]
  float* o_part;              // [M][n_q][nsplit][128]
  float* ml_part;             // [M][n_q][nsplit][2]
  int* attn_tickets;          // [n_kv]
  unsigned* bar;              // [0] arrivals, [1] abort, [2] exits
  float eps, scale_log2;
  int nsplit, span_pages;
  int n_phases;               // phases to run (1 + 5 * n_layers for a whole step; fewer: a debugging cut)
  int variant;                // measurement switches (environment B2_MEGA_VARIANT; results are wrong with any bit set):
                              // 1 consumers skip the maths, 2 no weight copies, 4 no activation copies, 8 no attention work,
  unsigned long long* dbg;    // optional [nCTA][8][32] timestamps per phase: arrival, barrier seen by the activation producer,
                              // consumers done with their last stage, consumers holding their first stage; the epilogue
                              // warp's last run end: handed over, sums stored, ticket known, folded
};

struct Smem {   // byte addresses in the shared window
  uint32_t ring, fullW, fullX, empty, kvbar, misc, attn;
  uint32_t out, outfull, outempty;   // run-end hand-off: [2 buffers][2 groups][M][128] floats and their barriers
  int stageB;
};

// ------------------------------------------------------------------ small helpers
__device__ __forceinline__ void cons_sync() { asm volatile("bar.sync 1, 512;" ::: "memory"); }
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
__device__ __forceinline__ uint32_t lds32v(uint32_t a) {
  uint32_t v;
  asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(v) : "r"(a) : "memory");
  return v;
}
__device__ __forceinline__ void sts32(uint32_t a, uint32_t v) {
  asm volatile("st.shared.u32 [%0], %1;" ::"r"(a), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
// Ticket / arrival in one operation: the release covers the warp's earlier stores (ordered before it by the warp
// barrier in front), the acquire the loads that follow.
__device__ __forceinline__ int atom_add_acq_rel(int* p, int v) {
  int old;
  asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return old;
}
__device__ __forceinline__ void red_add_release(unsigned* p, unsigned v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Wait on an mbarrier, bounded.  After any wait of this CTA has run out (or the CTA has learnt that the launch is
// being abandoned) every wait fails: at once if it has not begun, else at its next look at the flag.
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
#ifdef B2_MEGA_PROF
#define MISS_ARG , long long* miss = nullptr
#define MISS_COUNT if (miss) ++*miss;
#else
#define MISS_ARG
#define MISS_COUNT
#endif
__device__ __forceinline__ bool mwait(uint32_t bar, uint32_t parity, uint32_t failed_addr, unsigned code MISS_ARG) {
  if (mbar_test(bar, parity)) return true;   // in the steady state the phase is complete already
  MISS_COUNT
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
      if (mbar_try(bar, parity)) return true;
    if (lds32v(failed_addr)) return false;
    if (clock64() - t0 > kWaitCycles) {
      record_error(code, (blockIdx.x << 8) | (threadIdx.x >> 5));
      sts32(failed_addr, 1u);
      return false;
    }
  }
}

// A whole warp waits: one lane polls (every lane's poll of one mbarrier is a shared-memory operation of its own, and
// they are served one after the other: 32 of them cost some 400 cycles even on a completed phase), the shuffle
// hands the result to the others and orders their reads after the lane's acquire.
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, uint32_t failed_addr, unsigned code, int lane MISS_ARG) {
  int r = 1;
#ifdef B2_MEGA_PROF
  if (lane == 0) r = mwait(bar, parity, failed_addr, code, miss) ? 1 : 0;
#else
  if (lane == 0) r = mwait(bar, parity, failed_addr, code) ? 1 : 0;
#endif
  return __shfl_sync(0xffffffffu, r, 0) != 0;
}

__device__ __forceinline__ void mma_u8s8_16832(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
// byte offset of (key row, dim d) inside a swizzled 64-key tile; d a multiple of 8
__device__ __forceinline__ uint32_t tile_off(int row, int d) {
  return (uint32_t)((d >> 6) * HALFB + row * 128 + ((((d & 63) >> 3) ^ (row & 7)) << 4));
}

// The CTA that owns stage s of a linear with T stages dealt to n CTAs in runs [T c / n, T (c + 1) / n).
// (32-bit arithmetic: the plan refuses shapes with T * n >= 2^31; a 64-bit division is a long subroutine on the GPU)
__host__ __device__ inline int stage_owner(int s, int n, int T) { return (int)((((unsigned)s + 1u) * (unsigned)n - 1u) / (unsigned)T); }
// First stage of CTA c's run: T c / n.
__host__ __device__ inline int run_begin(int T, int c, int n) { return (int)((unsigned)T * (unsigned)c / (unsigned)n); }

// ------------------------------------------------------------------ activation quantiser (the form of gemv_w4.cu)
// X = rint(x * 16383 / amax) = 128 X_hi + X_lo per 64-k group; eight lanes (one 8-vector each) hold a group and share
// amax and sum(X) by shuffles: every lane of the warp must call this.
struct StagedVec {
  uint32_t w[4];
  float scale;
  int m8sum;
};
__device__ __forceinline__ StagedVec stage_quant_f(const float (&xf)[8]) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(xf[i]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
  const bool live = amax > 0.f && amax < 3.0e38f;
  const float inv = live ? 16383.f / amax : 0.f;
  int X[8], sumX = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    X[i] = __float2int_rn(xf[i] * inv);
    sumX += X[i];
  }
  sumX += __shfl_xor_sync(0xffffffffu, sumX, 1);
  sumX += __shfl_xor_sync(0xffffffffu, sumX, 2);
  sumX += __shfl_xor_sync(0xffffffffu, sumX, 4);
  StagedVec o;
  o.w[0] = o.w[1] = o.w[2] = o.w[3] = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    o.w[0] |= (uint32_t)((X[i] >> 7) & 0xff) << (8 * i);
    o.w[1] |= (uint32_t)(X[i] & 127) << (8 * i);
    o.w[2] |= (uint32_t)((X[i + 4] >> 7) & 0xff) << (8 * i);
    o.w[3] |= (uint32_t)(X[i + 4] & 127) << (8 * i);
  }
  o.scale = live ? amax / 16383.f : 0.f;
  o.m8sum = -8 * sumX;
  return o;
}
__device__ __forceinline__ int stage_word(int vq) { return (vq & 1) * 16 + (vq >> 2) * 2 + ((vq & 3) >> 1); }

// Writes vector vq of (group, row) of a quantised activation buffer.
__device__ __forceinline__ void store_staged(const MegaParams& p, int which, int group, int row, int vq, const StagedVec& sv) {
  uint32_t* dst = reinterpret_cast<uint32_t*>(p.xq[which] + ((size_t)group * p.rows + row) * kXRow) + stage_word(vq);
  dst[0] = sv.w[0];
  dst[4] = sv.w[1];
  dst[8] = sv.w[2];
  dst[12] = sv.w[3];
  if (vq == 0) {
    p.gs[which][((size_t)group * 8 + row) * 2] = __float_as_uint(sv.scale);
    p.gs[which][((size_t)group * 8 + row) * 2 + 1] = (uint32_t)sv.m8sum;
  }
}

// Sum of the slots of an n-block for eight consecutive columns, in slot order.
__device__ __forceinline__ void sum_slots8(const float* base, int nslots, size_t slot_stride, float (&v)[8]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = 0.f;
#pragma unroll 4
  for (int ps = 0; ps < nslots; ++ps) {
    const float4 a = __ldcg(reinterpret_cast<const float4*>(base + (size_t)ps * slot_stride));
    const float4 b = __ldcg(reinterpret_cast<const float4*>(base + (size_t)ps * slot_stride + 4));
    v[0] += a.x; v[1] += a.y; v[2] += a.z; v[3] += a.w;
    v[4] += b.x; v[5] += b.y; v[6] += b.z; v[7] += b.w;
  }
}

// ------------------------------------------------------------------ grid barrier
// One arrival per CTA and phase; phase g is complete when the counter has reached (g + 1) * nCTA.  A CTA arrives for
// phase g only after it has seen phase g - 1 complete (its stages' activations, or an explicit wait), which is what
// makes the plain counter a barrier.
__device__ __forceinline__ void grid_arrive(const MegaParams& p, int tid, int phase = -1) {
  fence_proxy_async_all();   // this phase's generic-proxy stores are read by TMA / bulk copies of other CTAs next
  cons_sync();
  if (tid == 0) {
    if (p.dbg && phase >= 0 && phase < 32) p.dbg[((size_t)blockIdx.x * 8 + 0) * 32 + phase] = globaltimer_ns();
    red_add_release(p.bar, 1u);   // releases the consumers' stores of the phase (ordered before it by the barrier)
  }
}
// Consumer-side wait until `phases` phases are complete (tid 0 polls, bounded).
__device__ __forceinline__ bool grid_wait(const MegaParams& p, const Smem& sm, int phases, int tid) {
  if (tid == 0) {
    const unsigned need = (unsigned)phases * (unsigned)p.nCTA;
    bool ok = lds32v(sm.misc) == 0u;
    if (ok) {
      const long long t0 = clock64();
      int spins = 0;
      while (ld_acquire_gpu(p.bar) < need) {
        if (++spins > 64) {
          if (ld_acquire_gpu(p.bar + 1) != 0u || clock64() - t0 > 3000000000ll) {
            if (ld_acquire_gpu(p.bar + 1) == 0u) record_error(ERR_MEGA_GRID, (unsigned)phases << 16 | blockIdx.x);
            atomicExch(p.bar + 1, 1u);
            ok = false;
            break;
          }
          __nanosleep(32);
        }
      }
    }
    if (!ok) sts32(sm.misc, 1u);
    sts32(sm.misc + 4, ok ? 1u : 0u);
  }
  cons_sync();
  const bool ok = lds32v(sm.misc + 4) != 0u;
  cons_sync();   // the word is rewritten by the next wait
  return ok;
}

// ------------------------------------------------------------------ optional cycle accounting (compile with -DB2_MEGA_PROF)
// One thread per role adds up the cycles between marks; at its exit it stores the sums behind the phase timestamps
// of `dbg`: [nCTA][4 roles][8] after the first nCTA * 64 words.
#ifdef B2_MEGA_PROF
struct Prof {
  long long t, v[8];
  __device__ __forceinline__ void start() {
    t = clock64();
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0;
  }
  __device__ __forceinline__ void mark(int k) {
    const long long now = clock64();
    v[k] += now - t;
    t = now;
  }
  __device__ __forceinline__ void dump(const MegaParams& p, int role) {
    if (!p.dbg) return;
#pragma unroll
    for (int i = 0; i < 8; ++i) p.dbg[(size_t)p.nCTA * 256 + ((size_t)blockIdx.x * 4 + role) * 8 + i] = (unsigned long long)v[i];
  }
};
#define PROF_DECL Prof prof; prof.start();
#define PROF_MARK(k) prof.mark(k);
#define PROF_DUMP(role) prof.dump(p, role);
#else
#define PROF_DECL
#define PROF_MARK(k)
#define PROF_DUMP(role)
#endif

// ------------------------------------------------------------------ the schedule every role of a CTA walks
struct Cursor {
  int gphase;        // global phase of the linear the cursor is in
  int kind, layer;
  int s, s1;         // next stage, end of this CTA's run
  int ks;            // the stage's position inside its n-block (k groups kSB * ks ...)
  bool fresh;        // the cursor has just entered a linear
};
__device__ __forceinline__ bool cursor_load(const MegaParams& p, Cursor& c) {
  // positions the cursor on the first stage of this CTA's run of (layer, kind); false when past the last phase
  for (;;) {
    if (c.layer >= p.n_layers) return false;
    c.gphase = 1 + 5 * c.layer + (c.kind == 0 ? 0 : c.kind + 1);
    if (c.gphase >= p.n_phases) return false;
    const int T = p.T[c.kind];
    c.s = run_begin(T, blockIdx.x, p.nCTA);
    c.s1 = run_begin(T, blockIdx.x + 1, p.nCTA);
    c.ks = c.s % p.SG[c.kind];
    c.fresh = true;
    if (c.s < c.s1) return true;
    if (++c.kind == 4) { c.kind = 0; ++c.layer; }
  }
}
__device__ __forceinline__ bool cursor_next(const MegaParams& p, Cursor& c) {
  c.fresh = false;
  if (++c.ks == p.SG[c.kind]) c.ks = 0;
  if (++c.s < c.s1) return true;
  if (++c.kind == 4) { c.kind = 0; ++c.layer; }
  return cursor_load(p, c);
}

// One thread polls the arrival counter until `need` arrivals are in (phases 0 .. need / nCTA - 1 complete).
// Returns the counter, or 0xffffffff when the launch is being abandoned or the bound ran out.
__device__ __forceinline__ unsigned poll_arrivals(const MegaParams& p, const Smem& sm, unsigned need, unsigned code, int phase,
                                                  unsigned nap = 64) {
  unsigned v = ld_acquire_gpu(p.bar);
  if (v >= need) return v;
  const long long t0 = clock64();
  int spins = 0;
  for (;;) {
    v = ld_acquire_gpu(p.bar);
    if (v >= need) return v;
    if (++spins > 16) {
      __nanosleep(nap);
      if ((spins & 15) == 0) {
        const bool stale = clock64() - t0 > 3000000000ll;
        if (stale || lds32v(sm.misc) != 0u || ld_acquire_gpu(p.bar + 1) != 0u) {
          if (stale && ld_acquire_gpu(p.bar + 1) == 0u) record_error(code, (unsigned)phase << 16 | blockIdx.x);
          atomicExch(p.bar + 1, 1u);
          sts32(sm.misc, 1u);
          return 0xffffffffu;
        }
      }
    }
  }
}

// ------------------------------------------------------------------ the weight producer (one thread)
// Walks the schedule and refills every ring slot the consumers give back.  Weights depend on nothing, so this
// thread never looks at the grid barrier: the stream runs on through phase changes and through attention.
__device__ void w_producer(const MegaParams& p, const Smem& sm) {
  Cursor c{0, 0, 0, 0, 0, 0, true};
  bool more = cursor_load(p, c);
  int slot = 0, issued = 0;
  unsigned use = 0;
  bool ok = true;
  const uint8_t* wptr = nullptr;   // a CTA's run of a linear is one contiguous byte range of its W4B tensor
  int KG = 0;
  PROF_DECL
  while (more) {
#ifdef B2_MEGA_PROF
    ++prof.v[6];
    if (use > 0 && !mwait(sm.empty + 8 * slot, (use - 1) & 1u, sm.misc, ERR_MEGA_RING, &prof.v[7])) {
#else
    if (use > 0 && !mwait(sm.empty + 8 * slot, (use - 1) & 1u, sm.misc, ERR_MEGA_RING)) {
#endif
      ok = false;
      break;
    }
    if (c.fresh) {
      KG = p.KG[c.kind];
      const int j = c.s / p.SG[c.kind];
      wptr = p.layers[c.layer].w[c.kind] + ((size_t)j * KG + (size_t)c.ks * kSB) * kBlockBytes;
    }
    const uint32_t wbytes = (uint32_t)min(kSB, KG - c.ks * kSB) * kBlockBytes;
    if (p.variant & 2) {
      mbar_arrive(sm.fullW + 8 * slot);
    } else {
      mbar_expect_tx(sm.fullW + 8 * slot, wbytes);
      bulk_g2s(sm.ring + slot * sm.stageB, wptr, wbytes, sm.fullW + 8 * slot);
    }
    wptr += wbytes;
    ++issued;
    if (++slot == p.NS) { slot = 0; ++use; }
    more = cursor_next(p, c);
  }
  PROF_DUMP(0)
  if (!ok) {
    // drain: the copies that were issued must have landed before the CTA gives its shared memory back
    atomicExch(p.bar + 1, 1u);
    for (int G = (issued > p.NS ? issued - p.NS : 0); G < issued; ++G)
      mbar_wait(sm.fullW + 8 * (G % p.NS), (uint32_t)((G / p.NS) & 1), ERR_MEGA_RING);
  }
}

// ------------------------------------------------------------------ the activation producer (one thread)
// The two 64-k groups of a stage for every row (contiguous in the quantised buffer) and their {scale, -8 sum} words:
// two bulk copies into the stage's slot behind the weights, on the slot's second mbarrier.  A linear's rows exist
// once the phase before it is complete, so this thread is the one that meets the grid barrier; the consumers only
// ever wait on their stage's two mbarriers.  The rows were written with ordinary stores by other CTAs: their
// writers fence towards the async proxy before they arrive at the barrier, and so does this thread after it.
__device__ void x_producer(const MegaParams& p, const Smem& sm) {
  Cursor c{0, 0, 0, 0, 0, 0, true};
  bool more = cursor_load(p, c);
  int slot = 0, issued = 0;
  unsigned use = 0, seen = 0;
  bool ok = true;
  const uint32_t xgroup = (uint32_t)p.rows * kXRow;   // bytes of one 64-k group of every row
  int KG = 0;
  const uint8_t* xbase = nullptr;
  const uint8_t* gbase = nullptr;
  PROF_DECL
  while (more) {
#ifdef B2_MEGA_PROF
    ++prof.v[6];
    if (use > 0 && !mwait(sm.empty + 8 * slot, (use - 1) & 1u, sm.misc, ERR_MEGA_RING, &prof.v[7])) {
#else
    if (use > 0 && !mwait(sm.empty + 8 * slot, (use - 1) & 1u, sm.misc, ERR_MEGA_RING)) {
#endif
      ok = false;
      break;
    }
    const unsigned need = (unsigned)c.gphase * (unsigned)p.nCTA;   // the phase before this linear's is complete
    if (seen < need) {
      const unsigned v = poll_arrivals(p, sm, need, ERR_MEGA_PRODUCER, c.gphase);
      if (v == 0xffffffffu) {
        ok = false;
        break;
      }
      seen = v;
      __threadfence();
      fence_proxy_async_all();   // the copies below (async proxy) come after the other CTAs' stores
      if (p.dbg && c.gphase < 32) p.dbg[((size_t)blockIdx.x * 8 + 1) * 32 + c.gphase] = globaltimer_ns();
    }
    if (c.fresh) {
      const int which = c.kind == 1 ? 1 : (c.kind == 3 ? 2 : 0);
      xbase = p.xq[which];
      gbase = reinterpret_cast<const uint8_t*>(p.gs[which]);
      KG = p.KG[c.kind];
    }
    const uint32_t dst = sm.ring + slot * sm.stageB + kWStage;
    if (p.variant & 4) {
      mbar_arrive(sm.fullX + 8 * slot);
    } else {
      // the stage's k groups walk round and round the row: kSB * ks .. (an n-block's last stage may be short)
      const uint32_t ng = (uint32_t)min(kSB, KG - c.ks * kSB);
      mbar_expect_tx(sm.fullX + 8 * slot, ng * (xgroup + 64u));
      bulk_g2s(dst, xbase + (size_t)(c.ks * kSB) * xgroup, ng * xgroup, sm.fullX + 8 * slot);
      bulk_g2s(dst + kSB * xgroup, gbase + (size_t)(c.ks * kSB) * 64, ng * 64u, sm.fullX + 8 * slot);
    }
    ++issued;
    if (++slot == p.NS) { slot = 0; ++use; }
    more = cursor_next(p, c);
  }
  PROF_DUMP(1)
  if (!ok) {
    sts32(sm.misc, 1u);
    atomicExch(p.bar + 1, 1u);
    for (int G = (issued > p.NS ? issued - p.NS : 0); G < issued; ++G)
      mbar_wait(sm.fullX + 8 * (G % p.NS), (uint32_t)((G / p.NS) & 1), ERR_MEGA_RING);
  }
}

// ------------------------------------------------------------------ linear epilogues, run by the CTA that finishes an n-block last
// KIND 0 qkv: RoPE; q rows as bf16, k / v rows into the cache.  Items (row m, 8-vector v of the head's 128 dims).
__device__ void fold_qkv(const MegaParams& p, const MegaLayer& L, int j, int nslots, int tid, int nthreads) {
  const int warp = tid >> 5, lane = tid & 31;
  const int items = p.M * 16;
  const int pos0 = p.ctrl[CTRL_ROW_POS], req = p.ctrl[CTRL_ROW_REQ];
  const size_t slot_stride = (size_t)p.M * 128;
  const float* pbase = p.part + (size_t)j * 2 * p.maxseg[0] * slot_stride;   // qkv: half 0
  for (int it0 = warp * 32; it0 < items; it0 += nthreads) {
    const int it = it0 + lane;
    const bool act = it < items;
    const int m = act ? it >> 4 : 0, v = it & 15;
    float x[8];
    if (act) sum_slots8(pbase + (size_t)m * 128 + 8 * v, nslots, slot_stride, x);
    else {
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] = 0.f;
    }
    const int pos = pos0 + m;
    float y[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float px = __shfl_xor_sync(0xffffffffu, x[i], 8);   // the rotate-half partner: dim d +- 64
      if (j < p.n_q + p.n_kv) {
        const int d = (8 * v + i) & 63;
        const float cs = p.cos_t[(size_t)pos * 64 + d], sn = p.sin_t[(size_t)pos * 64 + d];
        y[i] = v >= 8 ? x[i] * cs + px * sn : x[i] * cs - px * sn;
      } else {
        y[i] = x[i];
      }
    }
    if (!act) continue;
    uint4 o;
    o.x = pack_bf16(y[0], y[1]); o.y = pack_bf16(y[2], y[3]); o.z = pack_bf16(y[4], y[5]); o.w = pack_bf16(y[6], y[7]);
    if (j < p.n_q) {
      *reinterpret_cast<uint4*>(p.q + (size_t)m * p.n_q * D + (size_t)j * D + 8 * v) = o;
    } else {
      const bool is_v = j >= p.n_q + p.n_kv;
      const int kh = j - p.n_q - (is_v ? p.n_kv : 0);
      const int page = p.block_table[(size_t)req * p.max_blocks + (pos >> 4)];
      __nv_bfloat16* base = (is_v ? p.v_cache : p.k_cache) + (size_t)L.kv_plane * p.num_pages * p.n_kv * 16 * D;
      *reinterpret_cast<uint4*>(base + (((size_t)page * p.n_kv + kh) * 16 + (pos & 15)) * D + 8 * v) = o;
    }
  }
}

// KIND 1 / 3 (and the embedding, nslots = 0 with `src` the rows' embedding vectors): residual add, bf16 stream,
// the block's sums of squares, next norm weight and quantised rows for the next hidden-wide linear.
__device__ void fold_resid(const MegaParams& p, int kind, const float* norm_next, int j, int nslots, int tid, int nthreads, bool embed) {
  const int warp = tid >> 5, lane = tid & 31;
  const int items = p.M * 16;
  const size_t slot_stride = (size_t)p.M * 128;
  const float* pbase = embed ? nullptr : p.part + (kind & 1) * p.part_half + (size_t)j * 2 * p.maxseg[kind] * slot_stride;
  for (int it0 = warp * 32; it0 < items; it0 += nthreads) {
    const int it = it0 + lane;
    const bool act = it < items;
    const int m = act ? it >> 4 : 0, v = it & 15;
    float x[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = 0.f;
    uint4 rv = make_uint4(0, 0, 0, 0);
    if (act) {
      if (embed) {
        int tok = p.ctrl[CTRL_CUR_TOKEN + m];
        if (tok < 0 || tok >= p.vocab) {
          if (p.flag) atomicExch(p.flag, 0xDEAD0001);
          tok = 0;
        }
        rv = *reinterpret_cast<const uint4*>(p.embed + (size_t)tok * p.H + (size_t)j * 128 + 8 * v);
      } else {
        sum_slots8(pbase + (size_t)m * 128 + 8 * v, nslots, slot_stride, x);
        rv = __ldcg(reinterpret_cast<const uint4*>(p.resid + (size_t)m * p.H + (size_t)j * 128 + 8 * v));
      }
    }
    const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
    uint32_t ow[4];
    float rf[8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      ow[i] = pack_bf16(bf16_lo(rw[i]) + x[2 * i], bf16_hi(rw[i]) + x[2 * i + 1]);
      rf[2 * i] = bf16_lo(ow[i]);
      rf[2 * i + 1] = bf16_hi(ow[i]);
      ss += rf[2 * i] * rf[2 * i] + rf[2 * i + 1] * rf[2 * i + 1];
    }
    ss += __shfl_xor_sync(0xffffffffu, ss, 1);
    ss += __shfl_xor_sync(0xffffffffu, ss, 2);
    ss += __shfl_xor_sync(0xffffffffu, ss, 4);
    ss += __shfl_xor_sync(0xffffffffu, ss, 8);
    if (act) {
      *reinterpret_cast<uint4*>(p.resid + (size_t)m * p.H + (size_t)j * 128 + 8 * v) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
      if (v == 0) p.ssq[(size_t)m * p.nbH + j] = ss;
    }
    if (norm_next) {
      float y[8];
      const float4 w0 = *reinterpret_cast<const float4*>(norm_next + (size_t)j * 128 + 8 * v);
      const float4 w1 = *reinterpret_cast<const float4*>(norm_next + (size_t)j * 128 + 8 * v + 4);
      y[0] = rf[0] * w0.x; y[1] = rf[1] * w0.y; y[2] = rf[2] * w0.z; y[3] = rf[3] * w0.w;
      y[4] = rf[4] * w1.x; y[5] = rf[5] * w1.y; y[6] = rf[6] * w1.z; y[7] = rf[7] * w1.w;
      const StagedVec sv = stage_quant_f(y);
      if (act) store_staged(p, 0, 2 * j + (v >> 3), m, v & 7, sv);
    }
  }
}

// KIND 2 gate||up (interleave16: runs of 16 gate, 16 up): SiLU(gate) * up -> one quantised group of down's input.
__device__ void fold_act(const MegaParams& p, int j, int nslots, int tid, int nthreads) {
  const int warp = tid >> 5, lane = tid & 31;
  const int items = p.M * 8;
  const size_t slot_stride = (size_t)p.M * 128;
  const float* pbase = p.part + (size_t)j * 2 * p.maxseg[2] * slot_stride;   // gate||up: half 0
  for (int it0 = warp * 32; it0 < items; it0 += nthreads) {
    const int it = it0 + lane;
    const bool act = it < items;
    const int m = act ? it >> 3 : 0, a = it & 7;
    const int gcol = (a >> 1) * 32 + (a & 1) * 8;
    float gsum[8], usum[8], y[8];
    if (act) {
      sum_slots8(pbase + (size_t)m * 128 + gcol, nslots, slot_stride, gsum);
      sum_slots8(pbase + (size_t)m * 128 + gcol + 16, nslots, slot_stride, usum);
    }
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
      const uint32_t pk = act ? pack_bf16(silu(gsum[i]) * usum[i], silu(gsum[i + 1]) * usum[i + 1]) : 0u;
      y[i] = bf16_lo(pk);
      y[i + 1] = bf16_hi(pk);
    }
    const StagedVec sv = stage_quant_f(y);
    if (act) store_staged(p, 2, j, m, a, sv);
  }
}

// ------------------------------------------------------------------ one linear: this CTA's run of stages
struct Lane {
  int tid, warp, lane, wq, gidx, g, t;
};
// What a consumer thread carries from phase to phase: stages and run ends of this CTA so far (every role counts
// them the same way), and the ring position of its group's next stage (the groups take alternate stages).
struct ConsState {
  int G, R, slot;
  uint32_t par;
#ifdef B2_MEGA_PROF
  Prof prof;
#endif
};
#ifdef B2_MEGA_PROF
#define CPROF(k) cs.prof.mark(k);
#else
#define CPROF(k)
#endif

__device__ __forceinline__ void sts_f32(uint32_t a, float v) { asm volatile("st.shared.f32 [%0], %1;" ::"r"(a), "f"(v) : "memory"); }
__device__ __forceinline__ float4 lds_f4(uint32_t a) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a));
  return v;
}

// Which runs meet in n-block j of a linear, and which of them is CTA c's (whose last stage there is s_last).  With
// at least one stage per CTA the runs belong to consecutive CTAs; a linear with fewer stages than CTAs gives
// single-stage runs to scattered CTAs, one per stage.
__device__ __forceinline__ void run_slots(const MegaParams& p, int kind, int c, int j, int s_last, int& nseg, int& seg) {
  const int T = p.T[kind], SG = p.SG[kind];
  if (T >= p.nCTA) {
    const int c_first = stage_owner(j * SG, p.nCTA, T), c_last = stage_owner((j + 1) * SG - 1, p.nCTA, T);
    nseg = c_last - c_first + 1;
    seg = c - c_first;
  } else {
    nseg = SG;
    seg = s_last - j * SG;
  }
}

// The consumer side: wait for a stage's two mbarriers, multiply, give the slot back.  At the end of a run inside an
// n-block the accumulators go to a shared-memory hand-off buffer and the warps carry on with the next stage at
// once: global stores, fences, tickets and folds are the epilogue warp's business.
template <int KIND>
__device__ void gemv_phase(const MegaParams& p, const Smem& sm, ConsState& cs, bool& ok, const Lane& ln, int layer_dbg) {
  const int T = p.T[KIND], SG = p.SG[KIND];
  const int c = blockIdx.x;
  const int s0 = run_begin(T, c, p.nCTA), s1 = run_begin(T, c + 1, p.nCTA);
  if (s0 == s1) return;
  // A warp of a group owns rows 32 wq .. 32 wq + 31 of the 128-row block as two 16-row tiles: two independent chains
  // of integer MMAs per 64-k group, and the activation fragments are read once for both.
  float acc[2][4];
#pragma unroll
  for (int h = 0; h < 2; ++h) acc[h][0] = acc[h][1] = acc[h][2] = acc[h][3] = 0.f;
  const uint32_t w_off = ln.wq * 1024 + ln.lane * 16;
  const uint32_t sc_off = 4096 + (ln.wq * 32 + 2 * ln.g) * 2;
  const uint32_t x_off = kWStage + min(ln.g, p.rows - 1) * kXRow + ln.t * 32;
  const uint32_t gs_off = kWStage + kSB * p.rows * kXRow + 2 * ln.t * 8;
  const int KG = p.KG[KIND];
  int ks = s0 % SG;   // the stage's position inside its n-block
  const uint32_t out_g = sm.out + ln.gidx * p.M * 512;
  constexpr uint32_t kMask = 0x0F0F0F0Fu;
  int jend = (s0 / SG + 1) * SG;   // first stage of the next n-block
  const int gphase_dbg = 1 + 5 * layer_dbg + (KIND == 0 ? 0 : KIND + 1);
  bool first_dbg = p.dbg != nullptr && ln.tid == 0 && gphase_dbg < 32;
  for (int s = s0; s < s1; ++s) {
    if (((cs.G + s - s0) & (kGroups - 1)) == ln.gidx) {
      const int slot = cs.slot;
      const uint32_t par = cs.par;
      // the shuffle inside keeps `ok` the same in every lane: the code below runs warp-wide
#ifdef B2_MEGA_PROF
      ++cs.prof.v[6];
      if (ok) ok = warp_wait(sm.fullW + 8 * slot, par, sm.misc, ERR_MEGA_RING, ln.lane, &cs.prof.v[0]);
      if (ok) ok = warp_wait(sm.fullX + 8 * slot, par, sm.misc, ERR_MEGA_RING, ln.lane, &cs.prof.v[1]);
#else
      if (ok) ok = warp_wait(sm.fullW + 8 * slot, par, sm.misc, ERR_MEGA_RING, ln.lane);
      if (ok) ok = warp_wait(sm.fullX + 8 * slot, par, sm.misc, ERR_MEGA_RING, ln.lane);
#endif
      if (first_dbg) {
        first_dbg = false;
        p.dbg[((size_t)blockIdx.x * 8 + 3) * 32 + gphase_dbg] = globaltimer_ns();
      }
      if (ok && !(p.variant & 1)) {
        const uint32_t st = sm.ring + slot * sm.stageB;
        const int ng = min(kSB, KG - ks * kSB);
#pragma unroll 2
        for (int q = 0; q < ng; ++q) {
          const uint4 xh = lds128(st + x_off + q * p.rows * kXRow);
          const uint4 xl = lds128(st + x_off + q * p.rows * kXRow + 16);
          const uint4 gsv = lds128(st + gs_off + q * 64);
          const float sx0 = __uint_as_float(gsv.x), sx1 = __uint_as_float(gsv.z);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint4 wv = lds128(st + q * kBlockBytes + w_off + h * 512);
            const uint32_t sc2 = lds32(st + q * kBlockBytes + sc_off + h * 32);
            const uint32_t l0 = wv.x & kMask, l1 = wv.y & kMask, l2 = wv.z & kMask, l3 = wv.w & kMask;
            const uint32_t h0 = (wv.x >> 4) & kMask, h1 = (wv.y >> 4) & kMask;
            const uint32_t h2 = (wv.z >> 4) & kMask, h3 = (wv.w >> 4) & kMask;
            const __half2 sh = *reinterpret_cast<const __half2*>(&sc2);
            const float s_lo = __low2float(sh), s_hi = __high2float(sh);
            int ih[4] = {0, 0, 0, 0};
            int il[4] = {(int)gsv.y, (int)gsv.w, (int)gsv.y, (int)gsv.w};
            mma_u8s8_16832(ih, l0, l1, h0, h1, xh.x, xh.y);
            mma_u8s8_16832(il, l0, l1, h0, h1, xl.x, xl.y);
            mma_u8s8_16832(ih, l2, l3, h2, h3, xh.z, xh.w);
            mma_u8s8_16832(il, l2, l3, h2, h3, xl.z, xl.w);
            acc[h][0] = fmaf(s_lo * sx0, (float)(ih[0] * 128 + il[0]), acc[h][0]);
            acc[h][1] = fmaf(s_lo * sx1, (float)(ih[1] * 128 + il[1]), acc[h][1]);
            acc[h][2] = fmaf(s_hi * sx0, (float)(ih[2] * 128 + il[2]), acc[h][2]);
            acc[h][3] = fmaf(s_hi * sx1, (float)(ih[3] * 128 + il[3]), acc[h][3]);
          }
        }
      }
      if (ok) {
        __syncwarp();
        if (ln.lane == 0) mbar_arrive(sm.empty + 8 * slot);
      }
      cs.slot += kGroups;
      if (cs.slot >= p.NS) {
        cs.slot -= p.NS;
        cs.par ^= 1u;
      }
    }
    if (++ks == SG) ks = 0;
    if (s + 1 < s1 && s + 1 < jend) continue;
    // ---- end of this CTA's run inside an n-block: hand the sums (zeros from a group without a stage) over
    jend += SG;
    const int buf = cs.R & 1;
    if (ok && cs.R >= 2) ok = warp_wait(sm.outempty + 8 * buf, (uint32_t)(((cs.R >> 1) - 1) & 1), sm.misc, ERR_MEGA_RING, ln.lane);
    if (ok) {
      const uint32_t o = out_g + buf * (kGroups * p.M * 512);
      const int m0 = 2 * ln.t, m1 = m0 + 1;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int n_lo = ln.wq * 32 + h * 16 + ln.g;
        if (m0 < p.M) {
          sts_f32(o + (m0 * 128 + n_lo) * 4, acc[h][0]);
          sts_f32(o + (m0 * 128 + n_lo + 8) * 4, acc[h][2]);
        }
        if (m1 < p.M) {
          sts_f32(o + (m1 * 128 + n_lo) * 4, acc[h][1]);
          sts_f32(o + (m1 * 128 + n_lo + 8) * 4, acc[h][3]);
        }
      }
      __syncwarp();
      if (ln.lane == 0) mbar_arrive(sm.outfull + 8 * buf);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) acc[h][0] = acc[h][1] = acc[h][2] = acc[h][3] = 0.f;
    ++cs.R;
  }
  cs.G += s1 - s0;
  if (p.dbg != nullptr && ln.tid == 256 && gphase_dbg < 32) p.dbg[((size_t)blockIdx.x * 8 + 2) * 32 + gphase_dbg] = globaltimer_ns();
}

// ------------------------------------------------------------------ the epilogue warp
// Takes every run end of this CTA from the hand-off buffer: adds the two groups' sums (times 1/rms of the row where
// the linear's input is RMS-normalised), stores them in the n-block's slot, takes a ticket; as the last of an
// n-block's runs it sums the slots in slot order and applies the linear's epilogue.  After the CTA's last run of a
// phase it makes the CTA's arrival at the grid barrier.  None of this holds the consumer warps up.
__device__ void epilogue(const MegaParams& p, const Smem& sm, const int lane) {
  const int c = blockIdx.x;
  int R = 0;
  bool ok = true;
  PROF_DECL
  for (int layer = 0; layer < p.n_layers && ok; ++layer) {
    const MegaLayer& L = p.layers[layer];
#pragma unroll 1
    for (int kind = 0; kind < 4 && ok; ++kind) {
      const int gphase = 1 + 5 * layer + (kind == 0 ? 0 : kind + 1);
      if (gphase >= p.n_phases) {
        if (lane == 0) { PROF_DUMP(3) }
        return;
      }
      const int T = p.T[kind], SG = p.SG[kind];
      const int s0 = run_begin(T, c, p.nCTA), s1 = run_begin(T, c + 1, p.nCTA);
      if (s0 == s1) {
        // no stage of this linear here: the arrival still has to come after the phase before
        unsigned v = 0;
        if (lane == 0) v = poll_arrivals(p, sm, (unsigned)gphase * (unsigned)p.nCTA, ERR_MEGA_GRID, gphase);
        if (__shfl_sync(0xffffffffu, v, 0) == 0xffffffffu) ok = false;
      } else {
        const bool normed = kind == 0 || kind == 2;   // the input is RMS-normalised: 1/rms multiplies the sums
        float rinv[kMaxRows];
#pragma unroll
        for (int m = 0; m < kMaxRows; ++m) rinv[m] = 1.f;
        if (normed) {
          // 1 / rms of the rows: their sums of squares are final once the phase before is complete.  This warp
          // has nothing else to do until the consumers hand their first run over, so it meets the barrier itself.
          unsigned v = 0;
          if (lane == 0) v = poll_arrivals(p, sm, (unsigned)gphase * (unsigned)p.nCTA, ERR_MEGA_GRID, gphase, 400);   // in no hurry
          if (__shfl_sync(0xffffffffu, v, 0) == 0xffffffffu) {
            ok = false;
            break;
          }
#pragma unroll
          for (int m = 0; m < kMaxRows; ++m) {
            if (m < p.M) {
              float s = 0.f;
              for (int jj = lane; jj < p.nbH; jj += 32) s += __ldcg(p.ssq + (size_t)m * p.nbH + jj);
              s = warp_sum(s);
              rinv[m] = rsqrtf(s / (float)p.H + p.eps);
            }
          }
        }
        for (int j = s0 / SG; j <= (s1 - 1) / SG && ok && !(p.variant & 64); ++j) {
          const int buf = R & 1;
          ok = warp_wait(sm.outfull + 8 * buf, (uint32_t)((R >> 1) & 1), sm.misc, ERR_MEGA_RING, lane);
          if (!ok) break;
          const bool stamp = p.dbg != nullptr && lane == 0 && gphase < 32 && j == (s1 - 1) / SG;
          if (stamp) p.dbg[((size_t)blockIdx.x * 8 + 4) * 32 + gphase] = globaltimer_ns();
          int nseg, seg;
          run_slots(p, kind, c, j, min(s1, (j + 1) * SG) - 1, nseg, seg);
          float* dst = p.part + (kind & 1) * p.part_half + ((size_t)j * 2 * p.maxseg[kind] + (size_t)seg) * p.M * 128;
          const uint32_t o = sm.out + buf * (kGroups * p.M * 512);
#pragma unroll
          for (int m = 0; m < kMaxRows; ++m) {
            if (m < p.M) {
              float4 a = lds_f4(o + (m * 128 + 4 * lane) * 4);
#pragma unroll
              for (int gq = 1; gq < kGroups; ++gq) {   // group order: the order the stages were dealt in
                const float4 b = lds_f4(o + gq * p.M * 512 + (m * 128 + 4 * lane) * 4);
                a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
              }
              const float r = rinv[m];
              *reinterpret_cast<float4*>(dst + m * 128 + 4 * lane) = make_float4(a.x * r, a.y * r, a.z * r, a.w * r);
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(sm.outempty + 8 * buf);
          if (stamp) p.dbg[((size_t)blockIdx.x * 8 + 5) * 32 + gphase] = globaltimer_ns();
          int last = 1;
          if (nseg > 1) {
            __syncwarp();
            if (lane == 0) {
              const int tk = atom_add_acq_rel(&p.tickets[j], 1);
              last = tk == nseg - 1;
              if (last) p.tickets[j] = 0;   // next used after a grid barrier
            }
            last = __shfl_sync(0xffffffffu, last, 0);
            __syncwarp();   // the other lanes' loads of the slots come after lane 0's acquire
          } else {
            __threadfence_block();   // the whole n-block is this CTA's: the fold below reads this warp's own stores
            __syncwarp();
          }
          if (stamp) p.dbg[((size_t)blockIdx.x * 8 + 6) * 32 + gphase] = globaltimer_ns();
          if (last) {
            if (kind == 0) fold_qkv(p, L, j, nseg, lane, 32);
            else if (kind == 2) fold_act(p, j, nseg, lane, 32);
            else {
              const float* nn = kind == 1 ? L.post_norm : (layer + 1 < p.n_layers ? p.layers[layer + 1].input_norm : nullptr);
              fold_resid(p, kind, nn, j, nseg, lane, 32, false);
            }
          }
          if (stamp) p.dbg[((size_t)blockIdx.x * 8 + 7) * 32 + gphase] = globaltimer_ns() | (last ? 1ull : 0ull);
          ++R;
        }
      }
      if (!ok) break;
      // ---- this CTA's arrival for the phase
      fence_proxy_async_all();   // the phase's generic-proxy stores are read by TMA / bulk copies of other CTAs next
      __syncwarp();
      if (lane == 0) {
        if (p.dbg && gphase < 32) p.dbg[((size_t)blockIdx.x * 8 + 0) * 32 + gphase] = globaltimer_ns();
        red_add_release(p.bar, 1u);
      }
    }
  }
  if (lane == 0) { PROF_DUMP(3) }
  if (!ok && lane == 0) {
    sts32(sm.misc, 1u);
    atomicExch(p.bar + 1, 1u);
  }
}

// ------------------------------------------------------------------ attention phase
__device__ void attn_phase(const MegaParams& p, const Smem& sm, int layer, int gphase, unsigned& use0, unsigned& use1, bool& ok,
                           const Lane& ln, ConsState& cs) {
  // What does not depend on this step's rows comes before the barrier: the split's key range and pages, and its
  // first two batches when they hold only keys of earlier steps (their K / V rows are not written in this launch).
  const int c = blockIdx.x, tid = ln.tid, warp = ln.warp, lane = ln.lane, g = ln.g, t = ln.t;
  const bool mine = c < p.n_kv * p.nsplit && !(p.variant & 8);
  const MegaLayer& L = p.layers[layer];
  const int kh = c / p.nsplit, split = c % p.nsplit;
  const int pos0 = p.ctrl[CTRL_ROW_POS], req = p.ctrl[CTRL_ROW_REQ];
  const int ctx_max = pos0 + p.M;
  const int total_pages = (ctx_max + 15) >> 4;
  int key0, key1;
  if (p.span_pages > 0) {
    key0 = split * p.span_pages * 16;
    key1 = min(ctx_max, (split + 1) * p.span_pages * 16);
  } else {
    const int pps = (total_pages + p.nsplit - 1) / p.nsplit;
    key0 = split * pps * 16;
    key1 = min(ctx_max, key0 + pps * 16);
  }
  const int nkeys = mine ? max(key1 - key0, 0) : 0;
  const int nbatch = (nkeys + KB - 1) / KB;
  const int* bt = p.block_table + (size_t)req * p.max_blocks + (key0 >> 4);
  const long long row_plane = L.kv_plane * (long long)p.num_pages;
  const uint32_t tiles = sm.attn;
  // batch b into buffer b & 1: warp 0 issues one tiled copy per (page, K | V, low | high dims)
  auto issue = [&](int b) {
    const int kb0 = key0 + b * KB, nk = min(KB, key1 - kb0), buf = b & 1;
    const int npages = (nk + 15) >> 4;
    const uint32_t bar = sm.kvbar + 8 * buf, base = tiles + buf * KVBUF;
    if (warp == 0) {
      if (lane == 0) mbar_expect_tx(bar, (uint32_t)npages * 8192u);
      __syncwarp();
      if (lane < 16) {
        const int pi = lane >> 2, which = lane & 3;
        if (pi < npages) {
          const int page = bt[((kb0 - key0) >> 4) + pi];
          const int row = (int)(((row_plane + page) * p.n_kv + kh) * 16);
          tma_load_2d(base + (which & 2 ? TILEB : 0) + (which & 1) * HALFB + pi * 2048, (which & 2) ? &p.v_map : &p.k_map,
                      (which & 1) * 64, row, bar);
        }
      }
    }
    if (tid < KB && tid >= npages * 16) {   // rows of pages that are not fetched: V must be finite (P = 0 there)
#pragma unroll
      for (int i = 0; i < 16; ++i)
        asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(base + TILEB + (i >> 3) * HALFB + tid * 128 + 16 * (i & 7)), "r"(0) : "memory");
    }
  };
  const bool stamp = p.dbg != nullptr && tid == 0 && gphase < 32;
  unsigned long long* stamps = p.dbg + ((size_t)blockIdx.x * 8) * 32 + gphase;   // rows 1..6 of this phase
  if (stamp) stamps[1 * 32] = globaltimer_ns();
  int issued = 0;
  while (ok && issued < 2 && issued < nbatch && key0 + (issued + 1) * KB <= pos0) issue(issued++);
  if (!grid_wait(p, sm, gphase, ln.tid)) ok = false;
  if (stamp) stamps[2 * 32] = globaltimer_ns();
  const bool run = lds32v(sm.misc + 4) != 0u;   // the wait's result: the same in every consumer thread
  fence_proxy_async_all();                       // the new K / V rows were stored by other CTAs; TMA reads them next
  if (!run && tid == 0)                          // abandoned: the copies in flight still have to land before the CTA exits
    for (int b = 0; b < issued; ++b) mbar_wait(sm.kvbar + 8 * (b & 1), ((b ? use1 : use0)) & 1u, ERR_MEGA_KV);
  if (mine && run) {
    const int QR = p.M * p.gqa;
    // 16 warps = (row groups x key slices) x 4 quarters of the head's 128 dims.  rgN groups of 16 query rows; with
    // fewer than four of them the 64 keys of a batch are cut into kqN slices, one per warp, and the slices meet in
    // shared memory after the last batch (slice order).  Every warp scores its keys for its rows (the four quarter
    // warps repeat that small product) and owns 32 dims of O.
    const int rgN = (QR + 15) >> 4;
    const int kqN = rgN == 1 ? 4 : (rgN == 2 ? 2 : 1);
    const int w4 = warp & 3, dq = warp >> 2;
    const int rg = rgN == 1 ? 0 : (rgN == 2 ? (w4 & 1) : w4);
    const int kq = rgN == 1 ? w4 : (rgN == 2 ? (w4 >> 1) : 0);
    const bool active = rg < rgN;
    const int kslice = KB / kqN;

    // The head group's query rows, once per CTA: 16-byte loads into the (idle) hand-off buffer, rows 272 bytes apart
    // (conflict-free fragment reads), then every warp takes its A fragments from there.
    constexpr uint32_t kQRow = 272;
    if (tid < QR * 16) {
      const int qr = tid >> 4, c16 = tid & 15;
      const int m = qr / p.gqa, h = qr % p.gqa;
      const uint4 v = __ldcg(reinterpret_cast<const uint4*>(p.q + (size_t)m * p.n_q * D + (size_t)(kh * p.gqa + h) * D + 8 * c16));
      asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(sm.out + qr * kQRow + c16 * 16), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
    }
    cons_sync();
    int ctx[2] = {0, 0};
    uint32_t qa[8][4];
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int qr = rg * 16 + g + 8 * hf;
      const bool okr = active && qr < QR;
      ctx[hf] = okr ? pos0 + qr / p.gqa + 1 : 0;
      const uint32_t qs = sm.out + (okr ? qr : 0) * kQRow + 4 * t;
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        qa[kk][hf] = okr ? lds32(qs + 32 * kk) : 0u;
        qa[kk][2 + hf] = okr ? lds32(qs + 32 * kk + 16) : 0u;
      }
    }
    float o[4][4];
#pragma unroll
    for (int jd = 0; jd < 4; ++jd) o[jd][0] = o[jd][1] = o[jd][2] = o[jd][3] = 0.f;
    float mx[2] = {-INFINITY, -INFINITY}, lsum[2] = {0.f, 0.f};

    if (issued == 0 && nbatch > 0) issue(issued++);
    for (int b = 0; b < nbatch; ++b) {
      const int buf = b & 1;
      cons_sync();   // batch b - 1 is consumed: its buffer may be refilled
      if (b + 1 < nbatch && issued < b + 2) issue(issued++);
      if (ok) ok = warp_wait(sm.kvbar + 8 * buf, ((buf ? use1 : use0) + (unsigned)(b >> 1)) & 1u, sm.misc, ERR_MEGA_KV, lane);
      if (stamp && b == 0) stamps[3 * 32] = globaltimer_ns();
      const int kb0 = key0 + b * KB, nk = min(KB, key1 - kb0);
      if (!ok || !active) continue;
      const uint32_t ks = tiles + buf * KVBUF, vs = ks + TILEB;
      const int kend = min(nk, (kq + 1) * kslice);
#pragma unroll 1
      for (int kofs = kq * kslice; kofs < kend; kofs += 16) {
        float s[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
          for (int kk = 0; kk < 8; kk += 2) {
            uint32_t b0, b1, b2, b3;
            ldsm_x4(ks + tile_off(kofs + 8 * j + (lane & 7), 16 * kk + 8 * (lane >> 3)), b0, b1, b2, b3);
            mma_bf16_16816(s[j], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], b0, b1);
            mma_bf16_16816(s[j], qa[kk + 1][0], qa[kk + 1][1], qa[kk + 1][2], qa[kk + 1][3], b2, b3);
          }
        }
        float mnew[2] = {mx[0], mx[1]};
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int key = kb0 + kofs + 8 * j + 2 * t + (e & 1);
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
          corr[hf] = mnew[hf] == -INFINITY ? 1.f : exp2f(mx[hf] - mnew[hf]);
          lsum[hf] *= corr[hf];
          mx[hf] = mnew[hf];
        }
#pragma unroll
        for (int jd = 0; jd < 4; ++jd) {
          o[jd][0] *= corr[0]; o[jd][1] *= corr[0]; o[jd][2] *= corr[1]; o[jd][3] *= corr[1];
        }
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int hf = e >> 1;
            const float pe = mnew[hf] == -INFINITY ? 0.f : exp2f(s[j][e] - mnew[hf]);
            s[j][e] = pe;
            lsum[hf] += pe;
          }
        const uint32_t pa0 = pack_bf16(s[0][0], s[0][1]), pa1 = pack_bf16(s[0][2], s[0][3]);
        const uint32_t pa2 = pack_bf16(s[1][0], s[1][1]), pa3 = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
        for (int jd = 0; jd < 4; jd += 2) {
          uint32_t b0, b1, b2, b3;
          const int mi = lane >> 3;
          ldsm_x4_trans(vs + tile_off(kofs + 8 * (mi & 1) + (lane & 7), 32 * dq + 8 * (jd + (mi >> 1))), b0, b1, b2, b3);
          mma_bf16_16816(o[jd], pa0, pa1, pa2, pa3, b0, b1);
          mma_bf16_16816(o[jd + 1], pa0, pa1, pa2, pa3, b2, b3);
        }
      }
    }
    if (stamp) stamps[4 * 32] = globaltimer_ns();
    use0 += (unsigned)((nbatch + 1) >> 1);   // batch b used buffer b & 1: the barriers' phase parities follow these counts
    use1 += (unsigned)(nbatch >> 1);
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      lsum[hf] += __shfl_xor_sync(0xffffffffu, lsum[hf], 1);
      lsum[hf] += __shfl_xor_sync(0xffffffffu, lsum[hf], 2);
    }
    if (kqN > 1) {
      // ---- the key slices of a row group meet: [slice][row][128] sums and [slice][row] (max, sum), slice order
      const int R16 = rgN * 16;
      const uint32_t oS = tiles, mlS = tiles + (uint32_t)(kqN * R16) * 512u;
      cons_sync();   // every warp is done with the K / V tiles
      if (active) {
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const int r = rg * 16 + g + 8 * hf;
          const uint32_t ob = oS + (uint32_t)((kq * R16 + r) * 128 + 32 * dq + 2 * t) * 4;
#pragma unroll
          for (int jd = 0; jd < 4; ++jd) {
            sts_f32(ob + 32 * jd, o[jd][2 * hf]);
            sts_f32(ob + 32 * jd + 4, o[jd][2 * hf + 1]);
          }
          if (t == 0 && dq == 0) {
            sts_f32(mlS + (uint32_t)(kq * R16 + r) * 8, mx[hf]);
            sts_f32(mlS + (uint32_t)(kq * R16 + r) * 8 + 4, lsum[hf]);
          }
        }
      }
      cons_sync();
      if (active && kq == 0) {
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const int r = rg * 16 + g + 8 * hf;
          float mm = -INFINITY;
          for (int k2 = 0; k2 < kqN; ++k2) mm = fmaxf(mm, __uint_as_float(lds32(mlS + (uint32_t)(k2 * R16 + r) * 8)));
          float lt = 0.f, acc2[4][2];
#pragma unroll
          for (int jd = 0; jd < 4; ++jd) acc2[jd][0] = acc2[jd][1] = 0.f;
          for (int k2 = 0; k2 < kqN; ++k2) {
            const float mk = __uint_as_float(lds32(mlS + (uint32_t)(k2 * R16 + r) * 8));
            const float wk = mk == -INFINITY ? 0.f : exp2f(mk - mm);
            lt = fmaf(__uint_as_float(lds32(mlS + (uint32_t)(k2 * R16 + r) * 8 + 4)), wk, lt);
            const uint32_t ob = oS + (uint32_t)((k2 * R16 + r) * 128 + 32 * dq + 2 * t) * 4;
#pragma unroll
            for (int jd = 0; jd < 4; ++jd) {
              acc2[jd][0] = fmaf(__uint_as_float(lds32(ob + 32 * jd)), wk, acc2[jd][0]);
              acc2[jd][1] = fmaf(__uint_as_float(lds32(ob + 32 * jd + 4)), wk, acc2[jd][1]);
            }
          }
          mx[hf] = mm;
          lsum[hf] = lt;
#pragma unroll
          for (int jd = 0; jd < 4; ++jd) {
            o[jd][2 * hf] = acc2[jd][0];
            o[jd][2 * hf + 1] = acc2[jd][1];
          }
        }
      }
    }
    // ---- this split's partials: unnormalised O against the running maximum, (max, sum)
    if (active && kq == 0) {
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int qr = rg * 16 + g + 8 * hf;
        if (qr < QR) {
          const int m = qr / p.gqa, h = qr % p.gqa;
          const size_t pb = ((size_t)m * p.n_q + kh * p.gqa + h) * p.nsplit + split;
#pragma unroll
          for (int jd = 0; jd < 4; ++jd)
            *reinterpret_cast<float2*>(p.o_part + pb * D + 32 * dq + 8 * jd + 2 * t) = make_float2(o[jd][2 * hf], o[jd][2 * hf + 1]);
          if (t == 0 && dq == 0) {
            p.ml_part[pb * 2] = mx[hf];
            p.ml_part[pb * 2 + 1] = lsum[hf];
          }
        }
      }
    }
    // ---- the last split CTA of this KV head merges all splits in split order and quantises the o-proj input
    cons_sync();
    if (tid == 0) {
      const int tk = atom_add_acq_rel(&p.attn_tickets[kh], 1);   // releases the CTA's stores (ordered by the barrier)
      const int last = tk == p.nsplit - 1;
      if (last) p.attn_tickets[kh] = 0;
      sts32(sm.misc + 8, (uint32_t)last);
    }
    cons_sync();
    const bool last = lds32v(sm.misc + 8) != 0u;
    if (stamp) stamps[5 * 32] = globaltimer_ns();
    if (last) {
      // Four lanes per (row, 8-vector): lane `sub` folds splits sub, sub + 4, ... in that order with a running
      // maximum (every load independent of the others: one trip to L2), then the four meet in a fixed butterfly.
      const int sub = lane & 3, iw = lane >> 2;
      const int items = QR * 16;
      for (int it0 = warp * 8; it0 < items; it0 += kConsWarps * 8) {
        const int it = it0 + iw;
        const bool act = it < items;
        const int qr = act ? it >> 4 : 0, v = it & 15;
        const int m = qr / p.gqa, h = qr % p.gqa;
        const size_t pb = ((size_t)m * p.n_q + kh * p.gqa + h) * p.nsplit;
        float mm = -INFINITY, lt = 0.f, y[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) y[i] = 0.f;
        if (act) {
#pragma unroll 5
          for (int sp = sub; sp < p.nsplit; sp += 4) {
            const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.ml_part + (pb + sp) * 2));
            const float4 a = __ldcg(reinterpret_cast<const float4*>(p.o_part + (pb + sp) * D + 8 * v));
            const float4 bq = __ldcg(reinterpret_cast<const float4*>(p.o_part + (pb + sp) * D + 8 * v + 4));
            const float mnew = fmaxf(mm, ml.x);
            const float c0 = mm == -INFINITY ? 0.f : exp2f(mm - mnew);
            const float c1 = ml.x == -INFINITY ? 0.f : exp2f(ml.x - mnew);
            lt = lt * c0 + ml.y * c1;
            y[0] = y[0] * c0 + a.x * c1; y[1] = y[1] * c0 + a.y * c1; y[2] = y[2] * c0 + a.z * c1; y[3] = y[3] * c0 + a.w * c1;
            y[4] = y[4] * c0 + bq.x * c1; y[5] = y[5] * c0 + bq.y * c1; y[6] = y[6] * c0 + bq.z * c1; y[7] = y[7] * c0 + bq.w * c1;
            mm = mnew;
          }
        }
        float mall = mm;
        mall = fmaxf(mall, __shfl_xor_sync(0xffffffffu, mall, 1));
        mall = fmaxf(mall, __shfl_xor_sync(0xffffffffu, mall, 2));
        const float cc = mm == -INFINITY ? 0.f : exp2f(mm - mall);
        lt *= cc;
#pragma unroll
        for (int i = 0; i < 8; ++i) y[i] *= cc;
#pragma unroll
        for (int d = 1; d < 4; d <<= 1) {
          lt += __shfl_xor_sync(0xffffffffu, lt, d);
#pragma unroll
          for (int i = 0; i < 8; ++i) y[i] += __shfl_xor_sync(0xffffffffu, y[i], d);
        }
        if (act && sub == 0) {
          const float inv = lt > 0.f ? 1.f / lt : 0.f;
          const uint32_t dst = tiles + (uint32_t)(qr * 128 + 8 * v) * 4;
#pragma unroll
          for (int i = 0; i < 8; ++i) sts_f32(dst + 4 * i, y[i] * inv);
        }
      }
      cons_sync();
      for (int it0 = warp * 32; it0 < items; it0 += kCons) {
        const int it = it0 + lane;
        const bool act = it < items;
        const int qr = act ? it >> 4 : 0, v = it & 15;
        const int m = qr / p.gqa, h = qr % p.gqa;
        float y[8];
        const float4 a = lds_f4(tiles + (uint32_t)(qr * 128 + 8 * v) * 4);
        const float4 bq = lds_f4(tiles + (uint32_t)(qr * 128 + 8 * v) * 4 + 16);
        y[0] = a.x; y[1] = a.y; y[2] = a.z; y[3] = a.w; y[4] = bq.x; y[5] = bq.y; y[6] = bq.z; y[7] = bq.w;
#pragma unroll
        for (int i = 0; i < 8; i += 2) {   // the attention output is a bf16 tensor, as in the launch-per-kernel form
          const uint32_t pk = act ? pack_bf16(y[i], y[i + 1]) : 0u;
          y[i] = bf16_lo(pk);
          y[i + 1] = bf16_hi(pk);
        }
        const StagedVec sv = stage_quant_f(y);
        if (act) store_staged(p, 1, (kh * p.gqa + h) * 2 + (v >> 3), m, v & 7, sv);
      }
    }
    cons_sync();
    if (stamp) stamps[6 * 32] = globaltimer_ns() | (last ? 1ull : 0ull);
  }
  grid_arrive(p, ln.tid, gphase);
}

// The consumers and the epilogue warp of every CTA sign out; the last one puts the barrier words back for the next
// launch (by then no CTA polls them: the activation producers are done before their consumers are).
__device__ __forceinline__ void leave(const MegaParams& p) {
  __threadfence();
  const unsigned n = atomicAdd(p.bar + 2, 1u);
  if (n == 2u * (unsigned)p.nCTA - 1u) {
    p.bar[0] = 0u;
    p.bar[1] = 0u;
    p.bar[2] = 0u;
    __threadfence();
  }
}

// ------------------------------------------------------------------ the kernel
__global__ void __launch_bounds__(kThreads, 1) decode_mega_kernel(const __grid_constant__ MegaParams p) {
  extern __shared__ uint8_t smem_raw[];
  Smem sm;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  sm.attn = base;                       // 1024-aligned: the swizzle pattern repeats every 1024 bytes
  sm.stageB = kWStage + kSB * p.rows * kXRow + kSB * 64;
  sm.fullW = base + kAttnBytes;
  sm.fullX = sm.fullW + 8 * kMaxNS;
  sm.empty = sm.fullX + 8 * kMaxNS;
  sm.kvbar = sm.empty + 8 * kMaxNS;
  sm.outfull = sm.kvbar + 16;
  sm.outempty = sm.outfull + 16;
  sm.misc = sm.outempty + 16;           // [0] failed, [4] grid-wait result, [8] ticket result
  sm.out = (sm.misc + 16 + 15u) & ~15u;
  sm.ring = (sm.out + 2u * kGroups * (uint32_t)p.M * 512u + 127u) & ~127u;

  const int tid = threadIdx.x;
  if (tid == 0) {
    for (int i = 0; i < p.NS; ++i) {
      mbar_init(sm.fullW + 8 * i, 1);
      mbar_init(sm.fullX + 8 * i, 1);
      mbar_init(sm.empty + 8 * i, kGroupWarps);
    }
    mbar_init(sm.kvbar, 1);
    mbar_init(sm.kvbar + 8, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(sm.outfull + 8 * i, kConsWarps);   // one arrival per consumer warp
      mbar_init(sm.outempty + 8 * i, 1);
    }
    sts32(sm.misc, 0u);
    sts32(sm.misc + 4, 0u);
    sts32(sm.misc + 8, 0u);
    mbar_fence_init();
    prefetch_tmap(&p.k_map);
    prefetch_tmap(&p.v_map);
  }
  __syncthreads();

  if (tid >= kCons) {
    const int role = (tid - kCons) >> 5, lane = tid & 31;
    if (role == 0) {
      if (lane == 0) w_producer(p, sm);
    } else if (role == 1) {
      if (lane == 0) x_producer(p, sm);
    } else {
      epilogue(p, sm, lane);
      if (lane == 0) leave(p);
    }
    return;
  }
  Lane ln;
  ln.tid = tid; ln.warp = tid >> 5; ln.lane = tid & 31; ln.wq = ln.warp & (kGroupWarps - 1); ln.gidx = ln.warp / kGroupWarps;
  ln.g = ln.lane >> 2; ln.t = ln.lane & 3;
  bool ok = true;
  ConsState cs;
  cs.G = 0; cs.R = 0; cs.slot = ln.gidx; cs.par = 0u;
#ifdef B2_MEGA_PROF
  cs.prof.start();
#endif
  unsigned use0 = 0u, use1 = 0u;

  // ---- phase 0: embedding rows -> residual stream, sums of squares, quantised rows for layer 0's qkv
  if (p.n_phases > 0) {
    if ((int)blockIdx.x < p.nbH) fold_resid(p, 1, p.layers[0].input_norm, blockIdx.x, 0, tid, kCons, true);
    grid_arrive(p, tid, 0);
  }
  for (int layer = 0; layer < p.n_layers; ++layer) {
    const int g0 = 1 + 5 * layer;
    if (g0 >= p.n_phases) break;
    gemv_phase<0>(p, sm, cs, ok, ln, layer);
    if (g0 + 1 >= p.n_phases) break;
    attn_phase(p, sm, layer, g0 + 1, use0, use1, ok, ln, cs);
    if (g0 + 2 >= p.n_phases) break;
    gemv_phase<1>(p, sm, cs, ok, ln, layer);
    if (g0 + 3 >= p.n_phases) break;
    gemv_phase<2>(p, sm, cs, ok, ln, layer);
    if (g0 + 4 >= p.n_phases) break;
    gemv_phase<3>(p, sm, cs, ok, ln, layer);
  }
#ifdef B2_MEGA_PROF
  if (tid == 0) cs.prof.dump(p, 2);
#endif
  cons_sync();
  if (tid == 0) leave(p);
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
int kv_map(CUtensorMap* out, const void* ptr, uint64_t rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -100;
  cuuint64_t dims[2] = {(cuuint64_t)D, rows};
  cuuint64_t strides[1] = {(cuuint64_t)D * 2};
  cuuint32_t box[2] = {64, 16};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -101;
}

struct Plan {
  int nb[4], SG[4], T[4], maxseg[4], KG[4];
  int rows, NS, nsplit, smem;
  long long part_floats;
  int max_nb;
};

// Shapes -> schedule constants.  Returns 0, or a negative code when the shape is outside what the kernel covers.
int make_plan(Plan& pl, int nCTA, int M, int H, int n_q, int n_kv, int ffn) {
  if (M < 1 || M > kMaxRows || nCTA < 1) return -1;
  if (H % 128 || ffn % 128 || n_q % n_kv || n_q / n_kv > 8 || M * (n_q / n_kv) > 62 || n_kv > nCTA) return -2;   // 62: the slice merge's scratch
  const int N[4] = {(n_q + 2 * n_kv) * D, H, 2 * ffn, H};
  const int Kd[4] = {H, n_q * D, H, ffn};
  pl.part_floats = 0;
  pl.max_nb = 0;
  for (int k = 0; k < 4; ++k) {
    pl.nb[k] = N[k] / 128;
    pl.KG[k] = Kd[k] / 64;
    pl.SG[k] = (pl.KG[k] + kSB - 1) / kSB;
    pl.T[k] = pl.nb[k] * pl.SG[k];
    if ((long long)(pl.T[k] + 1) * (nCTA + 1) >= (1ll << 31)) return -2;
    int mx = 0;
    for (int j = 0; j < pl.nb[k]; ++j) {
      const int a = stage_owner(j * pl.SG[k], nCTA, pl.T[k]), b = stage_owner((j + 1) * pl.SG[k] - 1, nCTA, pl.T[k]);
      const int runs = pl.T[k] >= nCTA ? b - a + 1 : pl.SG[k];   // fewer stages than CTAs: one single-stage run per stage
      if (runs > mx) mx = runs;
    }
    pl.maxseg[k] = mx;
    const long long f = (long long)pl.nb[k] * 2 * mx * M * 128;
    if (f > pl.part_floats) pl.part_floats = f;
    if (pl.nb[k] > pl.max_nb) pl.max_nb = pl.nb[k];
  }
  int rows = 1;
  while (rows < M) rows *= 2;
  pl.rows = rows;
  const int stageB = kWStage + kSB * rows * kXRow + kSB * 64;
  const int fixed = 1024 + kAttnBytes + 8 * kMaxNS * 3 + 16 + 32 + 16 + 16 + 2 * kGroups * M * 512 + 128;
  int ns = (232448 - fixed) / stageB;
  if (ns > kMaxNS) ns = kMaxNS;
  if (ns < kGroups + 1) return -3;   // every consumer group can hold a stage while one more is in flight
  pl.NS = ns;
  pl.smem = fixed + ns * stageB;
  int nsplit = nCTA / n_kv;
  if (nsplit > kMaxSplit) nsplit = kMaxSplit;
  pl.nsplit = nsplit;
  return 0;
}

}  // namespace

// Schedule constants for the buffers the caller owns.  out: [0] rows (token slots of the quantised buffers),
// [1] KV splits, [2] n-blocks of the widest linear (ticket words), [3] ring stages, [4] shared memory bytes;
// *part_floats: floats of the partial-sum buffer (two halves).  Also checks (on the host) that the runs cover every stage once.
extern "C" int b2_decode_mega_plan(int nCTA, int M, int H, int n_q, int n_kv, int ffn, int* out, long long* part_floats) {
  Plan pl;
  const int rc = make_plan(pl, nCTA, M, H, n_q, n_kv, ffn);
  if (rc) return rc;
  for (int k = 0; k < 4; ++k) {
    int prev_end = 0;
    for (int c = 0; c < nCTA; ++c) {
      const int s0 = run_begin(pl.T[k], c, nCTA), s1 = run_begin(pl.T[k], c + 1, nCTA);
      if (s0 != prev_end) return -20;
      for (int s = s0; s < s1; ++s)
        if (stage_owner(s, nCTA, pl.T[k]) != c) return -21;
      prev_end = s1;
    }
    if (prev_end != pl.T[k]) return -22;
  }
  out[0] = pl.rows; out[1] = pl.nsplit; out[2] = pl.max_nb; out[3] = pl.NS; out[4] = pl.smem;
  *part_floats = 2 * pl.part_floats;
  return 0;
}

extern "C" int b2_decode_mega_sms() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
  return n;
}

extern "C" int b2_decode_mega(const void* layers_dev, int n_layers, int M, int H, int n_q, int n_kv, int ffn,
                              const int* ctrl, const int* block_table, int max_blocks, int num_pages, int planes,
                              const void* embed, int vocab, int* flag, const float* cos_t, const float* sin_t,
                              void* k_cache, void* v_cache, void* resid, float* ssq, void* xq_h, void* xq_o, void* xq_f,
                              void* gs_h, void* gs_o, void* gs_f, float* part, int* tickets, void* q, float* o_part,
                              float* ml_part, int* attn_tickets, unsigned* bar, float eps, float scale, int span_pages,
                              int n_phases, int nCTA, int cooperative, unsigned long long* dbg, void* stream) {
  Plan pl;
  int rc = make_plan(pl, nCTA, M, H, n_q, n_kv, ffn);
  if (rc) return rc;
  if (((uintptr_t)k_cache | (uintptr_t)v_cache) & 15) return -4;
  MegaParams p;
  const uint64_t cache_rows = (uint64_t)planes * num_pages * n_kv * 16;
  if (cache_rows >= (1ull << 31)) return -5;
  rc = kv_map(&p.k_map, k_cache, cache_rows);
  if (rc == 0) rc = kv_map(&p.v_map, v_cache, cache_rows);
  if (rc) return rc;
  p.layers = reinterpret_cast<const MegaLayer*>(layers_dev);
  p.n_layers = n_layers; p.M = M; p.rows = pl.rows; p.nCTA = nCTA; p.NS = pl.NS;
  p.H = H; p.n_q = n_q; p.n_kv = n_kv; p.gqa = n_q / n_kv; p.nbH = H / 128;
  for (int k = 0; k < 4; ++k) { p.nb[k] = pl.nb[k]; p.SG[k] = pl.SG[k]; p.T[k] = pl.T[k]; p.maxseg[k] = pl.maxseg[k]; p.KG[k] = pl.KG[k]; }
  p.ctrl = ctrl; p.block_table = block_table; p.max_blocks = max_blocks; p.num_pages = num_pages;
  p.embed = (const __nv_bfloat16*)embed; p.vocab = vocab; p.flag = flag; p.cos_t = cos_t; p.sin_t = sin_t;
  p.k_cache = (__nv_bfloat16*)k_cache; p.v_cache = (__nv_bfloat16*)v_cache;
  p.resid = (__nv_bfloat16*)resid; p.ssq = ssq;
  p.xq[0] = (uint8_t*)xq_h; p.xq[1] = (uint8_t*)xq_o; p.xq[2] = (uint8_t*)xq_f;
  p.gs[0] = (uint32_t*)gs_h; p.gs[1] = (uint32_t*)gs_o; p.gs[2] = (uint32_t*)gs_f;
  p.part = part; p.part_half = pl.part_floats; p.tickets = tickets; p.q = (__nv_bfloat16*)q; p.o_part = o_part; p.ml_part = ml_part;
  p.attn_tickets = attn_tickets; p.bar = bar; p.eps = eps; p.scale_log2 = scale * 1.4426950408889634f;
  p.nsplit = pl.nsplit; p.span_pages = span_pages; p.dbg = dbg;
  { const char* v = getenv("B2_MEGA_VARIANT"); p.variant = v ? atoi(v) : 0; }
  const int all = 1 + 5 * n_layers;
  p.n_phases = (n_phases <= 0 || n_phases > all) ? all : n_phases;
  if (span_pages > 0 && (long long)span_pages * pl.nsplit < max_blocks) return -6;

  static int configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured[dev & 63] < pl.smem) {
    cudaError_t e = cudaFuncSetAttribute(decode_mega_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448);
    if (e != cudaSuccess) return (int)e;
    configured[dev & 63] = 232448;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(nCTA);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = pl.smem;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;   // every CTA resident at once, or the launch is refused
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = cooperative ? 1 : 0;
  return (int)cudaLaunchKernelEx(&cfg, decode_mega_kernel, p);
}

B2_DEFINE_STATUS(mega)
