// Shared device helpers for the sm_100a kernels: mbarrier, TMA (bulk and tiled),
// tcgen05 / TMEM, programmatic dependent launch, and bounded waits.
//
// Every wait in these kernels is bounded.  A wait that runs out records a code
// in a device-global status word (read by the host with b2_status()) and
// returns false; the caller then leaves its loops, the CTA drains what it has
// in flight, frees its tensor memory and returns, so the context stays usable.
// The reference takes the same stance for its cross-device waits
// (src/runtime/tp_protocol.h:35-60: bounded spin, status words, finish on
// garbage, host raises).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

namespace b2 {

// status[0]: first error code (0 = none); status[1]: detail; status[2]: count.
// One word set per translation unit (no relocatable device code is needed); each
// .cu file exports its own reader with B2_DEFINE_STATUS and the Python side reads them all.
static __device__ unsigned int g_status[4] = {0, 0, 0, 0};
// Optional word in pinned host memory: the first error code also lands there, so the serving loop can look for a
// failure after every step by reading host memory instead of copying every unit's status words from the device.
static __device__ unsigned int* g_host_flag = nullptr;

enum : unsigned int {
  ERR_NONE = 0,
  ERR_GEMV_FULL_WAIT = 0x101,
  ERR_GEMV_EMPTY_WAIT = 0x102,
  ERR_GEMM_FULL_WAIT = 0x201,
  ERR_GEMM_EMPTY_WAIT = 0x202,
  ERR_GEMM_TMEM_FULL_WAIT = 0x203,
  ERR_GEMM_TMEM_EMPTY_WAIT = 0x204,
  ERR_ATTN_WAIT = 0x301,
  ERR_MOE_WAIT = 0x401,
  ERR_COMM_FLAG_WAIT = 0x501,
  ERR_GDN_WAIT = 0x601,
  ERR_BAD_ARG = 0x901,
};

__device__ __forceinline__ void record_error(unsigned int code, unsigned int detail) {
  if (atomicCAS(&g_status[0], 0u, code) == 0u) {
    g_status[1] = detail;
    unsigned int* hf = g_host_flag;
    if (hf != nullptr) {
      *reinterpret_cast<volatile unsigned int*>(hf) = code;
      __threadfence_system();
    }
  }
  atomicAdd(&g_status[2], 1u);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// upper bound (ns) of one hardware-suspended poll; a completed phase wakes the thread at once
constexpr uint32_t kSuspendHintNs = 20000;
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(kSuspendHintNs)
      : "memory");
  return ok != 0;
}
// Bounded wait.  mbarrier.try_wait suspends the thread in hardware until the phase completes or a
// short system time limit passes, so the loop is not a hot spin.  The bound is kept on the SM's own
// cycle counter (%clock64 costs a few cycles; %globaltimer is a slow read that, taken on every
// wait, delayed each wake-up by most of a microsecond) and is only consulted after 256 failed
// polls: about 4e9 cycles, i.e. roughly two seconds at 2 GHz.
constexpr long long kWaitCycles = 4000000000ll;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned int code) {
#pragma unroll 1
  for (int i = 0; i < 256; ++i)
    if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_try(bar, parity)) return true;
    if (clock64() - t0 > kWaitCycles) {
      record_error(code, (blockIdx.x << 8) | (threadIdx.x >> 5));
      return false;
    }
  }
}

// ---------------------------------------------------------------- proxies / fences
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------- programmatic dependent launch
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---------------------------------------------------------------- TMA
// 1-D bulk copy global -> shared (both 16-byte aligned, size a multiple of 16)
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          dst),
      "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::
          "r"(dst),
      "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map), "r"(src),
               "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---------------------------------------------------------------- tcgen05 / TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]; kind::f16 covers fp16 and bf16 inputs
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same with each descriptor given as its two 32-bit words: a thread that issues many MMAs per tile keeps the
// (constant) high words and base low words in registers and pays one integer add per operand and MMA, instead of
// rebuilding 64-bit descriptors -- a lone issuing thread retires a dependent instruction only every ~10 cycles.
__device__ __forceinline__ void umma_f16_w(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %6, 0;\n\t"
      "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}" ::"r"(d_tmem),
      "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// A operand from tensor memory, B descriptor as two words
__device__ __forceinline__ void umma_f16_ts_w(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi,
                                              uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %5, 0;\n\tmov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// A operand from tensor memory (used by attention: P stays in TMEM)
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Shared-memory matrix descriptor for a K-major operand tile whose rows are 128
// bytes (64 bf16 or 128 int8) written with the 128-byte swizzle: 8-row groups are
// 1024 bytes apart (stride byte offset), the leading byte offset is unused (1).
__device__ __forceinline__ uint64_t make_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;   // descriptor version for sm_100
  d |= (uint64_t)2 << 61;   // SWIZZLE_128B
  return d;
}
// Instruction descriptor: dense, D format (1 = f32, 2 = s32), A/B format
// (kind::f16: 0 = f16, 1 = bf16; kind::i8: 0 = u8, 1 = s8), both operands K-major.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t dfmt, uint32_t abfmt, uint32_t m, uint32_t n) {
  return (dfmt << 4) | (abfmt << 7) | (abfmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

#define B2_TMEM_LD_32(taddr, r)                                                                              \
  asm volatile(                                                                                              \
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "                                                              \
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,"  \
      "%27,%28,%29,%30,%31}, [%32];"                                                                         \
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),      \
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),             \
        "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),           \
        "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),           \
        "=r"(r[29]), "=r"(r[30]), "=r"(r[31])                                                                \
      : "r"(taddr)                                                                                           \
      : "memory")

#define B2_TMEM_ST_32(taddr, r)                                                                              \
  asm volatile(                                                                                              \
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "                                                       \
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,"  \
      "%27,%28,%29,%30,%31};" ::"r"(r[0]),                                                                   \
      "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),     \
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),        \
      "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]),        \
      "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]), "r"(taddr)                     \
      : "memory")

__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------- small math helpers
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float silu(float x) { return x / (1.0f + __expf(-x)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// mma.sync m16n8k16 bf16 x bf16 -> fp32 (used by the small-M weight-streaming kernels,
// which are bound by HBM bandwidth, not by tensor throughput)
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---------------------------------------------------------------- activation rows for the integer GEMV
// Quantises a group's 64 activations (as rounded to bf16) to 15-bit integers with one scale,
// X = rint(x * 16383 / amax) = 128 X_hi + X_lo with X_hi in [-128, 127] and X_lo in [0, 127].  The eight
// lanes that hold a group (one 16-byte vector each) share amax and sum(X) by shuffles; every lane of the
// warp must call this.  w[0..3] = high limbs of k 0..3, low limbs of k 0..3, high of k 4..7, low of k 4..7.
struct StagedVec {
  uint32_t w[4];
  float scale;
  int m8sum;  // -8 sum(X) of the whole group
};
__device__ __forceinline__ StagedVec stage_quant(uint4 val) {
  float xf[8] = {bf16_lo(val.x), bf16_hi(val.x), bf16_lo(val.y), bf16_hi(val.y),
                 bf16_lo(val.z), bf16_hi(val.z), bf16_lo(val.w), bf16_hi(val.w)};
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
// Word index inside a group's 32 words where vector vq (k = 8 vq .. 8 vq + 7) puts its first word: 32-k step
// vq >> 2, operand register (vq & 3) >> 1, lanes t = 2 (vq & 1) and + 1.  Lane t's words sit at
// t * 8 + limb * 4 + step * 2 + register, so the main loop reads a limb's four words with one 16-byte load;
// the vector's four words go to +0 (high, k 0..3), +4 (low), +8 (high, k 4..7), +12 (low).
__device__ __forceinline__ int stage_word(int vq) { return (vq & 1) * 16 + (vq >> 2) * 2 + ((vq & 3) >> 1); }

}  // namespace b2

// Host-side launch helper: every kernel of the decode path is launched with the
// programmatic-stream-serialization attribute so its weight prefetch overlaps the
// tail of the kernel before it; kernels call b2::pdl_wait() before touching
// activations.
#define B2_DEFINE_STATUS(unit)                                                              \
  extern "C" int b2_status_##unit(unsigned int* out4) {                                     \
    return (int)cudaMemcpyFromSymbol(out4, b2::g_status, sizeof(unsigned int) * 4);         \
  }                                                                                         \
  extern "C" int b2_status_clear_##unit() {                                                 \
    unsigned int z[4] = {0, 0, 0, 0};                                                       \
    return (int)cudaMemcpyToSymbol(b2::g_status, z, sizeof(z));                             \
  }                                                                                         \
  extern "C" int b2_status_hostflag_##unit(void* pinned_word) {                             \
    return (int)cudaMemcpyToSymbol(b2::g_host_flag, &pinned_word, sizeof(pinned_word));     \
  }

template <typename... KArgs, typename... Args>
static inline int b2_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                            bool pdl, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  static const bool no_pdl = getenv("B2_NO_PDL") != nullptr;  // measurement switch: plain stream order
  cfg.numAttrs = (pdl && !no_pdl) ? 1 : 0;
  return (int)cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
