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
// consumer warps each own 16 output rows: they read their 16 bytes per lane,
// expand nibbles to exact bf16 integers with two logic ops and one subtract, and
// feed mma.m16n8k16 with the weights as the 16-row operand and up to 8 tokens as
// the 8-column operand (tokens beyond 8 reuse the dequantised registers, so the
// weights are read once for any M: weight-stationary).  Group scales are applied
// in fp32 to the per-group partial sums.  Split-K slices are written separately
// and summed by the consumer kernel in a fixed order: no atomics, bitwise
// reproducible, and a row's result does not depend on M (the split count is a
// function of N and K only) -- the reference's "property R"
// (src/kernels/gemm_sm.cl:44-50).
#include "common.cuh"

using namespace b2;

namespace {

constexpr int kBlockBytes = 4352;
constexpr int kG = 2;  // quantisation groups (W4B blocks) per ring stage
constexpr int kStages = 8;
constexpr int kStageBytes = kG * kBlockBytes;
constexpr int kConsumerThreads = 256;
constexpr int kThreads = kConsumerThreads + 32;

struct GemvParams {
  const uint8_t* w;  // [nb][KG][4352]
  const void* x;     // x_mode 0: bf16 [M][ldx];  x_mode 1: fp32 [s_in][M][ldx] (gate/up interleave16)
  float* out;        // [S][M][ldo]
  int M, N, KG, S, gps;
  int ldx, ldo;
  int x_mode, s_in;
  long long x_slice;  // elements between input slices (x_mode 1)
};

template <int T>
struct Cfg {
  static constexpr int XC = 2048 / T;           // k elements of x staged at a time
  static constexpr int XCG = XC / 64;           // groups per x chunk
  static constexpr int ROWS = 8 * T;            // token rows (padded)
  static constexpr int STRIDE_W = XC / 2 + 4;   // row stride in 32-bit words (+4: conflict-free B reads)
  static constexpr int X_BYTES = ROWS * STRIDE_W * 4;
  static constexpr int SMEM = kStages * kStageBytes + X_BYTES + 256 + 128;
};

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

template <int T>
__global__ void __launch_bounds__(kThreads, (T <= 2 ? 2 : 1)) gemv_w4_kernel(const GemvParams p) {
  using C = Cfg<T>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  uint8_t* ring = smem;
  uint32_t* xs = reinterpret_cast<uint32_t*>(smem + kStages * kStageBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes + C::X_BYTES);
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + kStages);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nblk = blockIdx.x, split = blockIdx.y;
  const int gbeg = split * p.gps;
  const int gend = min(p.KG, gbeg + p.gps);
  const int ngroups = max(0, gend - gbeg);
  const int nstage = (ngroups + kG - 1) / kG;

  if (tid == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(full0 + 8 * i, 1);
      mbar_init(empty0 + 8 * i, 8);
    }
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == 8) {
    // ---------------- producer: stream this CTA's blocks; weights do not depend on the previous kernel
    if (lane == 0) {
      const uint8_t* src = p.w + ((size_t)nblk * p.KG + gbeg) * kBlockBytes;
      bool ok = true;
      int issued = 0;
      for (int i = 0; i < nstage && ok; ++i) {
        const int s = i % kStages;
        if (i >= kStages) ok = mbar_wait(empty0 + 8 * s, ((i / kStages) - 1) & 1, ERR_GEMV_EMPTY_WAIT);
        if (!ok) break;
        const int ng = min(kG, ngroups - i * kG);
        const uint32_t bytes = ng * kBlockBytes;
        mbar_expect_tx(full0 + 8 * s, bytes);
        bulk_g2s(smem_u32(ring + s * kStageBytes), src + (size_t)i * kStageBytes, bytes, full0 + 8 * s);
        issued = i + 1;
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

  const int g = lane >> 2, t = lane & 3;
  float acc[T][4];
#pragma unroll
  for (int i = 0; i < T; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

  const uint32_t kMagic = 0x43004300u, kMask = 0x000F000Fu;
  const __nv_bfloat162 k136 = __floats2bfloat162_rn(136.f, 136.f);
  bool ok = true;

  for (int c0 = 0; c0 < ngroups; c0 += C::XCG) {
    const int cg = min(C::XCG, ngroups - c0);  // groups in this chunk
    consumer_sync();
    // ---- stage x[:, k0 : k0 + 64 cg] as bf16 rows
    {
      const int k0 = (gbeg + c0) * 64;
      const int nvec = cg * 8;  // 16-byte vectors per row
      for (int v = tid; v < C::ROWS * C::XC / 8; v += kConsumerThreads) {
        const int row = v / (C::XC / 8), col = v % (C::XC / 8);
        uint4 val = make_uint4(0, 0, 0, 0);
        if (row < p.M && col < nvec) {
          const int k = k0 + col * 8;
          if (p.x_mode == 0) {
            val = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.x) + (size_t)row * p.ldx + k);
          } else {
            // SiLU(gate) * up over summed fp32 slices; gate/up alternate in runs of 16
            const float* base = reinterpret_cast<const float*>(p.x) + (size_t)row * p.ldx + (k >> 4) * 32 + (k & 15);
            float gsum[8], usum[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) gsum[i] = usum[i] = 0.f;
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
        }
        *reinterpret_cast<uint4*>(xs + row * C::STRIDE_W + col * 4) = val;
      }
    }
    consumer_sync();

    // ---- consume the ring stages that cover this chunk
    // (after a failed wait the warp skips the rest of its work but still meets the others at
    //  the named barrier, so a lost copy costs one bounded wait and never a deadlock)
    for (int gi = 0; gi < cg; gi += kG) {
      const int i = (c0 + gi) / kG;  // stage index since kernel start
      const int s = i % kStages;
      if (ok) ok = mbar_wait(full0 + 8 * s, (i / kStages) & 1, ERR_GEMV_FULL_WAIT);
      if (!ok) continue;
      const uint8_t* st = ring + s * kStageBytes;
      const int ng = min(kG, cg - gi);
#pragma unroll
      for (int q = 0; q < kG; ++q) {
        if (q < ng) {
          const uint8_t* blk = st + q * kBlockBytes;
          const uint4 wv = *reinterpret_cast<const uint4*>(blk + warp * 512 + lane * 16);
          const __half* sc = reinterpret_cast<const __half*>(blk + 4096) + warp * 16;
          const float s_lo = __half2float(sc[g]), s_hi = __half2float(sc[g + 8]);
          float ag[T][4];
#pragma unroll
          for (int i2 = 0; i2 < T; ++i2) ag[i2][0] = ag[i2][1] = ag[i2][2] = ag[i2][3] = 0.f;
          const uint32_t* xrow = xs + g * C::STRIDE_W + (gi + q) * 32 + t;
          const uint32_t wa[2][2] = {{wv.x, wv.y}, {wv.z, wv.w}};
#pragma unroll
          for (int pr = 0; pr < 2; ++pr) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint32_t a[4];
              a[0] = ((wa[pr][0] >> (8 * h)) & kMask) | kMagic;
              a[1] = ((wa[pr][1] >> (8 * h)) & kMask) | kMagic;
              a[2] = ((wa[pr][0] >> (8 * h + 4)) & kMask) | kMagic;
              a[3] = ((wa[pr][1] >> (8 * h + 4)) & kMask) | kMagic;
#pragma unroll
              for (int r = 0; r < 4; ++r) {
                __nv_bfloat162 v = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&a[r]), k136);
                a[r] = *reinterpret_cast<uint32_t*>(&v);
              }
              const int step = 2 * pr + h;
#pragma unroll
              for (int tt = 0; tt < T; ++tt) {
                const uint32_t* xr = xrow + tt * 8 * C::STRIDE_W + step * 8;
                mma_bf16_16816(ag[tt], a[0], a[1], a[2], a[3], xr[0], xr[4]);
              }
            }
          }
#pragma unroll
          for (int tt = 0; tt < T; ++tt) {
            acc[tt][0] = fmaf(s_lo, ag[tt][0], acc[tt][0]);
            acc[tt][1] = fmaf(s_lo, ag[tt][1], acc[tt][1]);
            acc[tt][2] = fmaf(s_hi, ag[tt][2], acc[tt][2]);
            acc[tt][3] = fmaf(s_hi, ag[tt][3], acc[tt][3]);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + 8 * s);
    }
  }

  // ---- write this split's partial sums
  const int n_lo = nblk * 128 + warp * 16 + g, n_hi = n_lo + 8;
  float* outp = p.out + (size_t)split * p.M * p.ldo;
#pragma unroll
  for (int tt = 0; tt < T; ++tt) {
    const int m0 = tt * 8 + 2 * t, m1 = m0 + 1;
    if (m0 < p.M) {
      if (n_lo < p.N) outp[(size_t)m0 * p.ldo + n_lo] = acc[tt][0];
      if (n_hi < p.N) outp[(size_t)m0 * p.ldo + n_hi] = acc[tt][2];
    }
    if (m1 < p.M) {
      if (n_lo < p.N) outp[(size_t)m1 * p.ldo + n_lo] = acc[tt][1];
      if (n_hi < p.N) outp[(size_t)m1 * p.ldo + n_hi] = acc[tt][3];
    }
  }
}

template <int T>
int launch_t(const GemvParams& p, cudaStream_t stream) {
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(gemv_w4_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<T>::SMEM);
    if (e != cudaSuccess) return (int)e;
    configured[dev & 63] = true;
  }
  dim3 grid((p.N + 127) / 128, p.S);
  return b2_launch(gemv_w4_kernel<T>, grid, dim3(kThreads), Cfg<T>::SMEM, stream, true, p);
}

}  // namespace

// Number of k splits: a function of (N, K) only, so that a row's bits do not depend on M.
// The grid (N/128 x splits) is sized to one wave of 296 CTA slots (148 SMs x 2 resident CTAs):
// a second, partly filled wave would cost a full stream latency for a fraction of the work.
extern "C" int b2_gemv_w4_splits(int N, int K) {
  const int nb = (N + 127) / 128, kg = K / 64;
  int s = 296 / nb;
  int smax = kg / 8;  // at least 8 groups (512 k) per split
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

B2_DEFINE_STATUS(gemv)
