// Cross-GPU plumbing and the small collective kernels of the tensor-parallel decode step.
//
//  * symmetric buffers: plain cudaMalloc allocations whose CUDA IPC handles the ranks exchange, so
//    that every rank can store into every other rank's landing buffers from inside a kernel (the
//    reference maps its peer landing buffers the same way: src/runtime/tp_engine.h:26-96);
//  * vocabulary-parallel arg-max: every rank reduces its own slice of the vocabulary, pushes
//    (value, id) to all ranks and merges the parts on the device with the one-card tie rule (higher
//    value, then lower id), replacing the reference's host merge of the two halves
//    (src/runtime/tp_engine.cc:300-315, src/kernels/tp.cl:284-354);
//  * a one-shot all-reduce of small fp32 row blocks (push to all, local fold in rank order) for the
//    places that have no GEMV in front of them to fuse with (src/kernels/tp.cl:206-264 "tp_sum").
#include "wire.cuh"

using namespace b2;

namespace {

constexpr int CTRL_ROW_POS = 80, CTRL_CUR_TOKEN = 144, CTRL_OUT_TOKEN = 208, CTRL_OUT_VALUE = 272;

// grid M, 256 threads.  Landing layout per rank: [2 slots][world][mcap] x {value, id}; flags
// [2][world][mcap]; epoch [mcap].
__global__ void __launch_bounds__(256) argmax_finish_tp_kernel(const float* cand_val, const int* cand_idx, int ncand,
                                                               int vocab_offset, int* ctrl, int advance, Wire w,
                                                               int mcap) {
  __shared__ float sv[256];
  __shared__ int si[256];
  pdl_wait();
  pdl_launch_dependents();
  const int m = blockIdx.x, tid = threadIdx.x;
  float b = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = tid; i < ncand; i += 256) {
    const float v = cand_val[(size_t)m * ncand + i];
    const int id = cand_idx[(size_t)m * ncand + i];
    if (v > b || (v == b && id < bi)) { b = v; bi = id; }
  }
  sv[tid] = b;
  si[tid] = bi;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (tid < o) {
      const float v = sv[tid + o];
      const int id = si[tid + o];
      if (v > sv[tid] || (v == sv[tid] && id < si[tid])) { sv[tid] = v; si[tid] = id; }
    }
    __syncthreads();
  }
  if (tid >= 32) return;
  // one warp: lane r talks to rank r
  const int W = w.world, me = w.rank;
  int epoch = 0;
  if (tid == 0) {
    epoch = w.epoch[m] + 1;
    w.epoch[m] = epoch;
  }
  epoch = __shfl_sync(0xffffffffu, epoch, 0);
  const int slot = epoch & 1;
  const float myv = sv[0];
  const int myi = si[0] + vocab_offset;
  bool got = true;
  if (tid < W) {
    float* dst = wire_land(w, tid) + (((size_t)slot * W + me) * mcap + m) * 2;
    dst[0] = myv;
    dst[1] = __int_as_float(myi);
    __threadfence_system();
    if (tid != me) {
      st_release_sys(wire_flags(w, tid) + ((size_t)slot * W + me) * mcap + m, epoch);
      got = wire_wait(wire_flags(w, me) + ((size_t)slot * W + tid) * mcap + m, epoch, (unsigned)(0x80000000u | tid << 16 | m));
    }
  }
  if (__any_sync(0xffffffffu, !got)) return;
  float bv = -INFINITY;
  int bid = 0x7fffffff;
  if (tid < W) {
    const float* src = wire_land(w, me) + (((size_t)slot * W + tid) * mcap + m) * 2;
    bv = ld_sys_f32(src);
    bid = __float_as_int(ld_sys_f32(src + 1));
  }
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bid, o);
    if (ov > bv || (ov == bv && oi < bid)) { bv = ov; bid = oi; }
  }
  if (tid == 0) {
    ctrl[CTRL_OUT_TOKEN + m] = bid;
    ctrl[CTRL_OUT_VALUE + m] = __float_as_int(bv);
    if (advance) {
      ctrl[CTRL_CUR_TOKEN + m] = bid;
      ctrl[CTRL_ROW_POS + m] += 1;
    }
  }
}

// One-shot all-reduce of x[M][N] fp32 (N a multiple of 4): grid (ceil(N / 1024), M), 256 threads, one float4
// per thread.  Landing [2][world][mcap][N]; flags and epochs per (row, column block): [2][world][mcap * nblk].
__global__ void __launch_bounds__(256) allreduce_rows_kernel(const float* x, float* out, int M, int N, Wire w, int mcap) {
  pdl_wait();
  pdl_launch_dependents();
  const int m = blockIdx.y, cb = blockIdx.x, nblk = gridDim.x, tid = threadIdx.x;
  const int n = (cb * 256 + tid) * 4;
  const int W = w.world, me = w.rank;
  __shared__ int s_epoch, s_bad;
  if (tid == 0) {
    s_epoch = w.epoch[m * nblk + cb] + 1;
    w.epoch[m * nblk + cb] = s_epoch;
    s_bad = 0;
  }
  __syncthreads();
  const int epoch = s_epoch, slot = epoch & 1;
  const size_t src_stride = (size_t)mcap * N;
  if (n < N) {
    const float4 v = *reinterpret_cast<const float4*>(x + (size_t)m * N + n);
    const size_t off = ((size_t)slot * W + me) * src_stride + (size_t)m * N + n;
    for (int r = 0; r < W; ++r) *reinterpret_cast<float4*>(wire_land(w, r) + off) = v;
  }
  __threadfence_system();
  __syncthreads();
  if (tid < W && tid != me) {
    const int fi = m * nblk + cb, fn = mcap * nblk;
    st_release_sys(wire_flags(w, tid) + ((size_t)slot * W + me) * fn + fi, epoch);
    if (!wire_wait(wire_flags(w, me) + ((size_t)slot * W + tid) * fn + fi, epoch, (unsigned)(0x40000000u | tid << 16 | fi)))
      s_bad = 1;
  }
  __syncthreads();
  if (s_bad || n >= N) return;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  const float* land = wire_land(w, me) + (size_t)slot * W * src_stride + (size_t)m * N + n;
  for (int r = 0; r < W; ++r) {  // rank order: identical bits on every rank
    const float4 v = ld_sys_f32x4(land + (size_t)r * src_stride);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  *reinterpret_cast<float4*>(out + (size_t)m * N + n) = acc;
}

// ------------------------------------------------------------------ prefill: reduce-scatter fold + norm + all-gather push
// The owner side of the row-parallel GEMM -> reduce-scatter, fused with what follows it.  One warp per row
// this rank owns (eight rows per CTA).  Row r is token g = rank * rows_cap + r of the
// chunk.  The CTA waits (bounded) until every source rank's counter of the row's m-tile shows the whole tile
// has landed, adds the bf16 partial sums in rank order to the residual row, writes the residual back,
// applies RMSNorm with the NEXT layer's weight and pushes the normalised row into every rank's copy of the
// gathered activations, then counts one arrival for the row's m-tile on every rank: the column-parallel GEMM
// that follows waits on those counters tile by tile (all-gather -> GEMM).  nsrc = 0: no partial sums (first
// layer: the residual rows hold the embeddings).  One warp per row, eight rows per CTA.
struct RsFoldParams {
  const __nv_bfloat16* land;   // this rank's landing buffer [world][rows_cap][H]
  int* rs_cnt;                 // this rank's counters [world][tpr] (of the slot in use)
  int* done;                   // [tpr] local tickets: the last waiting row of a tile resets its counters
  int rs_expect;               // arrivals that complete one (source, m-tile)
  int nsrc;
  __nv_bfloat16* resid;        // [rows_cap][H]
  const float* norm_w;
  float eps;
  const unsigned long long* x_table;  // [2][kMaxRanks]: gathered activations [world rows_cap][H], tile counters
  int world, rank, H, tpr, c;
};

constexpr int kFoldRows = 8;   // rows (= warps) per CTA; divides the 128-row m-tile

__global__ void __launch_bounds__(32 * kFoldRows) rs_fold_kernel(const RsFoldParams p) {
  __shared__ int s_bad;
  pdl_wait();
  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int r = blockIdx.x * kFoldRows + warp;      // this warp's row; the CTA's rows share one m-tile
  const int rows_cap = p.tpr * 128, mtl = (blockIdx.x * kFoldRows) >> 7;
  const int g = p.rank * rows_cap + r;  // token index in the chunk
  const bool exists = g < p.c;
  const int tile_row0 = p.rank * rows_cap + mtl * 128;
  const int cta_row0 = p.rank * rows_cap + blockIdx.x * kFoldRows;
  const int cta_rows = max(0, min(kFoldRows, p.c - cta_row0));   // rows of this CTA that exist
  if (tid == 0) s_bad = 0;
  __syncthreads();
  if (cta_rows > 0 && p.nsrc > 0) {
    if (tid < p.nsrc && !wire_wait(p.rs_cnt + tid * p.tpr + mtl, p.rs_expect, (unsigned)(0x10000000u | tid << 16 | mtl)))
      s_bad = 1;
    __syncthreads();
    if (s_bad) return;
  }
  const int nvec = p.H / 8;
  float ss = 0.f;
  if (exists) {
    // pass 1: residual + the sources' partial sums in rank order (the same bits whichever rank owns the row),
    // written back as bf16; the sum of squares of what was stored
    __nv_bfloat16* rrow = p.resid + (size_t)r * p.H;
    for (int j0 = lane; j0 < nvec; j0 += 32 * 4) {
      uint4 rv[4], pv[4];
      float f[4][8];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int j = j0 + 32 * u;
        rv[u] = j < nvec ? *reinterpret_cast<const uint4*>(rrow + 8 * j) : make_uint4(0, 0, 0, 0);
        const uint32_t rw[4] = {rv[u].x, rv[u].y, rv[u].z, rv[u].w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          f[u][2 * q] = bf16_lo(rw[q]);
          f[u][2 * q + 1] = bf16_hi(rw[q]);
        }
      }
      for (int src = 0; src < p.nsrc; ++src) {
        const __nv_bfloat16* lrow = p.land + ((size_t)src * rows_cap + r) * p.H;
#pragma unroll
        for (int u = 0; u < 4; ++u) {   // four loads in flight per lane
          const int j = j0 + 32 * u;
          pv[u] = j < nvec ? ld_sys_u32x4(lrow + 8 * j) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const uint32_t pw[4] = {pv[u].x, pv[u].y, pv[u].z, pv[u].w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            f[u][2 * q] += bf16_lo(pw[q]);
            f[u][2 * q + 1] += bf16_hi(pw[q]);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int j = j0 + 32 * u;
        if (j < nvec) {
          uint4 ro;
          ro.x = pack_bf16(f[u][0], f[u][1]); ro.y = pack_bf16(f[u][2], f[u][3]);
          ro.z = pack_bf16(f[u][4], f[u][5]); ro.w = pack_bf16(f[u][6], f[u][7]);
          *reinterpret_cast<uint4*>(rrow + 8 * j) = ro;
          const uint32_t ow[4] = {ro.x, ro.y, ro.z, ro.w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {  // the norm sees the residual as stored (bf16)
            const float a = bf16_lo(ow[q]), b2v = bf16_hi(ow[q]);
            ss += a * a + b2v * b2v;
          }
        }
      }
    }
  }
  ss = warp_sum(ss);
  if (cta_rows > 0 && p.nsrc > 0) {
    // the CTA's rows have read their partial sums: the tile's last CTA puts the counters back to zero for the
    // next call (nobody can be a whole call ahead: the next push needs every rank's fold of this one)
    __syncthreads();
    if (tid == 0) {
      const int waiting = min(128, p.c - tile_row0);
      if (atomicAdd(p.done + mtl, cta_rows) == waiting - cta_rows) {
        p.done[mtl] = 0;
        for (int src = 0; src < p.nsrc; ++src) p.rs_cnt[src * p.tpr + mtl] = 0;
        __threadfence_system();
      }
    }
  }
  if (exists) {
    // pass 2: RMSNorm of the stored row (this warp wrote it: the reads hit L1 / L2) and the push to every rank
    const float rinv = rsqrtf(ss / (float)p.H + p.eps);
    const __nv_bfloat16* rrow = p.resid + (size_t)r * p.H;
    __syncwarp();
    for (int j = lane; j < nvec; j += 32) {
      const uint4 rv = *reinterpret_cast<const uint4*>(rrow + 8 * j);
      const float4 w0 = *reinterpret_cast<const float4*>(p.norm_w + 8 * j), w1 = *reinterpret_cast<const float4*>(p.norm_w + 8 * j + 4);
      uint4 xo;
      xo.x = pack_bf16(bf16_lo(rv.x) * rinv * w0.x, bf16_hi(rv.x) * rinv * w0.y);
      xo.y = pack_bf16(bf16_lo(rv.y) * rinv * w0.z, bf16_hi(rv.y) * rinv * w0.w);
      xo.z = pack_bf16(bf16_lo(rv.z) * rinv * w1.x, bf16_hi(rv.z) * rinv * w1.y);
      xo.w = pack_bf16(bf16_lo(rv.w) * rinv * w1.z, bf16_hi(rv.w) * rinv * w1.w);
      for (int d = 0; d < p.world; ++d) {
        __nv_bfloat16* xd = reinterpret_cast<__nv_bfloat16*>(p.x_table[d]);
        *reinterpret_cast<uint4*>(xd + (size_t)g * p.H + 8 * j) = xo;
      }
    }
  }
  // The CTA barrier orders every warp's stores before the releasing threads' fence; the release is at system
  // scope, so each destination sees the rows before the arrivals.  One arrival per row, added per CTA: rows
  // that do not exist in this chunk count too, so a tile is always complete at 128.
  __syncthreads();
  if (tid < p.world) {
    int* cnt = reinterpret_cast<int*>(p.x_table[kMaxRanks + tid]) + p.rank * p.tpr + mtl;
    __threadfence_system();
    asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(cnt), "r"(kFoldRows) : "memory");
  }
}

// One thread: bounded wait for a counter in this GPU's memory (orders later kernels of the stream after
// the peers' pushes, e.g. the lm_head after the last fold).
__global__ void wire_wait_kernel(const int* cnt, int expect) {
  pdl_wait();
  wire_wait(cnt, expect, 0x08000000u);
  pdl_launch_dependents();
}

}  // namespace

// ------------------------------------------------------------------ symmetric buffers (CUDA IPC)
extern "C" int b2_symm_alloc(void** ptr, unsigned long long bytes) {
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemset(*ptr, 0, bytes);
}
extern "C" int b2_symm_free(void* ptr) { return (int)cudaFree(ptr); }
extern "C" int b2_ipc_handle_bytes() { return (int)sizeof(cudaIpcMemHandle_t); }
extern "C" int b2_ipc_get(void* ptr, void* handle_out) {
  return (int)cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t*>(handle_out), ptr);
}
extern "C" int b2_ipc_open(const void* handle, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  return (int)cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
}
extern "C" int b2_ipc_close(void* ptr) { return (int)cudaIpcCloseMemHandle(ptr); }
extern "C" int b2_can_access_peer(int dev, int peer) {
  int ok = 0;
  if (cudaDeviceCanAccessPeer(&ok, dev, peer) != cudaSuccess) return 0;
  return ok;
}

// ------------------------------------------------------------------ kernels
extern "C" int b2_argmax_finish_tp(const float* cand_val, const int* cand_idx, int ncand, int M, int vocab_offset,
                                   int* ctrl, int advance, const void* table, int* epoch, int world, int rank, int mcap,
                                   void* stream) {
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world || M > mcap) return -1;
  Wire w;
  w.table = (const unsigned long long*)table; w.epoch = epoch; w.world = world; w.rank = rank;
  return b2_launch(argmax_finish_tp_kernel, dim3(M), dim3(256), 0, (cudaStream_t)stream, true, cand_val, cand_idx, ncand,
                   vocab_offset, ctrl, advance, w, mcap);
}

extern "C" int b2_allreduce_rows(const float* x, float* out, int M, int N, const void* table, int* epoch, int world,
                                 int rank, int mcap, void* stream) {
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world || M > mcap || N % 4) return -1;
  Wire w;
  w.table = (const unsigned long long*)table; w.epoch = epoch; w.world = world; w.rank = rank;
  return b2_launch(allreduce_rows_kernel, dim3((N + 1023) / 1024, M), dim3(256), 0, (cudaStream_t)stream, true, x, out, M,
                   N, w, mcap);
}

extern "C" int b2_rs_fold(const void* land, int* rs_cnt, int* done, int rs_expect, int nsrc, void* resid,
                          const float* norm_w, float eps, const void* x_table, int world, int rank, int H, int tpr, int c,
                          void* stream) {
  if (H % 8 || world < 1 || world > kMaxRanks || nsrc > kMaxRanks || tpr < 1) return -1;   // (nsrc > world: a loop-back test with several landing slots)
  RsFoldParams p;
  p.land = (const __nv_bfloat16*)land; p.rs_cnt = rs_cnt; p.done = done; p.rs_expect = rs_expect; p.nsrc = nsrc;
  p.resid = (__nv_bfloat16*)resid; p.norm_w = norm_w; p.eps = eps; p.x_table = (const unsigned long long*)x_table;
  p.world = world; p.rank = rank; p.H = H; p.tpr = tpr; p.c = c;
  return b2_launch(rs_fold_kernel, dim3(tpr * 128 / kFoldRows), dim3(32 * kFoldRows), 0, (cudaStream_t)stream, true, p);
}

extern "C" int b2_wire_wait(const int* cnt, int expect, void* stream) {
  return b2_launch(wire_wait_kernel, dim3(1), dim3(1), 0, (cudaStream_t)stream, true, cnt, expect);
}

B2_DEFINE_STATUS(comm)
