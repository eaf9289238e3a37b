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
// The owner side of the row-parallel GEMM -> reduce-scatter, fused with what follows it.  One CTA per row
// this rank owns (grid = rows_cap = 128 tpr, H / 8 threads).  Row r is token g = rank * rows_cap + r of the
// chunk.  The CTA waits (bounded) until every source rank's counter of the row's m-tile shows the whole tile
// has landed, adds the bf16 partial sums in rank order to the residual row, writes the residual back,
// applies RMSNorm with the NEXT layer's weight and pushes the normalised row into every rank's copy of the
// gathered activations, then counts one arrival for the row's m-tile on every rank: the column-parallel GEMM
// that follows waits on those counters tile by tile (all-gather -> GEMM).  nsrc = 0: no partial sums (first
// layer: the residual rows hold the embeddings).
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

__global__ void __launch_bounds__(1024) rs_fold_kernel(const RsFoldParams p) {
  __shared__ float red[32];
  __shared__ int s_bad;
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x, tid = threadIdx.x, nthr = blockDim.x;
  const int rows_cap = p.tpr * 128, mtl = r >> 7;
  const int g = p.rank * rows_cap + r;  // token index in the chunk
  const bool exists = g < p.c;
  const int tile_row0 = p.rank * rows_cap + mtl * 128;
  if (tid == 0) s_bad = 0;
  __syncthreads();
  if (exists && p.nsrc > 0) {
    if (tid < p.nsrc && !wire_wait(p.rs_cnt + tid * p.tpr + mtl, p.rs_expect, (unsigned)(0x10000000u | tid << 16 | mtl)))
      s_bad = 1;
    __syncthreads();
    if (s_bad) return;
  }
  const int col = tid * 8;
  float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  uint4 xo = make_uint4(0, 0, 0, 0);
  if (exists && col < p.H) {
    const uint4 rv = *reinterpret_cast<const uint4*>(p.resid + (size_t)r * p.H + col);
    const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      f[2 * q] = bf16_lo(rw[q]);
      f[2 * q + 1] = bf16_hi(rw[q]);
    }
    for (int src = 0; src < p.nsrc; ++src) {  // rank order: the same bits whichever rank owns the row
      const uint4 pv = ld_sys_u32x4(p.land + ((size_t)src * rows_cap + r) * p.H + col);
      const uint32_t pw[4] = {pv.x, pv.y, pv.z, pv.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        f[2 * q] += bf16_lo(pw[q]);
        f[2 * q + 1] += bf16_hi(pw[q]);
      }
    }
    uint4 ro;
    ro.x = pack_bf16(f[0], f[1]); ro.y = pack_bf16(f[2], f[3]); ro.z = pack_bf16(f[4], f[5]); ro.w = pack_bf16(f[6], f[7]);
    *reinterpret_cast<uint4*>(p.resid + (size_t)r * p.H + col) = ro;
    const uint32_t ow[4] = {ro.x, ro.y, ro.z, ro.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {  // the norm sees the residual as stored (bf16)
      f[2 * q] = bf16_lo(ow[q]);
      f[2 * q + 1] = bf16_hi(ow[q]);
    }
  }
  if (exists && p.nsrc > 0) {
    // this row has read its partial sums: the tile's last row puts the counters back to zero for the
    // call after next (the slots alternate; nobody can be two calls ahead)
    __syncthreads();
    if (tid == 0) {
      const int waiting = min(128, p.c - tile_row0);
      if (atomicAdd(p.done + mtl, 1) == waiting - 1) {
        p.done[mtl] = 0;
        for (int src = 0; src < p.nsrc; ++src) p.rs_cnt[src * p.tpr + mtl] = 0;
        __threadfence_system();
      }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
  ss = warp_sum(ss);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  if (tid < 32) {
    float v = tid < (nthr + 31) / 32 ? red[tid] : 0.f;
    v = warp_sum(v);
    if (tid == 0) red[0] = rsqrtf(v / (float)p.H + p.eps);
  }
  __syncthreads();
  const float rinv = red[0];
  if (exists && col < p.H) {
    const float4 w0 = *reinterpret_cast<const float4*>(p.norm_w + col), w1 = *reinterpret_cast<const float4*>(p.norm_w + col + 4);
    xo.x = pack_bf16(f[0] * rinv * w0.x, f[1] * rinv * w0.y);
    xo.y = pack_bf16(f[2] * rinv * w0.z, f[3] * rinv * w0.w);
    xo.z = pack_bf16(f[4] * rinv * w1.x, f[5] * rinv * w1.y);
    xo.w = pack_bf16(f[6] * rinv * w1.z, f[7] * rinv * w1.w);
    for (int d = 0; d < p.world; ++d) {
      __nv_bfloat16* xd = reinterpret_cast<__nv_bfloat16*>(p.x_table[d]);
      *reinterpret_cast<uint4*>(xd + (size_t)g * p.H + col) = xo;
    }
  }
  // The CTA barrier orders every thread's stores before the releasing threads' fence; the release is at system
  // scope, so each destination sees the row before the arrival (one fence per destination, not one per thread).
  __syncthreads();
  if (tid < p.world) {
    int* cnt = reinterpret_cast<int*>(p.x_table[kMaxRanks + tid]) + p.rank * p.tpr + mtl;
    __threadfence_system();
    asm volatile("red.release.sys.global.add.s32 [%0], 1;" ::"l"(cnt) : "memory");
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
  if (H % 8 || H / 8 > 1024 || world < 1 || world > kMaxRanks || nsrc > world || tpr < 1) return -1;
  RsFoldParams p;
  p.land = (const __nv_bfloat16*)land; p.rs_cnt = rs_cnt; p.done = done; p.rs_expect = rs_expect; p.nsrc = nsrc;
  p.resid = (__nv_bfloat16*)resid; p.norm_w = norm_w; p.eps = eps; p.x_table = (const unsigned long long*)x_table;
  p.world = world; p.rank = rank; p.H = H; p.tpr = tpr; p.c = c;
  const int threads = ((H / 8 + 31) / 32) * 32;
  return b2_launch(rs_fold_kernel, dim3(tpr * 128), dim3(threads), 0, (cudaStream_t)stream, true, p);
}

extern "C" int b2_wire_wait(const int* cnt, int expect, void* stream) {
  return b2_launch(wire_wait_kernel, dim3(1), dim3(1), 0, (cudaStream_t)stream, true, cnt, expect);
}

B2_DEFINE_STATUS(comm)
