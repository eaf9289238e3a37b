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

B2_DEFINE_STATUS(comm)
