// Expert parallelism: the all-to-all dispatch and the return path of a mixture-of-experts block
// whose experts are spread over the ranks of a group, written as peer stores over NVLink.
//
// The reference has no expert parallelism (its MoE models run every expert on each card:
// docs/17-running-models.md:455-470); this is the capability an 8-GPU NVSwitch box adds.  The plan
// follows the reference's one-card sort (src/kernels/prefill/pf_moe_sort_mw.cl): the host never
// reads a count, the tile table is padded to 128-row blocks and read on the device.
//
// Per chunk of T local tokens, on every rank:
//   1. route + count (moe.cu): counts[E], rank of every (token, slot) inside its expert;
//   2. ep_counts_push: counts -> every rank's cnt_all[source][E], one flag per (source -> destination);
//   3. ep_plan: waits (bounded) for all sources' counts; for the rank's OWN experts builds the block
//      table of the expert-sorted receive buffer (rows of source 0 first, then source 1, ...); for ALL
//      experts computes where this rank's rows start in the destination's buffer -- every rank runs the
//      same arithmetic on the same counts, so nothing else has to be exchanged;
//   4. ep_dispatch: one warp per (token, slot) stores the token's activation row straight into the
//      destination's receive buffer, records (source, token slot) beside it and counts one arrival on
//      the destination's 128-row block; the grouped GEMM there starts a block as soon as its rows are in
//      (gemm_tc.cu: blk_wait), so the transfer overlaps the expert GEMMs block by block;
//   5. the down GEMM's epilogue stores each result row into the source rank's return buffer
//      (gemm_tc.cu: EPI_EP_RETURN); ep_flag_all then tells every source "my rows are back";
//   6. ep_wait_all on the source, then the weighted sum over a token's slots in slot order (moe.cu:
//      moe_combine over the return buffer), so the bits do not depend on arrival order.
#include "wire.cuh"

using namespace b2;

namespace {

struct EpPlanParams {
  const unsigned long long* cnt_table;  // [2][kMaxRanks]: cnt_all [world][E] ints, flags [world]
  int epoch;
  int E, El, world, rank;
  int max_blk, cap_rows;
  int* send_base;   // [E] first row of this rank's rows of expert e in the destination's buffer
  int* blk_expert;  // block table of this rank's receive buffer (local expert ids)
  int* blk_row0;
  int* blk_rows;
  int* n_blk;
  int* total_rows;
  int* blk_cnt_next;  // arrival counters of the NEXT call (other parity): zeroed here
};

__global__ void __launch_bounds__(1024) ep_counts_push_kernel(const int* counts, int E, Wire w, int epoch) {
  pdl_wait();
  pdl_launch_dependents();
  const int tid = threadIdx.x;
  for (int e = tid; e < E; e += blockDim.x) {
    const int c = counts[e];
    for (int r = 0; r < w.world; ++r) reinterpret_cast<int*>(w.table[r])[(size_t)w.rank * E + e] = c;
  }
  __threadfence_system();
  __syncthreads();
  if (tid < w.world) st_release_sys(wire_flags(w, tid) + w.rank, epoch);
}

__global__ void __launch_bounds__(1024) ep_plan_kernel(const EpPlanParams p) {
  __shared__ int s_tot[1024];   // rows of expert e over all sources
  __shared__ int s_pad[1024];   // padded to whole blocks
  __shared__ int s_bad;
  pdl_wait();
  pdl_launch_dependents();
  const int tid = threadIdx.x;
  if (tid == 0) s_bad = 0;
  __syncthreads();
  const int* cnt_all = reinterpret_cast<const int*>(p.cnt_table[p.rank]);
  const int* flags = reinterpret_cast<const int*>(p.cnt_table[kMaxRanks + p.rank]);
  if (tid < p.world && !wire_wait(flags + tid, p.epoch, (unsigned)(0x04000000u | tid))) s_bad = 1;
  __syncthreads();
  if (s_bad) {
    if (tid == 0) {
      *p.n_blk = 0;
      *p.total_rows = 0;
    }
    return;
  }
  int tot = 0, before = 0;
  if (tid < p.E) {
    for (int s = 0; s < p.world; ++s) {
      int c;
      asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(c) : "l"(cnt_all + (size_t)s * p.E + tid) : "memory");
      if (s < p.rank) before += c;
      tot += c;
    }
  }
  s_tot[tid] = tot;
  s_pad[tid] = (tot + 127) & ~127;
  __syncthreads();
  if (tid < p.E) {
    // first row of expert e in its owner's buffer: padded rows of the owner's experts before it
    const int owner = tid / p.El;
    int base = 0;
    for (int e2 = owner * p.El; e2 < tid; ++e2) base += s_pad[e2];
    p.send_base[tid] = base + before;
    if (owner == p.rank) {
      const int el = tid - owner * p.El;
      const int b0 = base >> 7, nb = s_pad[tid] >> 7;
      for (int j = 0; j < nb && b0 + j < p.max_blk; ++j) {
        p.blk_expert[b0 + j] = el;
        p.blk_row0[b0 + j] = (b0 + j) * 128;
        p.blk_rows[b0 + j] = min(128, tot - j * 128);
      }
      if (el == p.El - 1) {
        const int rows = base + s_pad[tid];
        if (rows > p.cap_rows || (rows >> 7) > p.max_blk) record_error(ERR_BAD_ARG, (unsigned)rows);
        *p.n_blk = min(rows >> 7, p.max_blk);
        *p.total_rows = rows;
      }
    }
  }
  for (int i = tid; i < p.max_blk; i += blockDim.x) p.blk_cnt_next[i] = 0;
}

struct EpDispatchParams {
  const int* topk_idx;
  const int* rank_in_expert;
  const int* send_base;
  const __nv_bfloat16* x;   // [T][H]
  int k, H, El, me, cap_rows, parity, max_blk;
  const unsigned long long* recv_table;  // [2][kMaxRanks]: receive buffer [cap_rows][H] bf16, block counters [2][max_blk]
  const unsigned long long* src_table;   // [kMaxRanks]: recv_src [cap_rows] ints
};

// grid T (one CTA per token), one warp per slot.
__global__ void __launch_bounds__(1024) ep_dispatch_kernel(const EpDispatchParams p) {
  pdl_wait();
  pdl_launch_dependents();
  const int token = blockIdx.x, slot = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (slot >= p.k) return;
  const int i = token * p.k + slot;
  const int e = p.topk_idx[i];
  const int dest = e / p.El;
  const int row = p.send_base[e] + p.rank_in_expert[i];
  if (row >= p.cap_rows) {  // the destination's buffer is full: the token's slot is dropped and reported
    if (lane == 0) record_error(ERR_BAD_ARG, (unsigned)(0x80000000u | row));
    return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(p.x + (size_t)token * p.H);
  uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.recv_table[dest]) + (size_t)row * p.H);
  const int nvec = p.H / 8;
  for (int j0 = 0; j0 < nvec; j0 += 128) {   // four independent 16-byte loads per lane in flight
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (j0 + u * 32 + lane < nvec) v[u] = src[j0 + u * 32 + lane];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (j0 + u * 32 + lane < nvec) dst[j0 + u * 32 + lane] = v[u];
  }
  if (lane == 0) reinterpret_cast<int*>(p.src_table[dest])[row] = (p.me << 24) | i;
  // The warp's stores are ordered before lane 0's release by the warp barrier; the release is at system
  // scope, so the destination sees the row and its tag before the arrival.
  __syncwarp();
  if (lane == 0) {
    int* cnt = reinterpret_cast<int*>(p.recv_table[kMaxRanks + dest]) + p.parity * p.max_blk + (row >> 7);
    __threadfence_system();
    asm volatile("red.release.sys.global.add.s32 [%0], 1;" ::"l"(cnt) : "memory");
  }
}

// flags[me] = epoch on every rank (after everything earlier in the stream, whose peer stores are complete
// at the kernel boundary)
__global__ void ep_flag_all_kernel(Wire w, int epoch) {
  pdl_wait();
  __threadfence_system();
  if (threadIdx.x < w.world) st_release_sys(wire_flags(w, threadIdx.x) + w.rank, epoch);
  pdl_launch_dependents();
}

__global__ void ep_wait_all_kernel(Wire w, int epoch) {
  pdl_wait();
  if (threadIdx.x < w.world) wire_wait(wire_flags(w, w.rank) + threadIdx.x, epoch, (unsigned)(0x02000000u | threadIdx.x));
  pdl_launch_dependents();
}

// ---------------------------------------------------------------- decode rows on the experts' owner
// A decode step sends a handful of rows per expert, so the owner runs the batched W4 GEMV (one row against one
// expert's int4 weights, gemv_w4.cu) instead of a grouped GEMM over 128-row blocks.  The receive buffer is expert-
// sorted with every expert padded to whole blocks; ep_rows_gather waits (bounded) for each block's rows, packs
// them into consecutive batches and notes every batch's expert and (source rank, slot).  Batches past the last row
// get expert -1, which the GEMV skips.  ep_rows_return sums a batch's split-K slices in slice order and stores the
// bf16 row into the source rank's return buffer, where the usual slot-order combine finds it.
struct EpRowsParams {
  const int* blk_expert;
  const int* blk_row0;
  const int* blk_rows;
  const int* n_blk;
  const int* blk_cnt;          // arrival counters of this call's parity
  const __nv_bfloat16* recv_x; // [cap_rows][H]
  const int* recv_src;         // [cap_rows]
  int H, cap_pairs;
  __nv_bfloat16* cx;           // [cap_pairs][H]
  int* cexp;                   // [cap_pairs]
  int* csrc;                   // [cap_pairs]
  int* n_valid;
};

// grid max_blk (>= 1), 256 threads
__global__ void __launch_bounds__(256) ep_rows_gather_kernel(const EpRowsParams p) {
  __shared__ int s_before, s_total, s_ok;
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x, tid = threadIdx.x;
  const int nb = *p.n_blk;
  if (tid == 0) {
    int before = 0, total = 0;
    for (int j = 0; j < nb; ++j) {
      const int r = p.blk_rows[j];
      if (j < b) before += r;
      total += r;
    }
    s_before = before;
    s_total = total;
    s_ok = 1;
  }
  __syncthreads();
  if (b == 0) {
    for (int c = s_total + tid; c < p.cap_pairs; c += 256) p.cexp[c] = -1;
    if (tid == 0) {
      if (s_total > p.cap_pairs) record_error(ERR_BAD_ARG, (unsigned)s_total);
      *p.n_valid = min(s_total, p.cap_pairs);
    }
  }
  if (b >= nb) return;
  const int rows = p.blk_rows[b], row0 = p.blk_row0[b], before = s_before;
  if (rows <= 0) return;
  if (tid == 0 && !wire_wait(p.blk_cnt + b, rows, (unsigned)(0x05000000u | b))) s_ok = 0;
  __syncthreads();
  const int nvec = p.H / 8;
  for (int r = 0; r < rows; ++r) {
    const int c = before + r;
    if (c >= p.cap_pairs) break;
    if (!s_ok) {   // the rows never came: the batch is skipped, its source slot keeps what it held (reported)
      if (tid == 0) p.cexp[c] = -1;
      continue;
    }
    const uint8_t* src = reinterpret_cast<const uint8_t*>(p.recv_x + (size_t)(row0 + r) * p.H);
    uint4* dst = reinterpret_cast<uint4*>(p.cx + (size_t)c * p.H);
    for (int v = tid; v < nvec; v += 256) dst[v] = ld_sys_u32x4(src + 16 * (size_t)v);
    if (tid == 0) {
      p.cexp[c] = p.blk_expert[b];
      p.csrc[c] = ld_acquire_sys(p.recv_src + row0 + r);
    }
  }
}

struct EpRowsReturnParams {
  const float* part;   // [cap_pairs][S][H]
  const int* cexp;
  const int* csrc;
  int S, H;
  const unsigned long long* ret_table;   // [kMaxRanks]: return buffers [slots][H] bf16
};

// grid cap_pairs, 256 threads
__global__ void __launch_bounds__(256) ep_rows_return_kernel(const EpRowsReturnParams p) {
  pdl_wait();
  pdl_launch_dependents();
  const int c = blockIdx.x, tid = threadIdx.x;
  if (p.cexp[c] < 0) return;
  const int src = p.csrc[c];
  __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.ret_table[src >> 24]) + (size_t)(src & 0xffffff) * p.H;
  const float* base = p.part + (size_t)c * p.S * p.H;
  for (int v = tid; v < p.H / 8; v += 256) {
    float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < p.S; ++s) {
      const float4 x = *reinterpret_cast<const float4*>(base + (size_t)s * p.H + 8 * v);
      const float4 y = *reinterpret_cast<const float4*>(base + (size_t)s * p.H + 8 * v + 4);
      a[0] += x.x; a[1] += x.y; a[2] += x.z; a[3] += x.w; a[4] += y.x; a[5] += y.y; a[6] += y.z; a[7] += y.w;
    }
    uint4 o;
    o.x = pack_bf16(a[0], a[1]); o.y = pack_bf16(a[2], a[3]); o.z = pack_bf16(a[4], a[5]); o.w = pack_bf16(a[6], a[7]);
    *reinterpret_cast<uint4*>(dst + 8 * v) = o;
  }
}

}  // namespace

static Wire make_wire(const void* table, int world, int rank) {
  Wire w;
  w.table = (const unsigned long long*)table; w.epoch = nullptr; w.world = world; w.rank = rank;
  return w;
}

extern "C" int b2_ep_counts_push(const int* counts, int E, const void* cnt_table, int world, int rank, int epoch,
                                 void* stream) {
  if (world < 1 || world > kMaxRanks || E > 1024) return -1;
  return b2_launch(ep_counts_push_kernel, dim3(1), dim3(1024), 0, (cudaStream_t)stream, true, counts, E,
                   make_wire(cnt_table, world, rank), epoch);
}

extern "C" int b2_ep_plan(const void* cnt_table, int epoch, int E, int world, int rank, int max_blk, int cap_rows,
                          int* send_base, int* blk_expert, int* blk_row0, int* blk_rows, int* n_blk, int* total_rows,
                          int* blk_cnt_next, void* stream) {
  if (world < 1 || world > kMaxRanks || E > 1024 || E % world) return -1;
  EpPlanParams p;
  p.cnt_table = (const unsigned long long*)cnt_table; p.epoch = epoch; p.E = E; p.El = E / world; p.world = world;
  p.rank = rank; p.max_blk = max_blk; p.cap_rows = cap_rows; p.send_base = send_base; p.blk_expert = blk_expert;
  p.blk_row0 = blk_row0; p.blk_rows = blk_rows; p.n_blk = n_blk; p.total_rows = total_rows; p.blk_cnt_next = blk_cnt_next;
  return b2_launch(ep_plan_kernel, dim3(1), dim3(1024), 0, (cudaStream_t)stream, true, p);
}

extern "C" int b2_ep_dispatch(const int* topk_idx, const int* rank_in_expert, const int* send_base, const void* x, int T,
                              int k, int H, int E, int world, int me, int cap_rows, int parity, int max_blk,
                              const void* recv_table, const void* src_table, void* stream) {
  if (H % 8 || world < 1 || E % world || T * k >= (1 << 24) || k < 1 || k > 32) return -1;
  EpDispatchParams p;
  p.topk_idx = topk_idx; p.rank_in_expert = rank_in_expert; p.send_base = send_base; p.x = (const __nv_bfloat16*)x;
  p.k = k; p.H = H; p.El = E / world; p.me = me; p.cap_rows = cap_rows; p.parity = parity; p.max_blk = max_blk;
  p.recv_table = (const unsigned long long*)recv_table; p.src_table = (const unsigned long long*)src_table;
  return b2_launch(ep_dispatch_kernel, dim3(T), dim3(32 * k), 0, (cudaStream_t)stream, true, p);
}

extern "C" int b2_ep_flag_all(const void* table, int world, int rank, int epoch, void* stream) {
  return b2_launch(ep_flag_all_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream, true, make_wire(table, world, rank), epoch);
}

extern "C" int b2_ep_wait_all(const void* table, int world, int rank, int epoch, void* stream) {
  return b2_launch(ep_wait_all_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream, true, make_wire(table, world, rank), epoch);
}

extern "C" int b2_ep_rows_gather(const int* blk_expert, const int* blk_row0, const int* blk_rows, const int* n_blk, int max_blk,
                                 const int* blk_cnt, const void* recv_x, const int* recv_src, int H, int cap_pairs, void* cx,
                                 int* cexp, int* csrc, int* n_valid, void* stream) {
  if (H % 8 || max_blk < 1 || cap_pairs < 1) return -1;
  EpRowsParams p;
  p.blk_expert = blk_expert; p.blk_row0 = blk_row0; p.blk_rows = blk_rows; p.n_blk = n_blk; p.blk_cnt = blk_cnt;
  p.recv_x = (const __nv_bfloat16*)recv_x; p.recv_src = recv_src; p.H = H; p.cap_pairs = cap_pairs;
  p.cx = (__nv_bfloat16*)cx; p.cexp = cexp; p.csrc = csrc; p.n_valid = n_valid;
  return b2_launch(ep_rows_gather_kernel, dim3(max_blk), dim3(256), 0, (cudaStream_t)stream, true, p);
}

extern "C" int b2_ep_rows_return(const float* part, const int* cexp, const int* csrc, int cap_pairs, int S, int H,
                                 const void* ret_table, void* stream) {
  if (H % 8 || S < 1 || cap_pairs < 1) return -1;
  EpRowsReturnParams p;
  p.part = part; p.cexp = cexp; p.csrc = csrc; p.S = S; p.H = H; p.ret_table = (const unsigned long long*)ret_table;
  return b2_launch(ep_rows_return_kernel, dim3(cap_pairs), dim3(256), 0, (cudaStream_t)stream, true, p);
}

B2_DEFINE_STATUS(ep)
