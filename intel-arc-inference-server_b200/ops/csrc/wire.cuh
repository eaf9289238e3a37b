// Cross-GPU wire used by the fused compute+collective kernels.
//
// The reference's two-card wire (src/kernels/tp.cl:23-47, src/runtime/tp_protocol.h:1-17) keeps every
// landing buffer in the READER's memory: a writer stores its data into the peer, fences at system
// scope and then stores a flag; the reader spins (bounded) on a flag in its own memory, acquires,
// reads the data and folds the parts in a fixed rank order so every card computes identical bits.
// This is the same protocol for up to eight ranks behind an NVSwitch: peer memory is mapped into the
// address space (CUDA IPC), stores cross NVLink as ordinary st.global, flags carry a call number
// ("epoch") that only grows, so a CUDA graph that is replayed needs no reset between calls, and a
// landing buffer has two slots (epoch & 1) so call n + 1 never overwrites data call n still reads.
//
// A table of the ranks' buffer addresses lives in device memory (one 64-bit word per rank and
// buffer), so a captured graph holds no peer address in its kernel parameters.
#pragma once
#include "common.cuh"

namespace b2 {

constexpr int kMaxRanks = 8;

struct Wire {
  const unsigned long long* table;  // [2][kMaxRanks]: landing buffer address, flag array address of every rank
  int* epoch;                       // local call counters (one per tile of the caller's choosing)
  int world, rank;
};

__device__ __forceinline__ float* wire_land(const Wire& w, int r) {
  return reinterpret_cast<float*>(w.table[r]);
}
__device__ __forceinline__ int* wire_flags(const Wire& w, int r) {
  return reinterpret_cast<int*>(w.table[kMaxRanks + r]);
}

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float ld_sys_f32(const float* p) {
  float v;
  asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_sys_f32x4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_sys_u32x4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// Bounded wait for a flag in this GPU's own memory to reach `epoch` (flags only grow).  About a second
// at 2 GHz; on expiry the status word gets ERR_COMM_FLAG_WAIT with `detail` and the wait returns false -- the caller then
// skips its fold and leaves, the context stays usable and the host reads the status.
__device__ __forceinline__ bool wire_wait(const int* flag, int epoch, unsigned int detail) {
  for (int i = 0; i < 64; ++i)
    if (ld_acquire_sys(flag) - epoch >= 0) return true;
  if (g_status[0] != 0u) return false;  // an earlier wait already ran out: do not stack second-long waits
  const long long t0 = clock64();
  while (ld_acquire_sys(flag) - epoch < 0) {
    if (clock64() - t0 > 2000000000ll) {
      record_error(ERR_COMM_FLAG_WAIT, detail);
      return false;
    }
    __nanosleep(64);
  }
  return true;
}

}  // namespace b2
