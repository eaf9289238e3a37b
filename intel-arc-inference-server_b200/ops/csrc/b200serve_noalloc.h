/* Allocation-free entry point of libb200serve.so.
 *
 * This entry point has no counterpart in the reference project; it exists for embedders of this
 * library.
 *
 * Who it is for.  Some hosts of this library may not allocate device memory at the time they
 * call it: a plug-in running inside a process whose framework has already handed the whole GPU
 * to its own memory pool (a cudaMalloc there fails, or fragments what the pool believes it owns);
 * a serving thread with a latency bound, for which cudaMalloc / cudaFree are off limits because
 * they take driver-wide locks and may synchronise the device; and a caller that simply holds no
 * allocator at all (a C program handing over pointers it was given).  The regular entry point,
 * b2_attn_decode, needs two scratch buffers from its caller for the split-KV partial results.
 * b2_attn_decode_static runs the same kernels and keeps that scratch in a fixed array inside the
 * library image instead, so the call performs no cudaMalloc, no cudaFree and calls no allocating
 * library routine.  Inputs and outputs are still the caller's.
 *
 * Limits (the fixed array is 2 MiB + 32 KiB and stays resident on every GPU that loads the
 * library, until the process exits):
 *     M (rows)        1 .. 4
 *     n_q (heads)     1 .. 64, a multiple of n_kv with n_q / n_kv one of 1, 2, 4, 5, 8
 *     nsplit          1 .. 16
 *     D (head size)   64 or 128
 * A call beyond them (or on a device whose index is 64 or more) returns -10 and launches nothing; use
 * b2_attn_decode with your own buffers.
 *
 * Set-up.  The first call on each device resolves the array's device address (with that device
 * current); it launches nothing extra and allocates nothing, but it is a runtime query, so make
 * that first call before any stream capture begins on that device.
 *
 * Sharing.  Every call on a device uses the same array and leaves its contents behind.  Nothing in
 * it has to start at zero (each call writes every entry it later reads), so back-to-back calls on
 * one stream are fine.  Two calls that can overlap on the GPU -- different streams without an
 * ordering between them, or two host threads -- race on the array: order them, or give one of
 * them the regular entry point.
 *
 * Arguments are those of b2_attn_decode without o_part / ml_part:
 *   q            bf16 [M][n_q * D]                     k_cache, v_cache  paged cache [page][n_kv][16][D]
 *   k_scale, v_scale  fp32 [page][n_kv][16] (int8 cache) or NULL          block_table  int32 [slots][max_blocks]
 *   ctrl         int32 control block (row -> slot, position)             out  bf16 [M][n_q * D]
 * Returns 0, a CUDA error code, or a negative argument error.
 */
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
int b2_attn_decode_static(const void* q, const void* k_cache, const void* v_cache, const float* k_scale,
                          const float* v_scale, const int* block_table, const int* ctrl, void* out, int M, int n_q,
                          int n_kv, int D, int nsplit, int max_blocks, float scale, int kv_int8, void* stream);
#ifdef __cplusplus
}
#endif
