/* kindi_b200: the one entry point of the kernel library that allocates nothing.
 *
 * It has no counterpart in ahtx/kindi; it exists for hosts that cannot allocate device memory while they run (a
 * plug-in inside another program's CUDA context with a fixed memory limit, a real-time loop that keeps away from
 * the allocator, a process whose memory pool belongs to somebody else).
 *
 * kb_attn_decode_static runs this library's decode attention over the paged cache (bfloat16, head size 64 or 128,
 * one query row per sequence, up to 16 query heads per key/value head) like kb_attn_mma does, but keeps the scratch
 * of its position splits in a static device array inside the library instead of taking it from the caller:
 *   - 4 MiB per GPU that loads the library, held until the process exits;
 *   - a call needs B * nh * n_splits * (hd + 2) floats of at most 1 << 20; larger calls return
 *     cudaErrorInvalidValue (1) after one line on stderr and launch nothing;
 *   - the first call on a device looks the array's address up (cudaGetSymbolAddress): make that call before any
 *     stream capture;
 *   - all calls share the array: calls that overlap on the GPU race; calls on one stream are safe.
 * Arguments: q [B rows][>= nh * hd] bf16 with row stride ldq; out [B rows][nh * hd] bf16 with row stride ldo;
 * slot [B], q_start [B + 1] (row of each sequence), kv_len [B] (length of each sequence, its row being the last
 * position); pool = pages [n_pages][2][nkv][64][hd] bf16 of one cache entry; table [slots][table_stride] page of each
 * block of 64 positions; window 0 = all keys; n_splits 1..64; status = device int that collects error bits.
 * Returns 0 or a cudaError_t value. */
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

int kb_attn_decode_static(const void* q, int ldq, void* out, int ldo, const int* slot, const int* q_start,
                          const int* kv_len, int B, int nh, int nkv, int hd, float scale, int window, void* pool,
                          const int* table, int table_stride, int n_pages, int n_splits, int* status,
                          cudaStream_t st);

#ifdef __cplusplus
}
#endif
