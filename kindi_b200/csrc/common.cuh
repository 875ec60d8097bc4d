// Shared helpers of the kernel library: storage types, the status word, launch checks.
//
// Every entry point is extern "C", takes raw device pointers and a stream, and returns the cudaError_t of its
// launch as an int. Kernels never trap: an index that is out of range (a token id beyond the table, a page that is
// not mapped) sets a bit in the caller's status word and the access is skipped, so the context stays usable and
// the host can raise an error after the step.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define KB_F32 0
#define KB_BF16 1

#define KB_PAGE 64                 // positions per cache page

// status bits
#define KB_ST_BAD_TOKEN 1
#define KB_ST_BAD_PAGE 2
#define KB_ST_WAIT_TIMEOUT 4
#define KB_ST_BAD_ROW 8

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float kb_to_f(T v);
template <> __device__ __forceinline__ float kb_to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float kb_to_f<bf16>(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T kb_from_f(float v);
template <> __device__ __forceinline__ float kb_from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 kb_from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float kb_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float kb_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// where a sequence's keys and values live: pool of pages [page][2][n_kv][KB_PAGE][head_dim] for one cache entry,
// and the table that maps (slot, position / KB_PAGE) to a page
struct KbCacheView {
    void* pool;                 // this cache entry's pages
    const int* table;           // [n_slots][table_stride]
    int table_stride;
    int n_pages;
    int n_kv;
    int head_dim;
};

__device__ __forceinline__ size_t kb_kv_offset(const KbCacheView& c, int page, int kv, int head, int p_in_page) {
    return ((((size_t)page * 2 + kv) * c.n_kv + head) * KB_PAGE + p_in_page) * (size_t)c.head_dim;
}

#define KB_LAUNCH_RET() return (int)cudaGetLastError()
