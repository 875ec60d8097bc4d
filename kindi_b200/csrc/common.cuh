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

// Programmatic dependent launch. Every kernel of the library begins with kb_pdl_launch() (when its grid is small,
// the next kernel of the stream may be scheduled as soon as all CTAs of this one have started) and calls
// kb_pdl_wait() before its first
// read of anything an earlier kernel wrote and before its first global write (until then it may only set up
// barriers and tensor memory and fetch weights, which no kernel writes). The wait returns when the whole preceding
// kernel has finished and its writes are visible, so results are those of strictly ordered launches; what is
// gained is that launch latency and prologues overlap the predecessor's tail.
// Before its wait a kernel also reads the step's metadata (positions, lengths, slots, row lists, the page table)
// and cache pages of older positions. Callers therefore write those with operations that are complete before the
// step's first kernel starts: the engine brings the page table up to date and then copies the metadata to the
// device (a copy orders fully), and older pages were stored by earlier steps.
__device__ __forceinline__ void kb_pdl_launch_now() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// Small grids (decode steps) let their successor start at once; large grids (prompt steps) do not: a successor that
// was launched before its predecessor ended was measured to cost a prompt step several microseconds per kernel,
// whether the trigger came at the start of the blocks or after their last loads.
__device__ __forceinline__ void kb_pdl_launch() {
    if (gridDim.x * gridDim.y * gridDim.z <= 1024u) kb_pdl_launch_now();
}
__device__ __forceinline__ void kb_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// A kernel parameter that points at what an earlier kernel of the same step wrote (activations, split-K planes,
// partial results, logits) is marked KB_STEP_DATA and is NOT declared __restrict__: for a const __restrict__ pointer the
// compiler may take the data for read-only during the whole kernel and move its loads above the wait (seen with the
// 32-bit product: loads placed right after the wait were issued before it and read what the kernel before had not
// written yet). Weights, tables and the step's metadata are written before the step's first kernel and keep
// __restrict__: they are meant to be read early.
#define KB_STEP_DATA

extern int g_kb_pdl;            // 1: launches carry the programmatic-serialization attribute

#ifdef __cplusplus
#include <utility>
#include <mutex>
#include <unordered_set>
// true the first time it is asked about this kernel on the current device, false ever after: function attributes
// (the shared-memory opt-in, the carve-out) belong to a device, so they are set once per (device, kernel). Safe to
// call from several host threads.
static inline bool kb_first_use(const void* kern) {
    static std::mutex mu;
    static std::unordered_set<uint64_t> seen;
    int dev = 0;
    cudaGetDevice(&dev);
    const uint64_t key = ((uint64_t)(uintptr_t)kern << 8) ^ (uint64_t)(dev & 0xff);
    std::lock_guard<std::mutex> g(mu);
    return seen.insert(key).second;
}
// Every kernel of the library asks for the largest shared-memory partition of the SM, the one its tensor-core
// kernels need: an SM re-partitions L1 and shared memory only when it is idle, so a step whose kernels all want the
// same partition never waits for that, and a kernel launched early can become resident beside its predecessor.
static inline void kb_same_partition(const void* kern) {
    if (kb_first_use(kern))
        cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
}
template <typename... KArgs, typename... Args>
static inline cudaError_t kb_launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                    Args&&... args) {
    kb_same_partition((const void*)kern);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_kb_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...);
}
#endif
