// bfloat16 matrix products of prompt-sized steps on PAIRS of SMs: C = A W^T with tcgen05.mma.cta_group::2.
//
// Two CTAs that form a cluster work on one 256 x BN tile of C. Each brings 128 rows of A (tokens) and HALF of the
// weight tile (BN / 2 rows of W) into its own shared memory; one thread of the even CTA (the leader) issues MMAs of
// M 256, N BN, K 16 that read A and W from both CTAs' shared memory and leave 128 x BN accumulators in each CTA's
// tensor memory. Against one CTA that computes 128 x BN alone, a CTA takes in BN / 2 fewer weight rows per K block
// for the same arithmetic, and what an SM can take in from the L2 is what bounds the single-CTA kernel on wide tiles.
//
// Roles as in k_gemm_tc: warp 0 = TMA producer (both CTAs, each for its own tiles), warp 1 = tensor memory owner and,
// in the leader, the MMA thread, warps 2-5 = epilogue (each CTA writes its own 128 rows). Barriers:
//   full[s]      (leader's)  the leader's producer announces the bytes of BOTH CTAs' tiles; both CTAs' loads
//                            complete on it (cp.async.bulk.tensor with .cta_group::2 may signal the peer's barrier)
//   empty[s]     (each CTA's) tcgen05.commit with a multicast to both CTAs once the stage's MMAs are done
//   acc_full[a]  (each CTA's) the same commit after a tile's last MMA
//   acc_empty[a] (leader's)  eight arrivals: the four epilogue warps of each CTA (the peer's arrive remotely)
// Work is cut in one of two ways. Tile by tile: pair p takes tiles p, p + pairs, ... Or, when the tiles do not fill the
// pairs evenly (80 tiles on 74 pairs would take as long as 148), as one line of all (tile, K block) pairs, of which
// pair p takes the p-th stretch. A stretch is at least a tile long, so a tile is shared by at most two pairs: the one
// that holds its first K blocks at the END of its stretch (the owner) and the next pair, which holds the rest at the
// START of its own (the helper). The helper writes its 32-bit partial tile and raises the tile's flags as the first
// thing it does; the owner, when it comes to the tile at the end of its stretch, adds the part to its own sums in a
// fixed order (own + other), stores the result and lowers the flags.
// No TMA load is multicast. Every wait is bounded; a CTA leaves only after both have passed a cluster barrier, so no
// signal is sent to shared memory that has been given back.
#include "sm100.cuh"

#define GP_BM 128
#define GP_BK 64
#define GP_THREADS 192

template <int BN, int STAGES>
struct GpSmem {
    static constexpr int A_BYTES = GP_BM * GP_BK * 2;
    static constexpr int B_BYTES = (BN / 2) * GP_BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int EPI_OFF = STAGES * STAGE_BYTES;            // 4 KB per epilogue warp (see k_gemm_tc)
    static constexpr int BAR_OFF = EPI_OFF + 4 * 4096;
    static constexpr int N_BARS = 2 * STAGES + 4 + 4;               // + one per epilogue warp for a shared tile's part
    static constexpr int TOTAL = BAR_OFF + N_BARS * 8 + 16 + 1024;  // + alignment slack
    static_assert(4 * 32 * BN * 4 <= STAGES * STAGE_BYTES, "a shared tile's part is brought into the idle stages");
    static_assert(TOTAL <= 227 * 1024, "shared memory of a CTA");
    static_assert(BN % 32 == 0 && BN >= 64 && BN <= 256, "tile width");
};

__device__ __forceinline__ uint32_t gp_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void gp_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the address, in the cluster's shared window, of this CTA's shared address `addr` in CTA `rank`
__device__ __forceinline__ uint32_t gp_mapa(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void gp_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// tile load whose completion is counted on a barrier that may be the peer CTA's (no multicast)
__device__ __forceinline__ void gp_tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void gp_tmem_alloc(uint32_t smem_dst, uint32_t cols) {     // one warp of each CTA
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void gp_tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void gp_tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void gp_umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// one arrival on the barrier at this offset in BOTH CTAs when every MMA issued so far has completed
__device__ __forceinline__ void gp_umma_commit(uint32_t bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(bar), "h"((uint16_t)3)
        : "memory");
}

template <int BN, int STAGES, typename TC>
__global__ void __launch_bounds__(GP_THREADS) k_gemm_pair(const __grid_constant__ CUtensorMap mapA,
        const __grid_constant__ CUtensorMap mapW, TC* __restrict__ C, int M, int N, int K, int ldc, int* status,
        int swiglu_ld, float* part, int* flags) {      // (shared with other CTAs of this launch: no __restrict__)
    using S = GpSmem<BN, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar_full = sbase + S::BAR_OFF, bar_empty = bar_full + STAGES * 8;
    const uint32_t bar_acc_full = bar_empty + STAGES * 8, bar_acc_empty = bar_acc_full + 16;
    const uint32_t bar_part = bar_acc_empty + 16;
    volatile uint32_t* tmem_slot = (volatile uint32_t*)(smem + S::BAR_OFF + S::N_BARS * 8);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = gp_cta_rank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int tilesP = (M + 2 * GP_BM - 1) / (2 * GP_BM), tilesQ = (N + BN - 1) / BN;
    const int n_units = tilesP * tilesQ;
    const int total_kb = (K + GP_BK - 1) / GP_BK;
    constexpr uint32_t TMEM_COLS = BN <= 64 ? 128 : BN <= 128 ? 256 : 512;     // two accumulators
    constexpr uint32_t ACC_COLS = TMEM_COLS / 2;
    // the pair's work: segments (tile, first K block, one past the last K block). part != nullptr: the pair's stretch
    // of the line of all (tile, K block) pairs; else whole tiles.
    const bool line = part != nullptr;
    const int L0 = line ? (int)((long long)n_units * total_kb * pair / n_pairs) : 0;
    const int L1 = line ? (int)((long long)n_units * total_kb * (pair + 1) / n_pairs) : 0;
    auto seg_first = [&]() { return line ? L0 : pair; };
    auto seg_valid = [&](int pos) { return line ? pos < L1 : pos < n_units; };
    auto seg_get = [&](int pos, int& unit, int& kb0, int& kb1) {
        if (line) {
            unit = pos / total_kb;
            kb0 = pos % total_kb;
            kb1 = min(total_kb, kb0 + (L1 - pos));
        } else {
            unit = pos;
            kb0 = 0;
            kb1 = total_kb;
        }
    };
    auto seg_next = [&](int pos, int kb0, int kb1) { return line ? pos + (kb1 - kb0) : pos + n_pairs; };

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(bar_full + s * 8, 1);
            mbar_init(bar_empty + s * 8, 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(bar_acc_full + a * 8, 1);
            mbar_init(bar_acc_empty + a * 8, 8);
        }
        for (int w = 0; w < 4; w++) mbar_init(bar_part + w * 8, 1);
        mbar_fence_init();
        tma_prefetch_desc(&mapA);
        tma_prefetch_desc(&mapW);
    }
    if (warp == 1) {
        gp_tmem_alloc(smem_u32((const void*)tmem_slot), TMEM_COLS);
        gp_tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    gp_cluster_sync();                       // the peer's barriers are initialised before anything signals them
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t n = 0;
            bool ok = true;
            const uint32_t full0 = gp_mapa(bar_full, 0);         // the leader's full barriers
            kb_pdl_wait();                                       // A comes from the kernel before
            int u, kb0, kb1;
            for (int pos = seg_first(); seg_valid(pos) && ok; pos = seg_next(pos, kb0, kb1)) {
                seg_get(pos, u, kb0, kb1);
                const int tp = u % tilesP, tq = u / tilesP;
                for (int kb = kb0; kb < kb1; kb++, n++) {
                    const int s = n % STAGES;
                    if (!(ok = mbar_wait(bar_empty + s * 8, ((n / STAGES) & 1u) ^ 1u, status))) break;
                    if (leader) mbar_expect_tx(bar_full + s * 8, 2 * S::STAGE_BYTES);
                    const uint32_t dst = sbase + s * S::STAGE_BYTES;
                    gp_tma_load_2d(dst, &mapA, kb * GP_BK, (tp * 2 + (int)rank) * GP_BM, full0 + s * 8);
                    gp_tma_load_2d(dst + S::A_BYTES, &mapW, kb * GP_BK, tq * BN + (int)rank * (BN / 2), full0 + s * 8);
                }
            }
            // the MMAs' last commits signal this CTA's empty barriers: they must have landed before it may leave
            for (uint32_t m = n > (uint32_t)STAGES ? n - STAGES : 0; m < n && ok; m++)
                ok = mbar_wait(bar_empty + (m % STAGES) * 8, (m / STAGES) & 1u, status);
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = umma_idesc_bf16(2 * GP_BM, BN);
            uint32_t n = 0, it = 0;
            bool ok = true;
            int u, kb0, kb1;
            for (int pos = seg_first(); seg_valid(pos) && ok; pos = seg_next(pos, kb0, kb1), it++) {
                seg_get(pos, u, kb0, kb1);
                const uint32_t acc = it & 1u;
                if (!(ok = mbar_wait(bar_acc_empty + acc * 8, ((it >> 1) & 1u) ^ 1u, status))) break;
                tc_fence_after();
                const uint32_t d = tmem + acc * ACC_COLS;
                for (int kb = kb0; kb < kb1; kb++, n++) {
                    const int s = n % STAGES;
                    if (!(ok = mbar_wait(bar_full + s * 8, (n / STAGES) & 1u, status))) break;
                    tc_fence_after();
                    const uint32_t a = sbase + s * S::STAGE_BYTES, b = a + S::A_BYTES;
#pragma unroll
                    for (int k = 0; k < GP_BK / 16; k++)
                        gp_umma_bf16(d, umma_desc_sw128(a + k * 32), umma_desc_sw128(b + k * 32), idesc,
                                     (kb > kb0 || k > 0) ? 1u : 0u);
                    gp_umma_commit(bar_empty + s * 8);
                }
                gp_umma_commit(bar_acc_full + acc * 8);
            }
        }
    } else {
        // epilogue warps 2..5 own TMEM lanes 32 * (warp % 4) .. + 31 of this CTA's 128 rows
        const int quarter = warp & 3;
        const uint32_t acc_empty0 = gp_mapa(bar_acc_empty, 0);
        uint32_t it = 0;
        bool ok = true;
        kb_pdl_wait();                                   // C may be memory that an earlier kernel still reads
        int u, kb0, kb1;
        for (int pos = seg_first(); seg_valid(pos) && ok; pos = seg_next(pos, kb0, kb1), it++) {
            seg_get(pos, u, kb0, kb1);
            const int tp = u % tilesP, tq = u / tilesP;
            const int q0 = tq * BN;
            const uint32_t acc = it & 1u;
            const bool helper = kb0 > 0, owner = kb0 == 0 && kb1 < total_kb;      // of a shared tile
            // a warp's piece of a shared tile's part: [column][lane], so that both sides move whole 128-byte lines
            float* pw = part + ((size_t)(u * 2 + (int)rank) * 4 + quarter) * (size_t)(32 * BN) + lane;
            int* flag = flags + (u * 2 + (int)rank) * 4 + quarter;
            if (owner) {
                // the other part was written when the next pair began, long ago
                if (lane == 0) {
                    const uint64_t t0 = kb_globaltimer();
                    while (*((volatile int*)flag) == 0) {
                        __nanosleep(100);
                        if (kb_globaltimer() - t0 > KB_WAIT_NS) {
                            atomicOr(status, KB_ST_WAIT_TIMEOUT);
                            ok = false;
                            break;
                        }
                    }
                    __threadfence();
                }
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
            }
            if (!(ok = mbar_wait(bar_acc_full + acc * 8, (it >> 1) & 1u, status))) break;
            tc_fence_after();
            const float* ps = (const float*)(smem + quarter * (32 * BN * 4)) + lane;
            if (owner) {
                // This is the pair's last tile and its MMAs are done: the stages are idle. The warp's piece of the
                // other part comes into them as one bulk copy (it happens once in a launch: phase 0 of its barrier).
                if (lane == 0) {
                    mbar_expect_tx(bar_part + quarter * 8, 32 * BN * 4);
                    asm volatile(
                        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                        ::"r"(sbase + quarter * (32 * BN * 4)), "l"(pw - lane), "r"(32 * BN * 4),
                          "r"(bar_part + quarter * 8)
                        : "memory");
                }
                if (!(ok = mbar_wait(bar_part + quarter * 8, 0u, status))) break;
            }
            const int p0 = (tp * 2 + (int)rank) * GP_BM;
            const int prow = p0 + quarter * 32 + lane;
            const uint32_t tbase = tmem + acc * ACC_COLS + ((uint32_t)(quarter * 32) << 16);
            // 32 columns of this thread's row of the tile: the accumulator, plus the helper's part in a shared tile
            auto load32 = [&](int c0, uint32_t* r) {
                tmem_ld_32x32(tbase + c0, r);
                if (owner) {
                    float o[32];
#pragma unroll
                    for (int c = 0; c < 32; c++) o[c] = ps[(c0 + c) * 32];
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 32; c++) r[c] = __float_as_uint(__uint_as_float(r[c]) + o[c]);
                } else {
                    tmem_ld_wait();
                }
            };
            if (helper) {
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    uint32_t r[32];
                    tmem_ld_32x32(tbase + c0, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 32; c++) __stcg(pw + (size_t)(c0 + c) * 32, __uint_as_float(r[c]));
                }
                __threadfence();
                __syncwarp();
                if (lane == 0) atomicExch(flag, 1);
            } else if (swiglu_ld > 0) {
                // W's rows come as 16 gate rows followed by the 16 up rows of the same outputs: every 32 columns hold
                // both halves of 16 outputs, and silu(gate) * up leaves as bf16 (the 2F-wide product is never written)
                bf16* orow = (bf16*)C + (size_t)prow * swiglu_ld;
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    if (q0 + c0 >= N) continue;                       // past the end (uniform over the warp)
                    uint32_t gu[32];
                    tmem_ld_32x32(tbase + c0, gu);
                    tmem_ld_wait();
                    if (prow < M) {
                        uint32_t h[8];
#pragma unroll
                        for (int c = 0; c < 8; c++) {
                            const float g0 = __uint_as_float(gu[2 * c]), g1 = __uint_as_float(gu[2 * c + 1]);
                            __nv_bfloat162 v = __floats2bfloat162_rn(
                                __fdividef(g0, 1.0f + __expf(-g0)) * __uint_as_float(gu[16 + 2 * c]),
                                __fdividef(g1, 1.0f + __expf(-g1)) * __uint_as_float(gu[16 + 2 * c + 1]));
                            h[c] = *(uint32_t*)&v;
                        }
                        bf16* dst = orow + ((q0 + c0) >> 1);
                        *(uint4*)(dst) = make_uint4(h[0], h[1], h[2], h[3]);
                        *(uint4*)(dst + 8) = make_uint4(h[4], h[5], h[6], h[7]);
                    }
                }
            } else {
                // a thread holds one row of the accumulator; the warp's 32 rows x 128 bytes pass through its staging
                // area (16-byte pieces, swizzled by the row) and leave as whole 128-byte pieces of four rows a store
                constexpr int CW = 128 / (int)sizeof(TC);
                constexpr int PW = 16 / (int)sizeof(TC);
                uint8_t* stg = smem + S::EPI_OFF + quarter * 4096;
                const bool vec_ok = (((uintptr_t)C) & 15) == 0 && (ldc % PW) == 0;
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += CW) {
                    uint32_t r[32];
                    load32(c0, r);
                    if (sizeof(TC) == 4) {
#pragma unroll
                        for (int j = 0; j < 8; j++)
                            *(uint4*)(stg + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                                make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                    } else {
#pragma unroll
                        for (int half = 0; half < 2; half++) {
                            if (half == 1) load32(c0 + 32, r);
#pragma unroll
                            for (int j = 0; j < 4; j++) {
                                uint32_t h[4];
#pragma unroll
                                for (int c = 0; c < 4; c++) {
                                    __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[8 * j + 2 * c]),
                                                                             __uint_as_float(r[8 * j + 2 * c + 1]));
                                    h[c] = *(uint32_t*)&v;
                                }
                                *(uint4*)(stg + lane * 128 + (((half * 4 + j) ^ (lane & 7)) << 4)) =
                                    make_uint4(h[0], h[1], h[2], h[3]);
                            }
                        }
                    }
                    __syncwarp();
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        const int rr = i * 4 + (lane >> 3), jj = lane & 7;
                        const uint4 v = *(const uint4*)(stg + rr * 128 + ((jj ^ (rr & 7)) << 4));
                        const int grow = p0 + quarter * 32 + rr, ct = c0 + jj * PW, gcol = q0 + ct;
                        if (grow < M && ct < BN && gcol < N) {
                            TC* dst = C + (size_t)grow * ldc + gcol;
                            if (vec_ok && gcol + PW <= N) {
                                *(uint4*)dst = v;
                            } else {
                                const TC* e = (const TC*)&v;
#pragma unroll
                                for (int c = 0; c < PW; c++)
                                    if (gcol + c < N) dst[c] = e[c];
                            }
                        }
                    }
                    __syncwarp();
                }
                if (owner) {
                    __syncwarp();
                    if (lane == 0) atomicExch(flag, 0);          // lowered for the next call
                }
            }
            // this warp has read its lanes of the accumulator: tell the leader's MMA thread
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (leader) mbar_arrive(bar_acc_empty + acc * 8);
                else gp_arrive_remote(acc_empty0 + acc * 8);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    gp_cluster_sync();
    if (warp == 1) {
        tc_fence_after();
        gp_tmem_dealloc(tmem, TMEM_COLS);
    }
}

static int gp_sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

template <int BN, int STAGES, typename TC>
static int launch_pair(const CUtensorMap& ma, const CUtensorMap& mw, void* C, int M, int N, int K, int ldc, int* status,
                       cudaStream_t st, int swiglu_ld, float* part, int* flags) {
    using S = GpSmem<BN, STAGES>;
    auto kern = k_gemm_pair<BN, STAGES, TC>;
    static char once_tag;               // one per instantiation: the opt-in is per (device, kernel)
    if (kb_first_use(&once_tag)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
        if (e != cudaSuccess) return (int)e;
    }
    const int units = ((M + 2 * GP_BM - 1) / (2 * GP_BM)) * ((N + BN - 1) / BN);
    const int pairs = units < gp_sm_count() / 2 ? units : gp_sm_count() / 2;
    // the line of (tile, K block) pairs only where a stretch is at least a tile long and the epilogue is the plain one
    if (part && (units < pairs || swiglu_ld > 0 || !flags)) part = nullptr;
    kb_same_partition((const void*)kern);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(GP_THREADS);
    cfg.dynamicSmemBytes = S::TOTAL;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_kb_pdl ? 2 : 1;
    return (int)cudaLaunchKernelEx(&cfg, kern, ma, mw, (TC*)C, M, N, K, ldc, status, swiglu_ld, part, flags);
}

// C[M][N] = A[M][K] W[N][K]^T for prompt-sized M, on pairs of SMs. cdtype: KB_F32 or KB_BF16; bn: the pair's tile width
// (64, 128, 192 or 256). swiglu != 0 (bf16 out): W holds gate and up rows in groups of 16 + 16 and C is the bf16
// [M][N / 2] result silu(gate) * up with row stride ldc. part (fp32, tiles * 256 * bn elements with tiles =
// ceil(M / 256) * ceil(N / bn), 16-byte aligned) and flags (8 ints a tile, zero before the first call; the kernel
// lowers what it raised) are the scratch of tiles shared by two pairs; without them the work is cut tile by tile.
extern "C" int kb_gemm_pair(const void* A, const void* W, void* C, int cdtype, int M, int N, int K, int lda, int ldw,
                            int ldc, int bn, int* status, cudaStream_t st, int swiglu, float* part, int* flags) {
    if (swiglu && ((N % 32) || cdtype != KB_BF16 || (ldc % 8) || ((uintptr_t)C & 15))) return (int)cudaErrorInvalidValue;
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if ((K % 8) || (lda % 8) || (ldw % 8)) return (int)cudaErrorInvalidValue;
    if (cdtype != KB_F32 && cdtype != KB_BF16) return (int)cudaErrorInvalidValue;
    const int swiglu_ld = swiglu ? ldc : 0;
    CUtensorMap ma, mw;
    int rc;
    if ((rc = kb_make_map_bf16(&ma, A, M, K, lda, GP_BM))) return rc;
    if ((rc = kb_make_map_bf16(&mw, W, N, K, ldw, bn / 2))) return rc;
#define GP_GO(BN, ST)                                                                                        \
    return cdtype == KB_F32 ? launch_pair<BN, ST, float>(ma, mw, C, M, N, K, ldc, status, st, swiglu_ld, part, flags) \
                            : launch_pair<BN, ST, bf16>(ma, mw, C, M, N, K, ldc, status, st, swiglu_ld, part, flags)
    switch (bn) {
        case 64: GP_GO(64, 8);
        case 128: GP_GO(128, 8);
        case 192: GP_GO(192, 7);
        case 256: GP_GO(256, 6);
        default: return (int)cudaErrorInvalidValue;
    }
#undef GP_GO
}
