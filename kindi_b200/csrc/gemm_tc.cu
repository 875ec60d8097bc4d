// bfloat16 matrix products on the 5th-generation tensor cores: C = A W^T with both operands K-major.
//
// A work unit is a 128 x BN tile of D = P Q^T over one range of K, where P ("the 128-row side") and Q ("the BN-row
// side") are [rows][K] bf16 tensors read by TMA (boxes of 64 K-elements, 128-byte swizzle, zero fill past the edges,
// no multicast) into a ring of shared-memory stages. CTAs are persistent: CTA c takes units c, c + gridDim.x, ...;
// a producer warp keeps the ring full across unit boundaries, one elected thread issues tcgen05.mma (M 128, N BN,
// K 16, fp32 accumulator in tensor memory), tcgen05.commit frees a stage when its MMAs are done, and four epilogue
// warps drain one of TWO accumulators with tcgen05.ld while the MMAs of the next unit fill the other.
//   - prefill form: P = activations (tokens), Q = weights (features): a TMEM lane is a token, a column a feature.
//   - decode form ("swap"): P = weights (128 features a tile), Q = the few activation rows (BN = 16..128 tokens):
//     the weights stream through the 128-row side at memory speed and the batch is the narrow side.
// K may be split: each split writes its own fp32 plane (no atomics: the consumer adds the planes in order, so
// results are the same on every run).
// The reference's counterparts are its int8 mma.sync prompt product (kindi/nbq_mm.cu:23-178) and its dp4a
// matrix-vector products (kindi/nbq.cu:266-296).
#include "sm100.cuh"

#define TC_BM 128
#define TC_BK 64
#ifndef TC_EARLY
#define TC_EARLY 1               // stages of weights requested before the programmatic wait (decode form)
#endif
#define TC_THREADS 192          // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2-5: epilogue

template <int BN, int STAGES, int MT = 1, bool SWAP = false>
struct TcSmem {
    static constexpr int A_BYTES = MT * TC_BM * TC_BK * 2;
    static constexpr int B_BYTES = BN * TC_BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    // prefill form: 4 KB per epilogue warp, where 32 rows of the accumulator are turned into whole 128-byte row pieces
    static constexpr int EPI_OFF = STAGES * STAGE_BYTES;
    static constexpr int EPI_BYTES = SWAP ? 0 : 4 * 4096;
    static constexpr int BAR_OFF = EPI_OFF + EPI_BYTES;
    static constexpr int N_BARS = 2 * STAGES + 4;
    static constexpr int TOTAL = BAR_OFF + N_BARS * 8 + 16 + 1024;     // + alignment slack
    static_assert(TOTAL <= 227 * 1024, "shared memory of a CTA");
};

// MT = 2 (prefill form only): a unit is TWO 128-row tiles of the same BN columns, so one weight tile in shared memory
// feeds two accumulators: less traffic from the L2 per FLOP, at the price of not overlapping the epilogue with the next
// unit (both accumulators are in use).
template <int BN, int STAGES, bool SWAP, typename TC, int MT = 1>
__global__ void __launch_bounds__(TC_THREADS) k_gemm_tc(const __grid_constant__ CUtensorMap mapP,
        const __grid_constant__ CUtensorMap mapQ, TC* __restrict__ C, int rowsP, int rowsQ, int K, int ldc,
        long long split_stride, int kb_per_split, int n_splits, int* status, int swiglu_ld) {
    using S = TcSmem<BN, STAGES, MT, SWAP>;
    static_assert(MT == 1 || (!SWAP && 2 * BN <= 512), "two row tiles: prefill form, both accumulators in tensor memory");
    extern __shared__ uint8_t smem_raw[];
    if (SWAP) kb_pdl_launch_now();               // decode steps only (see common.cuh)
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar_full = sbase + S::BAR_OFF, bar_empty = bar_full + STAGES * 8;
    const uint32_t bar_acc_full = bar_empty + STAGES * 8, bar_acc_empty = bar_acc_full + 16;
    volatile uint32_t* tmem_slot = (volatile uint32_t*)(smem + S::BAR_OFF + S::N_BARS * 8);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tilesP = (rowsP + MT * TC_BM - 1) / (MT * TC_BM), tilesQ = (rowsQ + BN - 1) / BN;
    const int n_units = tilesP * tilesQ * n_splits;
    const int total_kb = (K + TC_BK - 1) / TC_BK;
    // two accumulators: the second starts at half of the allocation (a power of two of at least 2 x BN columns)
    // (MT == 2: the two halves are the two row tiles' accumulators, and there is no second buffer)
    constexpr uint32_t TMEM_COLS = BN <= 16 ? 32 : BN <= 32 ? 64 : BN <= 64 ? 128 : BN <= 128 ? 256 : 512;
    constexpr uint32_t ACC_COLS = TMEM_COLS / 2;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(bar_full + s * 8, 1);
            mbar_init(bar_empty + s * 8, 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(bar_acc_full + a * 8, 1);
            mbar_init(bar_acc_empty + a * 8, 4);
        }
        mbar_fence_init();
        tma_prefetch_desc(&mapP);
        tma_prefetch_desc(&mapQ);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32((const void*)tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t n = 0;                                  // k-blocks loaded so far (ring position)
            bool ok = true;
            // In the decode form the 128-row side is the weights, which no kernel writes: the tiles of the first
            // TC_EARLY stages are requested BEFORE the wait on the preceding kernel, so the first MMAs can start as
            // soon as the activations are there. (Filling the whole ring early was measured slower: the loads of all
            // CTAs take the memory system from the small kernel that is still running.)
            constexpr int EARLY = SWAP ? TC_EARLY : 0;
            bool waited = EARLY == 0;
            int pend_kb[EARLY + 1], pend_tq[EARLY + 1], n_pend = 0;
            if (waited) kb_pdl_wait();
            for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
                const int tp = u % tilesP, rest = u / tilesP, tq = rest % tilesQ, sp = rest / tilesQ;
                const int kb0 = sp * kb_per_split, kb1 = min(total_kb, kb0 + kb_per_split);
                for (int kb = kb0; kb < kb1; kb++, n++) {
                    const int s = n % STAGES;
                    const uint32_t ph = (n / STAGES) & 1u;
                    if (!waited && n_pend == EARLY) {
                        kb_pdl_wait();
                        waited = true;
                        for (int j = 0; j < n_pend; j++)
                            tma_load_2d(sbase + j * S::STAGE_BYTES + S::A_BYTES, &mapQ, pend_kb[j] * TC_BK,
                                        pend_tq[j] * BN, bar_full + j * 8);
                    }
                    if (!(ok = mbar_wait(bar_empty + s * 8, ph ^ 1u, status))) break;
                    mbar_expect_tx(bar_full + s * 8, S::STAGE_BYTES);
                    const uint32_t dst = sbase + s * S::STAGE_BYTES;
#pragma unroll
                    for (int m = 0; m < MT; m++)
                        tma_load_2d(dst + m * (TC_BM * TC_BK * 2), &mapP, kb * TC_BK, (tp * MT + m) * TC_BM,
                                    bar_full + s * 8);
                    if (waited) {
                        tma_load_2d(dst + S::A_BYTES, &mapQ, kb * TC_BK, tq * BN, bar_full + s * 8);
                    } else {
                        pend_kb[n_pend] = kb;                // stage n_pend == s here: the ring has not wrapped yet
                        pend_tq[n_pend] = tq;
                        n_pend++;
                    }
                }
            }
            if (!waited) {
                kb_pdl_wait();
                for (int j = 0; j < n_pend; j++)
                    tma_load_2d(sbase + j * S::STAGE_BYTES + S::A_BYTES, &mapQ, pend_kb[j] * TC_BK, pend_tq[j] * BN,
                                bar_full + j * 8);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(TC_BM, BN);
            uint32_t n = 0, it = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x, it++) {
                const int sp = (u / tilesP) / tilesQ;
                const int kb0 = sp * kb_per_split, kb1 = min(total_kb, kb0 + kb_per_split);
                const uint32_t acc = MT == 2 ? 0u : (it & 1u);
                const uint32_t acc_ph = MT == 2 ? (it & 1u) : ((it >> 1) & 1u);
                if (!(ok = mbar_wait(bar_acc_empty + acc * 8, acc_ph ^ 1u, status))) break;
                tc_fence_after();
                const uint32_t d = tmem + acc * ACC_COLS;
                for (int kb = kb0; kb < kb1; kb++, n++) {
                    const int s = n % STAGES;
                    const uint32_t ph = (n / STAGES) & 1u;
                    if (!(ok = mbar_wait(bar_full + s * 8, ph, status))) break;
                    tc_fence_after();
                    const uint32_t a = sbase + s * S::STAGE_BYTES, b = a + S::A_BYTES;
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; k++)
#pragma unroll
                        for (int m = 0; m < MT; m++)
                            umma_bf16(d + m * ACC_COLS, umma_desc_sw128(a + m * (TC_BM * TC_BK * 2) + k * 32),
                                      umma_desc_sw128(b + k * 32), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                    umma_commit(bar_empty + s * 8);
                }
                umma_commit(bar_acc_full + acc * 8);
            }
        }
    } else {
        // epilogue warps 2..5 own TMEM lanes 32 * (warp % 4) .. + 31
        const int quarter = warp & 3;
        uint32_t it = 0;
        bool ok = true;
        kb_pdl_wait();                                   // C may be memory that an earlier kernel still reads
        for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x, it++) {
            const int tp = u % tilesP, rest = u / tilesP, tq = rest % tilesQ, sp = rest / tilesQ;
            const int q0 = tq * BN;
            const uint32_t acc = MT == 2 ? 0u : (it & 1u);
            const uint32_t acc_ph = MT == 2 ? (it & 1u) : ((it >> 1) & 1u);
            if (!(ok = mbar_wait(bar_acc_full + acc * 8, acc_ph, status))) break;
            tc_fence_after();
            TC* Cz = C + (size_t)sp * split_stride;
#pragma unroll 1
            for (int mt = 0; mt < MT; mt++) {
            const int p0 = (tp * MT + mt) * TC_BM;
            const int prow = p0 + quarter * 32 + lane;           // row of the 128-row side this thread holds
            const uint32_t tbase = tmem + (acc + mt) * ACC_COLS + ((uint32_t)(quarter * 32) << 16);
            if (!SWAP && BN % 32 == 0 && swiglu_ld > 0) {
                // the weights' rows come in groups of 16 gate rows followed by the 16 up rows of the same outputs, so
                // every 32 columns of a tile hold both halves of 16 outputs: out[token][j] = silu(gate) * up goes out
                // as bf16 and the 2F-wide product is never written
                // (every lane of the warp takes part in the warp-wide TMEM loads; only the stores depend on the row)
                bf16* orow = (bf16*)C + (size_t)prow * swiglu_ld;
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    if (q0 + c0 >= rowsQ) continue;                   // past the end (uniform over the warp)
                    uint32_t gu[32];
                    tmem_ld_32x32(tbase + c0, gu);
                    tmem_ld_wait();
                    if (prow < rowsP) {
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
            } else if (!SWAP) {
                // C[token][feature]: a thread holds one row of the accumulator. The warp's 32 rows x 128 bytes go through
                // its staging area (16-byte pieces, swizzled by the row so that neither side meets bank conflicts) and
                // leave as whole 128-byte pieces of four rows per store instruction.
                constexpr int CW = 128 / (int)sizeof(TC);            // columns per pass: 32 (float) or 64 (bf16)
                constexpr int PW = 16 / (int)sizeof(TC);             // columns per 16-byte piece
                uint8_t* stg = smem + S::EPI_OFF + quarter * 4096;
                const bool vec_ok = (((uintptr_t)Cz) & 15) == 0 && (ldc % PW) == 0;
                const int myrow = lane;
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += CW) {
                    uint32_t r[32];
                    tmem_ld_32x32(tbase + c0, r);
                    tmem_ld_wait();
                    if (sizeof(TC) == 4) {
#pragma unroll
                        for (int j = 0; j < 8; j++)
                            *(uint4*)(stg + myrow * 128 + ((j ^ (myrow & 7)) << 4)) =
                                make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                    } else {
#pragma unroll
                        for (int half = 0; half < 2; half++) {
                            if (half == 1) {
                                tmem_ld_32x32(tbase + c0 + 32, r);       // (columns past the accumulator are never stored)
                                tmem_ld_wait();
                            }
#pragma unroll
                            for (int j = 0; j < 4; j++) {
                                uint32_t h[4];
#pragma unroll
                                for (int c = 0; c < 4; c++) {
                                    __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[8 * j + 2 * c]),
                                                                             __uint_as_float(r[8 * j + 2 * c + 1]));
                                    h[c] = *(uint32_t*)&v;
                                }
                                *(uint4*)(stg + myrow * 128 + (((half * 4 + j) ^ (myrow & 7)) << 4)) =
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
                        if (grow < rowsP && ct < BN && gcol < rowsQ) {
                            TC* dst = Cz + (size_t)grow * ldc + gcol;
                            if (vec_ok && gcol + PW <= rowsQ) {
                                *(uint4*)dst = v;
                            } else {
                                const TC* e = (const TC*)&v;
#pragma unroll
                                for (int c = 0; c < PW; c++)
                                    if (gcol + c < rowsQ) dst[c] = e[c];
                            }
                        }
                    }
                    __syncwarp();
                }
            } else
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                // C[token q0 + c][feature prow]: a warp's 32 lanes write 32 consecutive features
                uint32_t r[16];
                tmem_ld_32x16(tbase + c0, r);
                tmem_ld_wait();
                if (prow < rowsP) {
#pragma unroll
                    for (int c = 0; c < 16; c++)
                        if (q0 + c0 + c < rowsQ)
                            Cz[(size_t)(q0 + c0 + c) * ldc + prow] = kb_from_f<TC>(__uint_as_float(r[c]));
                }
            }
            }
            // this warp has read its lanes of the accumulator(s): hand them back to the MMA thread
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_acc_empty + acc * 8);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

static int kb_sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

template <int BN, int STAGES, bool SWAP, typename TC, int MT = 1>
static int launch_tc(const CUtensorMap& mp, const CUtensorMap& mq, void* C, int rowsP, int rowsQ, int K, int ldc,
                     int splits, long long split_stride, int* status, cudaStream_t st, int swiglu_ld) {
    using S = TcSmem<BN, STAGES, MT, SWAP>;
    auto kern = k_gemm_tc<BN, STAGES, SWAP, TC, MT>;
    static char once_tag;               // one per instantiation: the opt-in is per (device, kernel)
    if (kb_first_use(&once_tag)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
        if (e != cudaSuccess) return (int)e;
    }
    const int total_kb = (K + TC_BK - 1) / TC_BK;
    int kbps = (total_kb + splits - 1) / splits;
    int z = (total_kb + kbps - 1) / kbps;               // every split has at least one k-block
    const int units = ((rowsP + MT * TC_BM - 1) / (MT * TC_BM)) * ((rowsQ + BN - 1) / BN) * z;
    const int grid = units < kb_sm_count() ? units : kb_sm_count();
    if (swiglu_ld > 0 && (SWAP || BN % 32 || sizeof(TC) != 2 || z != 1)) return (int)cudaErrorInvalidValue;
    kb_launch(kern, grid, TC_THREADS, S::TOTAL, st, mp, mq, (TC*)C, rowsP, rowsQ, K, ldc, split_stride, kbps, z, status,
              swiglu_ld);
    return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------------
// Gate/up product of a decode step with SwiGLU finished inside the product: H[M][F] = silu(g) * u, bf16.
//
// The decode form again (weights on the 128-row side, 16 gate rows then the 16 up rows of the same outputs, so a
// quarter of a tile's rows = one epilogue warp's lanes holds both halves of 16 outputs), but the work is cut
// differently: all (tile, K block) pairs are laid out in one line, tile after tile, and CTA c takes the c-th stretch of
// it. A stretch is at least one tile long, so a tile is shared by at most two CTAs: the one that holds its first K
// blocks at the END of its stretch (its owner) and the next CTA, which holds the rest at the START of its own
// stretch. The second writes its 32-bit partial tile and raises the tile's flag as the first thing it does; the owner
// meets the flag long set when it comes to the tile, adds the partial in a fixed order (own + other), applies
// SwiGLU and lowers the flag. No split-K planes are written or read again, no SwiGLU kernel follows, and every CTA
// streams the same number of K blocks. The owner's wait is bounded like every wait here.
template <int BN, int STAGES>
__global__ void __launch_bounds__(TC_THREADS) k_gemm_sk_swiglu(const __grid_constant__ CUtensorMap mapP,
        const __grid_constant__ CUtensorMap mapQ, bf16* __restrict__ H, int rowsP, int M, int K, int F, int ldh,
        float* part, int* flags, int* status) {      // (shared with other CTAs of this launch: no __restrict__)
    using S = TcSmem<BN, STAGES, 1, true>;
    extern __shared__ uint8_t smem_raw[];
    kb_pdl_launch_now();
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar_full = sbase + S::BAR_OFF, bar_empty = bar_full + STAGES * 8;
    const uint32_t bar_acc_full = bar_empty + STAGES * 8, bar_acc_empty = bar_acc_full + 16;
    volatile uint32_t* tmem_slot = (volatile uint32_t*)(smem + S::BAR_OFF + S::N_BARS * 8);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tilesP = (rowsP + TC_BM - 1) / TC_BM;
    const int KB = (K + TC_BK - 1) / TC_BK;
    const int total = tilesP * KB;                                       // (the launcher refuses sizes beyond an int)
    const int W = (total + (int)gridDim.x - 1) / (int)gridDim.x;         // >= KB because gridDim.x <= tilesP
    const int L0 = min(total, (int)blockIdx.x * W), L1 = min(total, L0 + W);
    constexpr uint32_t TMEM_COLS = BN <= 16 ? 32 : BN <= 32 ? 64 : BN <= 64 ? 128 : 256;
    constexpr uint32_t ACC_COLS = TMEM_COLS / 2;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(bar_full + s * 8, 1);
            mbar_init(bar_empty + s * 8, 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(bar_acc_full + a * 8, 1);
            mbar_init(bar_acc_empty + a * 8, 4);
        }
        mbar_fence_init();
        tma_prefetch_desc(&mapP);
        tma_prefetch_desc(&mapQ);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32((const void*)tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0 && L0 < L1) {
            // the first stage's weights are requested before the wait on the preceding kernel (see k_gemm_tc)
            bool ok = true;
            int tile = L0 / KB, kb = L0 % KB;
            mbar_expect_tx(bar_full, S::STAGE_BYTES);
            tma_load_2d(sbase, &mapP, kb * TC_BK, tile * TC_BM, bar_full);
            kb_pdl_wait();
            tma_load_2d(sbase + S::A_BYTES, &mapQ, kb * TC_BK, 0, bar_full);
            uint32_t n = 1;
            for (int L = L0 + 1; L < L1 && ok; L++, n++) {
                if (++kb == KB) {
                    kb = 0;
                    tile++;
                }
                const int s = n % STAGES;
                if (!(ok = mbar_wait(bar_empty + s * 8, ((n / STAGES) & 1u) ^ 1u, status))) break;
                mbar_expect_tx(bar_full + s * 8, S::STAGE_BYTES);
                const uint32_t dst = sbase + s * S::STAGE_BYTES;
                tma_load_2d(dst, &mapP, kb * TC_BK, tile * TC_BM, bar_full + s * 8);
                tma_load_2d(dst + S::A_BYTES, &mapQ, kb * TC_BK, 0, bar_full + s * 8);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(TC_BM, BN);
            uint32_t n = 0, seg = 0;
            bool ok = true;
            int kb = L0 % KB - 1;
            for (int L = L0; L < L1 && ok; L++, n++) {
                if (++kb == KB) kb = 0;
                const bool first = L == L0 || kb == 0, last = L == L1 - 1 || kb == KB - 1;
                const uint32_t acc = seg & 1u;
                if (first) {
                    if (!(ok = mbar_wait(bar_acc_empty + acc * 8, ((seg >> 1) & 1u) ^ 1u, status))) break;
                    tc_fence_after();
                }
                const int s = n % STAGES;
                if (!(ok = mbar_wait(bar_full + s * 8, (n / STAGES) & 1u, status))) break;
                tc_fence_after();
                const uint32_t a = sbase + s * S::STAGE_BYTES, b = a + S::A_BYTES;
#pragma unroll
                for (int k = 0; k < TC_BK / 16; k++)
                    umma_bf16(tmem + acc * ACC_COLS, umma_desc_sw128(a + k * 32), umma_desc_sw128(b + k * 32), idesc,
                              (!first || k > 0) ? 1u : 0u);
                umma_commit(bar_empty + s * 8);
                if (last) {
                    umma_commit(bar_acc_full + acc * 8);
                    seg++;
                }
            }
        }
    } else {
        // epilogue warps 2..5 own TMEM lanes 32 * (warp % 4) .. + 31 = one group of 16 gate + 16 up rows of a tile
        const int quarter = warp & 3;
        const bool leader = threadIdx.x == 64;                       // one thread of the four warps talks to the flags
        uint32_t seg = 0;
        bool ok = true;
        kb_pdl_wait();
        for (int L = L0; L < L1 && ok; seg++) {
            const int tile = L / KB, kb0 = L % KB;
            const int Lend = min(L1, L + (KB - kb0));          // one past the stretch's last K block of this tile
            const bool helper = kb0 > 0;                             // the tile's first K blocks belong to the CTA before
            const bool shared_owner = !helper && Lend - L < KB;
            L = Lend;
            const uint32_t acc = seg & 1u;
            float* ptile = part + (size_t)tile * BN * TC_BM + quarter * 32 + lane;     // + token * 128
            float other[BN];                      // the other CTA's partial sums of this thread's row (shared tiles)
            if (shared_owner) {
                // The other part was written when the next CTA began, long ago: fetch it now, while this CTA's own K
                // blocks of the tile are still being multiplied, and lower the flag for the next call.
                if (leader) {
                    const uint64_t t0 = kb_globaltimer();
                    while (*((volatile int*)(flags + tile)) == 0) {
                        if (kb_globaltimer() - t0 > KB_WAIT_NS) {
                            atomicOr(status, KB_ST_WAIT_TIMEOUT);
                            break;
                        }
                    }
                    __threadfence();
                }
                asm volatile("bar.sync 2, 128;" ::: "memory");
#pragma unroll
                for (int c = 0; c < BN; c++) other[c] = c < M ? __ldcg(ptile + (size_t)c * TC_BM) : 0.0f;
                // (every thread's loads above have returned before it passes this barrier: their values are used below
                // only after it, and the compiler keeps the loads before the barrier's memory clobber)
                asm volatile("bar.sync 2, 128;" ::: "memory");
                if (leader) atomicExch(flags + tile, 0);
            }
            ok = mbar_wait(bar_acc_full + acc * 8, (seg >> 1) & 1u, status);
            {
                // the four warps go on together or not at all (they meet at barriers, which have no time limit)
                uint32_t any_bad;
                asm volatile(
                    "{\n .reg .pred p, q;\n setp.ne.u32 p, %1, 0;\n bar.red.or.pred q, 2, 128, p;\n selp.u32 %0, 1, 0, q;\n}"
                    : "=r"(any_bad)
                    : "r"(ok ? 0u : 1u)
                    : "memory");
                if (any_bad) {
                    ok = false;
                    break;
                }
            }
            tc_fence_after();
            const uint32_t tbase = tmem + acc * ACC_COLS + ((uint32_t)(quarter * 32) << 16);
            const int feat = tile * 64 + quarter * 16 + (lane & 15);
#pragma unroll
            for (int c0 = 0; c0 < BN; c0 += 16) {
                uint32_t r[16];
                tmem_ld_32x16(tbase + c0, r);
                tmem_ld_wait();
                if (helper) {
#pragma unroll
                    for (int c = 0; c < 16; c++)
                        if (c0 + c < M) ptile[(size_t)(c0 + c) * TC_BM] = __uint_as_float(r[c]);
                    continue;
                }
#pragma unroll
                for (int c = 0; c < 16; c++) {
                    float v = __uint_as_float(r[c]);
                    if (shared_owner) v += other[c0 + c];
                    const float u = __shfl_xor_sync(0xffffffffu, v, 16);          // lanes 0..15: gate; their partners: up
                    if (lane < 16 && c0 + c < M && feat < F)
                        H[(size_t)(c0 + c) * ldh + feat] = __float2bfloat16_rn(__fdividef(v, 1.0f + __expf(-v)) * u);
                }
            }
            if (helper) {
                __threadfence();
                asm volatile("bar.sync 2, 128;" ::: "memory");
                if (leader) atomicExch(flags + tile, 1);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_acc_empty + acc * 8);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

template <int BN, int STAGES>
static int launch_sk_swiglu(const CUtensorMap& mp, const CUtensorMap& mq, void* H, int rowsP, int M, int K, int F,
                            int ldh, float* part, int* flags, int* status, cudaStream_t st) {
    using S = TcSmem<BN, STAGES, 1, true>;
    auto kern = k_gemm_sk_swiglu<BN, STAGES>;
    static char once_tag;               // one per instantiation: the opt-in is per (device, kernel)
    if (kb_first_use(&once_tag)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
        if (e != cudaSuccess) return (int)e;
    }
    const int tilesP = (rowsP + TC_BM - 1) / TC_BM;
    const int grid = tilesP < kb_sm_count() ? tilesP : kb_sm_count();
    kb_launch(kern, grid, TC_THREADS, S::TOTAL, st, mp, mq, (bf16*)H, rowsP, M, K, F, ldh, part, flags, status);
    return (int)cudaGetLastError();
}

// H[M][F] (bf16, row stride ldh) = silu(g) * u with [g | u] = A[M][K] W[2F][K]^T, W in groups of 16 gate rows and the 16
// up rows of the same outputs; M <= bn in {16, 32, 64, 128}. `part` ([ceil(2F / 128)][bn][128] floats) and `flags`
// ([ceil(2F / 128)] ints, zero before the first call and left zero by every call that ends without an error) are the
// caller's; calls that share them must be ordered on one stream.
extern "C" int kb_gemm_swiglu_decode(const void* A, const void* W, void* H, int M, int F, int K, int lda, int ldw, int ldh,
                                     int bn, float* part, int* flags, int* status, cudaStream_t st) {
    if (M <= 0 || F <= 0 || K <= 0) return 0;
    if ((K % 8) || (lda % 8) || (ldw % 8) || (F % 16) || M > bn || !part || !flags) return (int)cudaErrorInvalidValue;
    if ((long long)((2 * (long long)F + TC_BM - 1) / TC_BM) * ((K + TC_BK - 1) / TC_BK) > 0x3fffffffLL)
        return (int)cudaErrorInvalidValue;
    CUtensorMap mp, mq;
    int rc;
    if ((rc = kb_make_map_bf16(&mp, W, 2 * F, K, ldw, TC_BM))) return rc;
    if ((rc = kb_make_map_bf16(&mq, A, M, K, lda, bn))) return rc;
    switch (bn) {
        case 16: return launch_sk_swiglu<16, 8>(mp, mq, H, 2 * F, M, K, F, ldh, part, flags, status, st);
        case 32: return launch_sk_swiglu<32, 8>(mp, mq, H, 2 * F, M, K, F, ldh, part, flags, status, st);
        case 64: return launch_sk_swiglu<64, 8>(mp, mq, H, 2 * F, M, K, F, ldh, part, flags, status, st);
        case 128: return launch_sk_swiglu<128, 5>(mp, mq, H, 2 * F, M, K, F, ldh, part, flags, status, st);
        default: return (int)cudaErrorInvalidValue;
    }
}

// how many K splits the launch will use for a wanted number (the caller sizes the partial planes with it)
extern "C" int kb_gemm_tc_splits(int K, int wanted) {
    const int total_kb = (K + TC_BK - 1) / TC_BK;
    if (wanted < 1) wanted = 1;
    if (wanted > total_kb) wanted = total_kb;
    int kbps = (total_kb + wanted - 1) / wanted;
    return (total_kb + kbps - 1) / kbps;
}

// C[M][N] (+ split planes) = A[M][K] W[N][K]^T. cdtype: KB_F32 or KB_BF16 (bf16 only without splits).
// swap = 0: prefill form (tile 128 tokens x bn features); swap = 1: decode form (tile 128 features x bn tokens).
// swiglu != 0 (prefill form, bn a multiple of 32, bf16 out): W holds gate and up rows in groups of 16 + 16 and C is
// the bf16 [M][N / 2] result silu(gate) * up with row stride ldc.
extern "C" int kb_gemm_tc(const void* A, const void* W, void* C, int cdtype, int M, int N, int K, int lda, int ldw,
                          int ldc, int swap, int bn, int splits, long long split_stride, int* status,
                          cudaStream_t st, int swiglu = 0, int mt = 1) {
    if (mt != 1 && (mt != 2 || swap || splits != 1)) return (int)cudaErrorInvalidValue;
    if (swiglu && (swap || (N % 32) || cdtype != KB_BF16 || splits != 1 || (ldc % 8) || ((uintptr_t)C & 15)))
        return (int)cudaErrorInvalidValue;
    const int swiglu_ld = swiglu ? ldc : 0;
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if ((K % 8) || (lda % 8) || (ldw % 8)) return (int)cudaErrorInvalidValue;
    if (splits > 1 && cdtype != KB_F32) return (int)cudaErrorInvalidValue;
    CUtensorMap mp, mq;
    int rc;
    const void* P = swap ? W : A;
    const void* Q = swap ? A : W;
    const int rowsP = swap ? N : M, rowsQ = swap ? M : N;
    const int ldp = swap ? ldw : lda, ldq = swap ? lda : ldw;
    if ((rc = kb_make_map_bf16(&mp, P, rowsP, K, ldp, TC_BM))) return rc;
    if ((rc = kb_make_map_bf16(&mq, Q, rowsQ, K, ldq, bn))) return rc;
#define TC_GO(BN, ST, SW)                                                                                         \
    return cdtype == KB_F32                                                                                       \
               ? launch_tc<BN, ST, SW, float>(mp, mq, C, rowsP, rowsQ, K, ldc, splits, split_stride, status, st, swiglu_ld)  \
               : launch_tc<BN, ST, SW, bf16>(mp, mq, C, rowsP, rowsQ, K, ldc, splits, split_stride, status, st, swiglu_ld)
    if (swap) {
        switch (bn) {
            case 16: TC_GO(16, 8, true);
            case 32: TC_GO(32, 8, true);
            case 64: TC_GO(64, 8, true);
            case 128: TC_GO(128, 5, true);
            default: return (int)cudaErrorInvalidValue;
        }
    } else if (mt == 2) {
#define TC_GO2(BN, ST)                                                                                               \
    return cdtype == KB_F32                                                                                          \
               ? launch_tc<BN, ST, false, float, 2>(mp, mq, C, rowsP, rowsQ, K, ldc, splits, split_stride, status, st, swiglu_ld) \
               : launch_tc<BN, ST, false, bf16, 2>(mp, mq, C, rowsP, rowsQ, K, ldc, splits, split_stride, status, st, swiglu_ld)
        switch (bn) {
            case 128: TC_GO2(128, 4);
            case 144: TC_GO2(144, 4);
            case 160: TC_GO2(160, 4);
            case 176: TC_GO2(176, 3);
            case 192: TC_GO2(192, 3);
            case 208: TC_GO2(208, 3);
            case 224: TC_GO2(224, 3);
            case 240: TC_GO2(240, 3);
            case 256: TC_GO2(256, 3);
            default: return (int)cudaErrorInvalidValue;
        }
#undef TC_GO2
    } else {
        switch (bn) {
            case 64: TC_GO(64, 6, false);
            case 128: TC_GO(128, 6, false);
            case 144: TC_GO(144, 6, false);
            case 160: TC_GO(160, 5, false);
            case 176: TC_GO(176, 5, false);
            case 192: TC_GO(192, 5, false);
            case 208: TC_GO(208, 4, false);
            case 224: TC_GO(224, 4, false);
            case 240: TC_GO(240, 4, false);
            case 256: TC_GO(256, 4, false);
            default: return (int)cudaErrorInvalidValue;
        }
    }
#undef TC_GO
}

// ------------------------------------------------------------------------------------------------ self-test of the bounded wait
// One CTA waits on a barrier that nothing arrives at, with the given limit. The wait must give up after the limit, set
// KB_ST_WAIT_TIMEOUT and return, so that the kernel ends by itself and the context stays usable: the behaviour every
// kernel of the library relies on when an arrival is lost. out[0] = 1 when the wait reported a time-out (0: it claimed
// the phase had completed), out[1] = nanoseconds spent in it.
__global__ void k_wait_selftest(unsigned long long limit_ns, long long* out, int* status) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        mbar_fence_init();
        const uint64_t t0 = kb_globaltimer();
        const bool ok = mbar_wait_ns(smem_u32(&bar), 0, status, limit_ns);
        out[0] = ok ? 0 : 1;
        out[1] = (long long)(kb_globaltimer() - t0);
    }
}

extern "C" int kb_wait_selftest(unsigned long long limit_ns, long long* out, int* status, cudaStream_t st) {
    if (limit_ns > 100000000ull) limit_ns = 100000000ull;           // a tenth of a second at most
    k_wait_selftest<<<1, 32, 0, st>>>(limit_ns, out, status);
    KB_LAUNCH_RET();
}
