// Prefill attention on the 5th-generation tensor cores: S = Q K^T and O += P V are tcgen05.mma instructions with their
// accumulators in tensor memory; softmax runs in 32-bit on the CUDA cores between them.
//
// One CTA serves one key/value head of one sequence and up to 128 rows r = token * G + j (token of this step, query
// head j of the group: the reference packs rows the same way, kindi/nbq_fa.cu:3-5,40-49), TOK = 128 / G whole tokens.
// Warps 0-3 (one thread per row) do the softmax, warp 4 brings pages of 64 positions in by TMA (two 64-column tile
// loads per 128-wide head for K and for V, 128-byte swizzle, no multicast), one thread of warp 5 issues the MMAs:
//     S[j % 2] = Q K_j^T      M 128 x N 64 x K 128: Q and K both K-major in shared memory
//     O       += P_j V_j      M 128 x N 128 x K 64: P from TENSOR memory (the A operand), V as stored in the cache,
//                              i.e. MN-major, from shared memory
// S has two buffers in tensor memory so that Q K^T of the next page runs while the softmax of this one does. A softmax
// thread reads its row of S, and writes the row's probabilities back as bf16 pairs over the first 32 columns of the
// same buffer, from where P V reads them: P never passes through shared memory. The tensor pipe runs the products in
// the order of their issue (S_{j+1}, P V_j, S_{j+2}, ...), which is all the ordering the two buffers need.
// Key and value tiles of a stage are freed separately (keys as soon as Q K^T of the page is done). A CTA needs 96 KB
// of shared memory and 256 columns of tensor memory, so two CTAs share an SM and one's softmax hides the other's
// waits. The running maximum is applied lazily: the exponent's reference only moves (and O in tensor
// memory is only rescaled, by tcgen05.ld / tcgen05.st) when a row's maximum has grown by more than 8 (a factor 256 in
// the probabilities, which bf16 and the 32-bit sums hold without loss); the final division by the row sum makes the
// result the same as with an exact running maximum (kindi/nbq_fa.cu:31-151 is the recurrence this follows).
// Head sizes 64 and 128. Every wait is bounded (sm100.cuh); all tcgen05 loads and stores are executed by whole warps.
#include "sm100.cuh"

#define FT_THREADS 192
#define FT_STAGES 2
// per head size HD (64 or 128): a page of keys (or values) of one head is 64 * HD * 2 bytes, a stage holds one of
// each, Q is HD / 64 blocks of [128 rows][64 columns]
#define FT_LAZY 8.0f

__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t* r) { tmem_ld_32x32(taddr, r); }
__device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ float ft_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// two 32-bit floats in one 64-bit register and the packed arithmetic of sm_100 on them; a maximum of three
__device__ __forceinline__ uint64_t ft_pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void ft_unpack2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t ft_fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t ft_add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float ft_max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// shared-memory descriptor of an MN-major operand tile stored as rows of 128 bytes (64 elements of the MN dimension per
// row, one row per K index), 128-byte swizzle: leading byte offset = distance to the next block of 64 MN elements,
// stride byte offset = distance between groups of 8 K rows (1024)
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

template <int FT_HD>
__global__ void __launch_bounds__(FT_THREADS, 2) k_attn_tc(const __grid_constant__ CUtensorMap kvmap,
        const bf16* KB_STEP_DATA q, int ldq, bf16* __restrict__ out, int ldo, const int* __restrict__ slot,
        const int* __restrict__ q_start, const int* __restrict__ kv_len, int nkv, int G, float scale_log2e, int window,
        const int* __restrict__ table, int table_stride, int n_pages, int* status) {
    constexpr int FT_TILE_BYTES = 64 * FT_HD * 2, FT_STAGE_BYTES = 2 * FT_TILE_BYTES, FT_Q_BYTES = 128 * FT_HD * 2;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t s_q = sbase, s_kv = s_q + FT_Q_BYTES;
    const uint32_t bars = s_kv + FT_STAGES * FT_STAGE_BYTES;
    // keys and values of a stage have barriers of their own: a stage's key tile is free as soon as Q K^T of its page
    // is done, long before P V of that page frees the value tile, so the next keys are on their way a page earlier
    const uint32_t b_k_full = bars, b_k_empty = b_k_full + FT_STAGES * 8, b_v_full = b_k_empty + FT_STAGES * 8;
    const uint32_t b_v_empty = b_v_full + FT_STAGES * 8, b_s_full = b_v_empty + FT_STAGES * 8;
    const uint32_t b_p_ready = b_s_full + 16, b_pv_done = b_p_ready + 8;
    volatile uint32_t* tmem_slot = (volatile uint32_t*)(smem + FT_Q_BYTES + FT_STAGES * FT_STAGE_BYTES +
                                                        (4 * FT_STAGES + 4) * 8);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // grid: (key/value heads, tiles, sequences): the longest tiles of every head start first, the shortest fill the end
    const int b = blockIdx.z, hk = blockIdx.x;

    if (threadIdx.x == 0) {
        for (int s = 0; s < FT_STAGES; s++) {
            mbar_init(b_k_full + s * 8, 1);
            mbar_init(b_k_empty + s * 8, 1);
            mbar_init(b_v_full + s * 8, 1);
            mbar_init(b_v_empty + s * 8, 1);
        }
        for (int i = 0; i < 2; i++) mbar_init(b_s_full + i * 8, 1);
        mbar_init(b_p_ready, 4);
        mbar_init(b_pv_done, 1);
        mbar_fence_init();
        tma_prefetch_desc(&kvmap);
    }
    if (warp == 5) {
        tmem_alloc(smem_u32((const void*)tmem_slot), 256);
        tmem_relinquish();
    }
    kb_pdl_wait();                       // the step's metadata, Q and the newest keys come from earlier kernels
    const int qs0 = q_start[b], qlen = q_start[b + 1] - qs0, kvl = kv_len[b];
    const int pos0 = kvl - qlen;
    const int TOK = 128 / G;                         // whole tokens per CTA
    const int n_tiles = (qlen + TOK - 1) / TOK;
    const bool active = (int)blockIdx.y < n_tiles;   // uniform over the CTA
    const int tile = n_tiles - 1 - (int)blockIdx.y;  // the longest tiles first
    const int tok0 = tile * TOK;
    const int ntok = active ? min(TOK, qlen - tok0) : 0;
    const int nrows = ntok * G;
    // pages this CTA reads
    const int p_first = pos0 + tok0, p_last = pos0 + tok0 + ntok - 1;
    const int lo_cta = (window > 0 && p_first - window + 1 > 0) ? p_first - window + 1 : 0;
    const int pg_lo = lo_cta / KB_PAGE, pg_hi = p_last / KB_PAGE;
    const int n_iter = active ? pg_hi - pg_lo + 1 : 0;

    tc_fence_before();
    __syncthreads();                                 // the barriers and the tensor memory's address are there
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t t_s = tmem, t_o = tmem + 128;     // S buffers at columns 0 and 64, O at 128..255

    // ---- Q into shared memory: two K-blocks of [128 rows][64 columns], rows of 128 bytes, 128-byte swizzle. The five
    // warps that do not load keys and values bring it, every load in flight before the first store (one trip to the
    // L2 instead of one a piece), while the producer warp already fetches the first pages.
    if (warp != 4) {
        if (active) {
            constexpr int QT = FT_THREADS - 32, QV = 128 * (FT_HD / 8), QN = (QV + QT - 1) / QT;
            const int qt = warp < 4 ? (int)threadIdx.x : (int)threadIdx.x - 32;
            uint4 v[QN];
#pragma unroll
            for (int i = 0; i < QN; i++) {
                const int e = qt + i * QT, r = e / (FT_HD / 8), c = e % (FT_HD / 8);
                v[i] = make_uint4(0, 0, 0, 0);
                if (e < QV && r < nrows)
                    v[i] = *(const uint4*)(q + (size_t)(qs0 + tok0 + r / G) * ldq + (size_t)(hk * G + r % G) * FT_HD + c * 8);
            }
#pragma unroll
            for (int i = 0; i < QN; i++) {
                const int e = qt + i * QT, r = e / (FT_HD / 8), c = e % (FT_HD / 8);
                if (e < QV) *(uint4*)(smem + (c >> 3) * 16384 + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = v[i];
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        asm volatile("bar.sync 1, %0;" ::"n"(FT_THREADS - 32) : "memory");
    }

    if (warp == 4) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0 && n_iter > 0) {
            const int* trow = table + (size_t)slot[b] * table_stride;
            // two streams, keys and values, each held back only by its own tiles; one thread polls both
            auto page_of = [&](int i) {
                int page = trow[pg_lo + i];
                if (page < 0 || page >= n_pages) {
                    atomicOr(status, KB_ST_BAD_PAGE);
                    page = 0;
                }
                return page;
            };
            int ik = 0, iv = 0, spins = 0;
            uint64_t t0 = kb_globaltimer();
            while (iv < n_iter) {
                bool moved = false;
                if (ik < n_iter) {
                    const int s = ik % FT_STAGES;
                    if (mbar_poll(b_k_empty + s * 8, ((uint32_t)(ik / FT_STAGES) & 1u) ^ 1u)) {
                        const int krow = ((page_of(ik) * 2 + 0) * nkv + hk) * KB_PAGE;
                        const uint32_t dst = s_kv + s * FT_STAGE_BYTES;
                        mbar_expect_tx(b_k_full + s * 8, FT_TILE_BYTES);
#pragma unroll
                        for (int h = 0; h < FT_HD / 64; h++)
                            tma_load_2d(dst + h * 8192, &kvmap, h * 64, krow, b_k_full + s * 8);
                        ik++;
                        moved = true;
                    }
                }
                if (iv < ik) {
                    const int s = iv % FT_STAGES;
                    if (mbar_poll(b_v_empty + s * 8, ((uint32_t)(iv / FT_STAGES) & 1u) ^ 1u)) {
                        const int vrow = ((page_of(iv) * 2 + 1) * nkv + hk) * KB_PAGE;
                        const uint32_t dst = s_kv + s * FT_STAGE_BYTES + FT_TILE_BYTES;
                        mbar_expect_tx(b_v_full + s * 8, FT_TILE_BYTES);
#pragma unroll
                        for (int h = 0; h < FT_HD / 64; h++)
                            tma_load_2d(dst + h * 8192, &kvmap, h * 64, vrow, b_v_full + s * 8);
                        iv++;
                        moved = true;
                    }
                }
                if (moved) {
                    spins = 0;
                    continue;
                }
                __nanosleep(100);                    // an idle poller would take issue slots from the softmax warp beside it
                if (++spins >= 256) {
                    // nothing moved for a while: look at the clock (the limit of every wait of this library)
                    if (spins == 256) t0 = kb_globaltimer();
                    else if ((spins & 255) == 0 && kb_globaltimer() - t0 > KB_WAIT_NS) {
                        atomicOr(status, KB_ST_WAIT_TIMEOUT);
                        break;
                    }
                }
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0 && n_iter > 0) {
            constexpr uint32_t idesc_s = umma_idesc_bf16(128, 64);                  // Q K^T: both K-major
            constexpr uint32_t idesc_o = umma_idesc_bf16(128, FT_HD) | (1u << 16);  // P V: V is MN-major
            bool ok = true;
            auto issue_s = [&](int j) {
                const int s = j % FT_STAGES;
                const uint32_t kt = s_kv + s * FT_STAGE_BYTES;
                const uint32_t d = t_s + (uint32_t)(j & 1) * 64;
#pragma unroll
                for (int k = 0; k < FT_HD / 16; k++) // the head's columns in blocks of 64 = steps of 16
                    umma_bf16(d, umma_desc_sw128(s_q + (k >> 2) * 16384 + (k & 3) * 32),
                              umma_desc_sw128(kt + (k >> 2) * 8192 + (k & 3) * 32), idesc_s, k > 0 ? 1u : 0u);
                umma_commit(b_s_full + (j & 1) * 8);
                umma_commit(b_k_empty + s * 8);                   // the stage's keys have been read
            };
            ok = mbar_wait(b_k_full, 0, status);
            if (ok) {
                tc_fence_after();
                issue_s(0);
            }
            for (int j = 0; j < n_iter && ok; j++) {
                if (j + 1 < n_iter) {
                    const int s1 = (j + 1) % FT_STAGES;
                    if (!(ok = mbar_wait(b_k_full + s1 * 8, (uint32_t)((j + 1) / FT_STAGES) & 1u, status))) break;
                    // S buffer (j + 1) & 1 holds P of page j - 1, which P V of page j - 1, issued before this product,
                    // reads: the tensor pipe runs them in order, and the softmax threads were done with the buffer when
                    // they handed that P over
                    tc_fence_after();
                    issue_s(j + 1);
                }
                if (!(ok = mbar_wait(b_p_ready, (uint32_t)j & 1u, status))) break;
                if (!(ok = mbar_wait(b_v_full + (j % FT_STAGES) * 8, (uint32_t)(j / FT_STAGES) & 1u, status))) break;
                tc_fence_after();
                const uint32_t vt = s_kv + (j % FT_STAGES) * FT_STAGE_BYTES + FT_TILE_BYTES;
#pragma unroll
                for (int k = 0; k < 4; k++)          // 64 keys = 4 steps of 16; P: 8 columns of tensor memory a step
                    umma_bf16_ts(t_o, t_s + (uint32_t)(j & 1) * 64 + k * 8, umma_desc_mn_sw128(vt + k * 2048, 8192),
                                 idesc_o, (j > 0 || k > 0) ? 1u : 0u);
                umma_commit(b_pv_done);                           // O holds pages 0..j
                umma_commit(b_v_empty + (j % FT_STAGES) * 8);     // the stage's values have been read
            }
        }
    } else if (n_iter > 0) {
        // ------------------------------------------------------------ softmax: thread = row = TMEM lane
        const int r = warp * 32 + lane;
        const bool row_ok = r < nrows;
        // (a padding row, whose query is zero and whose result is not written, sees every key: with a span of its own
        // it would take its whole warp through the masked branch at every page)
        const int p_row = row_ok ? pos0 + tok0 + r / G : 0x3fffffff;
        const int lo_row = (row_ok && window > 0 && p_row - window + 1 > 0) ? p_row - window + 1 : 0;
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        float m_ref = -INFINITY, l = 0.0f;
        bool ok = true;
        for (int j = 0; j < n_iter && ok; j++) {
            const int bsel = j & 1;
            if (!(ok = mbar_wait(b_s_full + bsel * 8, (uint32_t)(j >> 1) & 1u, status))) break;
            __syncwarp();
            tc_fence_after();
            uint32_t sv[64];
            tmem_ld_x32(t_s + lane_base + bsel * 64, sv);
            tmem_ld_x32(t_s + lane_base + bsel * 64 + 32, sv + 32);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            // scale, mask, row maximum
            const int key0 = (pg_lo + j) * KB_PAGE;
            // four independent running maxima (one long dependent chain would leave the few resident warps idle)
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (key0 + 63 <= p_row && key0 >= lo_row) {
                // the whole page lies inside this row's span (all pages but the last one or two): no masks
#pragma unroll
                for (int c = 0; c < 64; c += 8) {
#pragma unroll
                    for (int k = 0; k < 4; k++)
                        mx4[k] = ft_max3(mx4[k], __uint_as_float(sv[c + 2 * k]), __uint_as_float(sv[c + 2 * k + 1]));
                }
            } else {
#pragma unroll
                for (int c = 0; c < 64; c++) {
                    const int p = key0 + c;
                    const float s = (p <= p_row && p >= lo_row) ? __uint_as_float(sv[c]) : -INFINITY;
                    sv[c] = __float_as_uint(s);
                    mx4[c & 3] = fmaxf(mx4[c & 3], s);
                }
            }
            // (the scores stay as the product left them; the scale, which is positive, is applied to the maximum here
            // and to each score inside the exponent's one multiply-add)
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2e;
            // lazy reference: move it only when the maximum has grown by more than FT_LAZY
            const bool grow = mx > m_ref + FT_LAZY || (m_ref == -INFINITY && mx > -INFINITY);
            float f = 1.0f;
            if (grow) {
                f = m_ref == -INFINITY ? 0.0f : ft_exp2(m_ref - mx);
                m_ref = mx;
                l *= f;
            }
            // P V of page j - 1 done means: O holds pages 0..j-1. Only a rescale of O has to wait for that here;
            // otherwise the wait comes just before this page's P is handed over (it is taken once per page, in order,
            // so that the barrier's phases cannot be mistaken for one another).
            const bool rescale = __any_sync(0xffffffffu, grow) && j > 0;
            bool waited_prev = j == 0;
            if (!waited_prev && rescale) {
                if (!(ok = mbar_wait(b_pv_done, (uint32_t)(j - 1) & 1u, status))) break;
                __syncwarp();
                tc_fence_after();
                waited_prev = true;
            }
            if (rescale) {
#pragma unroll 1
                for (int c0 = 0; c0 < FT_HD; c0 += 32) {
                    uint32_t ov[32];
                    tmem_ld_x32(t_o + lane_base + c0, ov);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 32; c++) ov[c] = __float_as_uint(__uint_as_float(ov[c]) * f);
                    tmem_st_x32(t_o + lane_base + c0, ov);
                }
                tmem_st_wait();
            }
            // probabilities (relative to the reference), their sum, and P as bf16 into tensor memory
            const float mr = m_ref == -INFINITY ? 0.0f : m_ref;
            // (two scores a time through the packed 32-bit multiply-add and add of sm_100: half as many instructions
            // beside the exponentials, which is what a softmax warp's time goes to)
            const uint64_t scale2 = ft_pack2(scale_log2e, scale_log2e), nmr2 = ft_pack2(-mr, -mr);
            uint64_t sum2[4] = {0ull, 0ull, 0ull, 0ull};         // four pairs of partial sums (bit pattern of 0.0f, 0.0f)
            uint32_t pv[32];                         // the row's 64 probabilities as bf16 pairs
#pragma unroll
            for (int c8 = 0; c8 < 8; c8++) {
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    float x0, x1;
                    ft_unpack2(ft_fma2(ft_pack2(__uint_as_float(sv[c8 * 8 + 2 * c]), __uint_as_float(sv[c8 * 8 + 2 * c + 1])),
                                       scale2, nmr2), x0, x1);
                    const float p0 = ft_exp2(x0), p1 = ft_exp2(x1);
                    sum2[c] = ft_add2(sum2[c], ft_pack2(p0, p1));
                    __nv_bfloat162 v = __floats2bfloat162_rn(p0, p1);
                    pv[c8 * 4 + c] = *(uint32_t*)&v;
                }
            }
            {
                float a0, a1, b0, b1, c0, c1, d0, d1;
                ft_unpack2(sum2[0], a0, a1);
                ft_unpack2(sum2[1], b0, b1);
                ft_unpack2(sum2[2], c0, c1);
                ft_unpack2(sum2[3], d0, d1);
                l += ((a0 + a1) + (b0 + b1)) + ((c0 + c1) + (d0 + d1));
            }
            // over the first 32 columns of this page's S buffer (the scores are in registers): the row's K index runs
            // along the columns, two bf16 to a column, which is how the MMA reads an A operand from tensor memory
            tmem_st_x32(t_s + lane_base + bsel * 64, pv);
            tmem_st_wait();
            if (!waited_prev) {
                if (!(ok = mbar_wait(b_pv_done, (uint32_t)(j - 1) & 1u, status))) break;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(b_p_ready);
        }
        // ---- O / l once the last P V is done
        if (ok) ok = mbar_wait(b_pv_done, (uint32_t)(n_iter - 1) & 1u, status);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            tc_fence_after();
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            bf16* dst = out + (size_t)(qs0 + tok0 + (row_ok ? r / G : 0)) * ldo + (size_t)(hk * G + (row_ok ? r % G : 0)) * FT_HD;
#pragma unroll 1
            for (int c0 = 0; c0 < FT_HD; c0 += 32) {
                uint32_t ov[32];
                tmem_ld_x32(t_o + lane_base + c0, ov);
                tmem_ld_wait();
                if (row_ok) {
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        uint32_t h[4];
#pragma unroll
                        for (int k = 0; k < 4; k++) {
                            __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(ov[c + 2 * k]) * inv,
                                                                     __uint_as_float(ov[c + 2 * k + 1]) * inv);
                            h[k] = *(uint32_t*)&v;
                        }
                        *(uint4*)(dst + c0 + c) = make_uint4(h[0], h[1], h[2], h[3]);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem, 256);
    }
}

// grid_x = the most tiles of a sequence: ceil(longest q_len / (128 / G)) with G = nh / nkv <= 128
template <int HD>
static int launch_attn_tc(const CUtensorMap& map, const void* q, int ldq, void* out, int ldo, const int* slot,
                          const int* q_start, const int* kv_len, int B, int nh, int nkv, float scale, int window,
                          const int* table, int table_stride, int n_pages, int grid_x, int* status, cudaStream_t st) {
    // tiles (Q and two stages of keys and values: 96 KB at head size 128) + barriers + what aligning the base to 1024
    // can cost when it is aligned to 128: two CTAs fit an SM
    const int sm = 128 * HD * 2 + FT_STAGES * 2 * 64 * HD * 2 + 256 + 768;
    static char once_tag;               // one per instantiation: the opt-in is per (device, kernel)
    if (kb_first_use(&once_tag)) {
        cudaError_t e = cudaFuncSetAttribute(k_attn_tc<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, sm);
        if (e != cudaSuccess) return (int)e;
    }
    dim3 grid(nkv, grid_x, B);
    cudaError_t e = kb_launch(k_attn_tc<HD>, grid, FT_THREADS, sm, st, map, (const bf16*)q, ldq, (bf16*)out, ldo, slot,
                              q_start, kv_len, nkv, nh / nkv, scale * 1.4426950408889634f, window, table, table_stride,
                              n_pages, status);
    return (int)e;
}

// grid_x = the most tiles of a sequence: ceil(longest q_len / (128 / G)) with G = nh / nkv <= 128; head size 64 or 128
extern "C" int kb_attn_tc(const void* q, int ldq, void* out, int ldo, const int* slot, const int* q_start,
                          const int* kv_len, int B, int nh, int nkv, int hd, float scale, int window, void* pool,
                          const int* table, int table_stride, int n_pages, int grid_x, int* status, cudaStream_t st) {
    if (B <= 0 || grid_x <= 0) return 0;
    if (grid_x > 65535 || B > 65535) return (int)cudaErrorInvalidValue;
    if ((hd != 64 && hd != 128) || nkv <= 0 || nh % nkv || nh / nkv > 128) return (int)cudaErrorInvalidValue;
    if ((ldq % 8) || (ldo % 8) || ((uintptr_t)q & 15) || ((uintptr_t)out & 15)) return (int)cudaErrorInvalidValue;
    CUtensorMap map;
    int rc = kb_make_map_bf16(&map, pool, (uint64_t)n_pages * 2 * nkv * KB_PAGE, hd, hd, 64);
    if (rc) return rc;
    if (hd == 128)
        return launch_attn_tc<128>(map, q, ldq, out, ldo, slot, q_start, kv_len, B, nh, nkv, scale, window, table,
                                   table_stride, n_pages, grid_x, status, st);
    return launch_attn_tc<64>(map, q, ldq, out, ldo, slot, q_start, kv_len, B, nh, nkv, scale, window, table,
                              table_stride, n_pages, grid_x, status, st);
}
