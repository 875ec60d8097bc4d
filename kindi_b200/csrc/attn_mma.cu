// bfloat16 attention over the paged cache for prefill and for decode.
//
// One CTA serves one key/value head of one sequence: its rows are the (token, query head of the group) pairs that
// read this head, r = token * G + j (the reference packs rows the same way, kindi/nbq_fa.cu:3-5,40-49), so a tile of
// keys and values is fetched once for all G query heads. Pages of 64 positions are brought in by TMA (two tile loads
// of 64 columns per 128 bytes of head, 128-byte swizzle, no multicast) by a producer warp into a ring of stages;
// four consumer warps compute S = Q K^T and O += P V with tensor-core MMAs (bf16 in, fp32 accumulate), softmax in
// 32-bit with a running maximum and sum (kindi/nbq_fa.cu:31-151: the same flash-attention recurrence).
//   - prefill form: 64 rows a CTA, 16 a warp; every warp walks all keys up to its rows' own positions.
//   - decode form: the G rows of one token; the four warps split each page's 64 keys, gridDim.x splits the pages
//     (kindi/nbq.cu:525-633: position splits and per-warp running maxima), and the parts are merged in a fixed order
//     (kindi/nbq.cu:635-649).
//   - decode form with rotation ("ROPE"): the kernel takes the 32-bit planes of the QKV product instead of finished
//     queries. Every CTA sums and rotates the queries of its G heads itself (rotate-half pairs, the expressions of
//     k_rope_store); the CTA whose pages hold the newest position also sums and rotates that position's key, takes its
//     value, stores both in the cache for later steps and writes them into its shared-memory tile of the last page
//     over what the TMA load brought. The rotate-and-store kernel and its round trip of Q through memory fall away.
// Head sizes 64 and 128; any number of heads and groups for prefill, groups up to 16 for decode. Other shapes run
// the general kernel.
#include <stdio.h>
#include "sm100.cuh"

#define AT_THREADS 160          // warps 0-3: MMA + softmax, warp 4: TMA producer
#define AT_ROWS 64              // rows per CTA in the prefill form

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *(uint32_t*)&v;
}
// byte offset of (row, 16-byte chunk) in a [64 rows][HD] tile stored as HD/64 swizzled boxes of [64][128 bytes]
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
    return (uint32_t)((chunk >> 3) * 8192 + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

#ifndef AT_EARLY
#define AT_EARLY 2                   // pages of older positions requested before the programmatic wait (decode form)
#endif
// what the decode form with rotation reads instead of finished queries
struct AtRopeIn {
    const float* planes;        // [n_planes][rows][ld]: the QKV product, a row = [q heads | k heads | v heads]
    int n_planes;
    size_t plane_stride;
    int ld;
    const float* inv_freq;      // [HD / 2]
    bf16* pool;                 // the cache entry's pages, for the newest key and value; null: nothing is stored
};
// v[j][0..W-1] = sum over the planes, in order, of the W floats at p[j]: NS places at once, the loads of four planes of
// all places in flight together (a chain of dependent round trips to the L2 would cost more than the kernel saved)
template <int NS, int W>
__device__ __forceinline__ void at_ld_sum(const float* const (&p)[NS], const bool (&on)[NS], int n_planes,
                                          size_t plane_stride, float (&v)[NS][W]) {
    auto ld = [](const float* q, float* o) {
        if (W == 2) {
            const float2 t = *(const float2*)q;
            o[0] = t.x;
            o[W - 1] = t.y;
        } else {
            o[0] = *q;
        }
    };
#pragma unroll
    for (int j = 0; j < NS; j++) {
        v[j][0] = v[j][W - 1] = 0.0f;
        if (on[j]) ld(p[j], v[j]);
    }
    for (int s0 = 1; s0 < n_planes; s0 += 4) {
        float t[4][NS][W];
#pragma unroll
        for (int k = 0; k < 4; k++)
#pragma unroll
            for (int j = 0; j < NS; j++)
                if (s0 + k < n_planes && on[j]) ld(p[j] + (size_t)(s0 + k) * plane_stride, t[k][j]);
#pragma unroll
        for (int k = 0; k < 4; k++)
#pragma unroll
            for (int j = 0; j < NS; j++)
                if (s0 + k < n_planes && on[j]) {
#pragma unroll
                    for (int c = 0; c < W; c++) v[j][c] += t[k][j][c];
                }
    }
}
template <int HD, bool DEC, bool ROPE = false>
__global__ void __launch_bounds__(AT_THREADS, 2) k_attn_mma(const __grid_constant__ CUtensorMap kvmap,
        const bf16* KB_STEP_DATA q, int ldq, bf16* __restrict__ out, int ldo, float* __restrict__ part_o,
        float* __restrict__ part_ml, const int* __restrict__ slot, const int* __restrict__ q_start,
        const int* __restrict__ kv_len, int nh, int nkv, int G, float scale_log2e, int window,
        const int* __restrict__ table, int table_stride, int n_pages, int* status, AtRopeIn rp) {
    static_assert(!ROPE || DEC, "rotation inside the kernel: decode form only");
    constexpr int AT_STAGES = DEC ? 3 : 2;      // pages in flight (two CTAs fit an SM in both forms)
    constexpr int KT = HD / 16;                 // k-steps of Q K^T
    constexpr int NT = DEC ? 2 : 8;             // 8-key tiles a warp takes from each page
    constexpr int DT = HD / 8;                  // 8-column tiles of the output
    constexpr int TILE_BYTES = 64 * HD * 2;     // one page of keys (or values) of one head
    constexpr int STAGE_BYTES = 2 * TILE_BYTES;
    constexpr int QS = HD + 8;                  // padded row of the Q staging tile (elements)
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar_full = sbase + AT_STAGES * STAGE_BYTES, bar_empty = bar_full + AT_STAGES * 8;
    // Q staging: [4 warps][16][QS] (prefill); one shared [16][QS] for decode, where every warp has the same rows and
    // writes the same values
    bf16* qs = (bf16*)(smem + AT_STAGES * STAGE_BYTES + 2 * AT_STAGES * 8 + 16);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.z, hk = blockIdx.y;
    // The step's metadata (lengths, slots, page table) was written before the step's first kernel, and the pages of
    // older positions by earlier steps. In the decode form only Q and the page of the newest position come from the
    // kernel just before this one, so each thread waits for that kernel where it first needs them.
    if (DEC) kb_pdl_launch_now();
    else kb_pdl_wait();
    const int qs0 = q_start[b], qlen = q_start[b + 1] - qs0, kvl = kv_len[b];
    const int pos0 = kvl - qlen;                 // position of the sequence's first row of this step
    const int n_rows = qlen * G;
    int row0, pg_lo, pg_hi;                      // the CTA's first row; its pages [pg_lo, pg_hi]
    if (DEC) {
        row0 = 0;
        const int lo = (window > 0 && kvl - window > 0) ? kvl - window : 0;       // row position is kvl - 1
        const int first = lo / KB_PAGE, last = (kvl - 1) / KB_PAGE;
        const int per = (last - first + (int)gridDim.x) / (int)gridDim.x;        // ceil(pages / splits)
        pg_lo = first + (int)blockIdx.x * per;
        pg_hi = min(last, pg_lo + per - 1);
    } else {
        const int n_tiles = (n_rows + AT_ROWS - 1) / AT_ROWS;
        if ((int)blockIdx.x >= n_tiles) return;
        row0 = (n_tiles - 1 - (int)blockIdx.x) * AT_ROWS;          // the longest tiles first
        const int last_row = min(n_rows, row0 + AT_ROWS) - 1;
        const int p_first = pos0 + row0 / G, p_last = pos0 + last_row / G;
        const int lo = (window > 0 && p_first - window + 1 > 0) ? p_first - window + 1 : 0;
        pg_lo = lo / KB_PAGE;
        pg_hi = p_last / KB_PAGE;
    }
    const int n_iter = pg_hi - pg_lo + 1;        // may be <= 0 for an empty decode split

    if (threadIdx.x == 0) {
        for (int s = 0; s < AT_STAGES; s++) {
            mbar_init(bar_full + s * 8, 1);
            mbar_init(bar_empty + s * 8, 4);
        }
        mbar_fence_init();
    }
    __syncthreads();

    // per-thread accumulators (consumer warps)
    float o[DT][4];
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.0f, l_b = 0.0f;
#pragma unroll
    for (int i = 0; i < DT; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;

    if (warp == 4) {
        // ---------------------------------------------------------------- producer
        if (lane == 0 && n_iter > 0) {
            tma_prefetch_desc(&kvmap);
            const int* trow = table + (size_t)slot[b] * table_stride;
            bool waited = !DEC;
            for (int i = 0; i < n_iter; i++) {
                const int s = i % AT_STAGES;
                const uint32_t ph = (uint32_t)(i / AT_STAGES) & 1u;
                // (with rotation and a key of its own the newest row is patched in shared memory, so its page may come early too)
                if (DEC && !waited && (i >= AT_EARLY || (pg_lo + i == (kvl - 1) / KB_PAGE && !(ROPE && rp.pool)))) {
                    kb_pdl_wait();
                    waited = true;
                }
                if (!mbar_wait(bar_empty + s * 8, ph ^ 1u, status)) break;
                int page = trow[pg_lo + i];
                if (page < 0 || page >= n_pages) {
                    if (!waited) kb_pdl_wait();              // the status word is shared with earlier kernels
                    waited = true;
                    atomicOr(status, KB_ST_BAD_PAGE);
                    page = 0;
                }
                mbar_expect_tx(bar_full + s * 8, STAGE_BYTES);
                const uint32_t dst = sbase + s * STAGE_BYTES;
                const int krow = ((page * 2 + 0) * nkv + hk) * KB_PAGE, vrow = ((page * 2 + 1) * nkv + hk) * KB_PAGE;
#pragma unroll
                for (int h = 0; h < HD / 64; h++) {
                    tma_load_2d(dst + h * 8192, &kvmap, h * 64, krow, bar_full + s * 8);
                    tma_load_2d(dst + TILE_BYTES + h * 8192, &kvmap, h * 64, vrow, bar_full + s * 8);
                }
            }
        }
    } else {
        // ---------------------------------------------------------------- consumers
        // this warp's 16 rows: r = wrow0 + 0..15; thread rows ra = lane / 4, rb = ra + 8
        const int wrow0 = row0 + (DEC ? 0 : warp * 16);
        bf16* qw = qs + (DEC ? 0 : warp) * 16 * QS;
        constexpr int PPL = HD / 64;                 // pairs of the newest key a lane takes: i0 .. i0 + PPL - 1
        constexpr int HALF = HD / 2;
        const int i0 = lane * PPL;
        const int tid = threadIdx.x;                 // 0..127 here: the consumer threads
        float knew_lo[PPL], knew_hi[PPL], vnew[2][PPL];
        const int p_new = kvl - 1;
        const bool owns_new = ROPE && rp.pool != nullptr && p_new / KB_PAGE >= pg_lo && p_new / KB_PAGE <= pg_hi &&
                              warp == (p_new % KB_PAGE) / 16;
        if (ROPE) {
            // Queries: pair e = tid + 128 k is (row e / HALF, pair e % HALF of the head) and 128 is a multiple of HALF,
            // so a thread's pairs all have the same angle. Everything that does not come from the QKV product is
            // done before the wait for it.
            const float ang = __fmul_rn((float)p_new, rp.inv_freq[tid % HALF]);
            const float qc = cosf(ang), qsn = sinf(ang);
            float kc[PPL], ks[PPL];
            int page_new = 0;
            if (owns_new) {
#pragma unroll
                for (int j = 0; j < PPL; j++) {
                    const float ak = __fmul_rn((float)p_new, rp.inv_freq[i0 + j]);
                    kc[j] = cosf(ak);
                    ks[j] = sinf(ak);
                }
                page_new = table[(size_t)slot[b] * table_stride + p_new / KB_PAGE];
                if (page_new < 0 || page_new >= n_pages) page_new = -1;          // reported by the producer
            }
            // rows past G are zero
            for (int e = G * (HD / 8) + tid; e < 16 * (HD / 8); e += 128)
                *(uint4*)(qs + (e / (HD / 8)) * QS + (e % (HD / 8)) * 8) = make_uint4(0, 0, 0, 0);
            kb_pdl_wait();
            const float* prow = rp.planes + (size_t)qs0 * rp.ld;
            const int n_pairs = G * HALF;
            for (int e0 = tid; e0 < n_pairs; e0 += 4 * 128) {
                const float* ptr[8];
                bool on[8];
                float val[8][1];
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const int e = e0 + 128 * k;
                    on[2 * k] = on[2 * k + 1] = e < n_pairs;
                    const int r = e / HALF, i = e % HALF;
                    ptr[2 * k] = prow + (size_t)(hk * G + r) * HD + i;
                    ptr[2 * k + 1] = ptr[2 * k] + HALF;
                }
                at_ld_sum<8, 1>(ptr, on, rp.n_planes, rp.plane_stride, val);
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const int e = e0 + 128 * k;
                    if (e < n_pairs) {
                        const int r = e / HALF, i = e % HALF;
                        const float a = val[2 * k][0], bb = val[2 * k + 1][0];
                        qs[r * QS + i] = __float2bfloat16_rn(__fsub_rn(__fmul_rn(a, qc), __fmul_rn(bb, qsn)));
                        qs[r * QS + HALF + i] = __float2bfloat16_rn(__fadd_rn(__fmul_rn(bb, qc), __fmul_rn(a, qsn)));
                    }
                }
            }
            if (owns_new) {
                // the newest key (rotated) and value of this head: into the cache for later steps, and kept for the patch
                const float* ksrc = prow + (size_t)(nh + hk) * HD, *vsrc = prow + (size_t)(nh + nkv + hk) * HD;
                const float* ptr[4] = {ksrc + i0, ksrc + HALF + i0, vsrc + 2 * i0, vsrc + 2 * i0 + PPL};
                const bool on[4] = {true, true, true, true};
                float val[4][PPL];
                at_ld_sum<4, PPL>(ptr, on, rp.n_planes, rp.plane_stride, val);
#pragma unroll
                for (int j = 0; j < PPL; j++) {
                    knew_lo[j] = __fsub_rn(__fmul_rn(val[0][j], kc[j]), __fmul_rn(val[1][j], ks[j]));
                    knew_hi[j] = __fadd_rn(__fmul_rn(val[1][j], kc[j]), __fmul_rn(val[0][j], ks[j]));
                    vnew[0][j] = val[2][j];
                    vnew[1][j] = val[3][j];
                }
                if (page_new >= 0) {
                    const size_t base = (size_t)page_new * 2 * nkv;
                    bf16* kd = rp.pool + ((base + hk) * KB_PAGE + p_new % KB_PAGE) * HD;
                    bf16* vd = rp.pool + ((base + nkv + hk) * KB_PAGE + p_new % KB_PAGE) * HD;
#pragma unroll
                    for (int j = 0; j < PPL; j++) {
                        kd[i0 + j] = __float2bfloat16_rn(knew_lo[j]);
                        kd[HALF + i0 + j] = __float2bfloat16_rn(knew_hi[j]);
                        vd[2 * i0 + j] = __float2bfloat16_rn(vnew[0][j]);
                        vd[2 * i0 + PPL + j] = __float2bfloat16_rn(vnew[1][j]);
                    }
                }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");          // the four consumer warps: Q is whole
        } else {
        if (DEC) kb_pdl_wait();
        for (int e = lane; e < 16 * (HD / 8); e += 32) {
            const int r = e / (HD / 8), c = e % (HD / 8);
            const int gr = wrow0 + r;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (gr < n_rows) {
                const int t = gr / G, j = gr % G;
                v = *(const uint4*)(q + (size_t)(qs0 + t) * ldq + (size_t)(hk * G + j) * HD + c * 8);
            }
            *(uint4*)(qw + r * QS + c * 8) = v;
        }
        __syncwarp();
        }
        uint32_t qf[KT][4];
#pragma unroll
        for (int ks = 0; ks < KT; ks++) {
            const int r = (lane & 7) + ((lane >> 3) & 1) * 8, c = ks * 2 + (lane >> 4);
            ldsm_x4(smem_u32(qw + r * QS + c * 8), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
        }
        const int ra = wrow0 + (lane >> 2), rb = ra + 8;
        const int pa = ra < n_rows ? pos0 + ra / G : -1, pb = rb < n_rows ? pos0 + rb / G : -1;
        const int la = (window > 0 && pa - window + 1 > 0) ? pa - window + 1 : 0;
        const int lb = (window > 0 && pb - window + 1 > 0) ? pb - window + 1 : 0;
        // the last position any row of this warp reads: later pages are skipped by the whole warp
        int wlast = max(pa, pb);
        wlast = max(wlast, __shfl_xor_sync(0xffffffffu, wlast, 4));
        wlast = max(wlast, __shfl_xor_sync(0xffffffffu, wlast, 8));
        wlast = max(wlast, __shfl_xor_sync(0xffffffffu, wlast, 16));
        const int kw0 = DEC ? warp * 16 : 0;          // the warp's first key inside a page

        for (int i = 0; i < n_iter; i++) {
            const int s = i % AT_STAGES;
            const uint32_t ph = (uint32_t)(i / AT_STAGES) & 1u;
            if (!mbar_wait(bar_full + s * 8, ph, status)) break;
            if (ROPE && owns_new && pg_lo + i == p_new / KB_PAGE) {
                // the newest position's row of this page: the values computed above, over what the load brought
                uint8_t* kt8 = smem + s * STAGE_BYTES;
                const int row = p_new % KB_PAGE;
#pragma unroll
                for (int j = 0; j < PPL; j++) {
                    const int cl = i0 + j, ch = HALF + i0 + j;
                    *(bf16*)(kt8 + tile_off(row, cl >> 3) + (cl & 7) * 2) = __float2bfloat16_rn(knew_lo[j]);
                    *(bf16*)(kt8 + tile_off(row, ch >> 3) + (ch & 7) * 2) = __float2bfloat16_rn(knew_hi[j]);
                }
#pragma unroll
                for (int j = 0; j < 2 * PPL; j++) {
                    const int c = 2 * i0 + j;
                    *(bf16*)(kt8 + TILE_BYTES + tile_off(row, c >> 3) + (c & 7) * 2) =
                        __float2bfloat16_rn(vnew[j / PPL][j % PPL]);
                }
                __syncwarp();
            }
            const int key0 = (pg_lo + i) * KB_PAGE + kw0;           // absolute position of the warp's first key
            if (key0 <= wlast) {
                const uint32_t kt = sbase + s * STAGE_BYTES, vt = kt + TILE_BYTES;
                float sc[NT][4];
#pragma unroll
                for (int n = 0; n < NT; n++) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.0f;
#pragma unroll
                for (int n2 = 0; n2 < NT / 2; n2++) {
                    const int krow = kw0 + n2 * 16 + (lane & 7) + (lane >> 4) * 8;
#pragma unroll
                    for (int ks = 0; ks < KT; ks++) {
                        uint32_t r0, r1, r2, r3;
                        ldsm_x4(kt + tile_off(krow, ks * 2 + ((lane >> 3) & 1)), r0, r1, r2, r3);
                        mma_bf16(sc[2 * n2], qf[ks], r0, r1);
                        mma_bf16(sc[2 * n2 + 1], qf[ks], r2, r3);
                    }
                }
                // scale, mask, running maximum
                float mxa = -INFINITY, mxb = -INFINITY;
#pragma unroll
                for (int n = 0; n < NT; n++) {
                    const int p = key0 + n * 8 + (lane & 3) * 2;
                    sc[n][0] = (p <= pa && p >= la) ? sc[n][0] * scale_log2e : -INFINITY;
                    sc[n][1] = (p + 1 <= pa && p + 1 >= la) ? sc[n][1] * scale_log2e : -INFINITY;
                    sc[n][2] = (p <= pb && p >= lb) ? sc[n][2] * scale_log2e : -INFINITY;
                    sc[n][3] = (p + 1 <= pb && p + 1 >= lb) ? sc[n][3] * scale_log2e : -INFINITY;
                    mxa = fmaxf(mxa, fmaxf(sc[n][0], sc[n][1]));
                    mxb = fmaxf(mxb, fmaxf(sc[n][2], sc[n][3]));
                }
                mxa = fmaxf(mxa, __shfl_xor_sync(0xffffffffu, mxa, 1));
                mxa = fmaxf(mxa, __shfl_xor_sync(0xffffffffu, mxa, 2));
                mxb = fmaxf(mxb, __shfl_xor_sync(0xffffffffu, mxb, 1));
                mxb = fmaxf(mxb, __shfl_xor_sync(0xffffffffu, mxb, 2));
                const float na = fmaxf(m_a, mxa), nb = fmaxf(m_b, mxb);
                const float ua = na == -INFINITY ? 0.0f : na, ub = nb == -INFINITY ? 0.0f : nb;
                const float fa = exp2f(m_a - ua), fb = exp2f(m_b - ub);
                m_a = na;
                m_b = nb;
                float sa = 0.0f, sb = 0.0f;
                uint32_t pf[NT][2];
#pragma unroll
                for (int n = 0; n < NT; n++) {
                    const float p0 = exp2f(sc[n][0] - ua), p1 = exp2f(sc[n][1] - ua);
                    const float p2 = exp2f(sc[n][2] - ub), p3 = exp2f(sc[n][3] - ub);
                    sa += p0 + p1;
                    sb += p2 + p3;
                    pf[n][0] = pack_bf16(p0, p1);
                    pf[n][1] = pack_bf16(p2, p3);
                }
                l_a = l_a * fa + sa;
                l_b = l_b * fb + sb;
#pragma unroll
                for (int d = 0; d < DT; d++) {
                    o[d][0] *= fa;
                    o[d][1] *= fa;
                    o[d][2] *= fb;
                    o[d][3] *= fb;
                }
#pragma unroll
                for (int k2 = 0; k2 < NT / 2; k2++) {
                    const uint32_t a[4] = {pf[2 * k2][0], pf[2 * k2][1], pf[2 * k2 + 1][0], pf[2 * k2 + 1][1]};
                    const int vrow = kw0 + k2 * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
                    for (int d2 = 0; d2 < DT / 2; d2++) {
                        uint32_t r0, r1, r2, r3;
                        ldsm_x4_t(vt + tile_off(vrow, d2 * 2 + (lane >> 4)), r0, r1, r2, r3);
                        mma_bf16(o[2 * d2], a, r0, r1);
                        mma_bf16(o[2 * d2 + 1], a, r2, r3);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + s * 8);
        }
        l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
        l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
        l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
        l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
        if (!DEC) {
            // every row is whole in its warp: normalise and write
            const float ia = l_a > 0.0f ? 1.0f / l_a : 0.0f, ib = l_b > 0.0f ? 1.0f / l_b : 0.0f;
            if (ra < n_rows) {
                bf16* dst = out + (size_t)(qs0 + ra / G) * ldo + (size_t)(hk * G + ra % G) * HD + (lane & 3) * 2;
#pragma unroll
                for (int d = 0; d < DT; d++) *(uint32_t*)(dst + d * 8) = pack_bf16(o[d][0] * ia, o[d][1] * ia);
            }
            if (rb < n_rows) {
                bf16* dst = out + (size_t)(qs0 + rb / G) * ldo + (size_t)(hk * G + rb % G) * HD + (lane & 3) * 2;
#pragma unroll
                for (int d = 0; d < DT; d++) *(uint32_t*)(dst + d * 8) = pack_bf16(o[d][2] * ib, o[d][3] * ib);
            }
        }
    }
    if (!DEC) return;

    // ---------------------------------------------------------------- decode: merge the four warps, then write
    __syncthreads();                                   // every stage has been consumed: the ring is free
    float* mo = (float*)smem;                          // [4][16][HD]
    float* mml = mo + 4 * 16 * HD;                     // [4][16][2]
    if (warp < 4) {
        const int r = lane >> 2;
#pragma unroll
        for (int d = 0; d < DT; d++) {
            const int c = d * 8 + (lane & 3) * 2;
            *(float2*)(mo + (warp * 16 + r) * HD + c) = make_float2(o[d][0], o[d][1]);
            *(float2*)(mo + (warp * 16 + r + 8) * HD + c) = make_float2(o[d][2], o[d][3]);
        }
        if ((lane & 3) == 0) {
            mml[(warp * 16 + r) * 2] = m_a;
            mml[(warp * 16 + r) * 2 + 1] = l_a;
            mml[(warp * 16 + r + 8) * 2] = m_b;
            mml[(warp * 16 + r + 8) * 2 + 1] = l_b;
        }
    }
    __syncthreads();
    const int n_splits = gridDim.x, split = blockIdx.x;
    for (int e = threadIdx.x; e < G * HD; e += AT_THREADS) {
        const int r = e / HD, d = e % HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; w++) M = fmaxf(M, mml[(w * 16 + r) * 2]);
        const float U = M == -INFINITY ? 0.0f : M;
        float ov = 0.0f, lv = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; w++) {
            const float f = exp2f(mml[(w * 16 + r) * 2] - U);
            ov = fmaf(f, mo[(w * 16 + r) * HD + d], ov);
            lv = fmaf(f, mml[(w * 16 + r) * 2 + 1], lv);
        }
        const int h = hk * G + r;
        if (n_splits == 1) {
            out[(size_t)qs0 * ldo + (size_t)h * HD + d] = __float2bfloat16_rn(lv > 0.0f ? ov / lv : 0.0f);
        } else {
            const size_t pi = ((size_t)b * nh + h) * n_splits + split;
            part_o[pi * HD + d] = ov;
            if (d == 0) {
                part_ml[pi * 2] = M;
                part_ml[pi * 2 + 1] = lv;
            }
        }
    }
}

// merge the position splits of a decode step in split order: out = sum_s 2^(m_s - M) o_s / sum_s 2^(m_s - M) l_s
// (kindi/nbq.cu:635-649)
__global__ void k_attn_merge(const float* KB_STEP_DATA part_o, const float* KB_STEP_DATA part_ml, int n_splits,
                             bf16* __restrict__ out, int ldo, const int* __restrict__ q_start, int nh, int HD) {
    // blockDim = 4 * HD: group g = threadIdx.x / HD adds the splits 16 g .. 16 g + 15 for its column, then the four
    // group sums are added in group order: every sum has a fixed order
    __shared__ float sf[64], sl[64];              // at most 64 splits: each split's weight 2^(m_s - M), and its sum
    __shared__ float so[4][256];
    kb_pdl_launch();
    kb_pdl_wait();
    const int h = blockIdx.x, b = blockIdx.y;
    const size_t base = ((size_t)b * nh + h) * n_splits;
    if (threadIdx.x < 32) {
        float m0 = threadIdx.x < n_splits ? part_ml[(base + threadIdx.x) * 2] : -INFINITY;
        float m1 = threadIdx.x + 32 < n_splits ? part_ml[(base + threadIdx.x + 32) * 2] : -INFINITY;
        const float M = kb_warp_max(fmaxf(m0, m1));
        const float U = M == -INFINITY ? 0.0f : M;
        sf[threadIdx.x] = exp2f(m0 - U);
        sf[threadIdx.x + 32] = exp2f(m1 - U);
        sl[threadIdx.x] = threadIdx.x < n_splits ? part_ml[(base + threadIdx.x) * 2 + 1] : 0.0f;
        sl[threadIdx.x + 32] = threadIdx.x + 32 < n_splits ? part_ml[(base + threadIdx.x + 32) * 2 + 1] : 0.0f;
    }
    const int g = threadIdx.x / HD, d = threadIdx.x % HD;
    float t[16];
#pragma unroll
    for (int j = 0; j < 16; j++) t[j] = (g * 16 + j < n_splits) ? part_o[(base + g * 16 + j) * HD + d] : 0.0f;
    __syncthreads();
    float o = 0.0f;
#pragma unroll
    for (int j = 0; j < 16; j++)
        if (g * 16 + j < n_splits) o = fmaf(sf[g * 16 + j], t[j], o);
    so[g][d] = o;
    __syncthreads();
    if (g == 0) {
        float l = 0.0f;
        for (int s = 0; s < n_splits; s++) l = fmaf(sf[s], sl[s], l);
        o = ((so[0][d] + so[1][d]) + so[2][d]) + so[3][d];
        out[(size_t)q_start[b] * ldo + (size_t)h * HD + d] = __float2bfloat16_rn(l > 0.0f ? o / l : 0.0f);
    }
}

template <int HD, bool DEC>
static int attn_smem_bytes() {
    const int stages = DEC ? 3 : 2;
    int ring = stages * 2 * 64 * HD * 2;
    int tail = 2 * stages * 8 + 16 + (DEC ? 1 : 4) * 16 * (HD + 8) * 2;
    int merge = DEC ? (4 * 16 * HD * 4 + 4 * 16 * 2 * 4) : 0;
    int body = ring + tail;
    return (body > merge ? body : merge) + 1024;
}

static int kb_sm_count_attn() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

template <int HD, bool DEC, bool ROPE = false>
static int launch_attn(const CUtensorMap& map, const void* q, int ldq, void* out, int ldo, float* part_o,
                       float* part_ml, const int* slot, const int* q_start, const int* kv_len, int B, int nh, int nkv,
                       float scale, int window, const int* table, int table_stride, int n_pages, int grid_x,
                       int* status, cudaStream_t st, AtRopeIn rp = AtRopeIn()) {
    auto kern = k_attn_mma<HD, DEC, ROPE>;
    int sm = attn_smem_bytes<HD, DEC>();
    constexpr int ALONE = 118 * 1024;   // more than half of an SM's shared memory: a CTA that asks for it has the SM to itself
    static char once_tag;               // one per instantiation: the opt-in is per (device, kernel)
    if (kb_first_use(&once_tag)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, sm > ALONE ? sm : ALONE);
        if (e != cudaSuccess) return (int)e;
    }
    // A decode step with no more CTAs than SMs: every CTA gets an SM of its own. Placed while the kernel before still
    // holds some SMs, the CTAs were otherwise put two by two on the free ones, where two position streams share
    // what one SM can take in (32 sequences x 4 heads at context 8192: 4.97 -> 4.68 ms a step).
    if (DEC && (long long)grid_x * nkv * B <= kb_sm_count_attn() && sm < ALONE) sm = ALONE;
    dim3 grid(grid_x, nkv, B);
    kb_launch(kern, grid, AT_THREADS, sm, st, map, (const bf16*)q, ldq, (bf16*)out, ldo, part_o, part_ml, slot, q_start,
                                       kv_len, nh, nkv, nh / nkv, scale * 1.4426950408889634f, window, table,
                                       table_stride, n_pages, status, rp);
    return (int)cudaGetLastError();
}

// decode != 0: every sequence brings one token; grid_x = number of position splits (part_o [B][nh][splits][hd] and
// part_ml [B][nh][splits][2] are scratch when splits > 1). decode == 0: grid_x = ceil(max rows of a sequence / 64)
// with rows = tokens * (nh / nkv).
extern "C" int kb_attn_mma(const void* q, int ldq, void* out, int ldo, float* part_o, float* part_ml,
                           const int* slot, const int* q_start, const int* kv_len, int B, int nh, int nkv, int hd,
                           float scale, int window, void* pool, const int* table, int table_stride, int n_pages,
                           int decode, int grid_x, int* status, cudaStream_t st) {
    if (B <= 0 || grid_x <= 0) return 0;
    if (decode && grid_x > 64) return (int)cudaErrorInvalidValue;
    if ((hd != 64 && hd != 128) || nkv <= 0 || nh % nkv) return (int)cudaErrorInvalidValue;
    if (decode && nh / nkv > 16) return (int)cudaErrorInvalidValue;
    if ((ldq % 8) || (ldo % 2) || ((uintptr_t)q & 15)) return (int)cudaErrorInvalidValue;
    CUtensorMap map;
    int rc = kb_make_map_bf16(&map, pool, (uint64_t)n_pages * 2 * nkv * KB_PAGE, hd, hd, 64);
    if (rc) return rc;
#define AT_GO(HD, DEC)                                                                                          \
    rc = launch_attn<HD, DEC>(map, q, ldq, out, ldo, part_o, part_ml, slot, q_start, kv_len, B, nh, nkv, scale, \
                              window, table, table_stride, n_pages, grid_x, status, st)
    if (hd == 128) {
        if (decode) AT_GO(128, true); else AT_GO(128, false);
    } else {
        if (decode) AT_GO(64, true); else AT_GO(64, false);
    }
#undef AT_GO
    if (rc) return rc;
    if (decode && grid_x > 1) {
        dim3 grid(nh, B);
        kb_launch(k_attn_merge, grid, 4 * hd, 0, st, part_o, part_ml, grid_x, (bf16*)out, ldo, q_start, nh, hd);
        return (int)cudaGetLastError();
    }
    return 0;
}

// Decode attention that rotates and stores by itself: qkv = the 32-bit planes [n_planes][rows][ld_qkv] of the QKV product
// (a row = nh query heads, nkv key heads, nkv value heads of size hd), rotated over the whole head (rotary dimension =
// hd) with inv_freq [hd / 2] at each sequence's newest position kv_len - 1. store != 0: the newest key and value go
// into `pool` (the cache entry's own pages); store == 0: the entry reads another entry's pages and stores nothing.
extern "C" int kb_attn_decode_rope(const float* qkv, int n_planes, long long plane_stride, int ld_qkv,
                                   const float* inv_freq, void* out, int ldo, float* part_o, float* part_ml,
                                   const int* slot, const int* q_start, const int* kv_len, int B, int nh, int nkv,
                                   int hd, float scale, int window, void* pool, int store, const int* table,
                                   int table_stride, int n_pages, int grid_x, int* status, cudaStream_t st) {
    if (B <= 0 || grid_x <= 0) return 0;
    if (grid_x > 64 || n_planes < 1) return (int)cudaErrorInvalidValue;
    if ((hd != 64 && hd != 128) || nkv <= 0 || nh % nkv || nh / nkv > 16) return (int)cudaErrorInvalidValue;
    if ((ldo % 2) || (ld_qkv % 2) || (plane_stride % 2) || ((uintptr_t)qkv & 7)) return (int)cudaErrorInvalidValue;
    CUtensorMap map;
    int rc = kb_make_map_bf16(&map, pool, (uint64_t)n_pages * 2 * nkv * KB_PAGE, hd, hd, 64);
    if (rc) return rc;
    AtRopeIn rp;
    rp.planes = qkv;
    rp.n_planes = n_planes;
    rp.plane_stride = (size_t)plane_stride;
    rp.ld = ld_qkv;
    rp.inv_freq = inv_freq;
    rp.pool = store ? (bf16*)pool : nullptr;
    if (hd == 128)
        rc = launch_attn<128, true, true>(map, nullptr, 0, out, ldo, part_o, part_ml, slot, q_start, kv_len, B, nh, nkv,
                                          scale, window, table, table_stride, n_pages, grid_x, status, st, rp);
    else
        rc = launch_attn<64, true, true>(map, nullptr, 0, out, ldo, part_o, part_ml, slot, q_start, kv_len, B, nh, nkv,
                                         scale, window, table, table_stride, n_pages, grid_x, status, st, rp);
    if (rc) return rc;
    if (grid_x > 1) {
        dim3 grid(nh, B);
        kb_launch(k_attn_merge, grid, 4 * hd, 0, st, part_o, part_ml, grid_x, (bf16*)out, ldo, q_start, nh, hd);
        return (int)cudaGetLastError();
    }
    return 0;
}

// ------------------------------------------------------------------------------------------------------------------
// Decode attention for callers that cannot allocate device memory (declared in kindi_b200_noalloc.h; the reference has
// no counterpart). Some hosts of this library may not call cudaMalloc at all: a plug-in that runs inside another
// program's CUDA context under a fixed memory limit, a real-time loop that must not touch the allocator once it is
// running, a process whose memory pool is owned by somebody else. kb_attn_mma above needs scratch for the partial
// results of its position splits and takes it from its caller (who gets it from an allocator); this entry point runs
// the same kernels with that scratch in the file-scope array below instead, so it allocates nothing: no cudaMalloc,
// no cudaFree, no library routine that allocates. The caller still passes every input and output.
//
// The array is part of the loaded library: every GPU that loads it holds KB_STATIC_SCRATCH_FLOATS * 4 bytes (4 MiB)
// until the process exits. A call needs B * nh * n_splits * (hd + 2) floats of it; a call that needs more is
// refused (cudaErrorInvalidValue, with a line on stderr that gives both numbers) and launches nothing.
// In host code the array's NAME is only a stand-in (a host-side shadow symbol), not a device address; the address
// the kernels get is looked up with cudaGetSymbolAddress, once per device, on the first call made while that device is
// current. That first call should therefore come before any stream capture (the lookup is not a stream operation).
// All calls share the one array, and it keeps what the last call left there. Nothing in it has to start at zero:
// every split of every (sequence, head) writes its maximum, its sum and its whole output row before the merge
// reads them. Two calls that overlap on the GPU (different streams, or graphs replayed side by side) race on the
// array; calls on one stream are ordered and safe.
#define KB_STATIC_SCRATCH_FLOATS (1 << 20)
static __device__ __align__(256) float g_attn_static_scratch[KB_STATIC_SCRATCH_FLOATS];

extern "C" int kb_attn_decode_static(const void* q, int ldq, void* out, int ldo, const int* slot,
                                     const int* q_start, const int* kv_len, int B, int nh, int nkv, int hd,
                                     float scale, int window, void* pool, const int* table, int table_stride,
                                     int n_pages, int n_splits, int* status, cudaStream_t st) {
    static float* base_of_device[64] = {nullptr};
    if (B <= 0) return 0;
    if (n_splits < 1 || n_splits > 64 || nh <= 0 || hd <= 0) return (int)cudaErrorInvalidValue;
    const long long need = (long long)B * nh * n_splits * (hd + 2);
    if (need > (long long)KB_STATIC_SCRATCH_FLOATS) {
        fprintf(stderr,
                "kb_attn_decode_static: this call needs %lld floats of scratch (B %d x heads %d x splits %d x (head "
                "size %d + 2)) and the static array holds %d; use fewer splits or a smaller batch, or kb_attn_mma "
                "with scratch of your own\n", need, B, nh, n_splits, hd, KB_STATIC_SCRATCH_FLOATS);
        return (int)cudaErrorInvalidValue;
    }
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
    if (!base_of_device[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_attn_static_scratch);
        if (e != cudaSuccess || !p) return (int)(e != cudaSuccess ? e : cudaErrorInvalidSymbol);
        base_of_device[dev] = (float*)p;
    }
    float* part_o = base_of_device[dev];
    float* part_ml = part_o + (size_t)B * nh * n_splits * hd;
    return kb_attn_mma(q, ldq, out, ldo, part_o, part_ml, slot, q_start, kv_len, B, nh, nkv, hd, scale, window, pool,
                       table, table_stride, n_pages, 1, n_splits, status, st);
}
