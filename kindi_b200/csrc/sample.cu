// Picking the next token on the GPU: greedy, or temperature sampling with top-k, top-p and min-p, and the repeat
// penalty. A row of logits is shared by a thread-block cluster of up to eight CTAs (their histograms meet through the
// cluster's shared-memory window); nothing but the chosen token ids leaves the device.
//
// The distribution is the reference's (kindi/sampling.py:91-114): keep the top_k best (0: all); of those keep the
// best-first prefix in which the probability mass before a token is below top_p (probabilities at temperature 1, or
// at the temperature when hf_order is set: kindi/sampling.py:19,103); keep tokens with z >= z_max + ln(min_p); then
// p = softmax((z - z_max) / temperature). Greedy is the argmax with ties to the lowest id (kindi/nbq.cu:670-694).
// The reference finds its candidates on the GPU and finishes on the host (kindi/kindi.cu:743-787, a threshold found by
// bisection); here the three cuts become one threshold on the logit value, found by radix selection (counts for
// top-k, probability mass for top-p), and the draw is an inverse-CDF walk over the kept tokens in token-id order with
// a uniform number that the caller supplies per row. Masses are summed as 64-bit fixed-point integers, so every sum
// is exact in any order and the result is the same on every run, however the row is cut between CTAs. Every pass
// reads the row in coalesced order; a warp's lanes that fall into the same histogram bin add once between them (most
// logits of a row share their leading byte: one atomic per element on the same word took 2.7 ms for top-p alone over
// 166,144 logits, against 0.14 ms now; top-k 20 with top-p 0.8: 0.43 -> 0.09 ms).
#include "common.cuh"

#define SM_THREADS 1024
#define SM_FIX 1099511627776.0          // 2^40: weights in (0, 1] as fixed point

// a logit as an unsigned key of the same order; -0 and +0, equal as numbers, get the same key
__device__ __forceinline__ unsigned sm_key(float f) {
    unsigned u = __float_as_uint(f);
    if (u == 0x80000000u) u = 0u;
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ unsigned long long sm_fix(float w) { return (unsigned long long)((double)w * SM_FIX); }

// block-wide argmax with ties to the lowest index
__device__ void sm_argmax(const float* z, int V, float* s_v, int* s_i, float& best, int& best_i) {
    float v = -INFINITY;
    int idx = 0x7fffffff;
    // within a thread indices rise, so ">" keeps the lowest index of a tie
    int i;
    if ((((uintptr_t)z) & 15) == 0) {
        // four neighbouring logits per load, four loads in flight per thread
        const float4* z4 = (const float4*)z;
        const int n4 = V >> 2;
        int j = threadIdx.x;
#define SM_TAKE4(q, base)                                                        \
        do {                                                                     \
            if (q.x > v || idx == 0x7fffffff) { v = q.x; idx = (base); }         \
            if (q.y > v) { v = q.y; idx = (base) + 1; }                          \
            if (q.z > v) { v = q.z; idx = (base) + 2; }                          \
            if (q.w > v) { v = q.w; idx = (base) + 3; }                          \
        } while (0)
        for (; j + 3 * SM_THREADS < n4; j += 4 * SM_THREADS) {
            const float4 q0 = z4[j], q1 = z4[j + SM_THREADS], q2 = z4[j + 2 * SM_THREADS], q3 = z4[j + 3 * SM_THREADS];
            SM_TAKE4(q0, 4 * j);
            SM_TAKE4(q1, 4 * (j + SM_THREADS));
            SM_TAKE4(q2, 4 * (j + 2 * SM_THREADS));
            SM_TAKE4(q3, 4 * (j + 3 * SM_THREADS));
        }
        for (; j < n4; j += SM_THREADS) {
            const float4 q0 = z4[j];
            SM_TAKE4(q0, 4 * j);
        }
#undef SM_TAKE4
        i = 4 * n4 + threadIdx.x;                       // the last V % 4 logits
    } else {
        i = threadIdx.x;
        for (; i + 3 * SM_THREADS < V; i += 4 * SM_THREADS) {
            const float x0 = z[i], x1 = z[i + SM_THREADS], x2 = z[i + 2 * SM_THREADS], x3 = z[i + 3 * SM_THREADS];
            if (x0 > v || idx == 0x7fffffff) { v = x0; idx = i; }
            if (x1 > v) { v = x1; idx = i + SM_THREADS; }
            if (x2 > v) { v = x2; idx = i + 2 * SM_THREADS; }
            if (x3 > v) { v = x3; idx = i + 3 * SM_THREADS; }
        }
    }
    for (; i < V; i += SM_THREADS) {
        float x = z[i];
        if (x > v || idx == 0x7fffffff) { v = x; idx = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float v2 = __shfl_xor_sync(0xffffffffu, v, o);
        int i2 = __shfl_xor_sync(0xffffffffu, idx, o);
        if (v2 > v || (v2 == v && i2 < idx)) { v = v2; idx = i2; }
    }
    if ((threadIdx.x & 31) == 0) { s_v[threadIdx.x >> 5] = v; s_i[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < SM_THREADS / 32; w++)
            if (s_v[w] > v || (s_v[w] == v && s_i[w] < idx)) { v = s_v[w]; idx = s_i[w]; }
        s_v[0] = v;
        s_i[0] = idx;
    }
    __syncthreads();
    best = s_v[0];
    best_i = s_i[0];
    __syncthreads();
}

// Every logit of the row once, in coalesced order (four neighbouring logits a thread where the row is 16-byte aligned,
// several loads in flight): f(i, x, live) with live = false past the row's end. Every thread of the block calls f the
// same number of times, so f may use warp-wide operations.
template <class F>
__device__ __forceinline__ void sm_scan(const float* z, int V, F f) {
    const int tid = threadIdx.x;
    if ((((uintptr_t)z) & 15) == 0) {
        const float4* z4 = (const float4*)z;
        const int n4 = V >> 2, n_it = (n4 + SM_THREADS - 1) / SM_THREADS;
        for (int it = 0; it < n_it; it += 4) {
            float4 q[4];
            bool live[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int j = (it + u) * SM_THREADS + tid;
                live[u] = it + u < n_it && j < n4;
                q[u] = live[u] ? z4[j] : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                if (it + u < n_it) {                                 // (the same for the whole block)
                    const int i = 4 * ((it + u) * SM_THREADS + tid);
                    f(i, q[u].x, live[u]);
                    f(i + 1, q[u].y, live[u]);
                    f(i + 2, q[u].z, live[u]);
                    f(i + 3, q[u].w, live[u]);
                }
            }
        }
        const int i = 4 * n4 + tid;                                  // the last V % 4 logits
        const bool live = tid < 4 && i < V;
        f(i, live ? z[i] : 0.0f, live);
    } else {
        const int n_it = (V + SM_THREADS - 1) / SM_THREADS;
        for (int it = 0; it < n_it; it += 4) {
            float q[4];
            bool live[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int i = (it + u) * SM_THREADS + tid;
                live[u] = it + u < n_it && i < V;
                q[u] = live[u] ? z[i] : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < 4; u++)
                if (it + u < n_it) f((it + u) * SM_THREADS + tid, q[u], live[u]);
        }
    }
}

// One more in bin `bin` of a 256-bin histogram in shared memory (bin < 0: nothing). The lanes of a warp that hit the same
// bin add once between them: with logits, most of a row shares a few leading bytes, and one atomic per lane on the
// same word would take the pass a hundred times longer. The warp goes through its distinct bins one by one (there are
// two or three). Called by all 32 lanes.
__device__ __forceinline__ void sm_hist_count(unsigned* s_cnt, int bin) {
    unsigned todo = __ballot_sync(0xffffffffu, bin >= 0);
    const int lane = threadIdx.x & 31;
    while (todo) {
        const int leader = __ffs(todo) - 1;
        const int b = __shfl_sync(0xffffffffu, bin, leader);
        const unsigned same = __ballot_sync(0xffffffffu, bin == b);
        if (lane == leader) atomicAdd(&s_cnt[b], (unsigned)__popc(same));
        todo &= ~same;
    }
}
// The same for fixed-point masses (each at most 2^40): the lanes of a bin add their masses in two 20-bit halves, whose
// sums over 32 lanes fit 32 bits, and one lane adds the 64-bit sum to the histogram.
__device__ __forceinline__ void sm_hist_mass(unsigned long long* s_mass, int bin, unsigned long long w) {
    unsigned todo = __ballot_sync(0xffffffffu, bin >= 0);
    const int lane = threadIdx.x & 31;
    while (todo) {
        const int leader = __ffs(todo) - 1;
        const int b = __shfl_sync(0xffffffffu, bin, leader);
        const unsigned same = __ballot_sync(0xffffffffu, bin == b);
        if (bin == b) {
            const unsigned lo = __reduce_add_sync(same, (unsigned)(w & 0xFFFFFull));
            const unsigned hi = __reduce_add_sync(same, (unsigned)(w >> 20));
            if (lane == leader) atomicAdd(&s_mass[b], ((unsigned long long)hi << 20) + (unsigned long long)lo);
        }
        todo &= ~same;
    }
}

__device__ __forceinline__ unsigned long long sm_shfl_up64(unsigned long long v, int o) {
    return __shfl_up_sync(0xffffffffu, v, o);
}

#define SM_CTA_CHUNKS 1024      // pieces of a row whose masses a CTA keeps for the draw (one a thread)
#define SM_MAX_SLICES 8         // the most CTAs (one thread-block cluster) that share a row

// ---- the cluster's shared window: every CTA of a row's cluster reads the others' histograms and sums
__device__ __forceinline__ unsigned sm_cta_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void sm_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ unsigned sm_remote(const void* mine, unsigned rank) {     // `mine` as CTA `rank` has it
    unsigned r;
    const unsigned a = (unsigned)__cvta_generic_to_shared(mine);
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
    return r;
}
__device__ __forceinline__ unsigned sm_ld32(unsigned cluster_addr) {
    unsigned v;
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(cluster_addr) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long sm_ld64(unsigned cluster_addr) {
    unsigned long long v;
    asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(cluster_addr) : "memory");
    return v;
}

// One row is shared by a cluster of SM_SLICES CTAs (eight when a step has few rows, fewer when the rows alone fill the
// SMs): CTA s scans the s-th stretch of the row (whole pieces of 128 m
// logits), histograms are built per CTA in its own shared memory and, after a cluster barrier, every CTA adds up all
// of them and makes the same choice (the sums are integers, so all agree). The histograms alternate between two
// buffers, so a CTA may clear the next pass's while a neighbour still reads this pass's.
template <int SM_SLICES>
__global__ void __cluster_dims__(SM_SLICES, 1, 1) __launch_bounds__(SM_THREADS)
k_sample(const float* KB_STEP_DATA logits, long long ld, int V, float temperature, int top_k, float top_p,
         float min_p, int hf_order, const float* __restrict__ uniform, int* __restrict__ out) {
    __shared__ float s_v[32];
    __shared__ int s_i[32];
    __shared__ unsigned s_cnt[2][256];
    __shared__ unsigned long long s_mass[2][256];
    __shared__ unsigned s_tot32[256];
    __shared__ unsigned long long s_tot64[256];
    __shared__ unsigned long long s_red[32];
    __shared__ unsigned s_sel[2];
    __shared__ unsigned long long s_sel64[2];
    __shared__ unsigned long long s_chunk[SM_CTA_CHUNKS];
    __shared__ float s_best_v;
    __shared__ int s_best_i;
    __shared__ unsigned long long s_slice_total;
    static_assert(SM_CTA_CHUNKS <= SM_THREADS, "a thread per piece");
    kb_pdl_launch();
    kb_pdl_wait();
    const int row = blockIdx.x / SM_SLICES, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const unsigned rank = sm_cta_rank();
    const float* z = logits + (size_t)row * ld;
    // the row in pieces of 128 m logits; this CTA's stretch of whole pieces
    const int m = (V + 128 * SM_CTA_CHUNKS * SM_SLICES - 1) / (128 * SM_CTA_CHUNKS * SM_SLICES);
    const int piece = 128 * m, n_pieces = (V + piece - 1) / piece;
    const int pps = (n_pieces + SM_SLICES - 1) / SM_SLICES;                 // pieces per CTA (at most SM_CTA_CHUNKS)
    const int pc0 = min(n_pieces, (int)rank * pps), pc1 = min(n_pieces, pc0 + pps);
    const int lo = pc0 * piece, hi = min(V, pc1 * piece), n = max(0, hi - lo);
    const float* zs = z + lo;

    // ---- the best logit of the row (ties: the lowest token id)
    float zmax;
    int imax;
    sm_argmax(zs, n, s_v, s_i, zmax, imax);
    if (tid == 0) {
        s_best_v = n > 0 ? zmax : -INFINITY;
        s_best_i = n > 0 ? imax + lo : 0x7fffffff;
    }
    __syncthreads();
    sm_cluster_sync();
    {
        float v = -INFINITY;
        int idx = 0x7fffffff;
        if (lane < SM_SLICES) {
            v = __uint_as_float(sm_ld32(sm_remote(&s_best_v, lane)));
            idx = (int)sm_ld32(sm_remote(&s_best_i, lane));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float v2 = __shfl_xor_sync(0xffffffffu, v, o);
            const int i2 = __shfl_xor_sync(0xffffffffu, idx, o);
            if (v2 > v || (v2 == v && i2 < idx)) { v = v2; idx = i2; }
        }
        zmax = v;
        imax = idx;
    }
    if (!(temperature > 0.0f)) {
        if (tid == 0 && rank == 0) out[row] = imax;
        sm_cluster_sync();                      // nobody leaves while a neighbour may still read its shared memory
        return;
    }
    int pass = 0;                               // which histogram buffer
    // ---- top-k: the key of the k-th best logit, by radix selection on the keys, eight bits a pass
    unsigned thr = 0;
    if (top_k > 0 && top_k < V) {
        unsigned prefix = 0, mask = 0;
        unsigned kk = (unsigned)top_k;
        for (int shift = 24; shift >= 0; shift -= 8, pass ^= 1) {
            unsigned* cnt = s_cnt[pass];
            if (tid < 256) cnt[tid] = 0;
            __syncthreads();
            sm_scan(zs, n, [&](int, float x, bool live) {
                const unsigned key = sm_key(x);
                sm_hist_count(cnt, (live && (key & mask) == prefix) ? (int)((key >> shift) & 255u) : -1);
            });
            __syncthreads();
            sm_cluster_sync();
            if (tid < 256) {                    // the cluster's histogram: a thread a bin
                unsigned t = 0;
#pragma unroll
                for (unsigned r = 0; r < SM_SLICES; r++) t += sm_ld32(sm_remote(&cnt[tid], r));
                s_tot32[tid] = t;
            }
            __syncthreads();
            if (warp == 0) {
                // from bin 255 down: the first bin with which the count reaches kk. Lane l has the bins 255 - 8 l - j.
                unsigned c[8], sum = 0;
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    c[j] = s_tot32[255 - 8 * lane - j];
                    sum += c[j];
                }
                unsigned incl = sum;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const unsigned nn = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) incl += nn;
                }
                const unsigned excl = incl - sum;
                const bool mine = excl < kk && kk <= incl;
                if (mine) {
                    unsigned run = excl;
                    int digit = 255 - 8 * lane - 7;
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        if (run + c[j] >= kk) { digit = 255 - 8 * lane - j; break; }
                        run += c[j];
                    }
                    s_sel[0] = (unsigned)digit;
                    s_sel[1] = kk - run;
                }
                if (__ballot_sync(0xffffffffu, mine) == 0u && lane == 31) {      // (fewer than kk keys: cannot happen)
                    s_sel[0] = 0u;
                    s_sel[1] = kk - incl;
                }
            }
            __syncthreads();
            prefix |= s_sel[0] << shift;
            mask |= 255u << shift;
            kk = s_sel[1];
            __syncthreads();
        }
        thr = prefix;
    }
    // ---- top-p: the key of the last token of the best-first prefix whose preceding mass is below top_p
    if (top_p > 0.0f && top_p < 1.0f) {
        const float inv_t = hf_order ? 1.0f / temperature : 1.0f;
        unsigned prefix = 0, mask = 0;
        unsigned long long above = 0, target = 0;
        for (int shift = 24; shift >= 0; shift -= 8, pass ^= 1) {
            unsigned long long* mass = s_mass[pass];
            if (tid < 256) mass[tid] = 0;
            __syncthreads();
            sm_scan(zs, n, [&](int, float x, bool live) {
                const unsigned key = sm_key(x);
                const bool in = live && key >= thr && (key & mask) == prefix;
                sm_hist_mass(mass, in ? (int)((key >> shift) & 255u) : -1, in ? sm_fix(expf((x - zmax) * inv_t)) : 0ull);
            });
            __syncthreads();
            sm_cluster_sync();
            if (tid < 256) {
                unsigned long long t = 0;
#pragma unroll
                for (unsigned r = 0; r < SM_SLICES; r++) t += sm_ld64(sm_remote(&mass[tid], r));
                s_tot64[tid] = t;
            }
            __syncthreads();
            if (warp == 0) {
                unsigned long long c[8], sum = 0;
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    c[j] = s_tot64[255 - 8 * lane - j];
                    sum += c[j];
                }
                unsigned long long incl = sum;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const unsigned long long nn = sm_shfl_up64(incl, o);
                    if (lane >= o) incl += nn;
                }
                const unsigned long long all = __shfl_sync(0xffffffffu, incl, 31);
                if (shift == 24) target = (unsigned long long)((double)top_p * (double)all);   // (the first pass sees all kept mass)
                const unsigned long long excl = incl - sum;
                // from bin 255 down: the first bin that holds mass and with which the mass reaches the target
                const unsigned hit = __ballot_sync(0xffffffffu, sum > 0 && above + incl >= target);
                const unsigned holds = __ballot_sync(0xffffffffu, sum > 0);
                if (hit) {
                    if (lane == __ffs(hit) - 1) {
                        unsigned long long run = above + excl;
                        int digit = -1;
#pragma unroll
                        for (int j = 0; j < 8; j++) {
                            if (digit < 0 && c[j] != 0) {
                                if (run + c[j] >= target) digit = 255 - 8 * lane - j;
                                else run += c[j];
                            }
                        }
                        s_sel[0] = (unsigned)digit;
                        s_sel64[0] = run;
                    }
                } else if (holds) {
                    // the target is never reached (rounding): the lowest bin that holds mass, with all the mass above it
                    if (lane == 31 - __clz(holds)) {
                        int last = 0;
#pragma unroll
                        for (int j = 0; j < 8; j++)
                            if (c[j] != 0) last = j;
                        s_sel[0] = (unsigned)(255 - 8 * lane - last);
                        s_sel64[0] = above + all - c[last];
                    }
                } else if (lane == 0) {
                    s_sel[0] = 0u;
                    s_sel64[0] = above;
                }
                if (lane == 0) s_sel64[1] = target;
            }
            __syncthreads();
            prefix |= s_sel[0] << shift;
            mask |= 255u << shift;
            above = s_sel64[0];
            target = s_sel64[1];
            __syncthreads();
        }
        if (prefix > thr) thr = prefix;
    }
    // ---- min-p
    if (min_p > 0.0f) {
        unsigned km = sm_key(zmax + logf(min_p));
        if (km > thr) thr = km;
    }
    // ---- the draw: the kept tokens in token-id order. A warp adds up a piece's masses with coalesced loads, the
    // pieces' sums are scanned (within the CTA, then over the cluster's CTAs in order), and the one piece that holds the
    // target is walked again by the CTA that has it. Masses are integers: every order gives the same sums.
    const float inv_temp = 1.0f / temperature;
    auto weight = [&](int i) -> unsigned long long {
        if (i >= hi) return 0ull;
        const float x = z[i];
        return sm_key(x) >= thr ? sm_fix(expf((x - zmax) * inv_temp)) : 0ull;
    };
    const int my_pieces = pc1 - pc0;
    for (int c0 = warp; c0 < my_pieces; c0 += 4 * (SM_THREADS / 32)) {
        unsigned long long sum[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int c = c0 + u * (SM_THREADS / 32);
            if (c < my_pieces)
                for (int r = 0; r < m; r++) {
                    const int i = lo + c * piece + r * 128 + lane;
                    sum[u] += weight(i) + weight(i + 32) + weight(i + 64) + weight(i + 96);
                }
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int c = c0 + u * (SM_THREADS / 32);
            unsigned long long v = sum[u];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && c < my_pieces) s_chunk[c] = v;
        }
    }
    __syncthreads();
    // exclusive scan of this CTA's pieces: thread t has piece t
    const unsigned long long mine = tid < my_pieces ? s_chunk[tid] : 0ull;
    unsigned long long incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long nn = sm_shfl_up64(incl, o);
        if (lane >= o) incl += nn;
    }
    if (lane == 31) s_red[warp] = incl;
    __syncthreads();
    unsigned long long warp_off = 0, cta_total = 0;
    for (int w = 0; w < SM_THREADS / 32; w++) {
        if (w < warp) warp_off += s_red[w];
        cta_total += s_red[w];
    }
    if (tid == 0) s_slice_total = cta_total;
    __syncthreads();
    sm_cluster_sync();
    unsigned long long before = 0, total = 0;               // the mass in the CTAs before this one; in the whole row
#pragma unroll
    for (unsigned r = 0; r < SM_SLICES; r++) {
        const unsigned long long t = sm_ld64(sm_remote(&s_slice_total, r));
        if (r < rank) before += t;
        total += t;
    }
    const unsigned long long excl = before + warp_off + incl - mine;
    float u = uniform[row];
    u = u < 0.0f ? 0.0f : u;
    unsigned long long target = (unsigned long long)((double)u * (double)total);
    if (total > 0 && target >= total) target = total - 1;
    if (tid == 0) s_sel[0] = 0xffffffffu;
    if (total == 0 && rank == 0 && tid == 0) out[row] = imax;     // cannot happen (the best token always weighs 1); be safe
    __syncthreads();
    if (total > 0 && mine > 0 && target >= excl && target < excl + mine) {
        s_sel[0] = (unsigned)tid;
        s_sel64[0] = excl;
    }
    __syncthreads();
    if (warp == 0 && s_sel[0] != 0xffffffffu) {
        // the piece with the target: 32 logits at a time, in token order
        const int c = (int)s_sel[0];
        unsigned long long run = s_sel64[0];
        bool done = false;
        for (int i0 = lo + c * piece; i0 < lo + c * piece + piece && i0 < hi && !done; i0 += 32) {
            const unsigned long long w = weight(i0 + lane);
            unsigned long long in = w;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned long long nn = sm_shfl_up64(in, o);
                if (lane >= o) in += nn;
            }
            const bool here = w > 0 && target >= run + in - w && target < run + in;
            const unsigned found = __ballot_sync(0xffffffffu, here);
            if (found) {
                if (here) out[row] = i0 + lane;
                done = true;
            }
            run += __shfl_sync(0xffffffffu, in, 31);
        }
    }
    sm_cluster_sync();                          // nobody leaves while a neighbour may still read its shared memory
}

extern "C" int kb_sample(const float* logits, long long ld, int R, int V, float temperature, int top_k, float top_p,
                         float min_p, int hf_order, const float* uniform, int* out, cudaStream_t st) {
    if (R <= 0) return 0;
    // As many CTAs a row as keep the whole launch in one wave. A CTA of 1024 threads has an SM to itself, and a cluster
    // has to fit into one GPC: measured on a B200 (148 SMs), 96 CTAs in clusters of eight and 128 in clusters of four
    // or two run at once; one row more and the launch takes two rounds (top-k + top-p, 166,144 logits: 12 rows in
    // eights 108 us, 16 rows 198 us in eights and 133 us in fours).
    int sms = 148, dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    const int room8 = sms * 2 / 3, room = sms - sms / 8;
#define SM_GO(S)                                                                                                      \
    kb_launch(k_sample<S>, R * S, SM_THREADS, 0, st, logits, ld, V, temperature, top_k, top_p, min_p, hf_order, uniform, \
              out)
    // (a cluster size this device or partition cannot place is answered with an error at the launch: the next
    // smaller one is tried then)
    cudaError_t e = cudaErrorUnknown;
    if (R * 8 <= room8) e = SM_GO(8);
    if (e != cudaSuccess && R * 4 <= room) { cudaGetLastError(); e = SM_GO(4); }
    if (e != cudaSuccess && R * 2 <= room) { cudaGetLastError(); e = SM_GO(2); }
    if (e != cudaSuccess) { cudaGetLastError(); e = SM_GO(1); }
#undef SM_GO
    return (int)(e != cudaSuccess ? e : cudaGetLastError());
}

// the repeat penalty: z[t] /= rp when positive, *= rp when negative, for each listed token of the row
// (kindi/sampling.py:117-123). recent: [R][n_recent], each row's distinct recent tokens, padded with -1.
__global__ void k_penalize(float* KB_STEP_DATA logits, long long ld, int V, const int* __restrict__ recent,
                           int n_recent, float rp) {
    kb_pdl_launch();
    kb_pdl_wait();
    const int row = blockIdx.x;
    float* z = logits + (size_t)row * ld;
    for (int j = threadIdx.x; j < n_recent; j += blockDim.x) {
        const int t = recent[(size_t)row * n_recent + j];
        if (t >= 0 && t < V) {
            const float v = z[t];
            z[t] = v > 0.0f ? v / rp : v * rp;
        }
    }
}

extern "C" int kb_penalize(float* logits, long long ld, int R, int V, const int* recent, int n_recent, float rp,
                           cudaStream_t st) {
    if (R <= 0 || n_recent <= 0) return 0;
    kb_launch(k_penalize, R, 256, 0, st, logits, ld, V, recent, n_recent, rp);
    KB_LAUNCH_RET();
}
