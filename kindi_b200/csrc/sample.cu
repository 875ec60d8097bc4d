// Picking the next token on the GPU: greedy, or temperature sampling with top-k, top-p and min-p, and the repeat
// penalty. One block per row of logits; nothing but the chosen token ids leaves the device.
//
// The distribution is the reference's (kindi/sampling.py:91-114): keep the top_k best (0: all); of those keep the
// best-first prefix in which the probability mass before a token is below top_p (probabilities at temperature 1, or
// at the temperature when hf_order is set: kindi/sampling.py:19,103); keep tokens with z >= z_max + ln(min_p); then
// p = softmax((z - z_max) / temperature). Greedy is the argmax with ties to the lowest id (kindi/nbq.cu:670-694).
// The reference finds its candidates on the GPU and finishes on the host (kindi/kindi.cu:743-787, a threshold found by
// bisection); here the three cuts become one threshold on the logit value, found by radix selection (counts for
// top-k, probability mass for top-p), and the draw is an inverse-CDF walk over the kept tokens in token-id order with
// a uniform number that the caller supplies per row. Masses are summed as 64-bit fixed-point integers, so every sum
// is exact in any order and the result is the same on every run.
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

// exact block sum of 64-bit integers; the result is returned to every thread
__device__ unsigned long long sm_block_sum(unsigned long long v, unsigned long long* s_red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = v;
    __syncthreads();
    unsigned long long t = 0;
    for (int w = 0; w < SM_THREADS / 32; w++) t += s_red[w];
    __syncthreads();
    return t;
}

__global__ void __launch_bounds__(SM_THREADS) k_sample(const float* KB_STEP_DATA logits, long long ld, int V,
        float temperature, int top_k, float top_p, float min_p, int hf_order, const float* __restrict__ uniform,
        int* __restrict__ out) {
    __shared__ float s_v[32];
    __shared__ int s_i[32];
    __shared__ unsigned s_cnt[256];
    __shared__ unsigned long long s_mass[256];
    __shared__ unsigned long long s_red[32];
    __shared__ unsigned s_sel[2];
    __shared__ unsigned long long s_sel64[2];
    kb_pdl_launch();
    kb_pdl_wait();
    const int row = blockIdx.x, tid = threadIdx.x;
    const float* z = logits + (size_t)row * ld;
    float zmax;
    int imax;
    sm_argmax(z, V, s_v, s_i, zmax, imax);
    if (!(temperature > 0.0f)) {
        if (tid == 0) out[row] = imax;
        return;
    }
    // ---- top-k: the key of the k-th best logit
    unsigned thr = 0;
    if (top_k > 0 && top_k < V) {
        unsigned prefix = 0, mask = 0;
        unsigned kk = (unsigned)top_k;
        for (int shift = 24; shift >= 0; shift -= 8) {
            if (tid < 256) s_cnt[tid] = 0;
            __syncthreads();
            for (int i = tid; i < V; i += SM_THREADS) {
                unsigned key = sm_key(z[i]);
                if ((key & mask) == prefix) atomicAdd(&s_cnt[(key >> shift) & 255u], 1u);
            }
            __syncthreads();
            if (tid == 0) {
                unsigned run = 0;
                int digit = 0;
                for (int b = 255; b >= 0; b--) {
                    if (run + s_cnt[b] >= kk) { digit = b; break; }
                    run += s_cnt[b];
                }
                s_sel[0] = (unsigned)digit;
                s_sel[1] = kk - run;
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
        unsigned long long mine = 0;
        for (int i = tid; i < V; i += SM_THREADS)
            if (sm_key(z[i]) >= thr) mine += sm_fix(expf((z[i] - zmax) * inv_t));
        const unsigned long long total = sm_block_sum(mine, s_red);
        const unsigned long long target = (unsigned long long)((double)top_p * (double)total);
        unsigned prefix = 0, mask = 0;
        unsigned long long above = 0;
        for (int shift = 24; shift >= 0; shift -= 8) {
            if (tid < 256) s_mass[tid] = 0;
            __syncthreads();
            for (int i = tid; i < V; i += SM_THREADS) {
                unsigned key = sm_key(z[i]);
                if (key >= thr && (key & mask) == prefix)
                    atomicAdd(&s_mass[(key >> shift) & 255u], sm_fix(expf((z[i] - zmax) * inv_t)));
            }
            __syncthreads();
            if (tid == 0) {
                unsigned long long run = above;
                int digit = -1, lowest = 0;
                for (int b = 255; b >= 0; b--) {
                    if (s_mass[b] == 0) continue;
                    lowest = b;
                    if (run + s_mass[b] >= target) { digit = b; break; }
                    run += s_mass[b];
                }
                if (digit < 0) { digit = lowest; run -= s_mass[lowest]; }
                s_sel[0] = (unsigned)digit;
                s_sel64[0] = run;
            }
            __syncthreads();
            prefix |= s_sel[0] << shift;
            mask |= 255u << shift;
            above = s_sel64[0];
            __syncthreads();
        }
        if (prefix > thr) thr = prefix;
    }
    // ---- min-p
    if (min_p > 0.0f) {
        unsigned km = sm_key(zmax + logf(min_p));
        if (km > thr) thr = km;
    }
    // ---- the draw: walk the kept tokens in token-id order
    const float inv_temp = 1.0f / temperature;
    const int chunk = (V + SM_THREADS - 1) / SM_THREADS;
    const int lo = tid * chunk, hi = min(V, lo + chunk);
    unsigned long long mine = 0;
    for (int i = lo; i < hi; i++)
        if (sm_key(z[i]) >= thr) mine += sm_fix(expf((z[i] - zmax) * inv_temp));
    // exclusive scan of the per-thread sums (integers: exact)
    unsigned long long incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        unsigned long long n = __shfl_up_sync(0xffffffffu, incl, o);
        if ((tid & 31) >= o) incl += n;
    }
    if ((tid & 31) == 31) s_red[tid >> 5] = incl;
    __syncthreads();
    unsigned long long warp_off = 0, total = 0;
    for (int w = 0; w < SM_THREADS / 32; w++) {
        if (w < (tid >> 5)) warp_off += s_red[w];
        total += s_red[w];
    }
    const unsigned long long excl = warp_off + incl - mine;
    float u = uniform[row];
    u = u < 0.0f ? 0.0f : u;
    unsigned long long target = (unsigned long long)((double)u * (double)total);
    if (total > 0 && target >= total) target = total - 1;
    if (tid == 0) out[row] = imax;              // total == 0 cannot happen (the best token always weighs 1); be safe
    __syncthreads();
    if (mine > 0 && target >= excl && target < excl + mine) {
        unsigned long long run = excl;
        int pick = imax;
        for (int i = lo; i < hi; i++) {
            if (sm_key(z[i]) >= thr) {
                unsigned long long w = sm_fix(expf((z[i] - zmax) * inv_temp));
                if (target < run + w) { pick = i; break; }
                run += w;
            }
        }
        out[row] = pick;
    }
}

extern "C" int kb_sample(const float* logits, long long ld, int R, int V, float temperature, int top_k, float top_p,
                         float min_p, int hf_order, const float* uniform, int* out, cudaStream_t st) {
    if (R <= 0) return 0;
    kb_launch(k_sample, R, SM_THREADS, 0, st, logits, ld, V, temperature, top_k, top_p, min_p, hf_order, uniform, out);
    KB_LAUNCH_RET();
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
