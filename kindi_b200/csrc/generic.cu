// Plain kernels for every operation of a step, templated on the storage type.
//
// With float storage they ARE the true 32-bit path of the model: no tensor cores, no reduced-precision matrix
// mode, no fast-math intrinsics; every sum is taken in an order that depends only on absolute positions and on the
// operand's own indices, never on how many rows share the launch, so logits do not change with the way the work is
// cut. With bfloat16 storage they are the slow-but-general versions of the serving kernels (every head size in
// steps of 2, any number of heads and groups), kept as the reference beside each fast kernel.
//
// Formulas follow the reference's order of operations: fused residual add + RMS norm (kindi/nbq.cu:412-453),
// rotary position encoding with individually rounded products (kindi/nbq.cu:127-130; rotate-half pairing as
// kindi/dspine.cu:151-174), attention with an online softmax over runs of 32 positions and a running maximum that
// starts at -1e30 (kindi/nbq.cu:525-633), SwiGLU g / (1 + exp(-g)) * u (kindi/nbq.cu:461-467).
#include "common.cuh"

int g_kb_pdl = 1;
extern "C" void kb_set_pdl(int on) { g_kb_pdl = on ? 1 : 0; }

// ------------------------------------------------------------------------------------------------ embedding
// x[t][:] = table[tok[t]][:] as 32-bit (no scaling: kindi/nbq.cu:472-487)
template <typename TW>
__global__ void k_embed(const TW* __restrict__ table, const int* __restrict__ tok, float* __restrict__ x, int E,
                        int vocab, float scale, int* status) {
    kb_pdl_launch();
    kb_pdl_wait();
    const int t = blockIdx.x;
    const int id = tok[t];
    float* xr = x + (size_t)t * E;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicOr(status, KB_ST_BAD_TOKEN);
        for (int i = threadIdx.x; i < E; i += blockDim.x) xr[i] = 0.0f;
        return;
    }
    const TW* row = table + (size_t)id * E;
    if (scale == 1.0f) {
        for (int i = threadIdx.x; i < E; i += blockDim.x) xr[i] = kb_to_f<TW>(row[i]);
    } else {
        for (int i = threadIdx.x; i < E; i += blockDim.x) xr[i] = kb_to_f<TW>(row[i]) * scale;
    }
}

// x[t] = table[tok[t]] * scale (scale 1: the row as stored, the reference's embedding: kindi/nbq.cu:472-487)
extern "C" int kb_embed(const void* table, int wdtype, const int* tok, float* x, int T, int E, int vocab,
                        float scale, int* status, cudaStream_t st) {
    if (T <= 0) return 0;
    if (wdtype == KB_F32)
        kb_launch(k_embed<float>, T, 256, 0, st, (const float*)table, tok, x, E, vocab, scale, status);
    else kb_launch(k_embed<bf16>, T, 256, 0, st, (const bf16*)table, tok, x, E, vocab, scale, status);
    KB_LAUNCH_RET();
}

// ------------------------------------------------------------------------------------------------ logits: scale, soft cap
// z = z * scale, then (cap > 0) z = cap * tanh(z / cap), in place: the options a head part may carry
__global__ void k_logit_post(float* KB_STEP_DATA z, long long n, float scale, float cap) {
    kb_pdl_launch();
    kb_pdl_wait();
    const float inv = cap > 0.0f ? 1.0f / cap : 0.0f;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        float v = z[i] * scale;
        if (cap > 0.0f) v = cap * tanhf(v * inv);
        z[i] = v;
    }
}

extern "C" int kb_logit_post(float* z, long long n, float scale, float cap, cudaStream_t st) {
    if (n <= 0) return 0;
    const int blocks = (int)((n + 1023) / 1024 < 1184 ? (n + 1023) / 1024 : 1184);
    kb_launch(k_logit_post, blocks, 256, 0, st, z, n, scale, cap);
    KB_LAUNCH_RET();
}

// ------------------------------------------------------------------------------------------------ add + RMS norm
// row r of the output is row t = rows ? rows[r] : r of the residual. v = x[t] + sum_s delta[s][t] (s in order);
// written back to x when write_back; y = (rsqrt(mean(v^2) + eps) * v) * w, the two products rounded one after the
// other as the reference does (kindi/nbq.cu:428-430).
// The planes are read with independent loads (eight in flight per element) and then added in order, so the sum is
// the same as a plain loop's while the few blocks of a decode step are not bound by load latency.
#define NORM_THREADS 1024
#define NORM_MAX_E 51200
__device__ __forceinline__ float kb_sum_planes(float v, const float* __restrict__ d, int n, size_t stride) {
    for (int s0 = 0; s0 < n; s0 += 8) {
        float t[8];
#pragma unroll
        for (int j = 0; j < 8; j++) t[j] = (s0 + j < n) ? d[(size_t)(s0 + j) * stride] : 0.0f;
#pragma unroll
        for (int j = 0; j < 8; j++)
            if (s0 + j < n) v += t[j];
    }
    return v;
}
__device__ __forceinline__ float4 kb_sum_planes4(float4 v, const float* __restrict__ d, int n, size_t stride) {
    for (int s0 = 0; s0 < n; s0 += 8) {
        float4 t[8];
#pragma unroll
        for (int j = 0; j < 8; j++)
            t[j] = (s0 + j < n) ? *(const float4*)(d + (size_t)(s0 + j) * stride) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 8; j++)
            if (s0 + j < n) {
                v.x += t[j].x;
                v.y += t[j].y;
                v.z += t[j].z;
                v.w += t[j].w;
            }
    }
    return v;
}
// VEC: the width is a multiple of 4 and every row is 16-byte aligned: a thread takes four neighbouring elements (one
// pass for widths up to 4096) with all its loads in flight at once. Each element's own sum (residual, then the
// planes in order) is the same in both forms.
template <typename TY, typename TW, bool VEC>
__global__ void __launch_bounds__(NORM_THREADS) k_add_rmsnorm(float* KB_STEP_DATA x, const float* KB_STEP_DATA delta,
        int n_delta, size_t delta_stride, const TW* __restrict__ w, float eps, TY* __restrict__ y,
        const int* __restrict__ rows, int T, int E, int write_back, int* status) {
    extern __shared__ float sv[];
    __shared__ float red[NORM_THREADS / 32];
    kb_pdl_launch();
    const int r = blockIdx.x;
    int t = rows ? rows[r] : r;                  // (the row list is step metadata, written before the step's kernels)
    if (t < 0 || t >= T) {
        if (threadIdx.x == 0) atomicOr(status, KB_ST_BAD_ROW);
        t = 0;
    }
    float* xr = x + (size_t)t * E;
    const float* dr = delta + (size_t)t * E;
    float ss = 0.0f;
    if (VEC && E <= NORM_THREADS * 4) {
        // the whole row in one pass, four elements a thread, kept in registers; the gains are fetched before the wait
        // for the kernel that produces the row. Sums are those of the general form below.
        const int i = threadIdx.x * 4;
        float w4[4] = {0.f, 0.f, 0.f, 0.f};
        if (i < E) {
#pragma unroll
            for (int c = 0; c < 4; c++) w4[c] = kb_to_f<TW>(w[i + c]);
        }
        kb_pdl_wait();
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < E) {
            v = *(const float4*)(xr + i);
            if (n_delta > 0) v = kb_sum_planes4(v, dr + i, n_delta, delta_stride);
            if (write_back) *(float4*)(xr + i) = v;
            ss = fmaf(v.x, v.x, ss);
            ss = fmaf(v.y, v.y, ss);
            ss = fmaf(v.z, v.z, ss);
            ss = fmaf(v.w, v.w, ss);
        }
        ss = kb_warp_sum(ss);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
        __syncthreads();
        float tot = red[0];
#pragma unroll
        for (int k = 1; k < NORM_THREADS / 32; k++) tot += red[k];
        const float scale = rsqrtf(tot / (float)E + eps);
        if (i < E) {
            TY* yr = y + (size_t)r * E + i;
            yr[0] = kb_from_f<TY>(__fmul_rn(__fmul_rn(scale, v.x), w4[0]));
            yr[1] = kb_from_f<TY>(__fmul_rn(__fmul_rn(scale, v.y), w4[1]));
            yr[2] = kb_from_f<TY>(__fmul_rn(__fmul_rn(scale, v.z), w4[2]));
            yr[3] = kb_from_f<TY>(__fmul_rn(__fmul_rn(scale, v.w), w4[3]));
        }
        return;
    }
    kb_pdl_wait();
    if (VEC) {
        for (int i = threadIdx.x * 4; i < E; i += NORM_THREADS * 4) {
            float4 v = *(const float4*)(xr + i);
            if (n_delta > 0) v = kb_sum_planes4(v, dr + i, n_delta, delta_stride);
            if (write_back) *(float4*)(xr + i) = v;
            *(float4*)(sv + i) = v;
            ss = fmaf(v.x, v.x, ss);
            ss = fmaf(v.y, v.y, ss);
            ss = fmaf(v.z, v.z, ss);
            ss = fmaf(v.w, v.w, ss);
        }
    } else {
        for (int i = threadIdx.x; i < E; i += NORM_THREADS) {
            float v = xr[i];
            if (n_delta > 0) v = kb_sum_planes(v, dr + i, n_delta, delta_stride);
            if (write_back) xr[i] = v;
            sv[i] = v;
            ss = fmaf(v, v, ss);
        }
    }
    ss = kb_warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = red[0];
#pragma unroll
    for (int k = 1; k < NORM_THREADS / 32; k++) tot += red[k];
    const float scale = rsqrtf(tot / (float)E + eps);
    TY* yr = y + (size_t)r * E;
    for (int i = threadIdx.x; i < E; i += NORM_THREADS)
        yr[i] = kb_from_f<TY>(__fmul_rn(__fmul_rn(scale, sv[i]), kb_to_f<TW>(w[i])));
}

// The same operation with one warp per row, for prompt-sized steps of the bf16 path: no shared memory and no block
// barrier; the row is read twice (the second time from the cache, it has just been written). The sum of squares is
// taken in another order than in k_add_rmsnorm, so the true 32-bit path, whose results must not depend on how many rows
// a step has, never uses it.
template <typename TW>
__global__ void __launch_bounds__(256) k_add_rmsnorm_warp(float* KB_STEP_DATA x, const float* KB_STEP_DATA delta,
        int n_delta, size_t delta_stride, const TW* __restrict__ w, float eps, bf16* __restrict__ y, int T, int E) {
    kb_pdl_launch();
    kb_pdl_wait();
    const int t = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= T) return;
    float* xr = x + (size_t)t * E;
    const float* dr = delta + (size_t)t * E;
    float ss = 0.0f;
    // four chunks of the row at a time: all their loads are issued before the first sum is stored (a store to the
    // row would otherwise hold back the loads behind it)
    for (int i0 = lane * 4; i0 < E; i0 += 4 * 128) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; u++)
            if (i0 + u * 128 < E) v[u] = *(const float4*)(xr + i0 + u * 128);
        if (n_delta > 0) {
#pragma unroll
            for (int u = 0; u < 4; u++)
                if (i0 + u * 128 < E) v[u] = kb_sum_planes4(v[u], dr + i0 + u * 128, n_delta, delta_stride);
#pragma unroll
            for (int u = 0; u < 4; u++)
                if (i0 + u * 128 < E) *(float4*)(xr + i0 + u * 128) = v[u];
        }
#pragma unroll
        for (int u = 0; u < 4; u++)
            if (i0 + u * 128 < E) {
                ss = fmaf(v[u].x, v[u].x, ss);
                ss = fmaf(v[u].y, v[u].y, ss);
                ss = fmaf(v[u].z, v[u].z, ss);
                ss = fmaf(v[u].w, v[u].w, ss);
            }
    }
    ss = kb_warp_sum(ss);
    const float scale = rsqrtf(ss / (float)E + eps);
    bf16* yr = y + (size_t)t * E;
    for (int i = lane * 4; i < E; i += 128) {
        const float4 v = *(const float4*)(xr + i);
        const float w0 = kb_to_f<TW>(w[i]), w1 = kb_to_f<TW>(w[i + 1]), w2 = kb_to_f<TW>(w[i + 2]), w3 = kb_to_f<TW>(w[i + 3]);
        __nv_bfloat162 a = __floats2bfloat162_rn(__fmul_rn(__fmul_rn(scale, v.x), w0), __fmul_rn(__fmul_rn(scale, v.y), w1));
        __nv_bfloat162 b = __floats2bfloat162_rn(__fmul_rn(__fmul_rn(scale, v.z), w2), __fmul_rn(__fmul_rn(scale, v.w), w3));
        *(uint2*)(yr + i) = make_uint2(*(uint32_t*)&a, *(uint32_t*)&b);
    }
}

// One warp per row with the whole row in registers (widths up to NCH * 128): every load of the row and of the planes is
// in flight before the first sum, and the row is read once. Same sums in the same order as k_add_rmsnorm_warp.
template <typename TW, int NCH>
__global__ void __launch_bounds__(256, 2) k_add_rmsnorm_regs(float* KB_STEP_DATA x, const float* KB_STEP_DATA delta,
        int n_delta, size_t delta_stride, const TW* __restrict__ w, float eps, bf16* __restrict__ y, int T, int E) {
    kb_pdl_launch();
    kb_pdl_wait();
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= T) return;
    float* xr = x + (size_t)t * E;
    const float* dr = delta + (size_t)t * E;
    float4 v[NCH];
#pragma unroll
    for (int c = 0; c < NCH; c++) {
        const int i = (c * 32 + lane) * 4;
        v[c] = i < E ? *(const float4*)(xr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int s = 0; s < n_delta; s++) {
        const float* ds = dr + (size_t)s * delta_stride;
#pragma unroll
        for (int c0 = 0; c0 < NCH; c0 += 8) {
            float4 d[8];
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int i = ((c0 + j) * 32 + lane) * 4;
                d[j] = (c0 + j < NCH && i < E) ? *(const float4*)(ds + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int j = 0; j < 8; j++)
                if (c0 + j < NCH) {
                    v[c0 + j].x += d[j].x;
                    v[c0 + j].y += d[j].y;
                    v[c0 + j].z += d[j].z;
                    v[c0 + j].w += d[j].w;
                }
        }
    }
    float ss = 0.0f;
#pragma unroll
    for (int c = 0; c < NCH; c++) {
        const int i = (c * 32 + lane) * 4;
        if (i < E) {
            if (n_delta > 0) *(float4*)(xr + i) = v[c];
            ss = fmaf(v[c].x, v[c].x, ss);
            ss = fmaf(v[c].y, v[c].y, ss);
            ss = fmaf(v[c].z, v[c].z, ss);
            ss = fmaf(v[c].w, v[c].w, ss);
        }
    }
    ss = kb_warp_sum(ss);
    const float scale = rsqrtf(ss / (float)E + eps);
    bf16* yr = y + (size_t)t * E;
#pragma unroll
    for (int c = 0; c < NCH; c++) {
        const int i = (c * 32 + lane) * 4;
        if (i < E) {
            const float w0 = kb_to_f<TW>(w[i]), w1 = kb_to_f<TW>(w[i + 1]), w2 = kb_to_f<TW>(w[i + 2]),
                        w3 = kb_to_f<TW>(w[i + 3]);
            __nv_bfloat162 a = __floats2bfloat162_rn(__fmul_rn(__fmul_rn(scale, v[c].x), w0),
                                                     __fmul_rn(__fmul_rn(scale, v[c].y), w1));
            __nv_bfloat162 b = __floats2bfloat162_rn(__fmul_rn(__fmul_rn(scale, v[c].z), w2),
                                                     __fmul_rn(__fmul_rn(scale, v[c].w), w3));
            *(uint2*)(yr + i) = make_uint2(*(uint32_t*)&a, *(uint32_t*)&b);
        }
    }
}

// Four warps per row, each with a quarter of the row in registers (widths up to 4 * NC * 128), and the planes taken
// several at a time: a step of a few hundred rows has too few rows to hide the round trips of one warp per row
// behind other rows (a row of 2560 with six planes: 18 trips for one warp, 4 here). The planes are added in order;
// the four warps' sums of squares are added in warp order.
template <typename TW, int NC>
__global__ void __launch_bounds__(256, 2) k_add_rmsnorm_row4(float* KB_STEP_DATA x, const float* KB_STEP_DATA delta,
        int n_delta, size_t delta_stride, const TW* __restrict__ w, float eps, bf16* __restrict__ y, int T, int E) {
    constexpr int PB = 12 / NC > 0 ? 12 / NC : 1;          // planes in flight
    __shared__ float s_ss[8];
    kb_pdl_launch();
    kb_pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, part = warp & 3;
    const int t = blockIdx.x * 2 + (warp >> 2);
    const bool live = t < T;
    float* xr = x + (size_t)t * E;
    const float* dr = delta + (size_t)t * E;
    float4 v[NC];
#pragma unroll
    for (int c = 0; c < NC; c++) {
        const int i = ((part * NC + c) * 32 + lane) * 4;
        v[c] = (live && i < E) ? *(const float4*)(xr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int s0 = 0; s0 < n_delta; s0 += PB) {
        float4 d[PB][NC];
#pragma unroll
        for (int k = 0; k < PB; k++)
#pragma unroll
            for (int c = 0; c < NC; c++) {
                const int i = ((part * NC + c) * 32 + lane) * 4;
                d[k][c] = (live && s0 + k < n_delta && i < E) ? *(const float4*)(dr + (size_t)(s0 + k) * delta_stride + i)
                                                              : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
        for (int k = 0; k < PB; k++)
            if (s0 + k < n_delta) {
#pragma unroll
                for (int c = 0; c < NC; c++) {
                    v[c].x += d[k][c].x;
                    v[c].y += d[k][c].y;
                    v[c].z += d[k][c].z;
                    v[c].w += d[k][c].w;
                }
            }
    }
    float ss = 0.0f;
#pragma unroll
    for (int c = 0; c < NC; c++) {
        const int i = ((part * NC + c) * 32 + lane) * 4;
        if (live && i < E) {
            if (n_delta > 0) *(float4*)(xr + i) = v[c];
            ss = fmaf(v[c].x, v[c].x, ss);
            ss = fmaf(v[c].y, v[c].y, ss);
            ss = fmaf(v[c].z, v[c].z, ss);
            ss = fmaf(v[c].w, v[c].w, ss);
        }
    }
    ss = kb_warp_sum(ss);
    if (lane == 0) s_ss[warp] = ss;
    __syncthreads();
    if (!live) return;
    const float* q = s_ss + (warp & ~3);
    const float scale = rsqrtf((((q[0] + q[1]) + q[2]) + q[3]) / (float)E + eps);
    bf16* yr = y + (size_t)t * E;
#pragma unroll
    for (int c = 0; c < NC; c++) {
        const int i = ((part * NC + c) * 32 + lane) * 4;
        if (i < E) {
            const float w0 = kb_to_f<TW>(w[i]), w1 = kb_to_f<TW>(w[i + 1]), w2 = kb_to_f<TW>(w[i + 2]),
                        w3 = kb_to_f<TW>(w[i + 3]);
            __nv_bfloat162 a = __floats2bfloat162_rn(__fmul_rn(__fmul_rn(scale, v[c].x), w0),
                                                     __fmul_rn(__fmul_rn(scale, v[c].y), w1));
            __nv_bfloat162 b = __floats2bfloat162_rn(__fmul_rn(__fmul_rn(scale, v[c].z), w2),
                                                     __fmul_rn(__fmul_rn(scale, v[c].w), w3));
            *(uint2*)(yr + i) = make_uint2(*(uint32_t*)&a, *(uint32_t*)&b);
        }
    }
}

// Rows of a step for which four warps share a row. Below, a block per row is as fast or faster (128 rows of 2560
// with one plane: 2.6 against 3.6 us; 160: 4.2 against 3.7); beyond, one warp a row has rows enough to hide its
// round trips behind (one plane: 512 rows 9.7 against 4.0 us, 1024: 10.8 / 7.0, 1536: 11.9 / 10.0, 2000: 11.8 / 12.7).
#define NORM_ROW4_MIN_T 160
#define NORM_ROW4_MAX_T 1792

extern "C" int kb_add_rmsnorm(float* x, const float* delta, int n_delta, long long delta_stride, const void* w,
                              int wdtype, float eps, void* y, int ydtype, const int* rows, int n_out, int T, int E,
                              int write_back, int* status, cudaStream_t st) {
    if (n_out <= 0) return 0;
    size_t sm = (size_t)E * sizeof(float);
    if (E > NORM_MAX_E) return (int)cudaErrorInvalidValue;
    const bool vec = (E % 4 == 0) && (((uintptr_t)x) % 16 == 0) && (((uintptr_t)delta) % 16 == 0) &&
                     (delta_stride % 4 == 0);
    cudaError_t e = cudaSuccess;
    if (ydtype == KB_BF16 && vec && rows == nullptr && n_out == T && T >= NORM_ROW4_MIN_T && T < NORM_ROW4_MAX_T &&
        (write_back || n_delta == 0) && (((uintptr_t)y) % 8) == 0 && E <= 4 * 10 * 128) {
#define KB_NORM_ROW4(NC)                                                                                           \
    do {                                                                                                           \
        if (wdtype == KB_F32)                                                                                      \
            e = kb_launch(k_add_rmsnorm_row4<float, NC>, (T + 1) / 2, 256, 0, st, x, delta, n_delta,               \
                          (size_t)delta_stride, (const float*)w, eps, (bf16*)y, T, E);                             \
        else                                                                                                       \
            e = kb_launch(k_add_rmsnorm_row4<bf16, NC>, (T + 1) / 2, 256, 0, st, x, delta, n_delta,                \
                          (size_t)delta_stride, (const bf16*)w, eps, (bf16*)y, T, E);                              \
        return (int)e;                                                                                             \
    } while (0)
        if (E <= 4 * 2 * 128) KB_NORM_ROW4(2);
        if (E <= 4 * 4 * 128) KB_NORM_ROW4(4);
        if (E <= 4 * 6 * 128) KB_NORM_ROW4(6);
        KB_NORM_ROW4(10);
#undef KB_NORM_ROW4
    }
    if (ydtype == KB_BF16 && vec && rows == nullptr && n_out == T && T >= 512 && (write_back || n_delta == 0) &&
        (((uintptr_t)y) % 8) == 0) {
// rows (warps) per block (1, 2 and 4 were measured slower on a 2048-row step)
#ifndef NORM_RW
#define NORM_RW 8
#endif
#define KB_NORM_REGS(NCH)                                                                                          \
    do {                                                                                                           \
        if (wdtype == KB_F32)                                                                                      \
            e = kb_launch(k_add_rmsnorm_regs<float, NCH>, (T + NORM_RW - 1) / NORM_RW, 32 * NORM_RW, 0, st, x, delta, n_delta, \
                          (size_t)delta_stride, (const float*)w, eps, (bf16*)y, T, E);                             \
        else                                                                                                       \
            e = kb_launch(k_add_rmsnorm_regs<bf16, NCH>, (T + NORM_RW - 1) / NORM_RW, 32 * NORM_RW, 0, st, x, delta, n_delta, \
                          (size_t)delta_stride, (const bf16*)w, eps, (bf16*)y, T, E);                              \
        return (int)e;                                                                                             \
    } while (0)
        if (E <= 8 * 128) KB_NORM_REGS(8);
        if (E <= 16 * 128) KB_NORM_REGS(16);
        if (E <= 24 * 128) KB_NORM_REGS(24);
#undef KB_NORM_REGS
        if (wdtype == KB_F32)
            e = kb_launch(k_add_rmsnorm_warp<float>, (T + 7) / 8, 256, 0, st, x, delta, n_delta, (size_t)delta_stride,
                          (const float*)w, eps, (bf16*)y, T, E);
        else
            e = kb_launch(k_add_rmsnorm_warp<bf16>, (T + 7) / 8, 256, 0, st, x, delta, n_delta, (size_t)delta_stride,
                          (const bf16*)w, eps, (bf16*)y, T, E);
        return (int)e;
    }
#define KB_NORM1(TY, TW, V)                                                                                      \
    do {                                                                                                         \
        if (sm > 48 * 1024)                                                                                      \
            cudaFuncSetAttribute(k_add_rmsnorm<TY, TW, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm); \
        e = kb_launch(k_add_rmsnorm<TY, TW, V>, n_out, NORM_THREADS, sm, st, x, delta, n_delta,                  \
                      (size_t)delta_stride, (const TW*)w, eps, (TY*)y, rows, T, E, write_back, status);          \
    } while (0)
#define KB_NORM(TY, TW)                \
    do {                               \
        if (vec) KB_NORM1(TY, TW, true); \
        else KB_NORM1(TY, TW, false);    \
    } while (0)
    if (ydtype == KB_F32 && wdtype == KB_F32) KB_NORM(float, float);
    else if (ydtype == KB_F32) KB_NORM(float, bf16);
    else if (wdtype == KB_F32) KB_NORM(bf16, float);
    else KB_NORM(bf16, bf16);
#undef KB_NORM
#undef KB_NORM1
    return (int)e;
}

// ------------------------------------------------------------------------------------------------ matrix product
// C[m][n] = sum_k A[m][k] * W[n][k]; each output's sum runs over k = 0, 1, 2, ... in order with 32-bit fused
// multiply-adds, so an output does not depend on the tile it lands in or on how many rows there are.
#define GS_BM 64
#define GS_BN 64
#define GS_BK 32
template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256) k_gemm_simt(const TA* KB_STEP_DATA A, const TW* __restrict__ W,
        TC* __restrict__ C, int M, int N, int K, int lda, int ldw, int ldc) {
    __shared__ float As[GS_BK][GS_BM + 1];
    __shared__ float Ws[GS_BK][GS_BN + 1];
    kb_pdl_launch();
    kb_pdl_wait();
    const int m0 = blockIdx.y * GS_BM, n0 = blockIdx.x * GS_BN;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;
    // the next K block's elements are requested before this one is multiplied: their way from memory runs beside the
    // products (the order of every output's sum does not change)
    constexpr int PER = GS_BM * GS_BK / 256;
    float ra[PER], rw[PER];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int j = 0; j < PER; j++) {
            const int e = tid + 256 * j, r = e / GS_BK, c = e % GS_BK;
            const int m = m0 + r, n = n0 + r, k = k0 + c;
            ra[j] = (m < M && k < K) ? kb_to_f<TA>(A[(size_t)m * lda + k]) : 0.0f;
            rw[j] = (n < N && k < K) ? kb_to_f<TW>(W[(size_t)n * ldw + k]) : 0.0f;
        }
    };
    fetch(0);
    for (int k0 = 0; k0 < K; k0 += GS_BK) {
#pragma unroll
        for (int j = 0; j < PER; j++) {
            const int e = tid + 256 * j, r = e / GS_BK, c = e % GS_BK;
            As[c][r] = ra[j];
            Ws[c][r] = rw[j];
        }
        __syncthreads();
        if (k0 + GS_BK < K) fetch(k0 + GS_BK);
#pragma unroll
        for (int k = 0; k < GS_BK; k++) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) b[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int n = n0 + tx * 4 + j;
            if (n < N) C[(size_t)m * ldc + n] = kb_from_f<TC>(acc[i][j]);
        }
    }
}

extern "C" int kb_gemm_simt(const void* A, int adtype, const void* W, int wdtype, void* C, int cdtype, int M, int N,
                            int K, int lda, int ldw, int ldc, cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    dim3 grid((N + GS_BN - 1) / GS_BN, (M + GS_BM - 1) / GS_BM);
#define KB_G(TA, TW, TC) \
    kb_launch(k_gemm_simt<TA, TW, TC>, grid, 256, 0, st, (const TA*)A, (const TW*)W, (TC*)C, M, N, K, lda, ldw, ldc)
    int code = adtype * 4 + wdtype * 2 + cdtype;
    switch (code) {
        case 0: KB_G(float, float, float); break;
        case 1: KB_G(float, float, bf16); break;
        case 2: KB_G(float, bf16, float); break;
        case 3: KB_G(float, bf16, bf16); break;
        case 4: KB_G(bf16, float, float); break;
        case 5: KB_G(bf16, float, bf16); break;
        case 6: KB_G(bf16, bf16, float); break;
        default: KB_G(bf16, bf16, bf16); break;
    }
#undef KB_G
    KB_LAUNCH_RET();
}

// ------------------------------------------------------------------------------------------------ rotary + store
// qkv: [T][(nh + 2 nkv) * hd] (q heads, then k heads, then v heads). Query heads are rotated in place; key heads
// are rotated and written to the cache at (slot of the row's sequence, the row's position); value heads are
// copied there. The rotation pairs element i with i + rot/2 (i < rot/2; elements from rot on pass through); the
// angle is (float)pos * inv_freq[i] in 32-bit, cosine and sine by the accurate library functions, and the four
// products are rounded one by one (kindi/nbq.cu:127-130).
template <typename TIN, typename T>
__global__ void k_rope_store(const TIN* KB_STEP_DATA in, int n_planes, size_t plane_stride, int ld_in,
        T* __restrict__ qout, int ldq, const float* __restrict__ inv_freq, int rot,
        const int* __restrict__ pos, const int* __restrict__ seq, const int* __restrict__ slot, int nh, int nkv,
        int hd, KbCacheView cv, int* status) {
    kb_pdl_launch();
    // positions, slots and the page table were written before the step's first kernel: they are read, and the first
    // angle of each thread is computed, before the wait for the kernel that produces the rows
    const int t = blockIdx.x, h = blockIdx.y;
    const int p = pos[t];
    if (p < 0) return;                               // a padding row of a recorded step: nothing to rotate or store
    const TIN* src = in + (size_t)t * ld_in + (size_t)h * hd;
    T* dst;
    const bool is_q = h < nh, is_k = !is_q && h < nh + nkv;
    if (is_q) {
        dst = qout + (size_t)t * ldq + (size_t)h * hd;
    } else {
        const int hk = is_k ? h - nh : h - nh - nkv;
        const int s = slot[seq[t]];
        const int page = cv.table[(size_t)s * cv.table_stride + p / KB_PAGE];
        if (page < 0 || page >= cv.n_pages) {
            if (threadIdx.x == 0) atomicOr(status, KB_ST_BAD_PAGE);
            return;
        }
        dst = (T*)cv.pool + kb_kv_offset(cv, page, is_k ? 0 : 1, hk, p % KB_PAGE);
    }
    auto rd = [&](int i) {
        float v = kb_to_f<TIN>(src[i]);
        for (int s0 = 1; s0 < n_planes; s0 += 8) {
            float t[8];
#pragma unroll
            for (int j = 0; j < 8; j++)
                t[j] = (s0 + j < n_planes) ? kb_to_f<TIN>(src[(size_t)(s0 + j) * plane_stride + i]) : 0.0f;
#pragma unroll
            for (int j = 0; j < 8; j++)
                if (s0 + j < n_planes) v += t[j];
        }
        return v;
    };
    const int half = rot / 2;
    float c_first = 1.0f, sn_first = 0.0f;
    if ((is_q || is_k) && (int)threadIdx.x < half) {
        const float ang = __fmul_rn((float)p, inv_freq[threadIdx.x]);
        c_first = cosf(ang);
        sn_first = sinf(ang);
    }
    kb_pdl_wait();
    if (is_q || is_k) {
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            float c = c_first, sn = sn_first;
            if (i != (int)threadIdx.x) {
                const float ang = __fmul_rn((float)p, inv_freq[i]);
                c = cosf(ang);
                sn = sinf(ang);
            }
            const float a = rd(i), b = rd(i + half);
            dst[i] = kb_from_f<T>(__fsub_rn(__fmul_rn(a, c), __fmul_rn(b, sn)));
            dst[i + half] = kb_from_f<T>(__fadd_rn(__fmul_rn(b, c), __fmul_rn(a, sn)));
        }
        if ((const void*)dst != (const void*)src || n_planes > 1)
            for (int i = rot + threadIdx.x; i < hd; i += blockDim.x) dst[i] = kb_from_f<T>(rd(i));
    } else {
        for (int i = threadIdx.x; i < hd; i += blockDim.x) dst[i] = kb_from_f<T>(rd(i));
    }
}

// The same operation with one block per row: cosine and sine of the row's angles are computed once into shared
// memory and used by every head, and each thread moves two neighbouring elements (and their partners) at a time.
// Taken for steps of 32 rows or more (fewer rows want the many small blocks of k_rope_store) when rot % 4 == 0,
// hd % 2 == 0 and the rows are aligned for two-element accesses; values are computed by the
// same expressions as in k_rope_store, so both give the same bits.
template <typename T> struct Kb2;
template <> struct Kb2<float> { typedef float2 type; };
template <> struct Kb2<bf16> { typedef __nv_bfloat162 type; };
__device__ __forceinline__ float2 kb_ld2(const float* p) { return *(const float2*)p; }
__device__ __forceinline__ float2 kb_ld2(const bf16* p) { return __bfloat1622float2(*(const __nv_bfloat162*)p); }
__device__ __forceinline__ void kb_st2(float* p, float2 v) { *(float2*)p = v; }
__device__ __forceinline__ void kb_st2(bf16* p, float2 v) { *(__nv_bfloat162*)p = __floats2bfloat162_rn(v.x, v.y); }

template <typename TIN, typename T>
__global__ void __launch_bounds__(256) k_rope_store_row(const TIN* KB_STEP_DATA in, int n_planes, size_t plane_stride,
        int ld_in, T* __restrict__ qout, int ldq, const float* __restrict__ inv_freq, int rot,
        const int* __restrict__ pos, const int* __restrict__ seq, const int* __restrict__ slot, int nh, int nkv,
        int hd, KbCacheView cv, int* status) {
    extern __shared__ float2 cs[];                  // [rot / 2]: (cos, sin) of the row's angles
    kb_pdl_launch();
    kb_pdl_wait();
    const int t = blockIdx.x;
    const int p = pos[t];
    if (p < 0) return;                               // a padding row of a recorded step (the whole block leaves)
    const int half = rot / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float ang = __fmul_rn((float)p, inv_freq[i]);
        cs[i] = make_float2(cosf(ang), sinf(ang));
    }
    T* kdst = nullptr;
    T* vdst = nullptr;
    if (nkv > 0) {
        const int s = slot[seq[t]];
        const int page = cv.table[(size_t)s * cv.table_stride + p / KB_PAGE];
        if (page < 0 || page >= cv.n_pages) {
            if (threadIdx.x == 0) atomicOr(status, KB_ST_BAD_PAGE);
        } else {
            kdst = (T*)cv.pool + kb_kv_offset(cv, page, 0, 0, p % KB_PAGE);
            vdst = (T*)cv.pool + kb_kv_offset(cv, page, 1, 0, p % KB_PAGE);
        }
    }
    __syncthreads();
    const TIN* row = in + (size_t)t * ld_in;
    auto rd2 = [&](int e) {                          // elements e, e + 1 of the row: the planes added in order
        float2 v = kb_ld2(row + e);
        for (int s0 = 1; s0 < n_planes; s0 += 8) {
            float2 tt[8];
#pragma unroll
            for (int j = 0; j < 8; j++)
                tt[j] = (s0 + j < n_planes) ? kb_ld2(row + (size_t)(s0 + j) * plane_stride + e) : make_float2(0.f, 0.f);
#pragma unroll
            for (int j = 0; j < 8; j++)
                if (s0 + j < n_planes) {
                    v.x += tt[j].x;
                    v.y += tt[j].y;
                }
        }
        return v;
    };
    const size_t head_stride = (size_t)KB_PAGE * hd;       // from one key/value head to the next inside a page
    // rotated heads: query heads, then key heads; an item is two neighbouring pairs of one head
    const int per_head = half / 2, n_rot = (nh + nkv) * per_head;
    for (int it = threadIdx.x; it < n_rot; it += blockDim.x) {
        const int h = it / per_head, i = (it % per_head) * 2;
        T* dst;
        if (h < nh) dst = qout + (size_t)t * ldq + (size_t)h * hd;
        else if (kdst) dst = kdst + (size_t)(h - nh) * head_stride;
        else continue;
        const float2 a = rd2(h * hd + i), b = rd2(h * hd + i + half);
        const float2 c0 = cs[i], c1 = cs[i + 1];
        float2 lo, hi;
        lo.x = __fsub_rn(__fmul_rn(a.x, c0.x), __fmul_rn(b.x, c0.y));
        lo.y = __fsub_rn(__fmul_rn(a.y, c1.x), __fmul_rn(b.y, c1.y));
        hi.x = __fadd_rn(__fmul_rn(b.x, c0.x), __fmul_rn(a.x, c0.y));
        hi.y = __fadd_rn(__fmul_rn(b.y, c1.x), __fmul_rn(a.y, c1.y));
        kb_st2(dst + i, lo);
        kb_st2(dst + i + half, hi);
    }
    // what is only copied: the elements past the rotated part of q and k heads, and the value heads
    const int tail2 = (hd - rot) / 2;
    if (tail2 > 0) {
        for (int it = threadIdx.x; it < (nh + nkv) * tail2; it += blockDim.x) {
            const int h = it / tail2, i = rot + (it % tail2) * 2;
            T* dst;
            if (h < nh) dst = qout + (size_t)t * ldq + (size_t)h * hd;
            else if (kdst) dst = kdst + (size_t)(h - nh) * head_stride;
            else continue;
            kb_st2(dst + i, rd2(h * hd + i));
        }
    }
    if (vdst) {
        const int hd2 = hd / 2;
        for (int it = threadIdx.x; it < nkv * hd2; it += blockDim.x) {
            const int h = it / hd2, i = (it % hd2) * 2;
            kb_st2(vdst + (size_t)h * head_stride + i, rd2((nh + nkv + h) * hd + i));
        }
    }
}

// One block per row as above, eight neighbouring elements (16 or 32 bytes) per access: taken when rot % 16 == 0,
// hd % 8 == 0 and everything is aligned for it. Same expressions, same bits.
__device__ __forceinline__ void kb_ld8(const float* p, float* o) {
    const float4 a = *(const float4*)p, b = *(const float4*)(p + 4);
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
__device__ __forceinline__ void kb_ld8(const bf16* p, float* o) {
    const uint4 r = *(const uint4*)p;
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float2 f = __bfloat1622float2(*(const __nv_bfloat162*)&w[j]);
        o[2 * j] = f.x;
        o[2 * j + 1] = f.y;
    }
}
__device__ __forceinline__ void kb_st8(float* p, const float* v) {
    *(float4*)p = make_float4(v[0], v[1], v[2], v[3]);
    *(float4*)(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void kb_st8(bf16* p, const float* v) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
        w[j] = *(uint32_t*)&h;
    }
    *(uint4*)p = make_uint4(w[0], w[1], w[2], w[3]);
}

// PLANES: the row is the sum of several planes (a decode step of many sequences). Without planes (a prompt) a thread
// keeps few registers, so that most rows of a prompt are resident at once. Each thread requests its first item's
// elements before it does anything else: those loads, the row's angles and its page lookup then wait side by side.
// TABLE: the cosines and sines of every row's angles were computed once for the step (k_rope_table: the same
// expressions, so the same bits) and are read from there, 64 bytes per item beside the item's own loads; without it
// each block computes its row's and shares them through shared memory.
template <typename TIN, typename T, bool PLANES, bool TABLE = false>
__global__ void __launch_bounds__(256, PLANES ? 1 : 5) k_rope_store_row8(const TIN* KB_STEP_DATA in, int n_planes,
        size_t plane_stride, int ld_in, T* __restrict__ qout, int ldq, const float* __restrict__ inv_freq, int rot,
        const int* __restrict__ pos, const int* __restrict__ seq, const int* __restrict__ slot, int nh, int nkv,
        int hd, KbCacheView cv, int* status, const float2* KB_STEP_DATA cs_table) {
    extern __shared__ float2 cs[];                  // [rot / 2]: (cos, sin) of the row's angles
    kb_pdl_launch();
    kb_pdl_wait();
    const int t = blockIdx.x;
    if (pos[t] < 0) return;                          // a padding row of a recorded step (the whole block leaves)
    const int half = rot / 2;
    const float2* cst = TABLE ? cs_table + (size_t)t * half : nullptr;
    const TIN* row = in + (size_t)t * ld_in;
    auto rd8 = [&](int e, float* v) {                // elements e .. e + 7 of the row: the planes added in order
        kb_ld8(row + e, v);
        if (PLANES) {
            for (int s0 = 1; s0 < n_planes; s0 += 4) {
                float tt[4][8];
#pragma unroll
                for (int j = 0; j < 4; j++)
                    if (s0 + j < n_planes) kb_ld8(row + (size_t)(s0 + j) * plane_stride + e, tt[j]);
#pragma unroll
                for (int j = 0; j < 4; j++)
                    if (s0 + j < n_planes) {
#pragma unroll
                        for (int c = 0; c < 8; c++) v[c] += tt[j][c];
                    }
            }
        }
    };
    // items of a row: rotated runs of eight pairs (query heads, then key heads), the runs past the rotated part of
    // those heads, the runs of the value heads
    const int per_head = half / 8, n_rot = (nh + nkv) * per_head;
    const int tail8 = (hd - rot) / 8, n_tail = (nh + nkv) * tail8;
    const int hd8 = hd / 8, n_items = n_rot + n_tail + nkv * hd8;
    auto load_item = [&](int it, float* a, float* b) {
        if (it < n_rot) {
            const int h = it / per_head, i = (it % per_head) * 8;
            rd8(h * hd + i, a);
            rd8(h * hd + i + half, b);
        } else if (it < n_rot + n_tail) {
            const int h = (it - n_rot) / tail8, i = rot + ((it - n_rot) % tail8) * 8;
            rd8(h * hd + i, a);
        } else {
            const int h = (it - n_rot - n_tail) / hd8, i = ((it - n_rot - n_tail) % hd8) * 8;
            rd8((nh + nkv + h) * hd + i, a);
        }
    };
    float a[8], b[8];
    float4 k4[4];                                    // TABLE: (cos, sin) of this thread's first item's eight pairs
    if ((int)threadIdx.x < n_items) {
        load_item(threadIdx.x, a, b);
        if (TABLE && (int)threadIdx.x < n_rot) {
            const float4* kp = (const float4*)(cst + ((int)threadIdx.x % per_head) * 8);
#pragma unroll
            for (int j = 0; j < 4; j++) k4[j] = kp[j];
        }
    }

    const int p = pos[t];
    if (!TABLE) {
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const float ang = __fmul_rn((float)p, inv_freq[i]);
            cs[i] = make_float2(cosf(ang), sinf(ang));
        }
    }
    T* kdst = nullptr;
    T* vdst = nullptr;
    if (nkv > 0) {
        const int s = slot[seq[t]];
        const int page = cv.table[(size_t)s * cv.table_stride + p / KB_PAGE];
        if (page < 0 || page >= cv.n_pages) {
            if (threadIdx.x == 0) atomicOr(status, KB_ST_BAD_PAGE);
        } else {
            kdst = (T*)cv.pool + kb_kv_offset(cv, page, 0, 0, p % KB_PAGE);
            vdst = (T*)cv.pool + kb_kv_offset(cv, page, 1, 0, p % KB_PAGE);
        }
    }
    if (!TABLE) __syncthreads();
    const size_t head_stride = (size_t)KB_PAGE * hd;       // from one key/value head to the next inside a page
    for (int it = threadIdx.x; it < n_items; it += blockDim.x) {
        if (it != (int)threadIdx.x) {
            load_item(it, a, b);
            if (TABLE && it < n_rot) {
                const float4* kp = (const float4*)(cst + (it % per_head) * 8);
#pragma unroll
                for (int j = 0; j < 4; j++) k4[j] = kp[j];
            }
        }
        if (it < n_rot) {
            const int h = it / per_head, i = (it % per_head) * 8;
            T* dst;
            if (h < nh) dst = qout + (size_t)t * ldq + (size_t)h * hd;
            else if (kdst) dst = kdst + (size_t)(h - nh) * head_stride;
            else continue;
            float lo[8], hi[8];
#pragma unroll
            for (int c = 0; c < 8; c++) {
                float2 k;
                if (TABLE) k = (c & 1) ? make_float2(k4[c >> 1].z, k4[c >> 1].w) : make_float2(k4[c >> 1].x, k4[c >> 1].y);
                else k = cs[i + c];
                lo[c] = __fsub_rn(__fmul_rn(a[c], k.x), __fmul_rn(b[c], k.y));
                hi[c] = __fadd_rn(__fmul_rn(b[c], k.x), __fmul_rn(a[c], k.y));
            }
            kb_st8(dst + i, lo);
            kb_st8(dst + i + half, hi);
        } else if (it < n_rot + n_tail) {
            const int h = (it - n_rot) / tail8, i = rot + ((it - n_rot) % tail8) * 8;
            T* dst;
            if (h < nh) dst = qout + (size_t)t * ldq + (size_t)h * hd;
            else if (kdst) dst = kdst + (size_t)(h - nh) * head_stride;
            else continue;
            kb_st8(dst + i, a);
        } else if (vdst) {
            const int h = (it - n_rot - n_tail) / hd8, i = ((it - n_rot - n_tail) % hd8) * 8;
            kb_st8(vdst + (size_t)h * head_stride + i, a);
        }
    }
}

// (cos, sin) of angle = float(pos[t]) * inv_freq[i] for every row t and pair i of a step: the angles are the same in
// every layer, so a step computes them once and its rotate-and-store kernels read them (float2 [T][half])
__global__ void k_rope_table(const int* __restrict__ pos, const float* __restrict__ inv_freq, int half, int T,
                             float2* __restrict__ out) {
    kb_pdl_launch();
    kb_pdl_wait();
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= T * half) return;
    const float ang = __fmul_rn((float)pos[e / half], inv_freq[e % half]);
    out[e] = make_float2(cosf(ang), sinf(ang));
}

extern "C" int kb_rope_table(const int* pos, const float* inv_freq, int rot, int T, void* out, cudaStream_t st) {
    const int half = rot / 2;
    if (T <= 0 || half <= 0) return 0;
    kb_launch(k_rope_table, (T * half + 255) / 256, 256, 0, st, pos, inv_freq, half, T, (float2*)out);
    KB_LAUNCH_RET();
}

// in: [n_planes][T][ld_in] (the planes are summed in order); in_dtype may be 32-bit planes with a bf16 cache / qout
// cs_table (may be null): float2 [T][rot / 2] made by kb_rope_table for these rows; used where the kernel form takes it
// Fewer rows than this (decode steps) go through the small blocks of k_rope_store: a row-wise block with planes holds
// most of an SM's registers, and the few SMs that such blocks occupy are closed to the CTAs of the attention kernel
// that is launched beside them (32 sequences at context 8192: 4.97 -> 4.66 ms a step; 64: 7.39 -> 7.32).
#define KB_ROPE_ROW_MIN_T 96
// the fewest rows for which kb_rope_store reads a table of the step's cosines and sines (kb_rope_table)
extern "C" int kb_rope_table_min_rows() { return KB_ROPE_ROW_MIN_T; }

extern "C" int kb_rope_store(const void* in, int in_dtype, int n_planes, long long plane_stride, int ld_in,
                             void* qout, int dtype, int ldq, const float* inv_freq, int rot, const int* pos,
                             const int* seq, const int* slot, int T, int nh, int nkv, int hd, void* pool,
                             const int* table, int table_stride, int n_pages, int* status, cudaStream_t st,
                             const void* cs_table) {
    if (T <= 0) return 0;
    KbCacheView cv{pool, table, table_stride, n_pages, nkv, hd};
    dim3 grid(T, nh + 2 * nkv);
    int thr = hd / 2 < 32 ? 32 : (hd / 2 > 128 ? 128 : ((hd / 2 + 31) / 32) * 32);
    const int in_el = in_dtype == KB_F32 ? 4 : 2, out_el = dtype == KB_F32 ? 4 : 2;
    const bool by_row = T >= KB_ROPE_ROW_MIN_T && rot % 4 == 0 && hd % 2 == 0 && ld_in % 2 == 0 && ldq % 2 == 0 && plane_stride % 2 == 0 &&
                        ((uintptr_t)in % (2 * in_el)) == 0 && ((uintptr_t)qout % (2 * out_el)) == 0 &&
                        ((uintptr_t)pool % (2 * out_el)) == 0 && rot / 2 * 8 <= 32 * 1024;
    const bool by_row8 = by_row && rot % 16 == 0 && hd % 8 == 0 && ld_in % 8 == 0 && ldq % 8 == 0 &&
                         plane_stride % 8 == 0 && ((uintptr_t)in % (8 * in_el)) == 0 &&
                         ((uintptr_t)qout % (8 * out_el)) == 0 && ((uintptr_t)pool % (8 * out_el)) == 0;
    const float2* cst = (const float2*)cs_table;
    const bool tab = by_row8 && cst && ((uintptr_t)cst % 16) == 0;
#define KB_RS(TIN, T_)                                                                                        \
    if (by_row8 && n_planes > 1 && tab)                                                                       \
        kb_launch(k_rope_store_row8<TIN, T_, true, true>, T, 256, 0, st,                                      \
                  (const TIN*)in, n_planes, (size_t)plane_stride, ld_in, (T_*)qout, ldq, inv_freq, rot, pos,  \
                  seq, slot, nh, nkv, hd, cv, status, cst);                                                   \
    else if (by_row8 && tab)                                                                                  \
        kb_launch(k_rope_store_row8<TIN, T_, false, true>, T, 256, 0, st,                                     \
                  (const TIN*)in, n_planes, (size_t)plane_stride, ld_in, (T_*)qout, ldq, inv_freq, rot, pos,  \
                  seq, slot, nh, nkv, hd, cv, status, cst);                                                   \
    else if (by_row8 && n_planes > 1)                                                                         \
        kb_launch(k_rope_store_row8<TIN, T_, true>, T, 256, (size_t)(rot / 2) * sizeof(float2), st,           \
                  (const TIN*)in, n_planes, (size_t)plane_stride, ld_in, (T_*)qout, ldq, inv_freq, rot, pos,  \
                  seq, slot, nh, nkv, hd, cv, status, cst);                                                   \
    else if (by_row8)                                                                                         \
        kb_launch(k_rope_store_row8<TIN, T_, false>, T, 256, (size_t)(rot / 2) * sizeof(float2), st,          \
                  (const TIN*)in, n_planes, (size_t)plane_stride, ld_in, (T_*)qout, ldq, inv_freq, rot, pos,  \
                  seq, slot, nh, nkv, hd, cv, status, cst);                                                   \
    else if (by_row)                                                                                               \
        kb_launch(k_rope_store_row<TIN, T_>, T, 256, (size_t)(rot / 2) * sizeof(float2), st, (const TIN*)in,   \
                  n_planes, (size_t)plane_stride, ld_in, (T_*)qout, ldq, inv_freq, rot, pos, seq, slot, nh,   \
                  nkv, hd, cv, status);                                                                       \
    else                                                                                                      \
    kb_launch(k_rope_store<TIN, T_>, grid, thr, 0, st, (const TIN*)in, n_planes, (size_t)plane_stride, ld_in,        \
                                                (T_*)qout, ldq, inv_freq, rot, pos, seq, slot, nh, nkv, hd,   \
                                                cv, status)
    if (in_dtype == KB_F32 && dtype == KB_F32) KB_RS(float, float);
    else if (in_dtype == KB_F32 && dtype == KB_BF16) KB_RS(float, bf16);
    else if (in_dtype == KB_BF16 && dtype == KB_BF16) KB_RS(bf16, bf16);
    else return (int)cudaErrorInvalidValue;
#undef KB_RS
    KB_LAUNCH_RET();
}

// ------------------------------------------------------------------------------------------------ attention
// One warp per (row, query head). The row attends the keys of its sequence at positions lo..pos, lo = 0 or
// pos - window + 1, read from the cache. Keys are taken in runs of 32 that start at multiples of 32 of the absolute
// position (lane = position for the scores, lane = dimension for P V) with a running maximum and sum, so the order
// of every sum depends on positions only: the same row gives the same bits whether it came in a prompt or alone.
#define AG_MAX_HD 256
template <typename T>
__global__ void __launch_bounds__(128) k_attn_generic(const T* KB_STEP_DATA q, int ldq, T* __restrict__ out,
        int ldo, const int* __restrict__ pos, const int* __restrict__ seq, const int* __restrict__ slot, int Tn,
        int nh, int group, int hd, float scale, int window, KbCacheView cv, int* status) {
    __shared__ float qs[4][AG_MAX_HD];
    kb_pdl_launch();
    kb_pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * 4 + warp;
    if (item >= (long long)Tn * nh) return;
    const int t = (int)(item / nh), h = (int)(item % nh);
    const int hk = h / group;
    const int p_q = pos[t];
    if (p_q < 0) return;                             // a padding row of a recorded step (the whole warp leaves)
    const int s = slot[seq[t]];
    const T* qr = q + (size_t)t * ldq + (size_t)h * hd;
    for (int d = lane; d < hd; d += 32) qs[warp][d] = __fmul_rn(kb_to_f<T>(qr[d]), scale);
    __syncwarp();
    const int lo = (window > 0 && p_q - window + 1 > 0) ? p_q - window + 1 : 0;
    const int* trow = cv.table + (size_t)s * cv.table_stride;
    float m = -1e30f, l = 0.0f;
    float o[AG_MAX_HD / 32];
#pragma unroll
    for (int i = 0; i < AG_MAX_HD / 32; i++) o[i] = 0.0f;
    for (int c0 = lo & ~31; c0 <= p_q; c0 += 32) {
        const int p = c0 + lane;
        const bool live = p >= lo && p <= p_q;
        float sc = -1e30f;
        const T* vrow = nullptr;
        bool ok = live;
        if (live) {
            const int page = trow[p / KB_PAGE];
            if (page < 0 || page >= cv.n_pages) {
                atomicOr(status, KB_ST_BAD_PAGE);
                ok = false;
            } else {
                const T* kr = (const T*)cv.pool + kb_kv_offset(cv, page, 0, hk, p % KB_PAGE);
                vrow = (const T*)cv.pool + kb_kv_offset(cv, page, 1, hk, p % KB_PAGE);
                float a = 0.0f;
                for (int d = 0; d < hd; d++) a = fmaf(qs[warp][d], kb_to_f<T>(kr[d]), a);
                sc = a;
            }
        }
        const float mx = kb_warp_max(ok ? sc : -1e30f);
        const float mn = fmaxf(m, mx);
        const float f = expf(m - mn);
        const float pr = ok ? expf(sc - mn) : 0.0f;
        l = l * f + kb_warp_sum(pr);
        m = mn;
#pragma unroll
        for (int i = 0; i < AG_MAX_HD / 32; i++) o[i] *= f;
        const unsigned mask = __ballot_sync(0xffffffffu, ok);
        for (int j = 0; j < 32; j++) {
            if (!((mask >> j) & 1u)) continue;
            const float pj = __shfl_sync(0xffffffffu, pr, j);
            const T* vj = (const T*)__shfl_sync(0xffffffffu, (unsigned long long)vrow, j);
#pragma unroll
            for (int i = 0; i < AG_MAX_HD / 32; i++) {
                const int d = i * 32 + lane;
                if (d < hd) o[i] = fmaf(pj, kb_to_f<T>(vj[d]), o[i]);
            }
        }
    }
    T* orow = out + (size_t)t * ldo + (size_t)h * hd;
#pragma unroll
    for (int i = 0; i < AG_MAX_HD / 32; i++) {
        const int d = i * 32 + lane;
        if (d < hd) orow[d] = kb_from_f<T>(o[i] / l);
    }
}

extern "C" int kb_attn_generic(const void* q, int dtype, int ldq, void* out, int ldo, const int* pos, const int* seq,
                               const int* slot, int T, int nh, int nkv, int hd, float scale, int window, void* pool,
                               const int* table, int table_stride, int n_pages, int* status, cudaStream_t st) {
    if (T <= 0) return 0;
    if (hd > AG_MAX_HD || nkv <= 0 || nh % nkv) return (int)cudaErrorInvalidValue;
    KbCacheView cv{pool, table, table_stride, n_pages, nkv, hd};
    long long items = (long long)T * nh;
    int grid = (int)((items + 3) / 4);
    if (dtype == KB_F32)
        kb_launch(k_attn_generic<float>, grid, 128, 0, st, (const float*)q, ldq, (float*)out, ldo, pos, seq, slot, T, nh,
                                                   nh / nkv, hd, scale, window, cv, status);
    else
        kb_launch(k_attn_generic<bf16>, grid, 128, 0, st, (const bf16*)q, ldq, (bf16*)out, ldo, pos, seq, slot, T, nh,
                                                  nh / nkv, hd, scale, window, cv, status);
    KB_LAUNCH_RET();
}

// ------------------------------------------------------------------------------------------------ SwiGLU
// gu: [T][2F] = gate then up; out[t][i] = gate / (1 + exp(-gate)) * up (kindi/nbq.cu:461-467)
template <typename TIN, typename T>
__global__ void k_swiglu(const TIN* KB_STEP_DATA gu, int n_planes, size_t plane_stride, T* __restrict__ out, int F,
                         long long total, int group) {
    kb_pdl_launch();
    kb_pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long t = i / F;
    const int c = (int)(i % F);
    const int gc = (c / group) * 2 * group + c % group;        // the gate's column; the up's is `group` further
    float g = 0.0f, u = 0.0f;
    for (int s0 = 0; s0 < n_planes; s0 += 4) {
        float tg[4], tu[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const bool on = s0 + j < n_planes;
            tg[j] = on ? kb_to_f<TIN>(gu[(size_t)(s0 + j) * plane_stride + t * 2 * F + gc]) : 0.0f;
            tu[j] = on ? kb_to_f<TIN>(gu[(size_t)(s0 + j) * plane_stride + t * 2 * F + gc + group]) : 0.0f;
        }
#pragma unroll
        for (int j = 0; j < 4; j++)
            if (s0 + j < n_planes) {
                g += tg[j];
                u += tu[j];
            }
    }
    out[i] = kb_from_f<T>(g / (1.0f + expf(-g)) * u);
}

// the same with a row per blockIdx.y and two neighbouring columns per thread (F even, aligned rows)
template <typename TIN, typename T>
__global__ void __launch_bounds__(256) k_swiglu2(const TIN* KB_STEP_DATA gu, int n_planes, size_t plane_stride,
                                                  T* __restrict__ out, int F, int group) {
    kb_pdl_launch();
    kb_pdl_wait();
    const int c = (blockIdx.x * 256 + threadIdx.x) * 2;
    if (c >= F) return;
    const size_t t = blockIdx.y;
    const TIN* g0 = gu + t * 2 * F + (c / group) * 2 * group + c % group;
    float2 g = make_float2(0.f, 0.f), u = make_float2(0.f, 0.f);
    for (int s0 = 0; s0 < n_planes; s0 += 4) {
        float2 tg[4], tu[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const bool on = s0 + j < n_planes;
            tg[j] = on ? kb_ld2(g0 + (size_t)(s0 + j) * plane_stride) : make_float2(0.f, 0.f);
            tu[j] = on ? kb_ld2(g0 + (size_t)(s0 + j) * plane_stride + group) : make_float2(0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < 4; j++)
            if (s0 + j < n_planes) {
                g.x += tg[j].x;
                g.y += tg[j].y;
                u.x += tu[j].x;
                u.y += tu[j].y;
            }
    }
    kb_st2(out + t * F + c, make_float2(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y));
}

// bf16 rows in, bf16 out, eight columns per thread with 16-byte accesses; exp and the division by the fast
// intrinsics (their error is far below one bf16 rounding)
__global__ void __launch_bounds__(256) k_swiglu8_bf16(const bf16* KB_STEP_DATA gu, bf16* __restrict__ out, int F,
                                                      int group) {
    kb_pdl_launch();
    kb_pdl_wait();
    const int c = (blockIdx.x * 256 + threadIdx.x) * 8;
    if (c >= F) return;
    const size_t t = blockIdx.y;
    const bf16* g0 = gu + t * 2 * F + (c / group) * 2 * group + c % group;
    const uint4 gv = *(const uint4*)g0, uv = *(const uint4*)(g0 + group);
    const __nv_bfloat162* g2 = (const __nv_bfloat162*)&gv;
    const __nv_bfloat162* u2 = (const __nv_bfloat162*)&uv;
    uint4 ov;
    __nv_bfloat162* o2 = (__nv_bfloat162*)&ov;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float2 g = __bfloat1622float2(g2[j]), u = __bfloat1622float2(u2[j]);
        o2[j] = __floats2bfloat162_rn(__fdividef(g.x, 1.0f + __expf(-g.x)) * u.x,
                                      __fdividef(g.y, 1.0f + __expf(-g.y)) * u.y);
    }
    *(uint4*)(out + t * F + c) = ov;
}

// gu: [n_planes][T][2F] (planes summed in order), 32-bit or the output's type. Columns come in groups: `group` gate
// columns, then the `group` up columns of the same outputs (group == F: all gates, then all ups).
extern "C" int kb_swiglu(const void* gu, int in_dtype, int n_planes, long long plane_stride, void* out, int dtype,
                         int T, int F, int group, cudaStream_t st) {
    if (group <= 0 || F % group) return (int)cudaErrorInvalidValue;
    long long total = (long long)T * F;
    if (total <= 0) return 0;
    int grid = (int)((total + 255) / 256);
    const int in_el = in_dtype == KB_F32 ? 4 : 2, out_el = dtype == KB_F32 ? 4 : 2;
    if (in_dtype == KB_BF16 && dtype == KB_BF16 && n_planes == 1 && F % 8 == 0 && group % 8 == 0 && ((uintptr_t)gu % 16) == 0 &&
        ((uintptr_t)out % 16) == 0 && T <= 65535) {
        dim3 g8((F / 8 + 255) / 256, T);
        kb_launch(k_swiglu8_bf16, g8, 256, 0, st, (const bf16*)gu, (bf16*)out, F, group);
        KB_LAUNCH_RET();
    }
    if (F % 2 == 0 && group % 2 == 0 && plane_stride % 2 == 0 && ((uintptr_t)gu % (2 * in_el)) == 0 &&
        ((uintptr_t)out % (2 * out_el)) == 0 && T <= 65535) {
        dim3 g2((F / 2 + 255) / 256, T);
        if (in_dtype == KB_F32 && dtype == KB_F32)
            kb_launch(k_swiglu2<float, float>, g2, 256, 0, st, (const float*)gu, n_planes, (size_t)plane_stride, (float*)out, F, group);
        else if (in_dtype == KB_F32 && dtype == KB_BF16)
            kb_launch(k_swiglu2<float, bf16>, g2, 256, 0, st, (const float*)gu, n_planes, (size_t)plane_stride, (bf16*)out, F, group);
        else if (in_dtype == KB_BF16 && dtype == KB_BF16)
            kb_launch(k_swiglu2<bf16, bf16>, g2, 256, 0, st, (const bf16*)gu, n_planes, (size_t)plane_stride, (bf16*)out, F, group);
        else return (int)cudaErrorInvalidValue;
        KB_LAUNCH_RET();
    }
    if (in_dtype == KB_F32 && dtype == KB_F32)
        kb_launch(k_swiglu<float, float>, grid, 256, 0, st, (const float*)gu, n_planes, (size_t)plane_stride, (float*)out, F, total, group);
    else if (in_dtype == KB_F32 && dtype == KB_BF16)
        kb_launch(k_swiglu<float, bf16>, grid, 256, 0, st, (const float*)gu, n_planes, (size_t)plane_stride, (bf16*)out, F, total, group);
    else if (in_dtype == KB_BF16 && dtype == KB_BF16)
        kb_launch(k_swiglu<bf16, bf16>, grid, 256, 0, st, (const bf16*)gu, n_planes, (size_t)plane_stride, (bf16*)out, F, total, group);
    else return (int)cudaErrorInvalidValue;
    KB_LAUNCH_RET();
}
