// Host-side launchers around kernels of ahtx/kindi, which are included as they stand (kindi/nbq_grids.h, kindi/nbq.cu,
// kindi/nbq_fa.cu: the reference concatenates its sources in this order before it compiles them,
// kindi/nanbeige.py:49-51, with --use_fast_math, :58). Only the kernels that take and give 32-bit tensors are
// launched: the fused add + RMS norm, the rotation with the key/value store, the decode attention over position
// splits with its merge, the prompt attention, and the two-stage argmax, all for 5 query heads per key/value head of
// size 128. Grids and blocks are the reference's own (kindi/nanbeige.py:703-724, 944-952).
#include "nbq_grids.h"
#include "nbq.cu"
#include "nbq_fa.cu"

static int done() { cudaError_t e = cudaGetLastError(); if (e != cudaSuccess) return (int)e; return (int)cudaDeviceSynchronize(); }

extern "C" int ref_add_rms(const float* x, const float* add, const float* w, int n, float eps, float* y) {
    nbq_add_rms<<<1, 1024>>>(x, add, w, n, eps, y, nullptr, nullptr);
    return done();
}
extern "C" int ref_rope_store(float* q, const float* k, const float* v, const int* pos, int nh, int nkv,
                              float theta_scale, void* kc, void* vc, int ctx) {
    nbq_rope_store<<<nh + nkv, 64>>>(q, k, v, pos, nh, nkv, theta_scale, (__half*)kc, (__half*)vc, ctx);
    return done();
}
extern "C" int ref_attn_decode_g5(const float* q, const void* kc, const void* vc, const int* pos, int ctx, float scale,
                                  float* part_o, float* part_ms, int qstride, int nkv, int nsplit, int rows, float* out) {
    nbq_attn_part_g5<<<dim3(nkv, nsplit, rows), 256>>>(q, (const __half*)kc, (const __half*)vc, pos, ctx, scale, part_o,
                                                       part_ms, qstride);
    nbq_attn_merge<<<dim3(nkv * 5, rows), 128>>>(part_o, part_ms, nsplit, out);
    return done();
}
extern "C" int ref_fa_prefill_g5(const float* q, int ld, int nt, int pos0, const void* kc, const void* vc, int ctx,
                                 float scale, float* out, int nkv) {
    nbq_fa_prefill_g5<<<dim3((5 * nt + 63) / 64, nkv), 128, 2 * 64 * NBQ_FLD * 2>>>(q, ld, nt, pos0, (const __half*)kc,
                                                                                  (const __half*)vc, ctx, scale, out);
    return done();
}
extern "C" int ref_argmax(const float* x, int n, float* pv, int* pi, int* out) {
    nbq_argmax_part<<<256, 256>>>(x, n, pv, pi);
    nbq_argmax_final<<<1, 32>>>(pv, pi, 256, out, nullptr);
    return done();
}
