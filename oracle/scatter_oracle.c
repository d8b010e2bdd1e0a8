/*
 * CPU restatement of TorchEx's scatter path.  TEST INFRASTRUCTURE ONLY: it is
 * the checker for the CUDA library and the timed CPU baseline; nothing in the
 * shipped package links or calls it.
 *
 * Two families:
 *   oracle_ref_*  replay the arithmetic ORDER of the reference CUDA kernels
 *                 (torchex/src/scatter/scatter_kernel.cu) so that fp32 sums and
 *                 tie-breaking come out bit-identical to what those kernels
 *                 produce on a GPU;
 *   oracle_spec_* state the result the operators are meant to have: exact
 *                 (fp64) sums, maximum with the lowest row on ties, and the
 *                 backward of scatter_op.py.
 *
 * Build: gcc -O2 -fopenmp -ffp-contract=off -fPIC -shared (see oracle/Makefile).
 */
#include <float.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* Block width of the reference launchers: clamp(up_2n(max_cnt), 32, 1024)
 * (scatter_kernel.cu:14-24, 177-181). */
static int ref_block_x(int max_cnt) {
    int n = max_cnt, p = 1;
    if (n < 1) n = 1;
    while (p < n) p <<= 1;
    if (p > 1024) p = 1024;
    if (p < 32) p = 32;
    return p;
}

int oracle_ref_block_x(int max_cnt) { return ref_block_x(max_cnt); }

/* getPreSum kernel (scatter_kernel.cu:85-100): for sorted ids, the thread at
 * the end of each run stores i + 1 at preSum[id + 1]; the caller zero-fills
 * preSum beforehand (scatter_op.py:126), so preSum[0] stays 0. */
void oracle_ref_get_pre_sum(const int32_t* unq_inv, int32_t* pre_sum, int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
        if (i == n - 1 || unq_inv[i] != unq_inv[i + 1]) pre_sum[unq_inv[i] + 1] = (int32_t)(i + 1);
    }
}

/* Lane 0 of the reference's shfl_down tree (scatter_kernel.cu:26-39): at step
 * d lane i adds lane i + d; only lanes below d feed lane 0 afterwards. */
static float tree_sum(float* v, int width) {
    for (int d = width / 2; d >= 1; d >>= 1)
        for (int i = 0; i < d; ++i) v[i] = v[i] + v[i + d];
    return v[0];
}

/* scatter_sum kernel (scatter_kernel.cu:102-129): X threads per (segment,
 * channel); thread t adds rows begin + t, begin + t + X, ... in order; each
 * warp folds with the tree; lane-0 values of the warps are folded by warp 0
 * with a tree over num_valid_warp entries. */
void oracle_ref_scatter_sum(const float* feats, const int32_t* pre_sum, float* out,
                            int channel, int num_unq, int max_cnt) {
    const int X = ref_block_x(max_cnt);
    const int nwarp = X / 32;
#pragma omp parallel
    {
        float* part = (float*)malloc(sizeof(float) * (size_t)X);
        float wsum[32];
#pragma omp for schedule(dynamic, 16)
        for (int u = 0; u < num_unq; ++u) {
            const int begin = pre_sum[u], end = pre_sum[u + 1];
            for (int c = 0; c < channel; ++c) {
                for (int t = 0; t < X; ++t) {
                    float s = 0.f;
                    for (int f = begin + t; f < end; f += X) s += feats[(int64_t)f * channel + c];
                    part[t] = s;
                }
                for (int w = 0; w < nwarp; ++w) wsum[w] = tree_sum(part + 32 * w, 32);
                out[(int64_t)u * channel + c] = tree_sum(wsum, nwarp);
            }
        }
        free(part);
    }
}

/* Lane 0 of warpReduceMax (scatter_kernel.cu:41-83): the partner replaces the
 * holder only when strictly greater. */
static void tree_max(float* v, int32_t* ix, int width) {
    for (int d = width / 2; d >= 1; d >>= 1)
        for (int i = 0; i < d; ++i)
            if (v[i + d] > v[i]) { v[i] = v[i + d]; ix[i] = ix[i + d]; }
}

/* scatter_max kernel (scatter_kernel.cu:131-171): per-thread scan with >=
 * (the last of equal values wins inside a thread's stride), then the trees
 * with strict >.  Start value -FLT_MAX / -1. */
void oracle_ref_scatter_max(const float* feats, const int32_t* pre_sum, float* out, int32_t* arg,
                            int channel, int num_unq, int max_cnt) {
    const int X = ref_block_x(max_cnt);
    const int nwarp = X / 32;
#pragma omp parallel
    {
        float* pv = (float*)malloc(sizeof(float) * (size_t)X);
        int32_t* pi = (int32_t*)malloc(sizeof(int32_t) * (size_t)X);
        float wv[32];
        int32_t wi[32];
#pragma omp for schedule(dynamic, 16)
        for (int u = 0; u < num_unq; ++u) {
            const int begin = pre_sum[u], end = pre_sum[u + 1];
            for (int c = 0; c < channel; ++c) {
                for (int t = 0; t < X; ++t) {
                    float best = -FLT_MAX;
                    int32_t bi = -1;
                    for (int f = begin + t; f < end; f += X) {
                        const float x = feats[(int64_t)f * channel + c];
                        if (x >= best) { best = x; bi = f; }
                    }
                    pv[t] = best;
                    pi[t] = bi;
                }
                for (int w = 0; w < nwarp; ++w) {
                    tree_max(pv + 32 * w, pi + 32 * w, 32);
                    wv[w] = pv[32 * w];
                    wi[w] = pi[32 * w];
                }
                tree_max(wv, wi, nwarp);
                out[(int64_t)u * channel + c] = wv[0];
                arg[(int64_t)u * channel + c] = wi[0];
            }
        }
        free(pv);
        free(pi);
    }
}

/* ---- specification side ---------------------------------------------------- */

/* Exact segment sums in fp64 for ids in any order; out[M, C] zero for empty
 * segments; cnt[M] receives the row counts (may be NULL). */
void oracle_spec_scatter_sum_f64(const float* feats, const int64_t* ids, int64_t n, int channel,
                                 int64_t m, double* out, int64_t* cnt) {
    memset(out, 0, sizeof(double) * (size_t)(m * channel));
    if (cnt) memset(cnt, 0, sizeof(int64_t) * (size_t)m);
    for (int64_t i = 0; i < n; ++i) {
        const int64_t s = ids[i];
        double* o = out + s * channel;
        const float* f = feats + i * channel;
        for (int c = 0; c < channel; ++c) o[c] += (double)f[c];
        if (cnt) cnt[s] += 1;
    }
}

/* Maximum per segment and the LOWEST row holding it.  Empty segments and
 * segments whose values never exceed the start value keep -FLT_MAX / -1, the
 * reference kernel's initial state (scatter_kernel.cu:139-140); a value equal
 * to -FLT_MAX still records its row, as the reference's >= does.  NaN never
 * wins. */
void oracle_spec_scatter_max(const float* feats, const int64_t* ids, int64_t n, int channel,
                             int64_t m, float* out, int32_t* arg) {
    for (int64_t k = 0; k < m * channel; ++k) { out[k] = -FLT_MAX; arg[k] = -1; }
    for (int64_t i = 0; i < n; ++i) {
        const int64_t s = ids[i];
        for (int c = 0; c < channel; ++c) {
            const float x = feats[i * channel + c];
            float* o = out + s * channel + c;
            int32_t* a = arg + s * channel + c;
            if (x > *o || (x == *o && *a < 0)) { *o = x; *a = (int32_t)i; }
        }
    }
}

/* Backward of scatter_sum: g_in[i] = g[ids[i]] (scatter_op.py:47-50). */
void oracle_spec_sum_backward(const float* g, const int64_t* ids, int64_t n, int channel, float* g_in) {
    for (int64_t i = 0; i < n; ++i)
        memcpy(g_in + i * channel, g + ids[i] * channel, sizeof(float) * (size_t)channel);
}

/* Backward of scatter_mean: g_in[i] = g[ids[i]] / count (scatter_op.py:73-78),
 * an fp32 division by the count converted to fp32. */
void oracle_spec_mean_backward(const float* g, const int64_t* ids, const int64_t* cnt, int64_t n,
                               int channel, float* g_in) {
    for (int64_t i = 0; i < n; ++i) {
        const float d = (float)cnt[ids[i]];
        for (int c = 0; c < channel; ++c) g_in[i * channel + c] = g[ids[i] * channel + c] / d;
    }
}

/* Intended backward of scatter_max: zeros(N, C).scatter_(0, arg, g)
 * (scatter_op.py:105-111).  Entries with arg < 0 send no gradient. */
void oracle_spec_max_backward(const float* g, const int32_t* arg, int64_t n, int channel, int64_t m,
                              float* g_in) {
    memset(g_in, 0, sizeof(float) * (size_t)(n * channel));
    for (int64_t s = 0; s < m; ++s)
        for (int c = 0; c < channel; ++c) {
            const int32_t a = arg[s * channel + c];
            if (a >= 0) g_in[(int64_t)a * channel + c] = g[s * channel + c];
        }
}
