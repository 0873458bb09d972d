/*
 * CPU oracle for fused deformable multi-head scaled-dot-product attention.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is compared
 * against (tests, the smoke run, and the CPU-baseline leg of the benchmark).  The
 * product never calls it: there is no CPU fallback in the library.
 *
 * It restates, in plain C, what the reference's pure-PyTorch path computes
 * (reference file ops/torch.py, function deform_sdpa_torch, lines 5-28):
 *
 *   ops/torch.py:8-9    K and V of every key view are feature maps of H rows and
 *                       W columns; pixel (x, y) is row y*W + x of the [L, D] map.
 *   ops/torch.py:10-11  the sampling coordinates are shared by all heads.
 *   ops/torch.py:14-15  bilinear grid_sample of the map at grid = c*2-1 with
 *                       align_corners=True and the default zero padding, i.e. the
 *                       pixel position is c*(size-1) and every one of the four
 *                       corners contributes only if it lies inside the map.
 *   ops/torch.py:16-19  keys are ordered key-view-major, then sample.
 *   ops/torch.py:20     q is scaled by sm_scale*log2(e).
 *   ops/torch.py:21-25  softmax in base 2 over ALL V*S keys of the query
 *                       (a key whose four corners are all outside still takes
 *                       part with logit 0 and value 0).
 *   ops/torch.py:26-28  out = sum_n p_n * v_n.
 *
 * The backward restates the gradients autograd derives from those lines
 * (softmax backward, grid_sample backward w.r.t. input and w.r.t. grid).
 *
 * The pixel position follows ATen's CPU grid sampler for align_corners=True:
 * x = ((c*2 - 1) + 1) * ((W - 1) / 2), weights (1 - fx), fx with fx = x - floor(x).
 *
 * Parity pin: tests/golden holds inputs and outputs produced by importing the
 * reference's ops/torch.py (forward and autograd backward); tests/test_oracle_golden.py
 * checks this file against every one of them.
 *
 * All tensors are fp32, contiguous:
 *   q, k, v, out, dout, dq, dk, dv : [B, V, Hh, L, D]   L = W*H
 *   coords, dcoords                : [B, V, L, V, S, 2] (x, y) in units of the map
 *   lse                            : [B, V, Hh, L]      base-2 log-sum-exp of the logits
 * Accumulations run in double so that the oracle is more accurate than either
 * implementation it is compared with.
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <stdint.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_LOG2E 1.4426950408889634

typedef struct {
    int idx[4];    /* pixel index of each corner, -1 when outside the map */
    float w[4];    /* bilinear weight of each corner (not zeroed when outside) */
    float fx, fy;  /* fractional position inside the cell */
} corner_t;

/* ops/torch.py:14 -> ATen grid_sampler (bilinear, zeros, align_corners=True). */
static inline void decode_sample(float cx, float cy, int W, int H, corner_t* c)
{
    float gx = cx * 2.0f - 1.0f;
    float gy = cy * 2.0f - 1.0f;
    float x = (gx + 1.0f) * ((float)(W - 1) * 0.5f);
    float y = (gy + 1.0f) * ((float)(H - 1) * 0.5f);
    float xf = floorf(x), yf = floorf(y);
    float fx = x - xf, fy = y - yf;
    /* floorf of a huge or non-finite coordinate must not overflow the int cast */
    int x0, y0;
    if (!(xf >= -2.0f && xf <= (float)W + 1.0f)) x0 = -2; else x0 = (int)xf;
    if (!(yf >= -2.0f && yf <= (float)H + 1.0f)) y0 = -2; else y0 = (int)yf;
    int xs[2] = { x0, x0 + 1 }, ys[2] = { y0, y0 + 1 };
    float wx[2] = { 1.0f - fx, fx }, wy[2] = { 1.0f - fy, fy };
    for (int j = 0; j < 2; ++j)
        for (int i = 0; i < 2; ++i) {
            int ok = xs[i] >= 0 && xs[i] < W && ys[j] >= 0 && ys[j] < H;
            c->idx[j * 2 + i] = ok ? ys[j] * W + xs[i] : -1;
            c->w[j * 2 + i] = wx[i] * wy[j];
        }
    c->fx = fx;
    c->fy = fy;
}

static inline void sample_row(const float* map, const corner_t* c, int D, float* dst)
{
    for (int d = 0; d < D; ++d) dst[d] = 0.0f;
    for (int t = 0; t < 4; ++t) {
        if (c->idx[t] < 0) continue;
        const float* row = map + (size_t)c->idx[t] * D;
        float w = c->w[t];
        for (int d = 0; d < D; ++d) dst[d] += w * row[d];
    }
}

static int clamp_threads(int nthreads)
{
#ifdef _OPENMP
    if (nthreads <= 0) nthreads = omp_get_max_threads();
    return nthreads;
#else
    (void)nthreads;
    return 1;
#endif
}

/*
 * Forward for query-heads [qh_begin, qh_end) of the flattened [B, V, Hh, L] index
 * space (the whole problem is 0 .. B*V*Hh*L).  lse may be NULL.
 */
int dsdpa_oracle_forward_range(const float* q, const float* k, const float* v, const float* coords,
                               float* out, float* lse,
                               int B, int V, int Hh, int W, int H, int D, int S, float sm_scale,
                               long long qh_begin, long long qh_end, int nthreads)
{
    const int L = W * H, N = V * S;
    if (B <= 0 || V <= 0 || Hh <= 0 || W <= 0 || H <= 0 || D <= 0 || S <= 0) return 1;
    const long long QH = (long long)B * V * Hh * L;
    if (qh_begin < 0 || qh_end > QH || qh_begin > qh_end) return 1;
    nthreads = clamp_threads(nthreads);
    int fail = 0;
#pragma omp parallel num_threads(nthreads)
    {
        float* kt = (float*)malloc(sizeof(float) * (size_t)D);
        float* vs = (float*)malloc(sizeof(float) * (size_t)N * D);
        double* logit = (double*)malloc(sizeof(double) * (size_t)N);
        double* acc = (double*)malloc(sizeof(double) * (size_t)D);
        if (!kt || !vs || !logit || !acc) {
#pragma omp atomic write
            fail = 1;
        } else {
#pragma omp for schedule(dynamic, 64)
            for (long long qh = qh_begin; qh < qh_end; ++qh) {
                int l = (int)(qh % L);
                int h = (int)((qh / L) % Hh);
                int vq = (int)((qh / ((long long)L * Hh)) % V);
                int b = (int)(qh / ((long long)L * Hh * V));
                const float* qrow = q + (size_t)qh * D;
                const float* crow = coords + ((((size_t)b * V + vq) * L + l) * V) * (size_t)S * 2;
                double m = -INFINITY;
                for (int vk = 0; vk < V; ++vk) {
                    const float* kmap = k + (((size_t)b * V + vk) * Hh + h) * (size_t)L * D;
                    const float* vmap = v + (((size_t)b * V + vk) * Hh + h) * (size_t)L * D;
                    for (int s = 0; s < S; ++s) {
                        int n = vk * S + s;
                        corner_t c;
                        decode_sample(crow[(size_t)n * 2], crow[(size_t)n * 2 + 1], W, H, &c);
                        sample_row(kmap, &c, D, kt);
                        sample_row(vmap, &c, D, vs + (size_t)n * D);
                        double dot = 0.0;
                        for (int d = 0; d < D; ++d) dot += (double)qrow[d] * (double)kt[d];
                        /* ops/torch.py:20 */
                        logit[n] = dot * (double)sm_scale * ORACLE_LOG2E;
                        if (logit[n] > m) m = logit[n];
                    }
                }
                /* ops/torch.py:22-25 */
                double sum = 0.0;
                for (int d = 0; d < D; ++d) acc[d] = 0.0;
                for (int n = 0; n < N; ++n) {
                    double p = exp2(logit[n] - m);
                    sum += p;
                    const float* vr = vs + (size_t)n * D;
                    for (int d = 0; d < D; ++d) acc[d] += p * (double)vr[d];
                }
                float* orow = out + (size_t)qh * D;
                for (int d = 0; d < D; ++d) orow[d] = (float)(acc[d] / sum);
                if (lse) lse[qh] = (float)(m + log2(sum));
            }
        }
        free(kt); free(vs); free(logit); free(acc);
    }
    return fail;
}

int dsdpa_oracle_forward(const float* q, const float* k, const float* v, const float* coords,
                         float* out, float* lse,
                         int B, int V, int Hh, int W, int H, int D, int S, float sm_scale,
                         int nthreads)
{
    return dsdpa_oracle_forward_range(q, k, v, coords, out, lse, B, V, Hh, W, H, D, S, sm_scale,
                                      0, (long long)B * V * Hh * W * H, nthreads);
}

/*
 * Backward for the (batch, head) slices [bh_begin, bh_end) of the flattened [B, Hh]
 * index space.  dq, dk, dv rows of those slices are overwritten; other rows are not
 * touched.  dcoords may be NULL; when given, the sum over the heads of the range is
 * ADDED to it (coordinates are shared by all heads, ops/torch.py:10), so the caller
 * zero-fills it before the first call.
 *
 * One slice is handled by one thread, so that dk/dv of a slice are accumulated
 * without atomics and in a fixed order.
 */
int dsdpa_oracle_backward_range(const float* q, const float* k, const float* v, const float* coords,
                                const float* dout, float* dq, float* dk, float* dv, float* dcoords,
                                int B, int V, int Hh, int W, int H, int D, int S, float sm_scale,
                                int bh_begin, int bh_end, int nthreads)
{
    const int L = W * H, N = V * S;
    if (B <= 0 || V <= 0 || Hh <= 0 || W <= 0 || H <= 0 || D <= 0 || S <= 0) return 1;
    if (bh_begin < 0 || bh_end > B * Hh || bh_begin > bh_end) return 1;
    nthreads = clamp_threads(nthreads);
    int fail = 0;
    /* coordinate gradients of all heads of a batch element land on the same rows:
       sum them in double so that the order of the additions does not show in fp32 */
    const size_t ncoord = (size_t)B * V * L * N * 2;
    double* dcacc = NULL;
    if (dcoords) {
        dcacc = (double*)calloc(ncoord, sizeof(double));
        if (!dcacc) return 2;
    }
#pragma omp parallel num_threads(nthreads)
    {
        float* ks = (float*)malloc(sizeof(float) * (size_t)N * D);
        float* vs = (float*)malloc(sizeof(float) * (size_t)N * D);
        corner_t* cs = (corner_t*)malloc(sizeof(corner_t) * (size_t)N);
        double* logit = (double*)malloc(sizeof(double) * (size_t)N);
        double* dkacc = (double*)malloc(sizeof(double) * (size_t)V * L * D);
        double* dvacc = (double*)malloc(sizeof(double) * (size_t)V * L * D);
        double* dqacc = (double*)malloc(sizeof(double) * (size_t)D);
        if (!ks || !vs || !cs || !logit || !dkacc || !dvacc || !dqacc) {
#pragma omp atomic write
            fail = 1;
        } else {
#pragma omp for schedule(dynamic, 1)
            for (int bh = bh_begin; bh < bh_end; ++bh) {
                int b = bh / Hh, h = bh % Hh;
                memset(dkacc, 0, sizeof(double) * (size_t)V * L * D);
                memset(dvacc, 0, sizeof(double) * (size_t)V * L * D);
                for (int vq = 0; vq < V; ++vq)
                    for (int l = 0; l < L; ++l) {
                        size_t qh = (((size_t)b * V + vq) * Hh + h) * (size_t)L + l;
                        const float* qrow = q + qh * D;
                        const float* grow = dout + qh * D;
                        size_t cbase = ((((size_t)b * V + vq) * L + l) * V) * (size_t)S * 2;
                        double m = -INFINITY;
                        for (int n = 0; n < N; ++n) {
                            int vk = n / S;
                            const float* kmap = k + (((size_t)b * V + vk) * Hh + h) * (size_t)L * D;
                            const float* vmap = v + (((size_t)b * V + vk) * Hh + h) * (size_t)L * D;
                            decode_sample(coords[cbase + (size_t)n * 2], coords[cbase + (size_t)n * 2 + 1],
                                          W, H, &cs[n]);
                            sample_row(kmap, &cs[n], D, ks + (size_t)n * D);
                            sample_row(vmap, &cs[n], D, vs + (size_t)n * D);
                            double dot = 0.0;
                            for (int d = 0; d < D; ++d) dot += (double)qrow[d] * (double)ks[(size_t)n * D + d];
                            logit[n] = dot * (double)sm_scale * ORACLE_LOG2E;
                            if (logit[n] > m) m = logit[n];
                        }
                        double sum = 0.0;
                        for (int n = 0; n < N; ++n) sum += exp2(logit[n] - m);
                        /* delta = sum_n p_n * (dout . v_n) = dout . out */
                        double delta = 0.0;
                        for (int n = 0; n < N; ++n) {
                            double p = exp2(logit[n] - m) / sum;
                            double dp = 0.0;
                            for (int d = 0; d < D; ++d) dp += (double)grow[d] * (double)vs[(size_t)n * D + d];
                            delta += p * dp;
                        }
                        for (int d = 0; d < D; ++d) dqacc[d] = 0.0;
                        for (int n = 0; n < N; ++n) {
                            int vk = n / S;
                            double p = exp2(logit[n] - m) / sum;
                            double dp = 0.0;
                            for (int d = 0; d < D; ++d) dp += (double)grow[d] * (double)vs[(size_t)n * D + d];
                            /* gradient w.r.t. the natural-log-domain logit sm_scale * q.k_n */
                            double ds = p * (dp - delta) * (double)sm_scale;
                            const float* kr = ks + (size_t)n * D;
                            for (int d = 0; d < D; ++d) dqacc[d] += ds * (double)kr[d];
                            /* grid_sample backward w.r.t. its input: weighted scatter to valid corners */
                            double* dkm = dkacc + (size_t)vk * L * D;
                            double* dvm = dvacc + (size_t)vk * L * D;
                            for (int t = 0; t < 4; ++t) {
                                int pix = cs[n].idx[t];
                                if (pix < 0) continue;
                                double w = (double)cs[n].w[t];
                                double* dkr = dkm + (size_t)pix * D;
                                double* dvr = dvm + (size_t)pix * D;
                                for (int d = 0; d < D; ++d) {
                                    dkr[d] += ds * w * (double)qrow[d];
                                    dvr[d] += p * w * (double)grow[d];
                                }
                            }
                            if (dcoords) {
                                /* grid_sample backward w.r.t. the grid, chained through
                                   grid = c*2-1 and x = (grid+1)*(W-1)/2, i.e. dx/dc = W-1. */
                                const float* kmap = k + (((size_t)b * V + vk) * Hh + h) * (size_t)L * D;
                                const float* vmap = v + (((size_t)b * V + vk) * Hh + h) * (size_t)L * D;
                                double fx = (double)cs[n].fx, fy = (double)cs[n].fy;
                                double gx = 0.0, gy = 0.0;
                                for (int d = 0; d < D; ++d) {
                                    double kc[4], vc[4];
                                    for (int t = 0; t < 4; ++t) {
                                        int pix = cs[n].idx[t];
                                        kc[t] = pix < 0 ? 0.0 : (double)kmap[(size_t)pix * D + d];
                                        vc[t] = pix < 0 ? 0.0 : (double)vmap[(size_t)pix * D + d];
                                    }
                                    double dkd = ds * (double)qrow[d];
                                    double dvd = p * (double)grow[d];
                                    double dkx = (1.0 - fy) * (kc[1] - kc[0]) + fy * (kc[3] - kc[2]);
                                    double dky = (1.0 - fx) * (kc[2] - kc[0]) + fx * (kc[3] - kc[1]);
                                    double dvx = (1.0 - fy) * (vc[1] - vc[0]) + fy * (vc[3] - vc[2]);
                                    double dvy = (1.0 - fx) * (vc[2] - vc[0]) + fx * (vc[3] - vc[1]);
                                    gx += dkd * dkx + dvd * dvx;
                                    gy += dkd * dky + dvd * dvy;
                                }
                                double addx = gx * (double)(W - 1);
                                double addy = gy * (double)(H - 1);
#pragma omp atomic
                                dcacc[cbase + (size_t)n * 2] += addx;
#pragma omp atomic
                                dcacc[cbase + (size_t)n * 2 + 1] += addy;
                            }
                        }
                        float* dqrow = dq + qh * D;
                        for (int d = 0; d < D; ++d) dqrow[d] = (float)dqacc[d];
                    }
                for (int vk = 0; vk < V; ++vk) {
                    float* dkm = dk + (((size_t)b * V + vk) * Hh + h) * (size_t)L * D;
                    float* dvm = dv + (((size_t)b * V + vk) * Hh + h) * (size_t)L * D;
                    const double* sk = dkacc + (size_t)vk * L * D;
                    const double* sv = dvacc + (size_t)vk * L * D;
                    for (size_t i = 0; i < (size_t)L * D; ++i) {
                        dkm[i] = (float)sk[i];
                        dvm[i] = (float)sv[i];
                    }
                }
            }
        }
        free(ks); free(vs); free(cs); free(logit); free(dkacc); free(dvacc); free(dqacc);
    }
    if (dcoords) {
        for (size_t i = 0; i < ncoord; ++i)
            if (dcacc[i] != 0.0) dcoords[i] += (float)dcacc[i];
        free(dcacc);
    }
    return fail;
}

int dsdpa_oracle_backward(const float* q, const float* k, const float* v, const float* coords,
                          const float* dout, float* dq, float* dk, float* dv, float* dcoords,
                          int B, int V, int Hh, int W, int H, int D, int S, float sm_scale,
                          int nthreads)
{
    return dsdpa_oracle_backward_range(q, k, v, coords, dout, dq, dk, dv, dcoords,
                                       B, V, Hh, W, H, D, S, sm_scale, 0, B * Hh, nthreads);
}

int dsdpa_oracle_max_threads(void)
{
    return clamp_threads(0);
}
