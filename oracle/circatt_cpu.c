/*
 * circatt_cpu.c -- CPU restatement of circulant attention in plain C + OpenMP.
 *
 * TEST INFRASTRUCTURE ONLY: this is the checker and the timed CPU baseline, not
 * a product path.  The reference package has no CPU implementation
 * (README.md:20 "only CUDA compatible"), so this is a plain-array windowed
 * implementation of the same math:
 *   scores      src/similarity.jl:55-103 (Dot / negative half squared distance)
 *   scaling     src/attention.jl:20-21   (q, k each divided by c^(1/4))
 *   normaliser  src/similarity.jl:105-110 (softmax over the K window entries)
 *   apply       src/attention.jl:22-24    (y = A v)
 *   gradients   src/rrules.jl:1-72 composed (similarity, softmax, apply)
 * A is never materialised.  PARITY UNPINNED (the reference has no golden
 * vectors); tests/test_cpu_oracle.py checks this file against the float64
 * numpy oracle.
 *
 * Layout: Julia column-major (H, W, c, units); W = 1 and ndim = 1 for 1-D.
 * Built twice through the REAL macro: float (timed baseline) and double.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

int ca_cpu_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Overrides OMP_NUM_THREADS (process launchers often pin it to 1). */
void ca_cpu_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

static inline int wrapi(int x, int X) {
    if (x < 0) x += X;
    if (x >= X) x -= X;
    return x;
}

#define DEFINE_CPU(REAL, SUFFIX, EXP, LOG)                                                          \
    /* (Np, c) pixel-major copy of one unit so that the channel loop is contiguous */               \
    static void to_pixel_major_##SUFFIX(const REAL* x, REAL* t, int Np, int c) {                     \
        for (int ch = 0; ch < c; ++ch)                                                              \
            for (int pix = 0; pix < Np; ++pix) t[(size_t)pix * c + ch] = x[(size_t)ch * Np + pix];  \
    }                                                                                               \
    static void from_pixel_major_##SUFFIX(const REAL* t, REAL* x, int Np, int c) {                   \
        for (int ch = 0; ch < c; ++ch)                                                              \
            for (int pix = 0; pix < Np; ++pix) x[(size_t)ch * Np + pix] = t[(size_t)pix * c + ch];  \
    }                                                                                               \
    static inline REAL score_##SUFFIX(const REAL* a, const REAL* b, int c, int dist, REAL scale) {   \
        REAL s = 0;                                                                                 \
        if (dist) {                                                                                 \
            for (int m = 0; m < c; ++m) { REAL d = a[m] - b[m]; s += d * d; }                       \
            s *= (REAL)-0.5;                                                                        \
        } else {                                                                                    \
            for (int m = 0; m < c; ++m) s += a[m] * b[m];                                           \
        }                                                                                           \
        return s * scale;                                                                           \
    }                                                                                               \
    int ca_cpu_attention_fwd_##SUFFIX(int H, int W, int ndim, int c, int units, int ws, int dist,    \
                                      REAL scale, const REAL* q, const REAL* k, const REAL* v,      \
                                      REAL* y, REAL* lse) {                                         \
        const int Np = H * W, p = (ws - 1) / 2, wsw = ndim == 2 ? ws : 1, pw = ndim == 2 ? p : 0;   \
        if (ws % 2 != 1 || H < ws || (ndim == 2 && W < ws)) return -1;                              \
        _Pragma("omp parallel")                                                                     \
        {                                                                                           \
            REAL* qt = (REAL*)malloc(sizeof(REAL) * (size_t)Np * c * 4);                            \
            REAL *kt = qt + (size_t)Np * c, *vt = kt + (size_t)Np * c, *yt = vt + (size_t)Np * c;   \
            REAL* sc = (REAL*)malloc(sizeof(REAL) * (size_t)ws * wsw);                              \
            _Pragma("omp for schedule(dynamic, 1)")                                                 \
            for (int u = 0; u < units; ++u) {                                                       \
                const size_t uo = (size_t)u * c * Np;                                               \
                to_pixel_major_##SUFFIX(q + uo, qt, Np, c);                                         \
                to_pixel_major_##SUFFIX(k + uo, kt, Np, c);                                         \
                to_pixel_major_##SUFFIX(v + uo, vt, Np, c);                                         \
                for (int j = 0; j < Np; ++j) {                                                      \
                    const int h = j % H, w = j / H;                                                 \
                    const REAL* qj = qt + (size_t)j * c;                                            \
                    REAL m = -INFINITY;                                                             \
                    int n = 0;                                                                      \
                    for (int dw = -pw; dw <= pw; ++dw)                                              \
                        for (int dh = -p; dh <= p; ++dh) {                                          \
                            const int i = wrapi(h + dh, H) + H * wrapi(w + dw, W);                  \
                            const REAL s = score_##SUFFIX(qj, kt + (size_t)i * c, c, dist, scale);  \
                            sc[n++] = s;                                                            \
                            if (s > m) m = s;                                                       \
                        }                                                                           \
                    REAL l = 0;                                                                     \
                    REAL* yj = yt + (size_t)j * c;                                                  \
                    for (int mm = 0; mm < c; ++mm) yj[mm] = 0;                                      \
                    n = 0;                                                                          \
                    for (int dw = -pw; dw <= pw; ++dw)                                              \
                        for (int dh = -p; dh <= p; ++dh) {                                          \
                            const int i = wrapi(h + dh, H) + H * wrapi(w + dw, W);                  \
                            const REAL e = EXP(sc[n++] - m);                                        \
                            l += e;                                                                 \
                            const REAL* vi = vt + (size_t)i * c;                                    \
                            for (int mm = 0; mm < c; ++mm) yj[mm] += e * vi[mm];                    \
                        }                                                                           \
                    const REAL inv = (REAL)1 / l;                                                   \
                    for (int mm = 0; mm < c; ++mm) yj[mm] *= inv;                                   \
                    if (lse) lse[(size_t)u * Np + j] = m + LOG(l);                                  \
                }                                                                                   \
                from_pixel_major_##SUFFIX(yt, y + uo, Np, c);                                       \
            }                                                                                       \
            free(qt);                                                                               \
            free(sc);                                                                               \
        }                                                                                           \
        return 0;                                                                                   \
    }                                                                                               \
    /* Gradient: P from the saved log-sum-exp; dq is query-owned, dk and dv key-owned gathers */     \
    /* (window symmetry), so no accumulation races and a fixed summation order.              */     \
    int ca_cpu_attention_bwd_##SUFFIX(int H, int W, int ndim, int c, int units, int ws, int dist,    \
                                      REAL scale, const REAL* q, const REAL* k, const REAL* v,      \
                                      const REAL* y, const REAL* dy, const REAL* lse,               \
                                      REAL* dq, REAL* dk, REAL* dv) {                               \
        const int Np = H * W, p = (ws - 1) / 2, pw = ndim == 2 ? p : 0;                             \
        if (ws % 2 != 1 || H < ws || (ndim == 2 && W < ws)) return -1;                              \
        _Pragma("omp parallel")                                                                     \
        {                                                                                           \
            REAL* buf = (REAL*)malloc(sizeof(REAL) * ((size_t)Np * c * 7 + Np));                    \
            REAL *qt = buf, *kt = qt + (size_t)Np * c, *vt = kt + (size_t)Np * c,                   \
                 *dyt = vt + (size_t)Np * c, *dqt = dyt + (size_t)Np * c,                           \
                 *dkt = dqt + (size_t)Np * c, *dvt = dkt + (size_t)Np * c, *D = dvt + (size_t)Np * c; \
            _Pragma("omp for schedule(dynamic, 1)")                                                 \
            for (int u = 0; u < units; ++u) {                                                       \
                const size_t uo = (size_t)u * c * Np;                                               \
                const REAL* L = lse + (size_t)u * Np;                                               \
                to_pixel_major_##SUFFIX(q + uo, qt, Np, c);                                         \
                to_pixel_major_##SUFFIX(k + uo, kt, Np, c);                                         \
                to_pixel_major_##SUFFIX(v + uo, vt, Np, c);                                         \
                to_pixel_major_##SUFFIX(dy + uo, dyt, Np, c);                                       \
                to_pixel_major_##SUFFIX(y + uo, dqt, Np, c);                                        \
                for (int j = 0; j < Np; ++j) {                                                      \
                    REAL d = 0;                                                                     \
                    for (int mm = 0; mm < c; ++mm) d += dyt[(size_t)j * c + mm] * dqt[(size_t)j * c + mm]; \
                    D[j] = d;                                                                       \
                }                                                                                   \
                for (int j = 0; j < Np; ++j) {                                                      \
                    const int h = j % H, w = j / H;                                                 \
                    const REAL *qj = qt + (size_t)j * c, *dyj = dyt + (size_t)j * c;                \
                    const REAL *kj = kt + (size_t)j * c, *vj = vt + (size_t)j * c;                  \
                    REAL *gq = dqt + (size_t)j * c, *gk = dkt + (size_t)j * c, *gv = dvt + (size_t)j * c; \
                    REAL sq = 0, sk = 0;                                                            \
                    for (int mm = 0; mm < c; ++mm) gq[mm] = gk[mm] = gv[mm] = 0;                    \
                    for (int dw = -pw; dw <= pw; ++dw)                                              \
                        for (int dh = -p; dh <= p; ++dh) {                                          \
                            const int i = wrapi(h + dh, H) + H * wrapi(w + dw, W);                  \
                            const REAL *ki = kt + (size_t)i * c, *vi = vt + (size_t)i * c;          \
                            const REAL *qi = qt + (size_t)i * c, *dyi = dyt + (size_t)i * c;        \
                            /* row j, column i */                                                   \
                            REAL s = score_##SUFFIX(qj, ki, c, dist, scale), dp = 0;                \
                            for (int mm = 0; mm < c; ++mm) dp += dyj[mm] * vi[mm];                  \
                            REAL P = EXP(s - L[j]);                                                 \
                            REAL ds = P * (dp - D[j]);                                              \
                            sq += ds;                                                               \
                            for (int mm = 0; mm < c; ++mm) gq[mm] += ds * ki[mm];                   \
                            /* row i, column j (pixel j as a key) */                                \
                            s = score_##SUFFIX(qi, kj, c, dist, scale);                             \
                            dp = 0;                                                                 \
                            for (int mm = 0; mm < c; ++mm) dp += dyi[mm] * vj[mm];                  \
                            P = EXP(s - L[i]);                                                      \
                            ds = P * (dp - D[i]);                                                   \
                            sk += ds;                                                               \
                            for (int mm = 0; mm < c; ++mm) { gk[mm] += ds * qi[mm]; gv[mm] += P * dyi[mm]; } \
                        }                                                                           \
                    for (int mm = 0; mm < c; ++mm) {                                                \
                        gq[mm] = scale * (gq[mm] - (dist ? sq * qj[mm] : 0));                       \
                        gk[mm] = scale * (gk[mm] - (dist ? sk * kj[mm] : 0));                       \
                    }                                                                               \
                }                                                                                   \
                from_pixel_major_##SUFFIX(dqt, dq + uo, Np, c);                                     \
                from_pixel_major_##SUFFIX(dkt, dk + uo, Np, c);                                     \
                from_pixel_major_##SUFFIX(dvt, dv + uo, Np, c);                                     \
            }                                                                                       \
            free(buf);                                                                              \
        }                                                                                           \
        return 0;                                                                                   \
    }

DEFINE_CPU(float, f32, expf, logf)
DEFINE_CPU(double, f64, exp, log)
