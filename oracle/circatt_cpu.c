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

/* Work is shared between the threads as (unit, block of CA_CPU_BLOCK pixels) items, so that
 * every thread has work even when there are fewer units than cores. */
#define CA_CPU_BLOCK 256

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
        const size_t per = (size_t)Np * c, all = per * units;                                       \
        const int nblk = (Np + CA_CPU_BLOCK - 1) / CA_CPU_BLOCK;                                    \
        REAL* buf = (REAL*)malloc(sizeof(REAL) * all * 4);                                          \
        if (!buf) return -2;                                                                        \
        REAL *qt = buf, *kt = qt + all, *vt = kt + all, *yt = vt + all;                             \
        _Pragma("omp parallel")                                                                     \
        {                                                                                           \
            REAL* sc = (REAL*)malloc(sizeof(REAL) * (size_t)ws * wsw);                              \
            _Pragma("omp for schedule(dynamic, 1)")                                                 \
            for (int t = 0; t < 3 * units; ++t) {                                                   \
                const int u = t / 3, which = t % 3;                                                 \
                const REAL* src = which == 0 ? q : (which == 1 ? k : v);                            \
                REAL* dst = which == 0 ? qt : (which == 1 ? kt : vt);                               \
                to_pixel_major_##SUFFIX(src + per * u, dst + per * u, Np, c);                       \
            }                                                                                       \
            _Pragma("omp for schedule(dynamic, 1)")                                                 \
            for (int item = 0; item < units * nblk; ++item) {                                       \
                const int u = item / nblk, j0 = (item % nblk) * CA_CPU_BLOCK;                       \
                const int j1 = j0 + CA_CPU_BLOCK < Np ? j0 + CA_CPU_BLOCK : Np;                     \
                const REAL *qu = qt + per * u, *ku = kt + per * u, *vu = vt + per * u;              \
                REAL* yu = yt + per * u;                                                            \
                for (int j = j0; j < j1; ++j) {                                                     \
                    const int h = j % H, w = j / H;                                                 \
                    const REAL* qj = qu + (size_t)j * c;                                            \
                    REAL m = -INFINITY;                                                             \
                    int n = 0;                                                                      \
                    for (int dw = -pw; dw <= pw; ++dw)                                              \
                        for (int dh = -p; dh <= p; ++dh) {                                          \
                            const int i = wrapi(h + dh, H) + H * wrapi(w + dw, W);                  \
                            const REAL s = score_##SUFFIX(qj, ku + (size_t)i * c, c, dist, scale);  \
                            sc[n++] = s;                                                            \
                            if (s > m) m = s;                                                       \
                        }                                                                           \
                    REAL l = 0;                                                                     \
                    REAL* yj = yu + (size_t)j * c;                                                  \
                    for (int mm = 0; mm < c; ++mm) yj[mm] = 0;                                      \
                    n = 0;                                                                          \
                    for (int dw = -pw; dw <= pw; ++dw)                                              \
                        for (int dh = -p; dh <= p; ++dh) {                                          \
                            const int i = wrapi(h + dh, H) + H * wrapi(w + dw, W);                  \
                            const REAL e = EXP(sc[n++] - m);                                        \
                            l += e;                                                                 \
                            const REAL* vi = vu + (size_t)i * c;                                    \
                            for (int mm = 0; mm < c; ++mm) yj[mm] += e * vi[mm];                    \
                        }                                                                           \
                    const REAL inv = (REAL)1 / l;                                                   \
                    for (int mm = 0; mm < c; ++mm) yj[mm] *= inv;                                   \
                    if (lse) lse[(size_t)u * Np + j] = m + LOG(l);                                  \
                }                                                                                   \
            }                                                                                       \
            _Pragma("omp for schedule(dynamic, 1)")                                                 \
            for (int u = 0; u < units; ++u) from_pixel_major_##SUFFIX(yt + per * u, y + per * u, Np, c); \
            free(sc);                                                                               \
        }                                                                                           \
        free(buf);                                                                                  \
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
        const size_t per = (size_t)Np * c, all = per * units;                                       \
        const int nblk = (Np + CA_CPU_BLOCK - 1) / CA_CPU_BLOCK;                                    \
        REAL* buf = (REAL*)malloc(sizeof(REAL) * (all * 7 + (size_t)Np * units));                   \
        if (!buf) return -2;                                                                        \
        REAL *qt = buf, *kt = qt + all, *vt = kt + all, *dyt = vt + all, *dqt = dyt + all,          \
             *dkt = dqt + all, *dvt = dkt + all, *Dall = dvt + all;                                 \
        _Pragma("omp parallel")                                                                     \
        {                                                                                           \
            _Pragma("omp for schedule(dynamic, 1)")                                                 \
            for (int t = 0; t < 5 * units; ++t) {                                                   \
                const int u = t / 5, which = t % 5;                                                 \
                const REAL* src = which == 0 ? q : which == 1 ? k : which == 2 ? v : which == 3 ? dy : y; \
                REAL* dst = which == 0 ? qt : which == 1 ? kt : which == 2 ? vt : which == 3 ? dyt : dqt; \
                to_pixel_major_##SUFFIX(src + per * u, dst + per * u, Np, c);                       \
            }                                                                                       \
            _Pragma("omp for schedule(static)")                                                     \
            for (int u = 0; u < units; ++u)                                                         \
                for (int j = 0; j < Np; ++j) {                                                      \
                    REAL d = 0;                                                                     \
                    for (int mm = 0; mm < c; ++mm)                                                  \
                        d += dyt[per * u + (size_t)j * c + mm] * dqt[per * u + (size_t)j * c + mm]; \
                    Dall[(size_t)u * Np + j] = d;                                                   \
                }                                                                                   \
            _Pragma("omp for schedule(dynamic, 1)")                                                 \
            for (int item = 0; item < units * nblk; ++item) {                                       \
                const int u = item / nblk, j0 = (item % nblk) * CA_CPU_BLOCK;                       \
                const int j1 = j0 + CA_CPU_BLOCK < Np ? j0 + CA_CPU_BLOCK : Np;                     \
                const REAL* L = lse + (size_t)u * Np;                                               \
                const REAL* D = Dall + (size_t)u * Np;                                              \
                const REAL *qu = qt + per * u, *ku = kt + per * u, *vu = vt + per * u, *dyu = dyt + per * u; \
                for (int j = j0; j < j1; ++j) {                                                     \
                    const int h = j % H, w = j / H;                                                 \
                    const REAL *qj = qu + (size_t)j * c, *dyj = dyu + (size_t)j * c;                \
                    const REAL *kj = ku + (size_t)j * c, *vj = vu + (size_t)j * c;                  \
                    REAL *gq = dqt + per * u + (size_t)j * c, *gk = dkt + per * u + (size_t)j * c,  \
                         *gv = dvt + per * u + (size_t)j * c;                                       \
                    REAL sq = 0, sk = 0;                                                            \
                    for (int mm = 0; mm < c; ++mm) gq[mm] = gk[mm] = gv[mm] = 0;                    \
                    for (int dw = -pw; dw <= pw; ++dw)                                              \
                        for (int dh = -p; dh <= p; ++dh) {                                          \
                            const int i = wrapi(h + dh, H) + H * wrapi(w + dw, W);                  \
                            const REAL *ki = ku + (size_t)i * c, *vi = vu + (size_t)i * c;          \
                            const REAL *qi = qu + (size_t)i * c, *dyi = dyu + (size_t)i * c;        \
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
            }                                                                                       \
            _Pragma("omp for schedule(dynamic, 1)")                                                 \
            for (int t = 0; t < 3 * units; ++t) {                                                   \
                const int u = t / 3, which = t % 3;                                                 \
                const REAL* src = which == 0 ? dqt : (which == 1 ? dkt : dvt);                      \
                REAL* dst = which == 0 ? dq : (which == 1 ? dk : dv);                               \
                from_pixel_major_##SUFFIX(src + per * u, dst + per * u, Np, c);                     \
            }                                                                                       \
        }                                                                                           \
        free(buf);                                                                                  \
        return 0;                                                                                   \
    }

DEFINE_CPU(float, f32, expf, logf)
DEFINE_CPU(double, f64, exp, log)
