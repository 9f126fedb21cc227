// Generic windowed kernels: one thread per (pixel, unit), operands read
// straight from global memory through L1/L2.  They accept every shape the
// descriptor allows (1-D/2-D, real/complex, any window, band mode) and are the
// fallback behind the tiled sm_100a kernels, which cover the hot shapes.
#pragma once
#include "common.cuh"

namespace ca {

// Tensor accessor: real channel `cc` of unit `u` at pixel `pix` for a tensor
// with `npix` pixels per channel plane.
template <int CPE>
__device__ __forceinline__ int64_t elem_off(int u, int c, int cc, int npix, int pix) {
    if (CPE == 1) return ((int64_t)u * c + cc) * npix + pix;
    return (((int64_t)u * c + (cc >> 1)) * npix + pix) * 2 + (cc & 1);
}

struct FwdArgs {
    Geo g;
    float scale;
    int dist;
    const float* q;
    const float* k;
    const float* v;
    float* y;
    float* nz;      // nullable
    float* stats;   // nullable
};

// ---------------------------------------------------------------------------
// Fused forward, softmax: online softmax over the window, 8 offsets at a time.
// ---------------------------------------------------------------------------
template <int CMAX, int CPE>
__global__ void __launch_bounds__(128) fwd_softmax_generic(FwdArgs a) {
    const Geo& g = a.g;
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    const int u = blockIdx.y;
    if (j >= g.Np) return;
    const int h = j % g.H, w = j / g.H;
    const int cr = g.cr;

    float qr[CMAX], acc[CMAX];
#pragma unroll
    for (int cc = 0; cc < CMAX; ++cc) {
        qr[cc] = (cc < cr) ? __ldg(a.q + elem_off<CPE>(u, g.c, cc, g.Np, j)) : 0.f;
        acc[cc] = 0.f;
    }
    const float sl2 = a.scale * kLog2e;
    float m = -INFINITY, l = 0.f;
    float* nzrow = a.nz ? a.nz + ((int64_t)u * g.Np + j) * g.K : nullptr;

    constexpr int SB = 8;
    for (int iw = 0; iw < g.wsw; ++iw) {
        const int dw = (g.wsw == 1) ? 0 : iw - g.p;
        const int kw = wrap_axis(w + dw + g.wk_off, g.Wk);
        const int posw = (g.wsw == 1) ? 0 : axis_pos(dw, w, g.W, g.p, g.ws);
        for (int ih0 = 0; ih0 < g.ws; ih0 += SB) {
            float s[SB];
            int kpix[SB];
#pragma unroll
            for (int t = 0; t < SB; ++t) {
                const int ih = ih0 + t;
                const bool valid = ih < g.ws;
                const int dh = valid ? ih - g.p : 0;
                const int kh = wrap_axis(h + dh, g.H);
                kpix[t] = kh + g.H * kw;
                float sum = 0.f;
                if (a.dist) {
#pragma unroll
                    for (int cc = 0; cc < CMAX; ++cc)
                        if (cc < cr) {
                            float d = qr[cc] - __ldg(a.k + elem_off<CPE>(u, g.c, cc, g.Npk, kpix[t]));
                            sum = fmaf(d, d, sum);
                        }
                    sum *= -0.5f;
                } else {
#pragma unroll
                    for (int cc = 0; cc < CMAX; ++cc)
                        if (cc < cr)
                            sum = fmaf(qr[cc], __ldg(a.k + elem_off<CPE>(u, g.c, cc, g.Npk, kpix[t])), sum);
                }
                s[t] = valid ? sum * sl2 : -INFINITY;
            }
            float bm = s[0];
#pragma unroll
            for (int t = 1; t < SB; ++t) bm = fmaxf(bm, s[t]);
            const float mn = fmaxf(m, bm);
            const float corr = fast_exp2(m - mn);
            m = mn;
            l *= corr;
#pragma unroll
            for (int cc = 0; cc < CMAX; ++cc) acc[cc] *= corr;
#pragma unroll
            for (int t = 0; t < SB; ++t) {
                const int ih = ih0 + t;
                if (ih < g.ws) {
                    const float pt = fast_exp2(s[t] - mn);
                    l += pt;
#pragma unroll
                    for (int cc = 0; cc < CMAX; ++cc)
                        if (cc < cr)
                            acc[cc] = fmaf(pt, __ldg(a.v + elem_off<CPE>(u, g.c, cc, g.Npk, kpix[t])), acc[cc]);
                    if (nzrow) {
                        const int posh = axis_pos(ih - g.p, h, g.H, g.p, g.ws);
                        nzrow[posw * g.ws + posh] = s[t];   // log2-domain score, normalised below
                    }
                }
            }
        }
    }
    const float inv = 1.f / l;
#pragma unroll
    for (int cc = 0; cc < CMAX; ++cc)
        if (cc < cr) a.y[elem_off<CPE>(u, g.c, cc, g.Np, j)] = acc[cc] * inv;
    const float lse2 = m + log2f(l);
    if (a.stats) a.stats[(int64_t)u * g.Np + j] = lse2 * kLn2;
    if (nzrow)
        for (int k = 0; k < g.K; ++k) nzrow[k] = fast_exp2(nzrow[k] - lse2);
}

// ---------------------------------------------------------------------------
// Similarity: nz = scale * simfun(x[row], y[col]) for every stored entry.
// ---------------------------------------------------------------------------
template <int CPE>
__global__ void __launch_bounds__(128) similarity_generic(Geo g, float scale, int dist,
                                                          const float* __restrict__ x,
                                                          const float* __restrict__ y,
                                                          float* __restrict__ nz) {
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    const int u = blockIdx.y;
    if (j >= g.Np) return;
    const int h = j % g.H, w = j / g.H;
    float* nzrow = nz + ((int64_t)u * g.Np + j) * g.K;
    for (int iw = 0; iw < g.wsw; ++iw) {
        const int dw = (g.wsw == 1) ? 0 : iw - g.p;
        const int kw = wrap_axis(w + dw, g.W);
        const int posw = (g.wsw == 1) ? 0 : axis_pos(dw, w, g.W, g.p, g.ws);
        for (int ih = 0; ih < g.ws; ++ih) {
            const int dh = ih - g.p;
            const int kpix = wrap_axis(h + dh, g.H) + g.H * kw;
            float sum = 0.f;
            for (int cc = 0; cc < g.cr; ++cc) {
                const float xv = __ldg(x + elem_off<CPE>(u, g.c, cc, g.Np, j));
                const float yv = __ldg(y + elem_off<CPE>(u, g.c, cc, g.Np, kpix));
                if (dist) {
                    const float d = xv - yv;
                    sum = fmaf(d, d, sum);
                } else {
                    sum = fmaf(xv, yv, sum);
                }
            }
            if (dist) sum *= -0.5f;
            nzrow[posw * g.ws + axis_pos(dh, h, g.H, g.p, g.ws)] = sum * scale;
        }
    }
}

// ---------------------------------------------------------------------------
// Apply: out = A v ('N') or A^T v ('T'); optionally out -= (sum of the used
// values) * center, which is the Distance-similarity pullback correction.
// One thread per (pixel, real channel, unit).
// ---------------------------------------------------------------------------
struct ApplyArgs {
    Geo g;
    const float* nz;
    const float* v;
    const float* center;   // nullable
    float* out;
    float alpha;           // out = alpha * (...)
    int transpose;
    int a_bcast, v_bcast;
};

template <int CPE>
__global__ void __launch_bounds__(128) apply_generic(ApplyArgs a) {
    const Geo& g = a.g;
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    const int cc = blockIdx.y;
    const int u = blockIdx.z;
    if (j >= g.Np) return;
    const int h = j % g.H, w = j / g.H;
    const int ua = a.a_bcast ? 0 : u;
    const int uv = a.v_bcast ? 0 : u;
    const float* nzu = a.nz + (int64_t)ua * g.Np * g.K;
    float acc = 0.f, asum = 0.f;
    for (int iw = 0; iw < g.wsw; ++iw) {
        const int dw = (g.wsw == 1) ? 0 : iw - g.p;
        const int ow = wrap_axis(w + dw, g.W);           // the other pixel's column
        for (int ih = 0; ih < g.ws; ++ih) {
            const int dh = ih - g.p;
            const int oh = wrap_axis(h + dh, g.H);
            const int opix = oh + g.H * ow;
            float aval;
            if (!a.transpose) {
                // entry (row j, offset d)
                const int pos = ((g.wsw == 1) ? 0 : axis_pos(dw, w, g.W, g.p, g.ws) * g.ws) +
                                axis_pos(dh, h, g.H, g.p, g.ws);
                aval = __ldg(nzu + (int64_t)j * g.K + pos);
            } else {
                // entry (row opix, offset -d): A[opix, j]
                const int pos = ((g.wsw == 1) ? 0 : axis_pos(-dw, ow, g.W, g.p, g.ws) * g.ws) +
                                axis_pos(-dh, oh, g.H, g.p, g.ws);
                aval = __ldg(nzu + (int64_t)opix * g.K + pos);
            }
            acc = fmaf(aval, __ldg(a.v + elem_off<CPE>(uv, g.c, cc, g.Np, opix)), acc);
            asum += aval;
        }
    }
    if (a.center) acc -= asum * __ldg(a.center + elem_off<CPE>(u, g.c, cc, g.Np, j));
    a.out[elem_off<CPE>(u, g.c, cc, g.Np, j)] = a.alpha * acc;
}

// ---------------------------------------------------------------------------
// Backward.  P is recomputed from the saved row statistic:
//   softmax: P = exp(s - L);            dS = P * (dP - D),  D = sum_row P*dP
//   entmax : g = max(s/2 - tau, 0);     dS = g * (dP - D),  D = sum g*dP / sum g
// ---------------------------------------------------------------------------
struct BwdArgs {
    Geo g;
    float scale;
    int dist, entmax;
    const float* q;
    const float* k;
    const float* v;
    const float* y;
    const float* dy;
    const float* stats;
    const float* nz;   // nullable (saved A)
    const float* dA;   // nullable
    float* D;          // Np*units (query-side pixel count of the tensor it is read from)
    float* dq;
    float* dk;
    float* dv;
};

// D for softmax: dy . y (+ sum_k P_k dA_k).
template <int CPE>
__global__ void __launch_bounds__(128) bwd_pre_softmax(BwdArgs a) {
    const Geo& g = a.g;
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    const int u = blockIdx.y;
    if (j >= g.Np) return;
    float d = 0.f;
    for (int cc = 0; cc < g.cr; ++cc) {
        const int64_t o = elem_off<CPE>(u, g.c, cc, g.Np, j);
        d = fmaf(__ldg(a.dy + o), __ldg(a.y + o), d);
    }
    if (a.dA) {
        const int64_t r = ((int64_t)u * g.Np + j) * g.K;
        for (int k = 0; k < g.K; ++k) d = fmaf(__ldg(a.nz + r + k), __ldg(a.dA + r + k), d);
    }
    a.D[(int64_t)u * g.Np + j] = d;
}

// Query-owned sweep.  MODE 0: dq.  MODE 1: entmax D (= sum g dP / sum g) only.
template <int CMAX, int CPE, int MODE>
__global__ void __launch_bounds__(128) bwd_query_generic(BwdArgs a) {
    const Geo& g = a.g;
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    const int u = blockIdx.y;
    if (j >= g.Np) return;
    const int h = j % g.H, w = j / g.H;
    const int cr = g.cr;
    float qr[CMAX], dyr[CMAX], dq[CMAX];
#pragma unroll
    for (int cc = 0; cc < CMAX; ++cc) {
        const int64_t o = elem_off<CPE>(u, g.c, cc, g.Np, j);
        qr[cc] = (cc < cr) ? __ldg(a.q + o) : 0.f;
        dyr[cc] = (cc < cr) ? __ldg(a.dy + o) : 0.f;
        dq[cc] = 0.f;
    }
    const float st = __ldg(a.stats + (int64_t)u * g.Np + j);
    const float Dj = (MODE == 0) ? a.D[(int64_t)u * g.Np + j] : 0.f;
    const float* dArow = a.dA ? a.dA + ((int64_t)u * g.Np + j) * g.K : nullptr;
    float sum_ds = 0.f, sg = 0.f, sgd = 0.f;
    for (int iw = 0; iw < g.wsw; ++iw) {
        const int dw = (g.wsw == 1) ? 0 : iw - g.p;
        const int kw = wrap_axis(w + dw + g.wk_off, g.Wk);
        const int posw = (g.wsw == 1) ? 0 : axis_pos(dw, w, g.W, g.p, g.ws);
        for (int ih = 0; ih < g.ws; ++ih) {
            const int dh = ih - g.p;
            const int kpix = wrap_axis(h + dh, g.H) + g.H * kw;
            float s = 0.f, dp = 0.f;
            float kr[CMAX];
#pragma unroll
            for (int cc = 0; cc < CMAX; ++cc)
                if (cc < cr) {
                    const int64_t o = elem_off<CPE>(u, g.c, cc, g.Npk, kpix);
                    kr[cc] = __ldg(a.k + o);
                    if (a.dist) {
                        const float d = qr[cc] - kr[cc];
                        s = fmaf(d, d, s);
                    } else {
                        s = fmaf(qr[cc], kr[cc], s);
                    }
                    dp = fmaf(dyr[cc], __ldg(a.v + o), dp);
                }
            if (a.dist) s *= -0.5f;
            s *= a.scale;
            if (dArow) dp += __ldg(dArow + posw * g.ws + axis_pos(dh, h, g.H, g.p, g.ws));
            const float pg = a.entmax ? fmaxf(0.5f * s - st, 0.f) : __expf(s - st);
            if (MODE == 1) {
                sg += pg;
                sgd = fmaf(pg, dp, sgd);
            } else {
                const float ds = pg * (dp - Dj);
                sum_ds += ds;
#pragma unroll
                for (int cc = 0; cc < CMAX; ++cc)
                    if (cc < cr) dq[cc] = fmaf(ds, kr[cc], dq[cc]);
            }
        }
    }
    if (MODE == 1) {
        a.D[(int64_t)u * g.Np + j] = sgd / sg;
    } else {
#pragma unroll
        for (int cc = 0; cc < CMAX; ++cc)
            if (cc < cr) {
                float r = dq[cc];
                if (a.dist) r -= sum_ds * qr[cc];
                a.dq[elem_off<CPE>(u, g.c, cc, g.Np, j)] = a.scale * r;
            }
    }
}

// Key-owned sweep: dk, dv of key pixel i gather over the queries j = i + e whose
// window contains i (window symmetry), reading q, dy, stats and D of those
// queries.  In band mode the query-side tensors (q, dy, stats, D, dA rows) have
// Wk columns and the key-side ones (k, v, dk, dv) W columns.
template <int CMAX, int CPE>
__global__ void __launch_bounds__(128) bwd_key_generic(BwdArgs a) {
    const Geo& g = a.g;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const int u = blockIdx.y;
    if (i >= g.Np) return;
    const int h = i % g.H, w = i / g.H;
    const int cr = g.cr;
    float kr[CMAX], vr[CMAX], dk[CMAX], dv[CMAX];
#pragma unroll
    for (int cc = 0; cc < CMAX; ++cc) {
        const int64_t o = elem_off<CPE>(u, g.c, cc, g.Np, i);
        kr[cc] = (cc < cr) ? __ldg(a.k + o) : 0.f;
        vr[cc] = (cc < cr) ? __ldg(a.v + o) : 0.f;
        dk[cc] = 0.f;
        dv[cc] = 0.f;
    }
    float sum_ds = 0.f;
    for (int iw = 0; iw < g.wsw; ++iw) {
        const int ew = (g.wsw == 1) ? 0 : iw - g.p;
        const int jw = wrap_axis(w + ew + g.wk_off, g.Wk);
        for (int ih = 0; ih < g.ws; ++ih) {
            const int eh = ih - g.p;
            const int jh = wrap_axis(h + eh, g.H);
            const int jpix = jh + g.H * jw;
            float s = 0.f, dp = 0.f;
            float qv[CMAX], dyv[CMAX];
#pragma unroll
            for (int cc = 0; cc < CMAX; ++cc)
                if (cc < cr) {
                    const int64_t o = elem_off<CPE>(u, g.c, cc, g.Npk, jpix);
                    qv[cc] = __ldg(a.q + o);
                    dyv[cc] = __ldg(a.dy + o);
                    if (a.dist) {
                        const float d = qv[cc] - kr[cc];
                        s = fmaf(d, d, s);
                    } else {
                        s = fmaf(qv[cc], kr[cc], s);
                    }
                    dp = fmaf(dyv[cc], vr[cc], dp);
                }
            if (a.dist) s *= -0.5f;
            s *= a.scale;
            const int64_t jrow = (int64_t)u * g.Npk + jpix;
            if (a.dA) {
                // entry of row j at offset -e (band mode never materialises A)
                const int pos = ((g.wsw == 1) ? 0 : axis_pos(-ew, jw, g.W, g.p, g.ws) * g.ws) +
                                axis_pos(-eh, jh, g.H, g.p, g.ws);
                dp += __ldg(a.dA + jrow * g.K + pos);
            }
            const float st = __ldg(a.stats + jrow);
            const float Dj = __ldg(a.D + jrow);
            float P, gq;
            if (a.entmax) {
                gq = fmaxf(0.5f * s - st, 0.f);
                P = gq * gq;
            } else {
                P = __expf(s - st);
                gq = P;
            }
            const float ds = gq * (dp - Dj);
            sum_ds += ds;
#pragma unroll
            for (int cc = 0; cc < CMAX; ++cc)
                if (cc < cr) {
                    dk[cc] = fmaf(ds, qv[cc], dk[cc]);
                    dv[cc] = fmaf(P, dyv[cc], dv[cc]);
                }
        }
    }
#pragma unroll
    for (int cc = 0; cc < CMAX; ++cc)
        if (cc < cr) {
            const int64_t o = elem_off<CPE>(u, g.c, cc, g.Np, i);
            float r = dk[cc];
            if (a.dist) r -= sum_ds * kr[cc];
            a.dk[o] = a.scale * r;
            a.dv[o] = dv[cc];
        }
}

}  // namespace ca
