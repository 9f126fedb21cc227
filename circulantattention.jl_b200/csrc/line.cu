// Fused attention for 1-D signals (sm_100a): forward and backward, softmax and 1.5-entmax, Dot and
// Distance similarity, 8 or 16 real channels per unit, no A-sized memory and no packed copy.
//
// The window of a 1-D signal is a run of `ws` consecutive pixels, so NQ consecutive pixels owned by one
// thread pair with ws + NQ - 1 consecutive pixels of the other side: every vector a thread loads from
// shared memory is used for NQ pairs (a sliding register tile).  A block of 128 threads owns 128*NQ
// consecutive pixels of one unit and stages the 128*NQ + ws - 1 pixels they pair with straight from the
// planar tensors (circular indices), four channels of a pixel per 16-byte slot; the slots carry one slot of
// padding per NQ pixels, which makes the 128-bit loads of a warp (lanes NQ pixels apart) conflict-free.
//
// The softmax forward is one sweep with an online sum.  Without the scores of a row in memory, a row quantity
// that needs all of them is found by sweeping the window again: the entmax forward sweeps once for the row
// maximum and once to accumulate; the 1.5-entmax
// threshold tau (sum_k max(z_k - tau, 0)^2 = 1, z = s/2) takes a few sweeps in between, each of which
// solves the quadratic exactly on the current support {z > tau} and stops when that support reproduces
// itself; the backward recomputes the weights from the saved row statistic (log-sum-exp or tau).
//
// Reference semantics: src/attention.jl:19-25 (similarity -> normaliser -> apply), src/similarity.jl:55-103
// (Dot / Distance), src/rrules.jl:1-72 (pullbacks).
#include <type_traits>

#include "line.cuh"

namespace ca {
namespace {

constexpr int kLT = 128;                      // threads per block

template <int V>
using ic = std::integral_constant<int, V>;

// Slot of staged pixel `pos`: one slot of padding per NQ pixels, so that lanes NQ pixels apart are NQ + 1 (odd)
// slots apart and a warp's 128-bit and 32-bit loads touch every bank group once.
template <int NQ>
__host__ __device__ __forceinline__ int pad(int pos) { return pos + pos / NQ; }

__host__ __device__ inline int64_t eoff(int cpe, int u, int c, int cc, int n, int pix) {
    if (cpe == 1) return ((int64_t)u * c + cc) * n + pix;
    return (((int64_t)u * c + (cc >> 1)) * n + pix) * 2 + (cc & 1);
}

struct LineArgs {
    Geo g;
    float scale;
    const float* q;
    const float* k;
    const float* v;
    const float* y;
    const float* dy;
    const float* stats;
    float* o;
    float* ostats;
    float* D;
    float* dq;
    float* dk;
    float* dv;
    int P;        // staged pixels per block: 128*NQ + ws - 1
    int PP;       // slots per channel group or scalar plane (padded)
};

__device__ __forceinline__ void cp_async4(float* smem_dst, const float* gsrc) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(gsrc) : "memory");
}
// Waits for the calling thread's own asynchronous copies (other threads' need a barrier on top).
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}

// Stage CR channels of pixels first .. first+P-1 (circular) of unit u as CR/4 groups of slots, by asynchronous
// 4-byte copies (all of a thread's copies are in flight at once; no registers in between).
template <int CR, int NQ>
__device__ __forceinline__ void stage_groups(float4* dst, int PP, const float* __restrict__ src, const Geo& g, int u,
                                             int first, int P, int lt) {
    const int N = g.Np;
    int base = first % N;
    if (base < 0) base += N;
    float* d = reinterpret_cast<float*>(dst);
    for (int i = lt; i < P; i += kLT) {
        int pix = base + i;
        if (pix >= N) {
            pix -= N;
            if (pix >= N) pix %= N;
        }
        const int slot = pad<NQ>(i);
#pragma unroll
        for (int cc = 0; cc < CR; ++cc) {
            float* to = d + ((cc >> 2) * PP + slot) * 4 + (cc & 3);
            if (cc < g.cr) cp_async4(to, src + eoff(g.cpe, u, g.c, cc, N, pix));
            else *to = 0.f;
        }
    }
}

template <int CR>
__device__ __forceinline__ void ld_vec(const float4* grp, int PP, int slot, float (&x)[CR]) {
#pragma unroll
    for (int gi = 0; gi < CR / 4; ++gi) {
        const float4 t = grp[gi * PP + slot];
        x[4 * gi] = t.x; x[4 * gi + 1] = t.y; x[4 * gi + 2] = t.z; x[4 * gi + 3] = t.w;
    }
}

template <int CR>
__device__ __forceinline__ float dot(const float (&a)[CR], const float (&b)[CR], float start) {
    float s = start;
#pragma unroll
    for (int i = 0; i < CR; ++i) s = fmaf(a[i], b[i], s);
    return s;
}

__device__ __forceinline__ float fast_rcp(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int CR>
__device__ __forceinline__ void axpy(float w, const float (&x)[CR], float (&y)[CR]) {
#pragma unroll
    for (int i = 0; i < CR; ++i) y[i] = fmaf(w, x[i], y[i]);
}

// factor * |x|^2 per staged pixel, from the staged groups.
template <int CR, int NQ>
__device__ __forceinline__ void stage_norms(float* dst, const float4* grp, int PP, int P, float factor, int lt) {
    for (int i = lt; i < P; i += kLT) {
        float x[CR];
        ld_vec<CR>(grp, PP, pad<NQ>(i), x);
        dst[pad<NQ>(i)] = factor * dot<CR>(x, x, 0.f);
    }
}

// One sweep of a thread's NQ owned pixels over the ws + NQ - 1 staged pixels they pair with.  Step t pairs
// owned pixel r with staged pixel (tb + t) iff 0 <= t - r < ws; `f(mask, slot)` gets the paired r as a
// compile-time bit mask and the slot of the staged pixel.  tb = NQ * thread, so the slot of step NQ*j + i is
// (NQ + 1) * (thread + j) + i: the steps are walked in aligned groups of NQ whose slots are one running value
// plus a compile-time i, which leaves the loads with immediate offsets.  Needs ws >= NQ - 1.
template <int NQ, int T, class F>
__device__ __forceinline__ void sweep_head(F& f, int slot0) {
    if constexpr (T < NQ - 1) {
        f(ic<(1 << (T + 1)) - 1>{}, slot0 + T);
        sweep_head<NQ, T + 1>(f, slot0);
    }
}
template <int NQ, int I, class F>
__device__ __forceinline__ void sweep_group(F& f, int slot0) {
    if constexpr (I < NQ) {
        f(ic<(1 << NQ) - 1>{}, slot0 + I);
        sweep_group<NQ, I + 1>(f, slot0);
    }
}
template <int NQ, int E, class F>
__device__ __forceinline__ void sweep_tail(F& f, int tb, int ws) {
    if constexpr (E < NQ - 1) {
        f(ic<((1 << NQ) - 1) & ~((1 << (E + 1)) - 1)>{}, pad<NQ>(tb + ws + E));
        sweep_tail<NQ, E + 1>(f, tb, ws);
    }
}
template <int NQ, class F>
__device__ __forceinline__ void sweep(int tb, int ws, F&& f) {
    int slot0 = pad<NQ>(tb);                       // tb is a multiple of NQ
    sweep_head<NQ, 0>(f, slot0);
    f(ic<(1 << NQ) - 1>{}, slot0 + NQ - 1);        // step NQ - 1: the first one every owned pixel pairs with
    int t = NQ;
    slot0 += NQ + 1;
    for (; t + NQ <= ws; t += NQ, slot0 += NQ + 1) sweep_group<NQ, 0>(f, slot0);
    for (; t < ws; ++t) f(ic<(1 << NQ) - 1>{}, pad<NQ>(tb + t));
    sweep_tail<NQ, 0>(f, tb, ws);
}

// One step of the entmax threshold search from the statistics of a sweep at the current tau, with t = z - tau:
// n = |{t > 0}| (the support S), sa = sum_S t, sb = sum_S t^2, rmax = max 1/t = 1 / (smallest t > 0),
// rmin = min 1/t = 1 / (largest t < 0).  Returns the step d that solves sum_S (t - d)^2 = 1 and sets `same` when
// tau + d has the support S again (d < smallest t > 0, or d >= largest t < 0) -- then tau + d is exact for S -- and
// the step was short against the distances it was computed from (a long step leaves tau with the rounding error
// of those larger numbers: one more sweep, now around the new tau, removes it).  `late`: a row that keeps
// changing its support takes Newton steps on f(tau) = sum max(z - tau, 0)^2 - 1 (convex: they converge from
// either side).  An empty support cannot happen for tau < max; it ends the search where it is.
__device__ __forceinline__ float tau_step(float n, float sa, float sb, float rmax, float rmin, bool late, bool& same) {
    same = true;
    if (n == 0.f) return 0.f;
    const float disc = fmaxf(fmaf(sa, sa, -n * (sb - 1.f)), 0.f);
    float d = (sa - sqrtf(disc)) / n;
    same = (d >= 0.f ? d * rmax < 1.f : d * rmin <= 1.f) && d * n <= 0.75f * sa;
    if (!same && late) d = 0.5f * (sb - 1.f) / sa;
    return d;
}

// Scale of the stored scores: z = f * sim(q, k) is the log2-domain score (softmax) or s / 2 (entmax).
template <bool ENT>
__device__ __forceinline__ float score_factor(float scale) { return ENT ? 0.5f * scale : scale * kLog2e; }

constexpr int kMaxTauSweeps = 24;
constexpr int kNewtonAfter = 10;              // threshold steps before the search falls back to Newton steps
constexpr unsigned kCoopRows = 16;            // open rows per warp (of 32 * NQ) below which the warp finishes them together
constexpr float kLineHeadroom = 12.f;          // log2 units between the softmax reference and the score that set it

// ------------------------------------------------------------------------------------------------ forward
template <int CR, int NQ, bool DIST, bool ENT>
__global__ void __launch_bounds__(kLT, CR <= 8 ? 3 : 2) line_fwd_kernel(LineArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    const Geo& g = a.g;
    const int N = g.Np, ws = g.ws, lt = threadIdx.x, u = blockIdx.y;
    const int j0 = blockIdx.x * (kLT * NQ);
    float4* Kg = reinterpret_cast<float4*>(smem);
    float4* Vg = Kg + (CR / 4) * a.PP;
    float* bk = reinterpret_cast<float*>(Vg + (CR / 4) * a.PP);
    const float f = score_factor<ENT>(a.scale), invf = f != 0.f ? 1.f / f : 0.f;

    stage_groups<CR, NQ>(Kg, a.PP, a.k, g, u, j0 - g.p, a.P, lt);
    stage_groups<CR, NQ>(Vg, a.PP, a.v, g, u, j0 - g.p, a.P, lt);
    cp_async_wait_all();
    __syncthreads();
    if (DIST) {
        stage_norms<CR, NQ>(bk, Kg, a.PP, a.P, -0.5f * f, lt);
        __syncthreads();
    }

    const int tb = NQ * lt;
    float q[NQ][CR], bq[NQ];
#pragma unroll
    for (int r = 0; r < NQ; ++r) {
        const int pix = min(j0 + tb + r, N - 1);
#pragma unroll
        for (int cc = 0; cc < CR; ++cc) q[r][cc] = cc < g.cr ? f * __ldg(a.q + eoff(g.cpe, u, g.c, cc, N, pix)) : 0.f;
        bq[r] = DIST ? -0.5f * invf * dot<CR>(q[r], q[r], 0.f) : 0.f;
    }

    // entmax: the row maximum.  softmax: an online sum against a reference that starts kLineHeadroom above the
    // score of the centre key and moves only when a score climbs past it (then the sums are rescaled)
    float m[NQ];
#pragma unroll
    for (int r = 0; r < NQ; ++r) m[r] = -INFINITY;
    if (!ENT) {
#pragma unroll
        for (int r = 0; r < NQ; ++r) {
            float kk[CR];
            ld_vec<CR>(Kg, a.PP, pad<NQ>(tb + r + g.p), kk);
            m[r] = dot<CR>(q[r], kk, DIST ? bq[r] + bk[pad<NQ>(tb + r + g.p)] : 0.f) + kLineHeadroom;
        }
    }
    if (ENT) sweep<NQ>(tb, ws, [&](auto mk, int slot) {
        constexpr int M = decltype(mk)::value;
        float kk[CR];
        ld_vec<CR>(Kg, a.PP, slot, kk);
        const float bkk = DIST ? bk[slot] : 0.f;
#pragma unroll
        for (int r = 0; r < NQ; ++r)
            if ((M >> r) & 1) m[r] = fmaxf(m[r], dot<CR>(q[r], kk, DIST ? bq[r] + bkk : 0.f));
    });

    // offset of the weights: p = 2^(z - m) (softmax) or max(z - tau, 0)^2 (entmax)
    float off[NQ];
#pragma unroll
    for (int r = 0; r < NQ; ++r) off[r] = m[r];
    if (ENT) {
        // tau >= max - 1; every sweep solves sum_{S} (z - tau)^2 = 1 on the support S = {z > tau} of the
        // current tau and is final when the new tau has the same support
        bool done[NQ];
#pragma unroll
        for (int r = 0; r < NQ; ++r) {
            off[r] = m[r] - 1.f;
            done[r] = false;
        }
        for (int it = 0; it < kMaxTauSweeps; ++it) {
            // the support's nearest members on both sides of tau through reciprocals: max 1/t is 1/(smallest t > 0),
            // min 1/t is 1/(largest t < 0) -- one reciprocal and two min/max per pair, no selects
            float n[NQ], sa[NQ], sb[NQ], rmax[NQ], rmin[NQ];
#pragma unroll
            for (int r = 0; r < NQ; ++r) {
                n[r] = 0.f; sa[r] = 0.f; sb[r] = 0.f;
                rmax[r] = 0.f;
                rmin[r] = 0.f;
            }
            sweep<NQ>(tb, ws, [&](auto mk, int slot) {
                constexpr int M = decltype(mk)::value;
                float kk[CR];
                ld_vec<CR>(Kg, a.PP, slot, kk);
                const float bkk = DIST ? bk[slot] : 0.f;
#pragma unroll
                for (int r = 0; r < NQ; ++r)
                    if ((M >> r) & 1) {
                        const float tt = dot<CR>(q[r], kk, DIST ? (bq[r] - off[r]) + bkk : -off[r]);
                        const float tp = fmaxf(tt, 0.f);
                        sa[r] += tp;
                        sb[r] = fmaf(tp, tp, sb[r]);
                        n[r] += tt > 0.f ? 1.f : 0.f;
                        const float rt = fast_rcp(tt);
                        rmax[r] = fmaxf(rmax[r], rt);
                        rmin[r] = fminf(rmin[r], rt);
                    }
            });
#pragma unroll
            for (int r = 0; r < NQ; ++r)
                if (!done[r]) {
                    bool same;
                    off[r] += tau_step(n[r], sa[r], sb[r], rmax[r], rmin[r], it >= kNewtonAfter, same);
                    done[r] = same;
                }
            // rows of this warp that are still open; when only a few are left (after the fourth sweep about
            // one row in a hundred), the warp finishes them one at a time, the window's keys spread over its
            // lanes, instead of sweeping all 32 * NQ rows again for their sake
            unsigned open_rows = 0;
#pragma unroll
            for (int r = 0; r < NQ; ++r) open_rows += done[r] ? 0u : 1u;
            const unsigned warp_open = __reduce_add_sync(0xffffffffu, open_rows);
            if (warp_open == 0) break;
            if (warp_open > kCoopRows) continue;
            const int lane = lt & 31;
            unsigned pend = __ballot_sync(0xffffffffu, open_rows != 0);
            while (pend) {
                const int src = __ffs(pend) - 1;
                pend &= pend - 1;
#pragma unroll
                for (int r = 0; r < NQ; ++r) {
                    if (!__shfl_sync(0xffffffffu, done[r] ? 0 : 1, src)) continue;        // warp-uniform
                    float qq[CR];
#pragma unroll
                    for (int cc = 0; cc < CR; ++cc) qq[cc] = __shfl_sync(0xffffffffu, q[r][cc], src);
                    const float bqq = DIST ? __shfl_sync(0xffffffffu, bq[r], src) : 0.f;
                    float tau = __shfl_sync(0xffffffffu, off[r], src);
                    const int base = NQ * ((lt & ~31) + src) + r;        // staged pixel of the row's first key
                    for (int ci = 0; ci < kMaxTauSweeps; ++ci) {
                        float n1 = 0.f, sa1 = 0.f, sb1 = 0.f, rmx = 0.f, rmn = 0.f;
                        for (int d = lane; d < ws; d += 32) {
                            const int slot = pad<NQ>(base + d);
                            float kk[CR];
                            ld_vec<CR>(Kg, a.PP, slot, kk);
                            const float tt = dot<CR>(qq, kk, DIST ? (bqq - tau) + bk[slot] : -tau);
                            const float tp = fmaxf(tt, 0.f);
                            sa1 += tp;
                            sb1 = fmaf(tp, tp, sb1);
                            n1 += tt > 0.f ? 1.f : 0.f;
                            const float rt = fast_rcp(tt);
                            rmx = fmaxf(rmx, rt);
                            rmn = fminf(rmn, rt);
                        }
#pragma unroll
                        for (int m = 16; m >= 1; m >>= 1) {
                            n1 += __shfl_xor_sync(0xffffffffu, n1, m);
                            sa1 += __shfl_xor_sync(0xffffffffu, sa1, m);
                            sb1 += __shfl_xor_sync(0xffffffffu, sb1, m);
                            rmx = fmaxf(rmx, __shfl_xor_sync(0xffffffffu, rmx, m));
                            rmn = fminf(rmn, __shfl_xor_sync(0xffffffffu, rmn, m));
                        }
                        bool same;
                        tau += tau_step(n1, sa1, sb1, rmx, rmn, ci >= kNewtonAfter, same);
                        if (same) break;
                    }
                    if (lane == src) {
                        off[r] = tau;
                        done[r] = true;
                    }
                }
            }
            break;
        }
    }

    float acc[NQ][CR], l[NQ];
#pragma unroll
    for (int r = 0; r < NQ; ++r) {
        l[r] = 0.f;
#pragma unroll
        for (int cc = 0; cc < CR; ++cc) acc[r][cc] = 0.f;
    }
    sweep<NQ>(tb, ws, [&](auto mk, int slot) {
        constexpr int M = decltype(mk)::value;
        float kk[CR], vv[CR];
        ld_vec<CR>(Kg, a.PP, slot, kk);
        ld_vec<CR>(Vg, a.PP, slot, vv);
        const float bkk = DIST ? bk[slot] : 0.f;
#pragma unroll
        for (int r = 0; r < NQ; ++r)
            if ((M >> r) & 1) {
                float tt = dot<CR>(q[r], kk, DIST ? (bq[r] - off[r]) + bkk : -off[r]);
                float w;
                if (ENT) {
                    const float tp = fmaxf(tt, 0.f);
                    w = tp * tp;
                } else {
                    if (tt > 0.f) {                  // rare: this score is above the reference; move it up
                        const float up = tt + kLineHeadroom;
                        const float corr = fast_exp2(-up);
                        l[r] *= corr;
#pragma unroll
                        for (int cc = 0; cc < CR; ++cc) acc[r][cc] *= corr;
                        off[r] += up;
                        tt = -kLineHeadroom;
                    }
                    w = fast_exp2(tt);
                    l[r] += w;
                }
                axpy<CR>(w, vv, acc[r]);
            }
    });

#pragma unroll
    for (int r = 0; r < NQ; ++r) {
        const int pix = j0 + tb + r;
        if (pix < N) {
            const float inv = ENT ? 1.f : 1.f / l[r];
#pragma unroll
            for (int cc = 0; cc < CR; ++cc)
                if (cc < g.cr) a.o[eoff(g.cpe, u, g.c, cc, N, pix)] = acc[r][cc] * inv;
            if (a.ostats) a.ostats[(int64_t)u * N + pix] = ENT ? off[r] : (off[r] + log2f(l[r])) * kLn2;
        }
    }
}

// ------------------------------------------------------------------------------------------------ dq, D
// Query-owned.  softmax: D = dy . y, dS = P (dP - D); entmax: g = max(z - tau, 0), D = sum g dP / sum g,
// dS = g (dP - D).  dq = scale * sum dS k  (Distance: - scale * q * sum dS).
template <int CR, int NQ, bool DIST, bool ENT>
__global__ void __launch_bounds__(kLT, CR <= 8 ? 3 : 2) line_dq_kernel(LineArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    const Geo& g = a.g;
    const int N = g.Np, ws = g.ws, lt = threadIdx.x, u = blockIdx.y;
    const int j0 = blockIdx.x * (kLT * NQ);
    float4* Kg = reinterpret_cast<float4*>(smem);
    float4* Vg = Kg + (CR / 4) * a.PP;
    float* bk = reinterpret_cast<float*>(Vg + (CR / 4) * a.PP);
    const float f = score_factor<ENT>(a.scale), invf = f != 0.f ? 1.f / f : 0.f;

    stage_groups<CR, NQ>(Kg, a.PP, a.k, g, u, j0 - g.p, a.P, lt);
    stage_groups<CR, NQ>(Vg, a.PP, a.v, g, u, j0 - g.p, a.P, lt);
    cp_async_wait_all();
    __syncthreads();
    if (DIST) {
        stage_norms<CR, NQ>(bk, Kg, a.PP, a.P, -0.5f * f, lt);
        __syncthreads();
    }

    const int tb = NQ * lt;
    float q[NQ][CR], dy[NQ][CR], c0[NQ], Dq[NQ];
#pragma unroll
    for (int r = 0; r < NQ; ++r) {
        const int pix = min(j0 + tb + r, N - 1);
        float dyy = 0.f;
#pragma unroll
        for (int cc = 0; cc < CR; ++cc) {
            const int64_t o = eoff(g.cpe, u, g.c, cc, N, pix);
            q[r][cc] = cc < g.cr ? f * __ldg(a.q + o) : 0.f;
            dy[r][cc] = cc < g.cr ? __ldg(a.dy + o) : 0.f;
            if (!ENT && cc < g.cr) dyy = fmaf(dy[r][cc], __ldg(a.y + o), dyy);
        }
        const float st = __ldg(a.stats + (int64_t)u * N + pix);
        // start value of the score chain: (-0.5 f |q|^2) - (row statistic in the units of z)
        c0[r] = (DIST ? -0.5f * invf * dot<CR>(q[r], q[r], 0.f) : 0.f) - (ENT ? st : st * kLog2e);
        Dq[r] = dyy;
    }

    float dqa[NQ][CR], sds[NQ];
#pragma unroll
    for (int r = 0; r < NQ; ++r) {
        sds[r] = 0.f;
#pragma unroll
        for (int cc = 0; cc < CR; ++cc) dqa[r][cc] = 0.f;
    }
    if (ENT) {
        // one sweep: with w = g dP, dq = sum (w - D g) k = sum w k - D sum g k and D = sum w / sum g, so the
        // sums with and without dP are accumulated side by side and combined at the end (sum dS = 0 exactly)
        float gk[NQ][CR], num[NQ], den[NQ];
#pragma unroll
        for (int r = 0; r < NQ; ++r) {
            num[r] = 0.f; den[r] = 0.f;
#pragma unroll
            for (int cc = 0; cc < CR; ++cc) gk[r][cc] = 0.f;
        }
        sweep<NQ>(tb, ws, [&](auto mk, int slot) {
            constexpr int M = decltype(mk)::value;
            float kk[CR], vv[CR];
            ld_vec<CR>(Kg, a.PP, slot, kk);
            ld_vec<CR>(Vg, a.PP, slot, vv);
            const float bkk = DIST ? bk[slot] : 0.f;
#pragma unroll
            for (int r = 0; r < NQ; ++r)
                if ((M >> r) & 1) {
                    const float gg = fmaxf(dot<CR>(q[r], kk, DIST ? c0[r] + bkk : c0[r]), 0.f);
                    const float w = gg * dot<CR>(dy[r], vv, 0.f);
                    num[r] += w;
                    den[r] += gg;
                    axpy<CR>(w, kk, dqa[r]);
                    axpy<CR>(gg, kk, gk[r]);
                }
        });
#pragma unroll
        for (int r = 0; r < NQ; ++r) {
            Dq[r] = num[r] / den[r];
#pragma unroll
            for (int cc = 0; cc < CR; ++cc) dqa[r][cc] = fmaf(-Dq[r], gk[r][cc], dqa[r][cc]);
        }
    } else {
        sweep<NQ>(tb, ws, [&](auto mk, int slot) {
            constexpr int M = decltype(mk)::value;
            float kk[CR], vv[CR];
            ld_vec<CR>(Kg, a.PP, slot, kk);
            ld_vec<CR>(Vg, a.PP, slot, vv);
            const float bkk = DIST ? bk[slot] : 0.f;
#pragma unroll
            for (int r = 0; r < NQ; ++r)
                if ((M >> r) & 1) {
                    const float z = dot<CR>(q[r], kk, DIST ? c0[r] + bkk : c0[r]);
                    const float ds = fast_exp2(z) * dot<CR>(dy[r], vv, -Dq[r]);
                    if (DIST) sds[r] += ds;
                    axpy<CR>(ds, kk, dqa[r]);
                }
        });
    }

#pragma unroll
    for (int r = 0; r < NQ; ++r) {
        const int pix = j0 + tb + r;
        if (pix < N) {
#pragma unroll
            for (int cc = 0; cc < CR; ++cc)
                if (cc < g.cr) {
                    float x = dqa[r][cc];
                    if (DIST) x -= sds[r] * (q[r][cc] * invf);
                    a.dq[eoff(g.cpe, u, g.c, cc, N, pix)] = a.scale * x;
                }
            a.D[(int64_t)u * N + pix] = Dq[r];
        }
    }
}

// ------------------------------------------------------------------------------------------------ dk, dv
// Key-owned gather (the window is symmetric: key i is in the window of the queries i-p .. i+p): dv = sum P dy,
// dk = scale * sum dS q  (Distance: - scale * k * sum dS), with P, dS recomputed from the queries' row
// statistic and D.  Deterministic, no atomics.
template <int CR, int NQ, bool DIST, bool ENT>
__global__ void __launch_bounds__(kLT, CR <= 8 ? 3 : 2) line_dkdv_kernel(LineArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    const Geo& g = a.g;
    const int N = g.Np, ws = g.ws, lt = threadIdx.x, u = blockIdx.y;
    const int j0 = blockIdx.x * (kLT * NQ);
    float4* Qg = reinterpret_cast<float4*>(smem);            // q of the staged query pixels
    float4* Yg = Qg + (CR / 4) * a.PP;                       // dy
    float4* Sg = Yg + (CR / 4) * a.PP;                       // (score-chain start, -D, 0, 0)
    const float f = score_factor<ENT>(a.scale);

    stage_groups<CR, NQ>(Qg, a.PP, a.q, g, u, j0 - g.p, a.P, lt);
    stage_groups<CR, NQ>(Yg, a.PP, a.dy, g, u, j0 - g.p, a.P, lt);
    cp_async_wait_all();
    {
        int base = (j0 - g.p) % N;
        if (base < 0) base += N;
        for (int i = lt; i < a.P; i += kLT) {       // a thread reads back only the slots it wrote itself
            int pix = base + i;
            if (pix >= N) {
                pix -= N;
                if (pix >= N) pix %= N;
            }
            float x[CR];
            ld_vec<CR>(Qg, a.PP, pad<NQ>(i), x);
            const float st = __ldg(a.stats + (int64_t)u * N + pix);
            const float c = (DIST ? -0.5f * f * dot<CR>(x, x, 0.f) : 0.f) - (ENT ? st : st * kLog2e);
            Sg[pad<NQ>(i)] = make_float4(c, -__ldg(a.D + (int64_t)u * N + pix), 0.f, 0.f);
        }
    }
    __syncthreads();

    const int tb = NQ * lt;
    float k[NQ][CR], v[NQ][CR], bk[NQ];
#pragma unroll
    for (int r = 0; r < NQ; ++r) {
        const int pix = min(j0 + tb + r, N - 1);
#pragma unroll
        for (int cc = 0; cc < CR; ++cc) {
            const int64_t o = eoff(g.cpe, u, g.c, cc, N, pix);
            k[r][cc] = cc < g.cr ? __ldg(a.k + o) : 0.f;
            v[r][cc] = cc < g.cr ? __ldg(a.v + o) : 0.f;
        }
        bk[r] = DIST ? -0.5f * f * dot<CR>(k[r], k[r], 0.f) : 0.f;
    }
    float dka[NQ][CR], dva[NQ][CR], sds[NQ];
#pragma unroll
    for (int r = 0; r < NQ; ++r) {
        sds[r] = 0.f;
#pragma unroll
        for (int cc = 0; cc < CR; ++cc) { dka[r][cc] = 0.f; dva[r][cc] = 0.f; }
    }
    sweep<NQ>(tb, ws, [&](auto mk, int slot) {
        constexpr int M = decltype(mk)::value;
        float qq[CR], yy[CR];
        ld_vec<CR>(Qg, a.PP, slot, qq);
        ld_vec<CR>(Yg, a.PP, slot, yy);
        const float4 sc = Sg[slot];
#pragma unroll
        for (int r = 0; r < NQ; ++r)
            if ((M >> r) & 1) {
                const float z = fmaf(dot<CR>(qq, k[r], 0.f), f, DIST ? sc.x + bk[r] : sc.x);
                const float w = ENT ? fmaxf(z, 0.f) : fast_exp2(z);
                const float ds = w * dot<CR>(yy, v[r], sc.y);
                if (DIST) sds[r] += ds;
                axpy<CR>(ds, qq, dka[r]);
                axpy<CR>(ENT ? w * w : w, yy, dva[r]);
            }
    });

#pragma unroll
    for (int r = 0; r < NQ; ++r) {
        const int pix = j0 + tb + r;
        if (pix < N) {
#pragma unroll
            for (int cc = 0; cc < CR; ++cc)
                if (cc < g.cr) {
                    const int64_t o = eoff(g.cpe, u, g.c, cc, N, pix);
                    float x = a.scale * dka[r][cc];
                    if (DIST) x -= a.scale * sds[r] * k[r][cc];
                    a.dk[o] = x;
                    a.dv[o] = dva[r][cc];
                }
        }
    }
}

// ------------------------------------------------------------------------------------------------ host
int prepare(LineArgs& a, int nq, int groups, int scalar_planes, size_t* smem) {
    a.P = kLT * nq + a.g.ws - 1;
    a.PP = a.P + (a.P - 1) / nq + 1;
    *smem = (size_t)groups * a.PP * 16 + (size_t)scalar_planes * a.PP * 4;
    return *smem <= 220 * 1024 ? CA_OK : CA_ERR_UNSUPPORTED;
}

template <typename Kern>
int launch(Kern kern, const LineArgs& a, int nq, size_t smem, cudaStream_t st, const char* what) {
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute");
    }
    const dim3 grid((a.g.Np + kLT * nq - 1) / (kLT * nq), a.g.units);
    kern<<<grid, kLT, smem, st>>>(a);
    count_tiled_launch();
    CA_CHECK_LAUNCH(what);
    return CA_OK;
}

#define CA_LINE_DISPATCH(KERN, CRV, NQV, dist, ent, ...)                                         \
    ((dist) ? ((ent) ? launch(KERN<CRV, NQV, true, true>, __VA_ARGS__)                           \
                     : launch(KERN<CRV, NQV, true, false>, __VA_ARGS__))                         \
            : ((ent) ? launch(KERN<CRV, NQV, false, true>, __VA_ARGS__)                          \
                     : launch(KERN<CRV, NQV, false, false>, __VA_ARGS__)))

constexpr int kFwdNQ8 = 4, kFwdNQ16 = 4, kBwdNQ8 = 4, kBwdNQ16 = 2;

}  // namespace

bool line_shape_ok(const Geo& g) {
    // windows up to 511: every kernel's staged tile then fits the shared memory of one block
    return g.wsw == 1 && g.W == 1 && g.Wk == g.W && !g.bf16 && g.cr >= 1 && g.cr <= 16 && g.ws >= 5 && g.ws <= 511 &&
           g.Np >= g.ws;
}

int line_attention_fwd(const Geo& g, float scale, int dist, int entmax, const float* q, const float* k,
                       const float* v, float* y, float* stats, cudaStream_t st) {
    if (!line_shape_ok(g)) return CA_ERR_UNSUPPORTED;
    LineArgs a{};
    a.g = g; a.scale = scale; a.q = q; a.k = k; a.v = v; a.o = y; a.ostats = stats;
    size_t smem;
    if (g.cr <= 8) {
        const int rc = prepare(a, kFwdNQ8, 4, 1, &smem);
        if (rc) return rc;
        return CA_LINE_DISPATCH(line_fwd_kernel, 8, kFwdNQ8, dist, entmax, a, kFwdNQ8, smem, st, "1-D forward kernel");
    }
    const int rc = prepare(a, kFwdNQ16, 8, 1, &smem);
    if (rc) return rc;
    return CA_LINE_DISPATCH(line_fwd_kernel, 16, kFwdNQ16, dist, entmax, a, kFwdNQ16, smem, st, "1-D forward kernel");
}

int line_attention_bwd(const Geo& g, float scale, int dist, int entmax, const float* q, const float* k,
                       const float* v, const float* y, const float* dy, const float* stats, float* D, float* dq,
                       float* dk, float* dv, cudaStream_t st) {
    if (!line_shape_ok(g)) return CA_ERR_UNSUPPORTED;
    LineArgs a{};
    a.g = g; a.scale = scale; a.q = q; a.k = k; a.v = v; a.y = y; a.dy = dy; a.stats = stats;
    a.D = D; a.dq = dq; a.dk = dk; a.dv = dv;
    size_t smem_q, smem_k;
    int rc;
    if (g.cr <= 8) {
        if ((rc = prepare(a, kBwdNQ8, 4, 1, &smem_q))) return rc;
        if ((rc = CA_LINE_DISPATCH(line_dq_kernel, 8, kBwdNQ8, dist, entmax, a, kBwdNQ8, smem_q, st, "1-D dq kernel"))) return rc;
        if ((rc = prepare(a, kBwdNQ8, 5, 0, &smem_k))) return rc;
        return CA_LINE_DISPATCH(line_dkdv_kernel, 8, kBwdNQ8, dist, entmax, a, kBwdNQ8, smem_k, st, "1-D dk/dv kernel");
    }
    if ((rc = prepare(a, kBwdNQ16, 8, 1, &smem_q))) return rc;
    if ((rc = CA_LINE_DISPATCH(line_dq_kernel, 16, kBwdNQ16, dist, entmax, a, kBwdNQ16, smem_q, st, "1-D dq kernel"))) return rc;
    if ((rc = prepare(a, kBwdNQ16, 9, 0, &smem_k))) return rc;
    return CA_LINE_DISPATCH(line_dkdv_kernel, 16, kBwdNQ16, dist, entmax, a, kBwdNQ16, smem_k, st, "1-D dk/dv kernel");
}

}  // namespace ca
