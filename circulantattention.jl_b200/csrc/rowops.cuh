// Row-wise and elementwise kernels on the stored values of a Circulant:
// structure generation, row normalisers and their pullbacks, sums, algebra.
#pragma once
#include "common.cuh"

namespace ca {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---------------------------------------------------------------- structure
// One thread per stored entry of one batch slice; the slice is written to all
// nbatch replicas.  Entry n of row j: position pos -> window offset -> column.
__global__ void structure_kernel(int H, int W, int ws, int wsw, int64_t nbatch,
                                 int32_t* __restrict__ rowptr, int32_t* __restrict__ colval) {
    const int p = (ws - 1) / 2;
    const int K = ws * wsw;
    const int64_t Np = (int64_t)H * W;
    const int64_t n = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (n <= Np) {
        const int32_t r = (int32_t)(1 + (int64_t)K * n);
        for (int64_t b = 0; b < nbatch; ++b) rowptr[n + (Np + 1) * b] = r;
    }
    if (n >= Np * K) return;
    const int j = (int)(n / K);
    const int k = (int)(n - (int64_t)j * K);
    const int h = j % H, w = j / H;
    const int posh = k % ws, posw = k / ws;
    // invert axis_pos: the run of row coordinate x starts at the smallest column
    // of the window, so the column at position `pos` is the pos-th smallest of
    // {(x+d) mod X}.
    auto col_at = [&](int pos, int x, int X) {
        if (x < p) {
            const int nfront = x + p + 1;          // coordinates 0..x+p, then the wrapped tail
            return pos < nfront ? pos : X - (ws - nfront) + (pos - nfront);
        }
        if (x >= X - p) {
            const int nfront = x + p - X + 1;      // wrapped coordinates 0..x+p-X come first
            return pos < nfront ? pos : (x - p) + (pos - nfront);
        }
        return x - p + pos;
    };
    const int ch = col_at(posh, h, H);
    const int cw = (wsw == 1) ? 0 : col_at(posw, w, W);
    const int32_t col = (int32_t)(ch + H * cw + 1);
    for (int64_t b = 0; b < nbatch; ++b) colval[n + Np * K * b] = col;
}

// ---------------------------------------------------------------- row normalisers
// One warp per row; K entries of a row are contiguous.
__global__ void __launch_bounds__(256) row_softmax_kernel(int64_t rows, int K,
                                                          const float* s,
                                                          float* p,
                                                          float* __restrict__ stats) {
    const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float* sr = s + row * K;
    float* pr = p + row * K;
    float m = -INFINITY;
    for (int k = lane; k < K; k += 32) m = fmaxf(m, sr[k]);
    m = warp_max(m);
    float l = 0.f;
    for (int k = lane; k < K; k += 32) l += __expf(sr[k] - m);
    l = warp_sum(l);
    const float inv = 1.f / l;
    for (int k = lane; k < K; k += 32) pr[k] = __expf(sr[k] - m) * inv;
    if (stats && lane == 0) stats[row] = m + logf(l);
}

// 1.5-entmax: p = max(s/2 - tau, 0)^2 with sum p = 1.  tau is bracketed by
// bisection (which fixes the support), then solved in closed form on that
// support: tau = mean - sqrt((1 - sum (z-mean)^2) / n).
__global__ void __launch_bounds__(256) row_entmax15_kernel(int64_t rows, int K,
                                                           const float* s,
                                                           float* p,
                                                           float* __restrict__ stats) {
    const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float* sr = s + row * K;
    float* pr = p + row * K;
    float m = -INFINITY;
    for (int k = lane; k < K; k += 32) m = fmaxf(m, 0.5f * sr[k]);
    m = warp_max(m);
    // work with z - m for accuracy; tau' in [-1, 0)
    float lo = -1.f, hi = 0.f;
    for (int it = 0; it < 26; ++it) {
        const float mid = 0.5f * (lo + hi);
        float f = 0.f;
        for (int k = lane; k < K; k += 32) {
            const float t = fmaxf(0.5f * sr[k] - m - mid, 0.f);
            f = fmaf(t, t, f);
        }
        f = warp_sum(f);
        if (f > 1.f) lo = mid; else hi = mid;
    }
    const float tb = 0.5f * (lo + hi);
    float n = 0.f, sum = 0.f;
    for (int k = lane; k < K; k += 32) {
        const float z = 0.5f * sr[k] - m;
        if (z > tb) { n += 1.f; sum += z; }
    }
    n = warp_sum(n);
    sum = warp_sum(sum);
    const float mean = sum / n;
    float ss = 0.f;
    for (int k = lane; k < K; k += 32) {
        const float z = 0.5f * sr[k] - m;
        if (z > tb) ss = fmaf(z - mean, z - mean, ss);
    }
    ss = warp_sum(ss);
    const float tau = mean - sqrtf(fmaxf((1.f - ss) / n, 0.f));
    for (int k = lane; k < K; k += 32) {
        const float t = fmaxf(0.5f * sr[k] - m - tau, 0.f);
        pr[k] = t * t;
    }
    if (stats && lane == 0) stats[row] = tau + m;
}

// The same for rows of at most 32*R entries, held in registers (one global read, one write).  The
// bisection stops as soon as no entry lies between the two ends of the bracket: the support is then
// known, and the closed form gives tau.
template <int R>
__global__ void __launch_bounds__(256) row_entmax15_reg_kernel(int64_t rows, int K,
                                                               const float* s,
                                                               float* p,
                                                               float* __restrict__ stats) {
    const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float* sr = s + row * K;
    float* pr = p + row * K;
    float z[R];
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int k = lane + 32 * i;
        z[i] = k < K ? 0.5f * sr[k] : -INFINITY;
        m = fmaxf(m, z[i]);
    }
    m = warp_max(m);
#pragma unroll
    for (int i = 0; i < R; ++i) z[i] -= m;                 // z - m in (-inf, 0]; tau' in [-1, 0)
    float lo = -1.f, hi = 0.f;
    int n_lo = 0, n_hi = 0;                                // entries above lo / above hi
#pragma unroll
    for (int i = 0; i < R; ++i) n_lo += z[i] > lo;
    n_lo = __reduce_add_sync(0xffffffffu, n_lo);
    for (int it = 0; it < 26 && n_lo != n_hi; ++it) {
        const float mid = 0.5f * (lo + hi);
        float f = 0.f;
        int cnt = 0;
#pragma unroll
        for (int i = 0; i < R; ++i) {
            const float t = fmaxf(z[i] - mid, 0.f);
            f = fmaf(t, t, f);
            cnt += z[i] > mid;
        }
        f = warp_sum(f);
        cnt = __reduce_add_sync(0xffffffffu, cnt);
        if (f > 1.f) { lo = mid; n_lo = cnt; } else { hi = mid; n_hi = cnt; }
    }
    // support = entries above lo (equivalently above hi when the loop stopped early)
    float n = 0.f, sum = 0.f;
#pragma unroll
    for (int i = 0; i < R; ++i)
        if (z[i] > lo) { n += 1.f; sum += z[i]; }
    n = warp_sum(n);
    sum = warp_sum(sum);
    const float mean = sum / n;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < R; ++i)
        if (z[i] > lo) ss = fmaf(z[i] - mean, z[i] - mean, ss);
    ss = warp_sum(ss);
    const float tau = mean - sqrtf(fmaxf((1.f - ss) / n, 0.f));
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int k = lane + 32 * i;
        const float t = fmaxf(z[i] - tau, 0.f);
        if (k < K) pr[k] = t * t;
    }
    if (stats && lane == 0) stats[row] = tau + m;
}

__global__ void __launch_bounds__(256) row_normalize_bwd_kernel(int64_t rows, int K, int entmax,
                                                                const float* __restrict__ p,
                                                                const float* dp,
                                                                float* ds) {
    const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float* pr = p + row * K;
    const float* dr = dp + row * K;
    float* out = ds + row * K;
    float a = 0.f, b = 0.f;
    for (int k = lane; k < K; k += 32) {
        const float g = entmax ? sqrtf(pr[k]) : pr[k];
        a = fmaf(g, dr[k], a);
        b += g;
    }
    a = warp_sum(a);
    b = warp_sum(b);
    const float D = entmax ? a / b : a;
    for (int k = lane; k < K; k += 32) {
        const float g = entmax ? sqrtf(pr[k]) : pr[k];
        out[k] = g * (dr[k] - D);
    }
}

// ---------------------------------------------------------------- sums
__global__ void __launch_bounds__(256) sum_rows_kernel(int64_t rows, int K,
                                                       const float* __restrict__ nz,
                                                       float* __restrict__ out) {
    const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    float a = 0.f;
    for (int k = lane; k < K; k += 32) a += nz[row * K + k];
    a = warp_sum(a);
    if (lane == 0) out[row] = a;
}

// Column sums by window symmetry: column i collects A[j, i] from the rows
// j = i + e, stored in row j at the position of offset -e.  Deterministic gather.
__global__ void __launch_bounds__(128) sum_cols_kernel(Geo g, const float* __restrict__ nz,
                                                       float* __restrict__ out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const int u = blockIdx.y;
    if (i >= g.Np) return;
    const int h = i % g.H, w = i / g.H;
    const float* nzu = nz + (int64_t)u * g.Np * g.K;
    float a = 0.f;
    for (int iw = 0; iw < g.wsw; ++iw) {
        const int ew = (g.wsw == 1) ? 0 : iw - g.p;
        const int jw = wrap_axis(w + ew, g.W);
        for (int ih = 0; ih < g.ws; ++ih) {
            const int eh = ih - g.p;
            const int jh = wrap_axis(h + eh, g.H);
            const int pos = ((g.wsw == 1) ? 0 : axis_pos(-ew, jw, g.W, g.p, g.ws) * g.ws) +
                            axis_pos(-eh, jh, g.H, g.p, g.ws);
            a += __ldg(nzu + (int64_t)(jh + g.H * jw) * g.K + pos);
        }
    }
    out[(int64_t)u * g.Np + i] = a;
}

// ---------------------------------------------------------------- algebra
__global__ void __launch_bounds__(256) axpby_kernel(int64_t n, float alpha, const float* __restrict__ x,
                                                    float beta, const float* __restrict__ y,
                                                    float* __restrict__ out) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t n4 = n >> 2;
    const bool vec = ((((uintptr_t)x | (uintptr_t)out | (uintptr_t)(y ? y : x)) & 15) == 0);
    if (vec) {
        const float4* x4 = reinterpret_cast<const float4*>(x);
        const float4* y4 = reinterpret_cast<const float4*>(y);
        float4* o4 = reinterpret_cast<float4*>(out);
        for (int64_t t = i; t < n4; t += stride) {
            float4 a = x4[t], r;
            if (y) {
                float4 b = y4[t];
                r = make_float4(alpha * a.x + beta * b.x, alpha * a.y + beta * b.y,
                                alpha * a.z + beta * b.z, alpha * a.w + beta * b.w);
            } else {
                r = make_float4(alpha * a.x, alpha * a.y, alpha * a.z, alpha * a.w);
            }
            o4[t] = r;
        }
        for (int64_t t = (n4 << 2) + i; t < n; t += stride)
            out[t] = alpha * x[t] + (y ? beta * y[t] : 0.f);
    } else {
        for (int64_t t = i; t < n; t += stride) out[t] = alpha * x[t] + (y ? beta * y[t] : 0.f);
    }
}

__global__ void __launch_bounds__(256) scale_batch_kernel(int64_t inner, int o1, int o2,
                                                          const float* __restrict__ a, int a1, int a2,
                                                          const float* __restrict__ c, int c1, int c2,
                                                          float* __restrict__ out) {
    const int i1 = blockIdx.y, i2 = blockIdx.z;
    const int64_t ao = ((int64_t)(a1 > 1 ? i1 : 0) + (int64_t)a1 * (a2 > 1 ? i2 : 0)) * inner;
    const float cv = c[(c1 > 1 ? i1 : 0) + c1 * (c2 > 1 ? i2 : 0)];
    const int64_t oo = ((int64_t)i1 + (int64_t)o1 * i2) * inner;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < inner; t += stride)
        out[oo + t] = cv * a[ao + t];
}

// One block per batch slice, fixed summation order: deterministic, no scratch.
__global__ void __launch_bounds__(1024) dot_batch_kernel(int64_t inner, int o1,
                                                         const float* __restrict__ x, int x1, int x2,
                                                         const float* __restrict__ y, int y1, int y2,
                                                         float* __restrict__ out) {
    const int i1 = blockIdx.x, i2 = blockIdx.y;
    const int64_t xo = ((int64_t)(x1 > 1 ? i1 : 0) + (int64_t)x1 * (x2 > 1 ? i2 : 0)) * inner;
    const int64_t yo = y ? ((int64_t)(y1 > 1 ? i1 : 0) + (int64_t)y1 * (y2 > 1 ? i2 : 0)) * inner : 0;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    int64_t t = threadIdx.x;
    for (; t + 3 * 1024 < inner; t += 4 * 1024) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int64_t e = t + r * 1024;
            acc[r] = y ? fmaf(x[xo + e], y[yo + e], acc[r]) : acc[r] + x[xo + e];
        }
    }
    for (; t < inner; t += 1024) acc[0] = y ? fmaf(x[xo + t], y[yo + t], acc[0]) : acc[0] + x[xo + t];
    float a = (acc[0] + acc[1]) + (acc[2] + acc[3]);
    __shared__ float sm[32];
    a = warp_sum(a);
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = a;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = sm[threadIdx.x];
        v = warp_sum(v);
        if (threadIdx.x == 0) out[i1 + o1 * i2] = v;
    }
}

__global__ void __launch_bounds__(256) sum_batch_kernel(int64_t inner, int b1, int b2, int sum1, int sum2,
                                                        const float* __restrict__ in,
                                                        float* __restrict__ out) {
    const int o1 = sum1 ? 1 : b1, o2 = sum2 ? 1 : b2;
    const int64_t total = inner * o1 * o2;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
        const int64_t n = t % inner;
        const int64_t r = t / inner;
        const int i1 = (int)(r % o1), i2 = (int)(r / o1);
        float acc = 0.f;
        for (int j2 = sum2 ? 0 : i2; j2 < (sum2 ? b2 : i2 + 1); ++j2)
            for (int j1 = sum1 ? 0 : i1; j1 < (sum1 ? b1 : i1 + 1); ++j1)
                acc += in[((int64_t)j1 + (int64_t)b1 * j2) * inner + n];
        out[t] = acc;
    }
}

}  // namespace ca
