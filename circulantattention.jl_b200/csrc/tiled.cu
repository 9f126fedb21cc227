// Tiled sm_100a kernels for 2-D windows with 16 real channels per unit
// (16 Float32 or 8 ComplexF32 channels per head) and softmax.
//
// Work decomposition.  A CTA owns TH consecutive rows (the fast axis h) of FOUR
// consecutive columns w0..w0+3 of one unit.  A thread owns one row and the four
// pixels of that row ("centre" pixels: queries in the forward and dq kernels,
// keys in the dk/dv kernel) and keeps their 16-channel vectors in registers.
// The other side of the window is streamed through shared memory one image
// column at a time: column stage s holds column w0 - p + s (wrapped circularly,
// or taken from the neighbour halo in band mode) for rows h0-p' .. h0+TH+p'-1.
// Centre pixel r pairs with stage s iff r <= s <= r + 2p, so every loaded
// 16-float vector is used by up to four centre pixels from registers.
//
// Feeding the stages.  The reference layout is channel-planar, which no bulk
// copy can turn into pixel vectors, so a pack kernel first rewrites the
// streamed tensors as [unit][column][row'][16 channels] with the circular halo
// along h already unrolled (row' = h + p', p' = p rounded up to even, rows
// -p'..-1 and H..H+p'-1 are copies of the wrapped rows).  A column stage is
// then ONE contiguous box per tensor, fetched by cp.async.bulk.tensor (TMA) with
// the 64-byte hardware swizzle and tracked by an mbarrier; three stages are in
// flight.  The wrap along w is just the column coordinate of the box.
//
// Shared-memory layout: pixel (row) = 64 bytes = four 16-byte chunks; the TMA
// 64B swizzle stores chunk cq of row `row` at chunk position
// cq ^ ((row >> 1) & 3).  Eight consecutive rows then hit eight distinct
// 4-bank groups, so the 128-bit loads of a warp whose lanes hold consecutive
// rows are conflict free.
//
// Arithmetic: FP32 on the FMA pipe, issued as packed fma.rn.f32x2 so that a
// 16-channel dot product or axpy is 8 instructions; softmax in the log2 domain
// with ex2.approx; the running maximum is only rescaled when some lane of the
// warp actually raises it.
#include "tiled.cuh"
#include "tma.cuh"

namespace ca {
namespace {

typedef unsigned long long u64;

__device__ __forceinline__ u64 pack2(float a, float b) {
    u64 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void unpack2(u64 v, float& a, float& b) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ u64 fma2(u64 a, u64 b, u64 c) {
    u64 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ u64 mul2(u64 a, u64 b) {
    u64 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float hsum2(u64 v) {
    float a, b;
    unpack2(v, a, b);
    return a + b;
}

struct TileArgs {
    Geo g;
    float scale;
    int TH;                 // rows per CTA
    int roff;               // p' - p: first window row inside a stage buffer
    int stage_bytes;        // bytes of one stage buffer (multiple of 1024)
    const float* c0;        // centre tensors (reference layout)
    const float* c1;
    const float* cs0;       // centre scalars (dq kernel: stats, D)
    const float* cs1;
    float* o0;              // outputs
    float* o1;
    float* ostats;
};

// Number of CTAs that gave up waiting for a stage copy (stays 0 in a healthy run).
__device__ int g_stage_timeouts = 0;

constexpr int kStages = 3;

__device__ __forceinline__ int swz(int row, int cq) { return row * 16 + ((cq ^ ((row >> 1) & 3)) << 2); }

// One 16-channel pixel vector as eight packed pairs.
__device__ __forceinline__ void lds_vec16(const float* buf, int row, u64 (&v)[8]) {
#pragma unroll
    for (int cq = 0; cq < 4; ++cq) {
        const float4 t = *reinterpret_cast<const float4*>(buf + swz(row, cq));
        v[2 * cq] = pack2(t.x, t.y);
        v[2 * cq + 1] = pack2(t.z, t.w);
    }
}
// Half of it (channels 8*half .. 8*half+7) as four packed pairs.
__device__ __forceinline__ void lds_vec8(const float* buf, int row, int half, u64 (&v)[4]) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const float4 t = *reinterpret_cast<const float4*>(buf + swz(row, 2 * half + j));
        v[2 * j] = pack2(t.x, t.y);
        v[2 * j + 1] = pack2(t.z, t.w);
    }
}

// Global offset of real channel cc of unit u at pixel pix (npix pixels per plane).
template <int CPE>
__device__ __forceinline__ int64_t goff(int u, int cc, int npix, int pix) {
    if (CPE == 1) return ((int64_t)u * 16 + cc) * npix + pix;
    return (((int64_t)u * 8 + (cc >> 1)) * npix + pix) * 2 + (cc & 1);
}

__device__ __forceinline__ int stage_column(const Geo& g, int w0, int s) {
    int kc = (w0 - g.p + s + g.wk_off) % g.Wk;
    return kc < 0 ? kc + g.Wk : kc;
}

// Stage pipeline shared by the three kernels.  Thread 0 is the producer: it
// arms the stage's mbarrier with the byte count and issues the TMA boxes.
template <bool NSC>
struct StagePipe {
    uint64_t* full;
    unsigned char* base;
    const CUtensorMap* m0;
    const CUtensorMap* m1;
    const CUtensorMap* msc;
    int ROWS, stage_bytes, u, h0, w0;

    // Each vector region starts on a 512-byte boundary so that the swizzle phase
    // (address bits 7-8) equals (row >> 1) & 3; scalar rows start on 128 bytes.
    __device__ __forceinline__ int vstride() const { return (ROWS * 64 + 511) & ~511; }
    __device__ __forceinline__ int sstride() const { return (ROWS * 4 + 127) & ~127; }
    __device__ __forceinline__ float* vec0(int buf) const { return reinterpret_cast<float*>(base + (size_t)buf * stage_bytes); }
    __device__ __forceinline__ float* vec1(int buf) const { return reinterpret_cast<float*>(base + (size_t)buf * stage_bytes + vstride()); }
    __device__ __forceinline__ float* sc0(int buf) const { return reinterpret_cast<float*>(base + (size_t)buf * stage_bytes + 2 * vstride()); }
    __device__ __forceinline__ float* sc1(int buf) const { return reinterpret_cast<float*>(base + (size_t)buf * stage_bytes + 2 * vstride() + sstride()); }

    __device__ __forceinline__ void issue(const Geo& g, int s) const {
        const int buf = s % kStages;
        const int kc = stage_column(g, w0, s);
        mbar_arrive_expect_tx(&full[buf], (uint32_t)(ROWS * 128 + (NSC ? ROWS * 8 : 0)));
        tma_load_4d(vec0(buf), m0, 0, h0, kc, u, &full[buf]);
        tma_load_4d(vec1(buf), m1, 0, h0, kc, u, &full[buf]);
        if (NSC) {
            tma_load_3d(sc0(buf), msc, h0, kc, 2 * u, &full[buf]);
            tma_load_3d(sc1(buf), msc, h0, kc, 2 * u + 1, &full[buf]);
        }
    }
};

#define CA_PIPE_PROLOGUE(NSCV)                                                                      \
    extern __shared__ unsigned char smem_raw[];                                                     \
    __shared__ __align__(8) uint64_t full_bar[kStages];                                             \
    __shared__ int s_err;                                                                           \
    StagePipe<NSCV> pipe;                                                                           \
    pipe.full = full_bar;                                                                           \
    pipe.base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);                        \
    pipe.m0 = &m0; pipe.m1 = &m1; pipe.msc = &msc;                                                  \
    pipe.ROWS = ROWS; pipe.stage_bytes = a.stage_bytes; pipe.u = u; pipe.h0 = h0; pipe.w0 = w0;     \
    if (threadIdx.x == 0) {                                                                         \
        for (int i = 0; i < kStages; ++i) mbar_init(&full_bar[i], 1);                               \
        s_err = 0;                                                                                  \
        mbar_fence_init();                                                                          \
    }                                                                                               \
    __syncthreads();                                                                                \
    const int NS = g.ws + 3;                                                                        \
    if (threadIdx.x == 0)                                                                           \
        for (int s = 0; s < kStages && s < NS; ++s) pipe.issue(g, s);

// Consumer side of one stage: bounded wait, compute, then recycle the buffer.
#define CA_PIPE_LOOP(...)                                                                           \
    for (int s = 0; s < NS; ++s) {                                                                  \
        const int buf = s % kStages;                                                                \
        if (!mbar_wait(&full_bar[buf], (uint32_t)((s / kStages) & 1))) s_err = 1;                   \
        __VA_ARGS__                                                                                 \
        __syncthreads();                                                                            \
        if (s_err) break;                                                                           \
        if (threadIdx.x == 0 && s + kStages < NS) pipe.issue(g, s + kStages);                       \
    }                                                                                               \
    if (s_err) {                                                                                    \
        /* give copies still in flight a bounded chance to land before the CTA exits */             \
        if (threadIdx.x == 0) {                                                                     \
            for (int i = 0; i < kStages; ++i) mbar_wait(&full_bar[i], 0, 1u << 12);                 \
            atomicAdd(&g_stage_timeouts, 1);                                                        \
        }                                                                                           \
        return;                                                                                     \
    }

__device__ __forceinline__ int stage_mask(int s, int p) {
    int mask = 0;
#pragma unroll
    for (int r = 0; r < 4; ++r)
        if (s >= r && s <= r + 2 * p) mask |= 1 << r;
    return mask;
}

// Loads the 16-channel vectors of the four centre pixels of this thread, times `mul`.
template <int CPE>
__device__ __forceinline__ void load_centre(const float* src, const Geo& g, int u, int h, int w0, bool active,
                                            float mul, u64 (&dst)[4][8]) {
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const bool ok = active && (w0 + r < g.W);
        const int pix = h + g.H * (w0 + r);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float x = 0.f, y = 0.f;
            if (ok) {
                if (CPE == 1) {
                    x = __ldg(src + goff<1>(u, 2 * i, g.Np, pix));
                    y = __ldg(src + goff<1>(u, 2 * i + 1, g.Np, pix));
                } else {
                    const float2 t = __ldg(reinterpret_cast<const float2*>(src + goff<2>(u, 2 * i, g.Np, pix)));
                    x = t.x;
                    y = t.y;
                }
            }
            dst[r][i] = pack2(x * mul, y * mul);
        }
    }
}

template <int CPE>
__device__ __forceinline__ void store_centre(float* dst, const Geo& g, int u, int h, int w0, bool active, int r,
                                             int i, float x, float y) {
    if (!(active && (w0 + r < g.W))) return;
    const int pix = h + g.H * (w0 + r);
    if (CPE == 1) {
        dst[goff<1>(u, 2 * i, g.Np, pix)] = x;
        dst[goff<1>(u, 2 * i + 1, g.Np, pix)] = y;
    } else {
        *reinterpret_cast<float2*>(dst + goff<2>(u, 2 * i, g.Np, pix)) = make_float2(x, y);
    }
}

// =====================================================================
// Forward
// =====================================================================
template <int DC, bool DIST, int MASK>
__device__ __forceinline__ void fwd_stage(const float* kb, const float* vb, int lr, int ws, float sl2,
                                          const u64 (&q)[4][8], u64 (&acc)[4][8], float (&m)[4], float (&l)[4],
                                          const float (&bq)[4]) {
    for (int c0 = 0; c0 < ws; c0 += DC) {
        float sc[4][DC];
#pragma unroll
        for (int t = 0; t < DC; ++t) {
            if (c0 + t < ws) {
                u64 k2[8];
                lds_vec16(kb, lr + c0 + t, k2);
                float bk = 0.f;
                if (DIST) {
                    u64 n = 0ull;
#pragma unroll
                    for (int i = 0; i < 8; ++i) n = fma2(k2[i], k2[i], n);
                    bk = -0.5f * sl2 * hsum2(n);
                }
#pragma unroll
                for (int r = 0; r < 4; ++r)
                    if (MASK & (1 << r)) {
                        u64 s2 = 0ull;
#pragma unroll
                        for (int i = 0; i < 8; ++i) s2 = fma2(q[r][i], k2[i], s2);
                        sc[r][t] = hsum2(s2) + (DIST ? bq[r] + bk : 0.f);
                    }
            } else {
#pragma unroll
                for (int r = 0; r < 4; ++r) sc[r][t] = -INFINITY;
            }
        }
        float mn[4];
        bool raise = false;
#pragma unroll
        for (int r = 0; r < 4; ++r)
            if (MASK & (1 << r)) {
                float cm = sc[r][0];
#pragma unroll
                for (int t = 1; t < DC; ++t) cm = fmaxf(cm, sc[r][t]);
                mn[r] = fmaxf(m[r], cm);
                raise |= mn[r] > m[r];
            }
        if (__any_sync(0xffffffffu, raise)) {
#pragma unroll
            for (int r = 0; r < 4; ++r)
                if (MASK & (1 << r)) {
                    const float corr = fast_exp2(m[r] - mn[r]);
                    m[r] = mn[r];
                    l[r] *= corr;
                    const u64 c2 = pack2(corr, corr);
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[r][i] = mul2(acc[r][i], c2);
                }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r)
            if (MASK & (1 << r)) {
#pragma unroll
                for (int t = 0; t < DC; ++t) {
                    const float pt = fast_exp2(sc[r][t] - m[r]);
                    l[r] += pt;
                    sc[r][t] = pt;
                }
            }
#pragma unroll
        for (int t = 0; t < DC; ++t) {
            if (c0 + t < ws) {
                u64 v2[8];
                lds_vec16(vb, lr + c0 + t, v2);
#pragma unroll
                for (int r = 0; r < 4; ++r)
                    if (MASK & (1 << r)) {
                        const u64 p2 = pack2(sc[r][t], sc[r][t]);
#pragma unroll
                        for (int i = 0; i < 8; ++i) acc[r][i] = fma2(p2, v2[i], acc[r][i]);
                    }
            }
        }
    }
}

#define CA_MASK_SWITCH(mask, CALL)                       \
    switch (mask) {                                      \
        case 1:  { constexpr int MK = 1;  CALL; } break; \
        case 3:  { constexpr int MK = 3;  CALL; } break; \
        case 7:  { constexpr int MK = 7;  CALL; } break; \
        case 15: { constexpr int MK = 15; CALL; } break; \
        case 14: { constexpr int MK = 14; CALL; } break; \
        case 12: { constexpr int MK = 12; CALL; } break; \
        case 8:  { constexpr int MK = 8;  CALL; } break; \
        default: break;                                  \
    }

template <int DC, bool DIST, int CPE>
__global__ void __launch_bounds__(128) fwd_tiled_kernel(TileArgs a, const __grid_constant__ CUtensorMap m0,
                                                        const __grid_constant__ CUtensorMap m1,
                                                        const __grid_constant__ CUtensorMap msc) {
    const Geo& g = a.g;
    const int ROWS = a.TH + 2 * (g.p + a.roff);
    const int w0 = blockIdx.x * 4, h0 = blockIdx.y * a.TH, u = blockIdx.z;
    const int lr = threadIdx.x, h = h0 + lr;
    const bool active = h < g.H;
    const float sl2 = a.scale * kLog2e;
    CA_PIPE_PROLOGUE(false)

    u64 q[4][8], acc[4][8];
    load_centre<CPE>(a.c0, g, u, h, w0, active, sl2, q);
    float m[4], l[4], bq[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        m[r] = -INFINITY;
        l[r] = 0.f;
        bq[r] = 0.f;
        if (DIST) {
            u64 n = 0ull;
#pragma unroll
            for (int i = 0; i < 8; ++i) n = fma2(q[r][i], q[r][i], n);
            bq[r] = -0.5f * hsum2(n) / sl2;      // q is pre-scaled by sl2
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[r][i] = 0ull;
    }

    CA_PIPE_LOOP({
        const int mask = stage_mask(s, g.p);
        const float* kb = pipe.vec0(buf);
        const float* vb = pipe.vec1(buf);
        CA_MASK_SWITCH(mask, (fwd_stage<DC, DIST, MK>(kb, vb, lr + a.roff, g.ws, sl2, q, acc, m, l, bq)));
    })
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const float inv = 1.f / l[r];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float x, y;
            unpack2(acc[r][i], x, y);
            store_centre<CPE>(a.o0, g, u, h, w0, active, r, i, x * inv, y * inv);
        }
        if (a.ostats && active && w0 + r < g.W)
            a.ostats[(int64_t)u * g.Np + h + g.H * (w0 + r)] = (m[r] + log2f(l[r])) * kLn2;
    }
}

// =====================================================================
// Backward, query-owned: dq
// =====================================================================
template <bool DIST, int MASK>
__device__ __forceinline__ void dq_stage(const float* kb, const float* vb, int lr, int ws, float sl2,
                                         const u64 (&q)[4][8], const u64 (&dy)[4][8], u64 (&dq)[4][8],
                                         const float (&L2)[4], const float (&D)[4], const float (&bq)[4],
                                         float (&sumds)[4]) {
#pragma unroll 1
    for (int di = 0; di < ws; ++di) {
        float dp[4];
        {
            u64 v2[8];
            lds_vec16(vb, lr + di, v2);
#pragma unroll
            for (int r = 0; r < 4; ++r)
                if (MASK & (1 << r)) {
                    u64 t = 0ull;
#pragma unroll
                    for (int i = 0; i < 8; ++i) t = fma2(dy[r][i], v2[i], t);
                    dp[r] = hsum2(t);
                }
        }
        u64 k2[8];
        lds_vec16(kb, lr + di, k2);
        float bk = 0.f;
        if (DIST) {
            u64 n = 0ull;
#pragma unroll
            for (int i = 0; i < 8; ++i) n = fma2(k2[i], k2[i], n);
            bk = -0.5f * sl2 * hsum2(n);
        }
#pragma unroll
        for (int r = 0; r < 4; ++r)
            if (MASK & (1 << r)) {
                u64 t = 0ull;
#pragma unroll
                for (int i = 0; i < 8; ++i) t = fma2(q[r][i], k2[i], t);
                const float s2 = hsum2(t) + (DIST ? bq[r] + bk : 0.f);
                const float P = fast_exp2(s2 - L2[r]);
                const float ds = P * (dp[r] - D[r]);
                if (DIST) sumds[r] += ds;
                const u64 d2 = pack2(ds, ds);
#pragma unroll
                for (int i = 0; i < 8; ++i) dq[r][i] = fma2(d2, k2[i], dq[r][i]);
            }
    }
}

template <bool DIST, int CPE>
__global__ void __launch_bounds__(128) dq_tiled_kernel(TileArgs a, const __grid_constant__ CUtensorMap m0,
                                                       const __grid_constant__ CUtensorMap m1,
                                                       const __grid_constant__ CUtensorMap msc) {
    const Geo& g = a.g;
    const int ROWS = a.TH + 2 * (g.p + a.roff);
    const int w0 = blockIdx.x * 4, h0 = blockIdx.y * a.TH, u = blockIdx.z;
    const int lr = threadIdx.x, h = h0 + lr;
    const bool active = h < g.H;
    const float sl2 = a.scale * kLog2e;
    CA_PIPE_PROLOGUE(false)

    u64 q[4][8], dy[4][8], dq[4][8];
    load_centre<CPE>(a.c0, g, u, h, w0, active, sl2, q);
    load_centre<CPE>(a.c1, g, u, h, w0, active, 1.f, dy);
    float L2[4], D[4], bq[4], sumds[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const bool ok = active && (w0 + r < g.W);
        const int64_t o = (int64_t)u * g.Np + h + g.H * (w0 + r);
        L2[r] = ok ? __ldg(a.cs0 + o) * kLog2e : 0.f;
        D[r] = ok ? __ldg(a.cs1 + o) : 0.f;
        sumds[r] = 0.f;
        bq[r] = 0.f;
        if (DIST) {
            u64 n = 0ull;
#pragma unroll
            for (int i = 0; i < 8; ++i) n = fma2(q[r][i], q[r][i], n);
            bq[r] = -0.5f * hsum2(n) / sl2;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) dq[r][i] = 0ull;
    }

    CA_PIPE_LOOP({
        const int mask = stage_mask(s, g.p);
        const float* kb = pipe.vec0(buf);
        const float* vb = pipe.vec1(buf);
        CA_MASK_SWITCH(mask, (dq_stage<DIST, MK>(kb, vb, lr + a.roff, g.ws, sl2, q, dy, dq, L2, D, bq, sumds)));
    })
    // dq = scale * (sum ds*k - [distance] sum(ds) * q);  q registers hold q*scale*log2(e)
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float x, y, qx, qy;
            unpack2(dq[r][i], x, y);
            unpack2(q[r][i], qx, qy);
            x = a.scale * x - (DIST ? sumds[r] * qx * kLn2 : 0.f);
            y = a.scale * y - (DIST ? sumds[r] * qy * kLn2 : 0.f);
            store_centre<CPE>(a.o0, g, u, h, w0, active, r, i, x, y);
        }
}

// =====================================================================
// Backward, key-owned: dk and dv.  Two lanes share a row: lane&1 selects the
// channel half; partial dot products are completed with one shuffle.
// =====================================================================
template <bool DIST, int MASK>
__device__ __forceinline__ void dkdv_stage(const float* qb, const float* dyb, const float* Lb, const float* Db,
                                           int lr, int half, int ws, float sl2, const u64 (&k)[4][4],
                                           const u64 (&v)[4][4], u64 (&dk)[4][4], u64 (&dv)[4][4],
                                           const float (&bk)[4], float (&sumds)[4]) {
#pragma unroll 1
    for (int di = 0; di < ws; ++di) {
        const int row = lr + di;
        u64 q2[4], y2[4];
        lds_vec8(qb, row, half, q2);
        lds_vec8(dyb, row, half, y2);
        const float Lj = Lb[row], Dj = Db[row];
        float bqj = 0.f;
        if (DIST) {
            u64 n = 0ull;
#pragma unroll
            for (int i = 0; i < 4; ++i) n = fma2(q2[i], q2[i], n);
            float t = hsum2(n);
            t += __shfl_xor_sync(0xffffffffu, t, 1);
            bqj = -0.5f * sl2 * t;
        }
#pragma unroll
        for (int r = 0; r < 4; ++r)
            if (MASK & (1 << r)) {
                u64 t = 0ull, w = 0ull;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    t = fma2(k[r][i], q2[i], t);
                    w = fma2(v[r][i], y2[i], w);
                }
                float s2 = hsum2(t), dp = hsum2(w);
                s2 += __shfl_xor_sync(0xffffffffu, s2, 1);
                dp += __shfl_xor_sync(0xffffffffu, dp, 1);
                if (DIST) s2 += bk[r] + bqj;
                const float P = fast_exp2(s2 - Lj);
                const float ds = P * (dp - Dj);
                if (DIST) sumds[r] += ds;
                const u64 d2 = pack2(ds, ds), p2 = pack2(P, P);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    dk[r][i] = fma2(d2, q2[i], dk[r][i]);
                    dv[r][i] = fma2(p2, y2[i], dv[r][i]);
                }
            }
    }
}

template <bool DIST, int CPE>
__global__ void __launch_bounds__(256) dkdv_tiled_kernel(TileArgs a, const __grid_constant__ CUtensorMap m0,
                                                         const __grid_constant__ CUtensorMap m1,
                                                         const __grid_constant__ CUtensorMap msc) {
    const Geo& g = a.g;
    const int ROWS = a.TH + 2 * (g.p + a.roff);
    const int w0 = blockIdx.x * 4, h0 = blockIdx.y * a.TH, u = blockIdx.z;
    const int lr = threadIdx.x >> 1, half = threadIdx.x & 1, h = h0 + lr;
    const bool active = h < g.H;
    const float sl2 = a.scale * kLog2e;
    CA_PIPE_PROLOGUE(true)

    u64 k[4][4], v[4][4], dk[4][4], dv[4][4];
    float bk[4], sumds[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const bool ok = active && (w0 + r < g.W);
        const int pix = h + g.H * (w0 + r);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float kx = 0.f, ky = 0.f, vx = 0.f, vy = 0.f;
            if (ok) {
                const int cc = 8 * half + 2 * i;
                if (CPE == 1) {
                    kx = __ldg(a.c0 + goff<1>(u, cc, g.Np, pix));
                    ky = __ldg(a.c0 + goff<1>(u, cc + 1, g.Np, pix));
                    vx = __ldg(a.c1 + goff<1>(u, cc, g.Np, pix));
                    vy = __ldg(a.c1 + goff<1>(u, cc + 1, g.Np, pix));
                } else {
                    const float2 tk = __ldg(reinterpret_cast<const float2*>(a.c0 + goff<2>(u, cc, g.Np, pix)));
                    const float2 tv = __ldg(reinterpret_cast<const float2*>(a.c1 + goff<2>(u, cc, g.Np, pix)));
                    kx = tk.x; ky = tk.y; vx = tv.x; vy = tv.y;
                }
            }
            k[r][i] = pack2(kx * sl2, ky * sl2);
            v[r][i] = pack2(vx, vy);
            dk[r][i] = 0ull;
            dv[r][i] = 0ull;
        }
        sumds[r] = 0.f;
        bk[r] = 0.f;
        if (DIST) {
            u64 n = 0ull;
#pragma unroll
            for (int i = 0; i < 4; ++i) n = fma2(k[r][i], k[r][i], n);
            float t = hsum2(n);
            t += __shfl_xor_sync(0xffffffffu, t, 1);
            bk[r] = -0.5f * t / sl2;
        }
    }

    CA_PIPE_LOOP({
        const int mask = stage_mask(s, g.p);
        CA_MASK_SWITCH(mask, (dkdv_stage<DIST, MK>(pipe.vec0(buf), pipe.vec1(buf), pipe.sc0(buf), pipe.sc1(buf),
                                                   lr + a.roff, half, g.ws, sl2, k, v, dk, dv, bk, sumds)));
    })
    // dk = scale * (sum ds*q - [distance] sum(ds) * k);  k registers hold k*scale*log2(e)
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        if (!(active && (w0 + r < g.W))) continue;
        const int pix = h + g.H * (w0 + r);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float x, y, kx, ky, vx, vy;
            unpack2(dk[r][i], x, y);
            unpack2(k[r][i], kx, ky);
            unpack2(dv[r][i], vx, vy);
            x = a.scale * x - (DIST ? sumds[r] * kx * kLn2 : 0.f);
            y = a.scale * y - (DIST ? sumds[r] * ky * kLn2 : 0.f);
            const int cc = 8 * half + 2 * i;
            if (CPE == 1) {
                a.o0[goff<1>(u, cc, g.Np, pix)] = x;
                a.o0[goff<1>(u, cc + 1, g.Np, pix)] = y;
                a.o1[goff<1>(u, cc, g.Np, pix)] = vx;
                a.o1[goff<1>(u, cc + 1, g.Np, pix)] = vy;
            } else {
                *reinterpret_cast<float2*>(a.o0 + goff<2>(u, cc, g.Np, pix)) = make_float2(x, y);
                *reinterpret_cast<float2*>(a.o1 + goff<2>(u, cc, g.Np, pix)) = make_float2(vx, vy);
            }
        }
    }
}

// =====================================================================
// Pack kernel: reference layout -> [unit][column][row'][16] with the circular
// halo along h unrolled, plus (optionally) the two scalar planes
// [2*unit + {0: stats*log2(e), 1: D}][column][row'].  One thread per (row', column, unit).
// =====================================================================
struct PackArgs {
    Geo g;
    int pp;                 // p' (even)
    int Hp;                 // padded rows per column: roundup4(H + 2p')
    int nt;                 // number of tensors to pack (<= 4)
    const float* src[4];
    float* dst[4];
    float* planes;          // nullable
    const float* stats;     // with planes
    const float* Din;       // with planes: D given ...
    const float* y;         // ... or computed as dy . y
    const float* dy;
    float* Dout;            // nullable: D in the reference layout (interior rows)
};

template <int CPE>
__global__ void __launch_bounds__(128) pack_kernel(PackArgs a) {
    const Geo& g = a.g;
    const int rr = blockIdx.x * blockDim.x + threadIdx.x;
    const int w = blockIdx.y, u = blockIdx.z;
    if (rr >= a.Hp) return;
    const bool real_row = rr < g.H + 2 * a.pp;
    const int hs = real_row ? (rr - a.pp + g.H) % g.H : 0;
    const int pix = hs + g.H * w;
    const int64_t orow = ((int64_t)u * g.Wk + w) * a.Hp + rr;
    for (int t = 0; t < a.nt; ++t) {
        float4 c[4];
        if (real_row) {
            if (CPE == 1) {
                const float* sp = a.src[t] + goff<1>(u, 0, g.Npk, pix);
                float v[16];
#pragma unroll
                for (int cc = 0; cc < 16; ++cc) v[cc] = __ldg(sp + (int64_t)cc * g.Npk);
#pragma unroll
                for (int i = 0; i < 4; ++i) c[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 lo = __ldg(reinterpret_cast<const float2*>(a.src[t] + goff<2>(u, 4 * i, g.Npk, pix)));
                    const float2 hi = __ldg(reinterpret_cast<const float2*>(a.src[t] + goff<2>(u, 4 * i + 2, g.Npk, pix)));
                    c[i] = make_float4(lo.x, lo.y, hi.x, hi.y);
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) c[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        float4* dp = reinterpret_cast<float4*>(a.dst[t] + orow * 16);
#pragma unroll
        for (int i = 0; i < 4; ++i) dp[i] = c[i];
    }
    if (a.planes) {
        float L = 0.f, D = 0.f;
        if (real_row) {
            const int64_t so = (int64_t)u * g.Npk + pix;
            L = __ldg(a.stats + so) * kLog2e;
            if (a.Din) {
                D = __ldg(a.Din + so);
            } else {
#pragma unroll
                for (int cc = 0; cc < 16; ++cc) {
                    const int64_t o = goff<CPE>(u, cc, g.Npk, pix);
                    D = fmaf(__ldg(a.dy + o), __ldg(a.y + o), D);
                }
                if (a.Dout && rr >= a.pp && rr < a.pp + g.H) a.Dout[so] = D;
            }
        }
        const int64_t plane = (int64_t)g.Wk * a.Hp;
        a.planes[(2 * (int64_t)u) * plane + (int64_t)w * a.Hp + rr] = L;
        a.planes[(2 * (int64_t)u + 1) * plane + (int64_t)w * a.Hp + rr] = D;
    }
}

// ---------------------------------------------------------------- host side
struct Padded {
    int pp, Hp;
    size_t tensor_floats;   // one packed tensor
    size_t plane_floats;    // both scalar planes
};

Padded padded_of(const Geo& g) {
    Padded P;
    P.pp = (g.p + 1) & ~1;
    P.Hp = (g.H + 2 * P.pp + 3) & ~3;
    P.tensor_floats = (size_t)g.units * g.Wk * P.Hp * 16;
    P.plane_floats = (size_t)2 * g.units * g.Wk * P.Hp;
    return P;
}

bool tiled_shape_ok(const Geo& g) {
    return g.cr == 16 && g.wsw == g.ws && g.ws >= 3 && g.H >= 16 && g.ws <= 63;
}

int pick_rows(const Geo& g, int rows_per_warp, int max_warps) {
    int warps = (g.H + rows_per_warp - 1) / rows_per_warp;
    if (warps > max_warps) warps = max_warps;
    return warps;
}

int pick_dc(int ws) {
    int best = 5, waste = 1 << 30;
    for (int dc : {3, 4, 5, 7}) {
        const int w = (ws + dc - 1) / dc * dc - ws;
        if (w < waste || (w == waste && dc > best)) { waste = w; best = dc; }
    }
    return best;
}

int launch_pack(const PackArgs& a, cudaStream_t st) {
    dim3 grid((a.Hp + 127) / 128, a.g.Wk, a.g.units);
    if (a.g.cpe == 1) pack_kernel<1><<<grid, 128, 0, st>>>(a);
    else pack_kernel<2><<<grid, 128, 0, st>>>(a);
    CA_CHECK_LAUNCH("pack kernel");
    return CA_OK;
}

struct Launch {
    TileArgs a;
    CUtensorMap m0, m1, msc;
    dim3 grid;
    int threads;
    size_t smem;
};

// Fills the launch geometry and the tensor maps of the packed tensors t0, t1
// (and the scalar planes when given).
int prepare(const Geo& g, const Padded& P, int rows_per_warp, int max_warps, const float* t0, const float* t1,
            const float* planes, Launch* L) {
    const int warps = pick_rows(g, rows_per_warp, max_warps);
    TileArgs& a = L->a;
    a.g = g;
    a.TH = rows_per_warp * warps;
    a.roff = P.pp - g.p;
    const int ROWS = a.TH + 2 * P.pp;
    if (ROWS > 256) { set_error("tile of %d rows exceeds the TMA box limit", ROWS); return CA_ERR_UNSUPPORTED; }
    const int vstride = (ROWS * 64 + 511) & ~511, sstride = (ROWS * 4 + 127) & ~127;
    a.stage_bytes = (2 * vstride + (planes ? 2 * sstride : 0) + 1023) & ~1023;
    L->smem = (size_t)kStages * a.stage_bytes + 1024;
    L->grid = dim3((g.W + 3) / 4, (g.H + a.TH - 1) / a.TH, g.units);
    L->threads = 32 * warps;
    const uint64_t dims[4] = {16, (uint64_t)P.Hp, (uint64_t)g.Wk, (uint64_t)g.units};
    const uint64_t strides[3] = {64, (uint64_t)P.Hp * 64, (uint64_t)P.Hp * 64 * g.Wk};
    const uint32_t box[4] = {16, (uint32_t)ROWS, 1, 1};
    int rc;
    if ((rc = encode_tensor_map(&L->m0, t0, 4, dims, strides, box, true))) return rc;
    if ((rc = encode_tensor_map(&L->m1, t1, 4, dims, strides, box, true))) return rc;
    if (planes) {
        const uint64_t sdims[3] = {(uint64_t)P.Hp, (uint64_t)g.Wk, (uint64_t)2 * g.units};
        const uint64_t sstr[2] = {(uint64_t)P.Hp * 4, (uint64_t)P.Hp * 4 * g.Wk};
        const uint32_t sbox[3] = {(uint32_t)ROWS, 1, 1};
        if ((rc = encode_tensor_map(&L->msc, planes, 3, sdims, sstr, sbox, false))) return rc;
    } else {
        L->msc = L->m0;
    }
    return CA_OK;
}

template <typename K>
int set_smem(K kernel, size_t bytes) {
    if (bytes > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(shared memory)");
    }
    return CA_OK;
}

#define CA_LAUNCH_TILED(KERNEL, L, st)                                                        \
    do {                                                                                      \
        int rc__ = set_smem(KERNEL, (L).smem);                                                \
        if (rc__) return rc__;                                                                \
        KERNEL<<<(L).grid, (L).threads, (L).smem, st>>>((L).a, (L).m0, (L).m1, (L).msc);      \
    } while (0)

#define CA_DIST_CPE(KERNEL_T, dist, cpe, L, st)                                               \
    do {                                                                                      \
        if ((cpe) == 1) {                                                                     \
            if (dist) CA_LAUNCH_TILED((KERNEL_T<true, 1>), L, st);                            \
            else CA_LAUNCH_TILED((KERNEL_T<false, 1>), L, st);                                \
        } else {                                                                              \
            if (dist) CA_LAUNCH_TILED((KERNEL_T<true, 2>), L, st);                            \
            else CA_LAUNCH_TILED((KERNEL_T<false, 2>), L, st);                                \
        }                                                                                     \
    } while (0)

}  // namespace

// ---------------------------------------------------------------- tensor maps
int encode_tensor_map(CUtensorMap* map, const float* base, int rank, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box, bool swizzle64) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q);
        if (e != cudaSuccess || !sym) {
            set_error("cuTensorMapEncodeTiled is not available from the driver");
            return CA_ERR_CUDA;
        }
        fn = reinterpret_cast<EncodeFn>(sym);
    }
    cuuint64_t gdims[5], gstr[4];
    cuuint32_t gbox[5], estr[5];
    for (int i = 0; i < rank; ++i) { gdims[i] = dims[i]; gbox[i] = box[i]; estr[i] = 1; }
    for (int i = 0; i + 1 < rank; ++i) gstr[i] = strides_bytes[i];
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, (cuuint32_t)rank, const_cast<float*>(base), gdims, gstr,
                    gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
        return CA_ERR_CUDA;
    }
    return CA_OK;
}

// ---------------------------------------------------------------- entry points of this file
size_t tiled_fwd_workspace(const Geo& g) {
    if (!tiled_shape_ok(g)) return 0;
    return 2 * padded_of(g).tensor_floats * sizeof(float) + 256;
}

size_t tiled_bwd_stage_workspace(const Geo& g) {
    if (!tiled_shape_ok(g)) return 0;
    const Padded P = padded_of(g);
    return (2 * P.tensor_floats + P.plane_floats) * sizeof(float) + 256;
}

size_t tiled_bwd_workspace(const Geo& g) {
    if (!tiled_shape_ok(g)) return 0;
    const Padded P = padded_of(g);
    return (4 * P.tensor_floats + P.plane_floats) * sizeof(float) + 256;
}

int tiled_stage_timeouts(int* count) {
    cudaError_t e = cudaMemcpyFromSymbol(count, g_stage_timeouts, sizeof(int));
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyFromSymbol(stage timeouts)");
    return CA_OK;
}

int tiled_attention_fwd(const Geo& g, float scale, int dist, const float* q, const float* k, const float* v,
                        float* y, float* nz, float* stats, void* workspace, cudaStream_t st) {
    if (!tiled_shape_ok(g) || nz) return CA_ERR_UNSUPPORTED;
    if (!workspace) { set_error("workspace of ca_attention_fwd_workspace() bytes is NULL"); return CA_ERR_NULL; }
    const Padded P = padded_of(g);
    float* kT = static_cast<float*>(workspace);
    float* vT = kT + P.tensor_floats;
    PackArgs pa{};
    pa.g = g; pa.pp = P.pp; pa.Hp = P.Hp; pa.nt = 2;
    pa.src[0] = k; pa.src[1] = v; pa.dst[0] = kT; pa.dst[1] = vT;
    int rc = launch_pack(pa, st);
    if (rc) return rc;
    Launch L{};
    if ((rc = prepare(g, P, 32, 4, kT, vT, nullptr, &L))) return rc;
    L.a.scale = scale; L.a.c0 = q; L.a.o0 = y; L.a.ostats = stats;
    const int dc = pick_dc(g.ws);
#define CA_FWD(DCV)                                                                              \
    do {                                                                                         \
        if (g.cpe == 1) {                                                                        \
            if (dist) CA_LAUNCH_TILED((fwd_tiled_kernel<DCV, true, 1>), L, st);                  \
            else CA_LAUNCH_TILED((fwd_tiled_kernel<DCV, false, 1>), L, st);                      \
        } else {                                                                                 \
            if (dist) CA_LAUNCH_TILED((fwd_tiled_kernel<DCV, true, 2>), L, st);                  \
            else CA_LAUNCH_TILED((fwd_tiled_kernel<DCV, false, 2>), L, st);                      \
        }                                                                                        \
    } while (0)
    switch (dc) {
        case 3: CA_FWD(3); break;
        case 4: CA_FWD(4); break;
        case 7: CA_FWD(7); break;
        default: CA_FWD(5); break;
    }
#undef CA_FWD
    CA_CHECK_LAUNCH("tiled forward kernel");
    return CA_OK;
}

static int run_dq(const Geo& g, const Padded& P, float scale, int dist, const float* q, const float* dy,
                  const float* stats, const float* D, const float* kT, const float* vT, float* dq, cudaStream_t st) {
    Launch L{};
    int rc = prepare(g, P, 32, 4, kT, vT, nullptr, &L);
    if (rc) return rc;
    L.a.scale = scale; L.a.c0 = q; L.a.c1 = dy; L.a.cs0 = stats; L.a.cs1 = D; L.a.o0 = dq;
    CA_DIST_CPE(dq_tiled_kernel, dist, g.cpe, L, st);
    CA_CHECK_LAUNCH("tiled dq kernel");
    return CA_OK;
}

static int run_dkdv(const Geo& g, const Padded& P, float scale, int dist, const float* k, const float* v,
                    const float* qT, const float* dyT, const float* planes, float* dk, float* dv,
                    cudaStream_t st) {
    Launch L{};
    int rc = prepare(g, P, 16, 8, qT, dyT, planes, &L);
    if (rc) return rc;
    L.a.scale = scale; L.a.c0 = k; L.a.c1 = v; L.a.o0 = dk; L.a.o1 = dv;
    CA_DIST_CPE(dkdv_tiled_kernel, dist, g.cpe, L, st);
    CA_CHECK_LAUNCH("tiled dk/dv kernel");
    return CA_OK;
}

int tiled_attention_bwd_dq(const Geo& g, float scale, int dist, const float* q, const float* k, const float* v,
                           const float* dy, const float* stats, const float* D, float* dq, void* workspace,
                           cudaStream_t st) {
    if (!tiled_shape_ok(g)) return CA_ERR_UNSUPPORTED;
    if (!workspace) { set_error("workspace of ca_attention_bwd_stage_workspace() bytes is NULL"); return CA_ERR_NULL; }
    const Padded P = padded_of(g);
    float* kT = static_cast<float*>(workspace);
    float* vT = kT + P.tensor_floats;
    PackArgs pa{};
    pa.g = g; pa.pp = P.pp; pa.Hp = P.Hp; pa.nt = 2;
    pa.src[0] = k; pa.src[1] = v; pa.dst[0] = kT; pa.dst[1] = vT;
    int rc = launch_pack(pa, st);
    if (rc) return rc;
    return run_dq(g, P, scale, dist, q, dy, stats, D, kT, vT, dq, st);
}

int tiled_attention_bwd_dkdv(const Geo& g, float scale, int dist, const float* q, const float* k, const float* v,
                             const float* dy, const float* stats, const float* D, float* dk, float* dv,
                             void* workspace, cudaStream_t st) {
    if (!tiled_shape_ok(g)) return CA_ERR_UNSUPPORTED;
    if (!workspace) { set_error("workspace of ca_attention_bwd_stage_workspace() bytes is NULL"); return CA_ERR_NULL; }
    const Padded P = padded_of(g);
    float* qT = static_cast<float*>(workspace);
    float* dyT = qT + P.tensor_floats;
    float* planes = dyT + P.tensor_floats;
    PackArgs pa{};
    pa.g = g; pa.pp = P.pp; pa.Hp = P.Hp; pa.nt = 2;
    pa.src[0] = q; pa.src[1] = dy; pa.dst[0] = qT; pa.dst[1] = dyT;
    pa.planes = planes; pa.stats = stats; pa.Din = D;
    int rc = launch_pack(pa, st);
    if (rc) return rc;
    return run_dkdv(g, P, scale, dist, k, v, qT, dyT, planes, dk, dv, st);
}

// Whole backward in three launches: pack (all four tensors, D, planes), dq, dk/dv.
int tiled_attention_bwd(const Geo& g, float scale, int dist, const float* q, const float* k, const float* v,
                        const float* y, const float* dy, const float* stats, float* D, float* dq, float* dk,
                        float* dv, void* workspace, cudaStream_t st) {
    if (!tiled_shape_ok(g) || g.Wk != g.W) return CA_ERR_UNSUPPORTED;
    if (!workspace) { set_error("workspace is NULL"); return CA_ERR_NULL; }
    const Padded P = padded_of(g);
    float* kT = static_cast<float*>(workspace);
    float* vT = kT + P.tensor_floats;
    float* qT = vT + P.tensor_floats;
    float* dyT = qT + P.tensor_floats;
    float* planes = dyT + P.tensor_floats;
    PackArgs pa{};
    pa.g = g; pa.pp = P.pp; pa.Hp = P.Hp; pa.nt = 4;
    pa.src[0] = k; pa.src[1] = v; pa.src[2] = q; pa.src[3] = dy;
    pa.dst[0] = kT; pa.dst[1] = vT; pa.dst[2] = qT; pa.dst[3] = dyT;
    pa.planes = planes; pa.stats = stats; pa.y = y; pa.dy = dy; pa.Dout = D;
    int rc = launch_pack(pa, st);
    if (rc) return rc;
    if ((rc = run_dq(g, P, scale, dist, q, dy, stats, D, kT, vT, dq, st))) return rc;
    return run_dkdv(g, P, scale, dist, k, v, qT, dyT, planes, dk, dv, st);
}

int tiled_apply(const Geo&, const float*, const float*, float*, cudaStream_t) { return CA_ERR_UNSUPPORTED; }

}  // namespace ca
