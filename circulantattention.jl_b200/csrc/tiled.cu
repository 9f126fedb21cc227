// Tiled sm_100a kernels for 2-D windows with 16 real channels per unit
// (16 Float32 or 8 ComplexF32 channels per head) and softmax.
//
// Work decomposition.  A CTA owns TH consecutive rows (the fast axis h) of NQ
// consecutive columns w0..w0+NQ-1 of one unit (NQ = 4 in the forward and dq
// kernels, 3 in the dk/dv kernel).  A thread owns one row and the NQ pixels of
// that row ("centre" pixels: queries in the forward and dq kernels, keys in
// the dk/dv kernel) and keeps their 16-channel vectors in registers.  The other
// side of the window is streamed through shared memory one image column at a
// time: column stage s holds column w0 - p + s (wrapped circularly, or taken
// from the neighbour halo in band mode) for rows h0-p' .. h0+TH+p'-1.  Centre
// pixel r pairs with stage s iff r <= s <= r + 2p, so every loaded vector is
// used by up to NQ centre pixels straight from registers.
//
// Feeding the stages.  The reference layout is channel-planar, which no bulk
// copy can turn into pixel vectors, so a pack kernel first rewrites the two
// streamed tensors as ONE array [unit][column][row'][36] = (16 channels of the
// first | 16 of the second | 4 floats of padding) with the circular halo along
// h already unrolled (row' = h + p', p' = p rounded up to even; rows -p'..-1
// and H..H+p'-1 are copies of the wrapped rows).  A column stage is then a
// single contiguous box fetched by cp.async.bulk.tensor (TMA) and tracked by an
// mbarrier; three stages are in flight.  The wrap along w is just the column
// coordinate of the box.
//
// Shared-memory layout: a pixel row is 144 bytes (36 words).  The rows that the
// eight lanes of a 128-bit load phase touch are consecutive, 36 words apart,
// i.e. nine 4-bank groups apart: eight distinct groups, so the loads are
// conflict free without any address swizzle and every chunk of every row of a
// window column is the thread's row base plus a compile-time constant.
//
// Arithmetic: FP32 on the FMA pipe, channel pairs as two scalar FMAs.  Softmax in
// the log2 domain with ex2.approx.  The running maximum (forward) or the saved row
// statistic (backward) is folded into the initial value of the dot-product
// chain, and the forward only touches the maximum when the sign bits of a chunk
// of relative scores say that one of them is positive.
//
// Small grids.  When the grid would not fill the GPU, the column stages of a
// tile are split between two groups of warps of the same CTA (each with its own
// copy pipeline) whose partial results are merged through shared memory.
#include "tiled.cuh"
#include "tma.cuh"
#include <cuda_bf16.h>
#include <stdlib.h>
#include <algorithm>
#include <type_traits>
#include <mutex>
#include <atomic>

namespace ca {
namespace {

// Two-channel arithmetic: a channel pair lives in two ordinary registers and a pair operation is
// two scalar FMAs.  (Packed fma.rn.f32x2 was measured slower here: a dot product or an outer
// product has two fresh 64-bit operands per instruction, which the register file does not deliver
// at the packed rate.)
struct u64 { float x, y; };
__device__ __forceinline__ u64 pack2(float a, float b) { return u64{a, b}; }
__device__ __forceinline__ void unpack2(u64 v, float& a, float& b) { a = v.x; b = v.y; }
__device__ __forceinline__ u64 fma2(u64 a, u64 b, u64 c) { return u64{fmaf(a.x, b.x, c.x), fmaf(a.y, b.y, c.y)}; }
__device__ __forceinline__ u64 mul2(u64 a, u64 b) { return u64{a.x * b.x, a.y * b.y}; }
__device__ __forceinline__ u64 add2(u64 a, u64 b) { return u64{a.x + b.x, a.y + b.y}; }
__device__ __forceinline__ u64 zero2() { return u64{0.f, 0.f}; }
__device__ __forceinline__ void lds128(uint32_t addr, u64& lo, u64& hi) {
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(lo.x), "=f"(lo.y), "=f"(hi.x), "=f"(hi.y) : "r"(addr));
}
__device__ __forceinline__ float hsum2(u64 v) {
    float a, b;
    unpack2(v, a, b);
    return a + b;
}

// Sum of a per-lane partial over the NS lanes that share a pixel (NS = 1: nothing to do).
template <int NS>
__device__ __forceinline__ float lane_sum(float x) {
#pragma unroll
    for (int m = 1; m < NS; m <<= 1) x += __shfl_xor_sync(0xffffffffu, x, m);
    return x;
}

struct TileArgs {
    Geo g;
    float scale;
    int TH;                 // rows per CTA
    int roff;               // p' - p: first window row inside a stage buffer
    int stage_bytes;        // bytes of one stage buffer (multiple of 1024)
    int nsplit;             // 1 or 2 groups of warps sharing the stages of a tile
    int which;              // half of the packed pair a single-tensor kernel streams (0 or 1)
    int iter;               // entmax threshold search: number of the step (late steps fall back to Newton)
    int row_bytes;          // bytes of one packed pixel row: 144 per 16-channel slab
    int nstages;            // copy stages in flight per part: 2 or 3 (kStages)
    const float* c0;        // centre tensors (reference layout)
    const float* c1;
    const float* cs0;       // centre scalars (dq kernel: stats, D)
    const float* cs1;
    float* o0;              // outputs
    float* o1;
    float* ostats;
    int* status;            // nullable device word of the caller: bit 0 is set when a stage wait ran out
    uint32_t wait_tries;    // polls before a stage wait gives up
};

constexpr int kStages = 3;
constexpr uint32_t kWaitTries = 1u << 20;
constexpr int kEntmaxFwdSteps = 16;            // launches of the entmax threshold step (settled blocks leave at once)

// Number of CTAs that gave up waiting for a stage copy (stays 0 in a healthy run).
__device__ int g_stage_timeouts = 0;

constexpr int kRowFloats = 36;                 // 16 + 16 + 4 padding
constexpr int kRowBytes = kRowFloats * 4;      // 144
constexpr int kRunChunk = 32;                  // window rows whose entries of A are staged at a time
constexpr int kSingleFloats = 20;              // single-tensor rows: 16 + 4 padding (80 bytes, also conflict free)

// Units with 16*NS real channels ("slabs" of 16) pack a pixel row as 36*NS words: the first
// tensor's channels, then the second's, then 4*NS words of padding.  Inside a tensor's part the
// order is [4-channel chunk][slab][4]: chunk c of slab s sits 16*(c*NS + s) bytes in, so the NS
// lanes that share a pixel read consecutive 16-byte pieces, and the row stride (144*NS bytes:
// 16, 32 or 64 bytes past a multiple of 128) spreads the 8/NS pixels of a 128-bit load phase over
// distinct bank groups.  NS = 1 is the plain channel order.
// 16-channel slab `slab` of tensor `which` of the pixel row at shared-space byte address `a0`.
template <int NS>
__device__ __forceinline__ void lds_slab16(uint32_t a0, int which, int slab, u64 (&v)[8]) {
    const uint32_t b = a0 + which * (64 * NS) + slab * 16;
    lds128(b, v[0], v[1]);
    lds128(b + 16 * NS, v[2], v[3]);
    lds128(b + 32 * NS, v[4], v[5]);
    lds128(b + 48 * NS, v[6], v[7]);
}

// Global offset of real channel cc of unit u at pixel pix (npix pixels per plane, NCR real
// channels per unit).
template <int CPE, int NCR = 16>
__device__ __forceinline__ int64_t goff(int u, int cc, int npix, int pix) {
    if (CPE == 1) return ((int64_t)u * NCR + cc) * npix + pix;
    return (((int64_t)u * (NCR / 2) + (cc >> 1)) * npix + pix) * 2 + (cc & 1);
}

// Window radius along w: p for 2-D windows, 0 for a folded 1-D signal (wsw == 1), whose window
// runs along h only and continues into the neighbouring columns through the packed halo rows.
__device__ __forceinline__ int radius_w(const Geo& g) { return (g.wsw - 1) >> 1; }

__device__ __forceinline__ int stage_column(const Geo& g, int w0, int s) {
    int kc = (w0 - radius_w(g) + s + g.wk_off) % g.Wk;
    return kc < 0 ? kc + g.Wk : kc;
}

// Rotation of the sorted run of a CSR row: the entry of window offset d sits at (d + p + rot) mod ws,
// where the row's pixel has coordinate x on the window axis of length X (src/circulant.jl:11-15).
__device__ __forceinline__ int run_rot(int x, int X, int p, int ws) {
    return x < p ? x - p + ws : (x >= X - p ? x - p - X + ws : 0);
}
// Coordinate and length of the window axis for pixel (h, w): the image row in 2-D, the linear
// index in a folded 1-D signal.
__device__ __forceinline__ int axis_coord(const Geo& g, int h, int w) { return g.wsw == 1 ? h + g.H * w : h; }
__device__ __forceinline__ int axis_len(const Geo& g) { return g.wsw == 1 ? g.Np : g.H; }

template <int NQ>
__device__ __forceinline__ int stage_mask(int s, int p) {
    int mask = 0;
#pragma unroll
    for (int r = 0; r < NQ; ++r)
        if (s >= r && s <= r + 2 * p) mask |= 1 << r;
    return mask;
}

// Barrier of one group of warps (ids 1 and 2; id 0 stays the CTA-wide barrier).
__device__ __forceinline__ void part_sync(int part, int nthreads) {
    if (part == 0) asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
    else asm volatile("bar.sync 2, %0;" ::"r"(nthreads) : "memory");
}

// ---------------------------------------------------------------------------
// Stage pipeline of one group of warps ("part").  Thread 0 of the part is the
// producer: it arms the stage's mbarrier with the byte count and issues the
// TMA boxes; every consumer wait is bounded.
// ---------------------------------------------------------------------------
template <bool NSC>
struct StagePipe {
    uint64_t* full;          // kStages barriers of this part
    unsigned char* base;     // kStages stage buffers of this part
    const CUtensorMap* mv;
    const CUtensorMap* msc;
    int ROWS, stage_bytes, row_bytes, u, h0, w0;

    __device__ __forceinline__ unsigned char* vec(int buf) const { return base + (size_t)buf * stage_bytes; }
    __device__ __forceinline__ int sstride() const { return (ROWS * 4 + 127) & ~127; }
    __device__ __forceinline__ int vbytes() const { return (ROWS * row_bytes + 127) & ~127; }
    __device__ __forceinline__ float* sc0(int buf) const { return reinterpret_cast<float*>(vec(buf) + vbytes()); }
    __device__ __forceinline__ float* sc1(int buf) const { return reinterpret_cast<float*>(vec(buf) + vbytes() + sstride()); }

    __device__ __forceinline__ void issue(const Geo& g, int s, int buf) const {
        const int kc = stage_column(g, w0, s);
        mbar_arrive_expect_tx(&full[buf], (uint32_t)(ROWS * row_bytes + (NSC ? ROWS * 8 : 0)));
        tma_load_4d(vec(buf), mv, 0, h0, kc, u, &full[buf]);
        if (NSC) {
            tma_load_3d(sc0(buf), msc, h0, kc, 2 * u, &full[buf]);
            tma_load_3d(sc1(buf), msc, h0, kc, 2 * u + 1, &full[buf]);
        }
    }
};

// Declares the pipeline of this thread's part and starts the first copies.
// Needs in scope: a (TileArgs), g, ROWS, u, h0, w0, NSTAGES (stages of the tile), mv, msc.
#define CA_PIPE_PROLOGUE(NSCV)                                                                       \
    extern __shared__ unsigned char smem_raw[];                                                      \
    __shared__ __align__(8) uint64_t full_bar[2 * kStages];                                          \
    __shared__ int s_err;                                                                            \
    const int PT = blockDim.x / a.nsplit;          /* threads per part */                            \
    const int part = threadIdx.x / PT;                                                               \
    const int lt = threadIdx.x - part * PT;                                                          \
    const int s_begin = part * (NSTAGES / a.nsplit);                                                      \
    const int s_end = (part + 1 == a.nsplit) ? NSTAGES : (part + 1) * (NSTAGES / a.nsplit);                    \
    unsigned char* smem_al = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);            \
    StagePipe<NSCV> pipe;                                                                            \
    pipe.full = full_bar + part * kStages;                                                           \
    pipe.base = smem_al + (size_t)part * a.nstages * a.stage_bytes;                                  \
    pipe.mv = &mv; pipe.msc = &msc;                                                                  \
    pipe.ROWS = ROWS; pipe.stage_bytes = a.stage_bytes; pipe.row_bytes = a.row_bytes;                \
    pipe.u = u; pipe.h0 = h0; pipe.w0 = w0;                                                          \
    if (threadIdx.x == 0) {                                                                          \
        for (int i = 0; i < 2 * kStages; ++i) mbar_init(&full_bar[i], 1);                            \
        s_err = 0;                                                                                   \
        mbar_fence_init();                                                                           \
    }                                                                                                \
    __syncthreads();                                                                                 \
    if (lt == 0)                                                                                     \
        for (int i = 0; i < a.nstages && s_begin + i < s_end; ++i) pipe.issue(g, s_begin + i, i);

// Consumer loop over the stages of this part: bounded wait, BODY, recycle the buffer.
#define CA_PIPE_LOOP(...)                                                                            \
    for (int s = s_begin; s < s_end; ++s) {                                                          \
        const int it = s - s_begin;                                                                  \
        const int buf = it % a.nstages;                                                              \
        if (!mbar_wait(&pipe.full[buf], (uint32_t)((it / a.nstages) & 1), a.wait_tries)) s_err = 1;  \
        __VA_ARGS__                                                                                  \
        part_sync(part, PT);                                                                         \
        if (s_err) break;                                                                            \
        if (lt == 0 && s + a.nstages < s_end) pipe.issue(g, s + a.nstages, buf);                     \
    }                                                                                                \
    __syncthreads();                                                                                 \
    /* A wait that ran out: the CTA stops computing, reports (device counter, caller's status word)  \
       and poisons what it still stores with NaN, so that the failure cannot pass for a result. */   \
    float ca_poison = 0.f;                                                                           \
    if (s_err) {                                                                                     \
        /* give copies still in flight a bounded chance to land before the CTA exits */              \
        if (lt == 0)                                                                                 \
            for (int i = 0; i < a.nstages; ++i) mbar_wait(&pipe.full[i], 0, 1u << 12);               \
        if (threadIdx.x == 0) {                                                                      \
            atomicAdd(&g_stage_timeouts, 1);                                                         \
            if (a.status) atomicOr(a.status, 1);                                                     \
        }                                                                                            \
        ca_poison = __int_as_float(0x7fc00000);                                                      \
    }

// One real element of a dense tensor stored as Float32 or bfloat16 (element offset `off`).
// BF is a compile-time flag so that a batch of loads stays a batch of independent loads; callers
// branch once on Geo::bf16 around the whole batch.
template <bool BF>
__device__ __forceinline__ float ld_real(const float* base, int64_t off) {
    if (BF) {
        const unsigned short h = __ldg(reinterpret_cast<const unsigned short*>(base) + off);
        return __uint_as_float((unsigned)h << 16);
    }
    return __ldg(base + off);
}
template <bool BF>
__device__ __forceinline__ void st_real(float* base, int64_t off, float v) {
    if (BF) reinterpret_cast<__nv_bfloat16*>(base)[off] = __float2bfloat16_rn(v);
    else base[off] = v;
}

// Runs the statements once with `constexpr bool BF` (bfloat16 storage) and `constexpr int NCRV`
// (8 or 16 real channels per unit) set from the geometry: one uniform branch around a whole
// epilogue instead of one per element.  Needs CPE and g in scope.
#define CA_OUT_DISPATCH_NCR(NCRVAL, ...)               \
    if (CPE == 1 && g.bf16) {                          \
        constexpr bool BF = true;                      \
        constexpr int NCRV = NCRVAL;                   \
        __VA_ARGS__                                    \
    } else {                                           \
        constexpr bool BF = false;                     \
        constexpr int NCRV = NCRVAL;                   \
        __VA_ARGS__                                    \
    }
#define CA_BF_DISPATCH(...)                            \
    if (g.cr == 8) {                                   \
        CA_OUT_DISPATCH_NCR(8, __VA_ARGS__)            \
    } else {                                           \
        CA_OUT_DISPATCH_NCR(16, __VA_ARGS__)           \
    }

// Loads the 16-channel vectors of the NQ centre pixels of this thread, times `mul`.
template <int CPE, int NQ, int NCR, bool BF>
__device__ __forceinline__ void load_centre_impl(const float* src, const Geo& g, int u, int h, int w0, bool active,
                                                 float mul, u64 (&dst)[NQ][8], int ch0) {
#pragma unroll
    for (int r = 0; r < NQ; ++r) {
        const bool ok = active && (w0 + r < g.W);
        const int pix = h + g.H * (w0 + r);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float x = 0.f, y = 0.f;
            if (ok && (NCR >= 16 || 2 * i < NCR)) {         // units narrower than a slab are zero-extended
                if (CPE == 1) {
                    x = ld_real<BF>(src, goff<1, NCR>(u, ch0 + 2 * i, g.Np, pix));
                    y = ld_real<BF>(src, goff<1, NCR>(u, ch0 + 2 * i + 1, g.Np, pix));
                } else {
                    const float2 t = __ldg(reinterpret_cast<const float2*>(src + goff<2, NCR>(u, ch0 + 2 * i, g.Np, pix)));
                    x = t.x;
                    y = t.y;
                }
            }
            dst[r][i] = pack2(x * mul, y * mul);
        }
    }
}

template <int CPE, int NQ, int NCR = 16>
__device__ __forceinline__ void load_centre(const float* src, const Geo& g, int u, int h, int w0, bool active,
                                            float mul, u64 (&dst)[NQ][8], int ch0 = 0) {
    if (NCR == 16 && g.cr == 8) {
        // a kernel compiled for one 16-channel slab running on 8-channel units: zero-extended
        if (CPE == 1 && g.bf16) load_centre_impl<CPE, NQ, 8, true>(src, g, u, h, w0, active, mul, dst, ch0);
        else load_centre_impl<CPE, NQ, 8, false>(src, g, u, h, w0, active, mul, dst, ch0);
        return;
    }
    if (CPE == 1 && g.bf16) load_centre_impl<CPE, NQ, NCR, true>(src, g, u, h, w0, active, mul, dst, ch0);
    else load_centre_impl<CPE, NQ, NCR, false>(src, g, u, h, w0, active, mul, dst, ch0);
}

template <int CPE, int NCR = 16, bool BF = false>
__device__ __forceinline__ void store_centre(float* dst, const Geo& g, int u, int h, int w0, bool active, int r,
                                             int i, float x, float y, int ch0 = 0) {
    if (!(active && (w0 + r < g.W))) return;
    if (NCR < 16 && 2 * i >= NCR) return;
    const int pix = h + g.H * (w0 + r);
    if (CPE == 1) {
        st_real<BF>(dst, goff<1, NCR>(u, ch0 + 2 * i, g.Np, pix), x);
        st_real<BF>(dst, goff<1, NCR>(u, ch0 + 2 * i + 1, g.Np, pix), y);
    } else {
        *reinterpret_cast<float2*>(dst + goff<2, NCR>(u, ch0 + 2 * i, g.Np, pix)) = make_float2(x, y);
    }
}

// MASK != 0: all centre pixels pair with this stage (compile time);
// MASK == 0: the set is the run-time `rm` (warp-uniform branches).
#define CA_ON(r) ((MASK != 0) || ((rm >> (r)) & 1))

// =====================================================================
// Forward
// =====================================================================
// Scores are kept relative to a running reference ref = (largest score seen when
// the reference was last set) + kHeadroom: the dot-product chain starts at -ref,
// so sc = s - ref and p = 2^sc needs no subtraction.  The reference moves only
// when some relative score of the chunk is non-negative (a score jumped more than
// kHeadroom log2 units above every earlier one), which the AND of the sign bits
// of the chunk reveals; with O(1) scores that happens almost never after the
// first key.  2^-kHeadroom only rescales p, l and acc together; it cancels in y.
constexpr float kHeadroom = 12.f;
// NS lanes share a pixel (units of 16*NS real channels): every lane holds one 16-channel slab of q and
// of the accumulator, scores are the lane sums of the per-slab partial dot products, and the terms that
// enter a score once (the running reference, in nm2) sit on slab 0 only.
template <int DC, bool DIST, int MASK, int NQ, int NS = 1>
__device__ __forceinline__ void fwd_stage(uint32_t rowbase, int ws, int rm, float sl2, const u64 (&q)[NQ][8],
                                          u64 (&acc)[NQ][8], u64 (&nm2)[NQ], float (&l)[NQ], const float (&bq)[NQ],
                                          int slab = 0) {
    constexpr int RB = kRowBytes * NS;
    for (int c0 = 0; c0 < ws; c0 += DC) {
        const uint32_t cb = rowbase + c0 * RB;
        float sc[NQ][DC];
        // one vector ahead: the next key (or the first v) is requested before this key's FMAs
        u64 nxt[8];
        lds_slab16<NS>(cb, 0, slab, nxt);
#pragma unroll
        for (int t = 0; t < DC; ++t) {
            {
                u64 k2[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) k2[i] = nxt[i];
                if (t + 1 < DC) lds_slab16<NS>(cb + (t + 1) * RB, 0, slab, nxt);
                else lds_slab16<NS>(cb, 1, slab, nxt);
                float bk = 0.f;
                if (DIST) {
                    u64 n = zero2();
#pragma unroll
                    for (int i = 0; i < 8; ++i) n = fma2(k2[i], k2[i], n);
                    bk = -0.5f * sl2 * hsum2(n);
                }
                if (MASK != 0) {
                    // all four chains advance together (4 independent FMAs in flight)
                    u64 sa[NQ];
#pragma unroll
                    for (int r = 0; r < NQ; ++r) {
                        sa[r] = nm2[r];                           // (-ref, 0)
                        if (DIST) sa[r] = add2(sa[r], pack2(bq[r] + bk, 0.f));
                    }
#pragma unroll
                    for (int i = 0; i < 8; ++i)
#pragma unroll
                        for (int r = 0; r < NQ; ++r) sa[r] = fma2(q[r][i], k2[i], sa[r]);
#pragma unroll
                    for (int r = 0; r < NQ; ++r) sc[r][t] = lane_sum<NS>(hsum2(sa[r]));
                } else {
#pragma unroll
                    for (int r = 0; r < NQ; ++r)
                        if (CA_ON(r)) {
                            u64 sa = nm2[r];
                            if (DIST) sa = add2(sa, pack2(bq[r] + bk, 0.f));
#pragma unroll
                            for (int i = 0; i < 8; ++i) sa = fma2(q[r][i], k2[i], sa);
                            sc[r][t] = lane_sum<NS>(hsum2(sa));       // rm is warp-uniform: all lanes shuffle
                        } else {
                            sc[r][t] = -INFINITY;
                        }
                }
            }
        }
        // any relative score >= 0 ?  (sign bit clear)
        uint32_t allneg = 0x80000000u;
#pragma unroll
        for (int r = 0; r < NQ; ++r)
#pragma unroll
            for (int t = 0; t < DC; ++t) allneg &= __float_as_uint(sc[r][t]);
        if (__any_sync(0xffffffffu, allneg == 0u)) {
#pragma unroll
            for (int r = 0; r < NQ; ++r) {
                float cm = sc[r][0];
#pragma unroll
                for (int t = 1; t < DC; ++t) cm = fmaxf(cm, sc[r][t]);
                if (cm >= 0.f) {                // move the reference of this row up by cm + headroom
                    cm += kHeadroom;
                    const float corr = fast_exp2(-cm);
                    float nm, zero;
                    unpack2(nm2[r], nm, zero);
                    nm2[r] = pack2(nm - (NS == 1 || slab == 0 ? cm : 0.f), 0.f);
                    l[r] *= corr;
                    const u64 c2 = pack2(corr, corr);
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[r][i] = mul2(acc[r][i], c2);
#pragma unroll
                    for (int t = 0; t < DC; ++t) sc[r][t] -= cm;
                }
            }
        }
#pragma unroll
        for (int t = 0; t < DC; ++t) {
            {
                u64 v2[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) v2[i] = nxt[i];
                if (t + 1 < DC) lds_slab16<NS>(cb + (t + 1) * RB, 1, slab, nxt);
#pragma unroll
                for (int r = 0; r < NQ; ++r)
                    if (CA_ON(r)) {
                        const float pt = fast_exp2(sc[r][t]);
                        l[r] += pt;
                        const u64 p2 = pack2(pt, pt);
#pragma unroll
                        for (int i = 0; i < 8; ++i) acc[r][i] = fma2(p2, v2[i], acc[r][i]);
                    }
            }
        }
    }
}

// The ws keys of one window column.  EXACT: ws is a multiple of DC.  Otherwise (DC == 4): chunks of four keys, then
// the remaining one to three keys as one chunk of exactly that length, so that no chunk carries bounds checks
// (a checked chunk keeps its prefetched vector alive across branches, which costs a register copy per loaded
// word and made windows such as 13 slower than 15).
template <int DC, bool DIST, bool EXACT, int NQ, int NS>
__device__ __forceinline__ void fwd_window(uint32_t rowbase, int ws, int rm, float sl2, const u64 (&q)[NQ][8],
                                           u64 (&acc)[NQ][8], u64 (&nm2)[NQ], float (&l)[NQ], const float (&bq)[NQ],
                                           int slab) {
    constexpr int FULLM = (1 << NQ) - 1;
    if (EXACT) {
        fwd_stage<DC, DIST, FULLM, NQ, NS>(rowbase, ws, rm, sl2, q, acc, nm2, l, bq, slab);
        return;
    }
    static_assert(EXACT || DC == 4, "windows without a dividing chunk length run chunks of four plus a tail");
    const int main = ws & ~3;
    fwd_stage<4, DIST, FULLM, NQ, NS>(rowbase, main, rm, sl2, q, acc, nm2, l, bq, slab);
    const uint32_t tail = rowbase + main * (kRowBytes * NS);
    switch (ws - main) {                                     // warp-uniform
        case 1: fwd_stage<1, DIST, FULLM, NQ, NS>(tail, 1, rm, sl2, q, acc, nm2, l, bq, slab); break;
        case 2: fwd_stage<2, DIST, FULLM, NQ, NS>(tail, 2, rm, sl2, q, acc, nm2, l, bq, slab); break;
        case 3: fwd_stage<3, DIST, FULLM, NQ, NS>(tail, 3, rm, sl2, q, acc, nm2, l, bq, slab); break;
        default: break;
    }
}

// First score of each centre pixel that starts in this stage: the reference
// point of its running maximum.
template <bool DIST, int NQ, int NS = 1>
__device__ __forceinline__ void fwd_init_max(uint32_t rowbase, int init, float sl2, const u64 (&q)[NQ][8],
                                             u64 (&nm2)[NQ], const float (&bq)[NQ], int slab = 0) {
    u64 k2[8];
    lds_slab16<NS>(rowbase, 0, slab, k2);
    float bk = 0.f;
    if (DIST) {
        u64 n = zero2();
#pragma unroll
        for (int i = 0; i < 8; ++i) n = fma2(k2[i], k2[i], n);
        bk = -0.5f * sl2 * hsum2(n);
    }
#pragma unroll
    for (int r = 0; r < NQ; ++r)
        if ((init >> r) & 1) {
            u64 sa = zero2();
#pragma unroll
            for (int i = 0; i < 8; ++i) sa = fma2(q[r][i], k2[i], sa);
            const float s0 = lane_sum<NS>(hsum2(sa) + (DIST ? bq[r] + bk : 0.f));     // init is warp-uniform
            nm2[r] = pack2((NS == 1 || slab == 0) ? -s0 - kHeadroom : 0.f, 0.f);
        }
}

#define CA_MASK_SWITCH(FULL, mask, CALL)                            \
    if ((mask) == (FULL)) { constexpr int MK = (FULL); CALL; }      \
    else { constexpr int MK = 0; CALL; }

// NCRT = real channels per unit the kernel is compiled for: 16 (also runs 8-channel units, zero-extended),
// 32 or 64 (NS = 2 or 4 lanes per pixel, one 16-channel slab each; launched without a stage split).
template <int DC, bool DIST, int CPE, bool EXACT, int NQ, int NCRT = 16>
__global__ void __launch_bounds__(128, (NQ <= 2 ? 3 : 2)) fwd_tiled_kernel(TileArgs a, const __grid_constant__ CUtensorMap mv,
                                                           const __grid_constant__ CUtensorMap msc) {
    constexpr int NS = NCRT <= 16 ? 1 : NCRT / 16;
    constexpr int RB = kRowBytes * NS;
    const Geo& g = a.g;
    const int ROWS = a.TH + 2 * (g.p + a.roff);
    const int NSTAGES = g.wsw + NQ - 1;
    const int w0 = blockIdx.x * NQ, h0 = blockIdx.y * a.TH, u = blockIdx.z;
    const float sl2 = a.scale * kLog2e;
    CA_PIPE_PROLOGUE(false)
    const int slab = NS == 1 ? 0 : (lt % NS);
    const int lr = NS == 1 ? lt : (lt >> 5) * (32 / NS) + (lt & 31) / NS, h = h0 + lr;
    const bool active = h < g.H;

    u64 q[NQ][8], acc[NQ][8];
    load_centre<CPE, NQ, NCRT>(a.c0, g, u, h, w0, active, sl2, q, 16 * slab);
    u64 nm2[NQ];
    float l[NQ], bq[NQ];
#pragma unroll
    for (int r = 0; r < NQ; ++r) {
        nm2[r] = pack2(INFINITY, 0.f);           // (-m, 0); running maximum -inf: no key seen yet
        l[r] = 0.f;
        bq[r] = 0.f;
        if (DIST) {
            u64 n = zero2();
#pragma unroll
            for (int i = 0; i < 8; ++i) n = fma2(q[r][i], q[r][i], n);
            bq[r] = -0.5f * hsum2(n) / sl2;      // q is pre-scaled by sl2
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[r][i] = zero2();
    }

    CA_PIPE_LOOP({
        const int mask = stage_mask<NQ>(s, radius_w(g));
        const uint32_t rowbase = smem_u32(pipe.vec(buf)) + (lr + a.roff) * RB;
        // pixels whose first stage (of this part) is s
        const int init = (s == s_begin) ? mask : (mask & ~stage_mask<NQ>(s - 1, radius_w(g)));
        if (init) fwd_init_max<DIST, NQ, NS>(rowbase, init, sl2, q, nm2, bq, slab);
        if (mask != (1 << NQ) - 1) {
            // a stage that pairs with only some of the columns: the all-slots code (interleaved chains) with the
            // unpaired slots' scores forced to -inf, so that they contribute exact zeros; measured 6-7 % faster
            // over a forward than computing the paired slots one after the other
            u64 nmE[NQ];
#pragma unroll
            for (int r = 0; r < NQ; ++r) nmE[r] = ((mask >> r) & 1) ? nm2[r] : pack2(-INFINITY, 0.f);
            fwd_window<DC, DIST, EXACT, NQ, NS>(rowbase, g.ws, mask, sl2, q, acc, nmE, l, bq, slab);
#pragma unroll
            for (int r = 0; r < NQ; ++r)
                if ((mask >> r) & 1) nm2[r] = nmE[r];
        } else {
            fwd_window<DC, DIST, EXACT, NQ, NS>(rowbase, g.ws, mask, sl2, q, acc, nm2, l, bq, slab);
        }
    })

    float nm[NQ];
#pragma unroll
    for (int r = 0; r < NQ; ++r) {
        float zero;
        unpack2(nm2[r], nm[r], zero);
    }
    if (a.nsplit == 2) {
        // merge the two partial softmaxes: part 1 publishes (m, l, acc), part 0 combines
        float* xch = reinterpret_cast<float*>(smem_al);
        if (part == 1) {
#pragma unroll
            for (int r = 0; r < NQ; ++r) {
                xch[(r * 18 + 0) * PT + lt] = nm[r];
                xch[(r * 18 + 1) * PT + lt] = l[r];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float x, y;
                    unpack2(acc[r][i], x, y);
                    xch[(r * 18 + 2 + 2 * i) * PT + lt] = x;
                    xch[(r * 18 + 3 + 2 * i) * PT + lt] = y;
                }
            }
        }
        __syncthreads();
        if (part == 1) return;
#pragma unroll
        for (int r = 0; r < NQ; ++r) {
            const float nm1 = xch[(r * 18 + 0) * PT + lt], l1 = xch[(r * 18 + 1) * PT + lt];
            const float nmn = fminf(nm[r], nm1);           // -max(m0, m1)
            const float c0 = (nm[r] == INFINITY) ? 0.f : fast_exp2(nmn - nm[r]);
            const float c1 = (nm1 == INFINITY) ? 0.f : fast_exp2(nmn - nm1);
            l[r] = l[r] * c0 + l1 * c1;
            nm[r] = nmn;
            const u64 c02 = pack2(c0, c0), c12 = pack2(c1, c1);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const u64 o = pack2(xch[(r * 18 + 2 + 2 * i) * PT + lt], xch[(r * 18 + 3 + 2 * i) * PT + lt]);
                acc[r][i] = fma2(o, c12, mul2(acc[r][i], c02));
            }
        }
    }
    if (NS == 1) {
        CA_BF_DISPATCH(
            _Pragma("unroll")
            for (int r = 0; r < NQ; ++r) {
                const float inv = 1.f / l[r] + ca_poison;
                _Pragma("unroll")
                for (int i = 0; i < 8; ++i) {
                    float x, y;
                    unpack2(acc[r][i], x, y);
                    store_centre<CPE, NCRV, BF>(a.o0, g, u, h, w0, active, r, i, x * inv, y * inv);
                }
            })
    } else {
#pragma unroll
        for (int r = 0; r < NQ; ++r) {
            const float inv = 1.f / l[r] + ca_poison;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float x, y;
                unpack2(acc[r][i], x, y);
                store_centre<CPE, NCRT>(a.o0, g, u, h, w0, active, r, i, x * inv, y * inv, 16 * slab);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < NQ; ++r)
        if (a.ostats && active && slab == 0 && w0 + r < g.W)
            a.ostats[(int64_t)u * g.Np + h + g.H * (w0 + r)] = (log2f(l[r]) - nm[r]) * kLn2 + ca_poison;
}

// =====================================================================
// A in CSR order.  Second sweep over the same packed (k|v) stages: with the
// saved log-sum-exp the normalised entry is P = 2^(q.k - L) directly; without
// row statistics (cs0 == NULL) the kernel writes the scaled scores themselves,
// which is the stand-alone similarity operator.  A thread
// produces, per stage, the ws entries of one (row, window column) run, which
// are contiguous in the row's CSR segment; a warp stages its 32 rows x ws run
// in shared memory and writes it out with consecutive lanes on consecutive
// addresses, so the 4*K*heads bytes per pixel leave the SM in full sectors.
// =====================================================================
// NCRT = real channels per unit: 8 (zero-extended to one slab), 16, 32 or 64.
template <bool DIST, int CPE, int NCRT>
__global__ void __launch_bounds__(128, 3) emit_a_tiled_kernel(TileArgs a, const __grid_constant__ CUtensorMap mv,
                                                              const __grid_constant__ CUtensorMap msc) {
    constexpr int NS = NCRT <= 16 ? 1 : NCRT / 16;             // 16-channel slabs = lanes per pixel
    constexpr int RW = 32 / NS;                                // pixel rows per warp
    const Geo& g = a.g;
    const int RB = a.row_bytes;                                // packed row: pair (144*NS) or single tensor (80*NS)
    const int ROWS = a.TH + 2 * (g.p + a.roff);
    const int pw = radius_w(g);
    const int w0 = blockIdx.x * 4, h0 = blockIdx.y * a.TH, u = blockIdx.z;
    const int NSTAGES = g.wsw + min(3, g.W - 1 - w0);          // no stages for centre columns past the image
    const float sl2 = a.scale * kLog2e;
    CA_PIPE_PROLOGUE(false)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int slab = lane % NS, lrow = lane / NS;              // this lane's channel slab and row inside the warp
    const int lr = (lt >> 5) * RW + lrow, h = h0 + lr;         // row inside the tile, image row
    const bool active = h < g.H;
    // per-warp staging tile [4][RW][CH] after the stage buffers: the entries of CH = min(ws, 32)
    // consecutive window rows at a time, then the run rotations of the warp's rows [4][RW]
    const int CH = min(g.ws, kRunChunk);
    const int CHS = CH | 1;                                    // odd row stride: conflict-free column access
    const int nslots = g.wsw == 1 ? 1 : 4;                     // folded 1-D: a stage pairs with one centre column
    float* tile = reinterpret_cast<float*>(smem_al + (size_t)a.nsplit * a.nstages * a.stage_bytes) +
                  (size_t)warp * (nslots * RW * CHS + 4 * RW + RW * CH);     // tile, rotations, offset table
    int* rots = reinterpret_cast<int*>(tile + nslots * RW * CHS);
    // 2-D windows that fit one piece: the destination offset of every tile element is the same
    // for all stages and centre columns (row*K + sorted position) and comes from a table
    const bool tabled = g.ws <= kRunChunk && g.wsw != 1;
    int* etab = rots + 4 * RW;
    const int hw0 = h0 + (lt >> 5) * RW;                       // first image row of this warp
    for (int i = lane; i < 4 * RW; i += 32)
        rots[i] = run_rot(axis_coord(g, hw0 + i % RW, w0 + i / RW), axis_len(g), g.p, g.ws);
    if (tabled)
        for (int idx = lane; idx < RW * g.ws; idx += 32) {
            const int row = idx / g.ws, e = idx - row * g.ws;
            int posh = e + run_rot(hw0 + row, g.H, g.p, g.ws);
            posh -= (posh >= g.ws) ? g.ws : 0;
            etab[idx] = row * g.K + posh;
        }
    __syncwarp();

    const bool raw = a.cs0 == nullptr;
    u64 q[4][8];
    load_centre<CPE, 4, NCRT>(a.c0, g, u, h, w0, active, sl2, q, 16 * slab);
    u64 nL2[4];
    float bq[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const bool ok = active && (w0 + r < g.W) && slab == 0;   // the row statistic enters the lane sum once
        nL2[r] = pack2((ok && !raw) ? -__ldg(a.cs0 + (int64_t)u * g.Np + h + g.H * (w0 + r)) * kLog2e : 0.f, 0.f);
        bq[r] = 0.f;
        if (DIST) {
            u64 n = zero2();
#pragma unroll
            for (int i = 0; i < 8; ++i) n = fma2(q[r][i], q[r][i], n);
            bq[r] = -0.5f * hsum2(n) / sl2;
        }
    }
    const int64_t warp_row0 = (int64_t)u * g.Np + hw0;
    const int rows_here = min(RW, g.H - hw0);

    CA_PIPE_LOOP({
        const int mask = stage_mask<4>(s, pw);
        const uint32_t rowbase = smem_u32(pipe.vec(buf)) + (lr + a.roff) * RB;
        for (int d0 = 0; d0 < g.ws; d0 += CH) {
            const int len = min(CH, g.ws - d0);                // window rows d0 .. d0 + len - 1
            // FULL: the dot products of all four centre columns run interleaved (the columns that do
            // not pair with this stage are computed too and dropped: cheaper than four serial chains);
            // otherwise only the paired columns are computed (folded 1-D: one column per stage)
            auto sweep = [&](auto full_tag) {
                constexpr bool FULL = decltype(full_tag)::value;
                u64 kn[8];                                 // the next window row's vector, fetched one row ahead
                lds_slab16<NS>(rowbase + d0 * RB, 0, slab, kn);
#pragma unroll 2
                for (int e = 0; e < len; ++e) {
                    u64 k2[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) k2[i] = kn[i];
                    if (e + 1 < len) lds_slab16<NS>(rowbase + (d0 + e + 1) * RB, 0, slab, kn);
                    float bk = 0.f;
                    if (DIST) {
                        u64 n = zero2();
#pragma unroll
                        for (int i = 0; i < 8; ++i) n = fma2(k2[i], k2[i], n);
                        bk = -0.5f * sl2 * hsum2(n);
                    }
                    u64 t[4];
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        t[r] = nL2[r];
                        if (DIST) t[r] = add2(t[r], pack2(bq[r] + bk, 0.f));
                    }
                    if (FULL) {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
#pragma unroll
                            for (int r = 0; r < 4; ++r) t[r] = fma2(q[r][i], k2[i], t[r]);
                    } else {
#pragma unroll
                        for (int r = 0; r < 4; ++r)
                            if ((mask >> r) & 1) {
#pragma unroll
                                for (int i = 0; i < 8; ++i) t[r] = fma2(q[r][i], k2[i], t[r]);
                            }
                    }
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        if (!((mask >> r) & 1)) continue;
                        float sc = hsum2(t[r]);
#pragma unroll
                        for (int m = 1; m < NS; m <<= 1) sc += __shfl_xor_sync(0xffffffffu, sc, m);
                        if (slab == 0) tile[((nslots == 1 ? 0 : r) * RW + lrow) * CHS + e] = raw ? sc * kLn2 : fast_exp2(sc);
                    }
                }
            };
            if (mask == 15 || g.wsw != 1) sweep(std::true_type{});
            else sweep(std::false_type{});
            __syncwarp();
            // write this piece of the runs of the stage: row j, positions posw*ws + (d + rot_j) mod ws
#pragma unroll 1
            for (int r = 0; r < 4; ++r) {
                if (!((mask >> r) & 1) || w0 + r >= g.W) continue;
                const int posw = axis_pos(s - pw - r, w0 + r, g.W, pw, g.wsw);
                float* dst = a.o0 + ((warp_row0 + (int64_t)g.H * (w0 + r)) * g.K + posw * g.ws);
                const float* src = tile + (nslots == 1 ? 0 : r) * RW * CHS;
                const int n = rows_here * len;
                if (tabled) {                                      // CHS == len == ws: tile index == idx
#pragma unroll 4
                    for (int idx = lane; idx < n; idx += 32) dst[etab[idx]] = src[idx];
                    continue;
                }
                int row = lane / len, e = lane - row * len;        // element idx = row*len + e
                const int drow = 32 / len, de = 32 - drow * len;
                for (int idx = lane; idx < n; idx += 32) {
                    int posh = d0 + e + rots[r * RW + row];
                    posh -= (posh >= g.ws) ? g.ws : 0;
                    dst[(int64_t)row * g.K + posh] = src[row * CHS + e];
                    row += drow;
                    e += de;
                    if (e >= len) { e -= len; ++row; }
                }
            }
            __syncwarp();
        }
    })
}

// =====================================================================
// A (x) V and A^T (x) V from stored values.  The dense operand is streamed as
// packed column stages exactly like the keys of the forward; the values of A
// that pair with a stage are, for every centre column r, one run of ws
// consecutive entries per CSR row (window column fixed, window rows varying),
// which a warp copies into shared memory before the stage's FMAs:
//   plain     : rows = the warp's own 32 pixels, run at posw(s - p - r; w0 + r);
//   transposed: rows = the 32 + 2p pixels of the streamed column around the warp
//               (by window symmetry A[j, i] sits in row j at offset i - j), run at
//               posw(r + p - s; streamed column).
// out = alpha * (sum_e a_e v_e - (sum_e a_e) * centre) with centre optional: the
// second term is the Distance similarity pullback.
// =====================================================================
// Four-byte asynchronous copy global -> shared (the runs of A are only 4-byte aligned).
__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int CPE, bool TRANS, int NCRT>
__global__ void __launch_bounds__(128, 3) apply_tiled_kernel(TileArgs a, const __grid_constant__ CUtensorMap mv,
                                                             const __grid_constant__ CUtensorMap msc) {
    constexpr int NS = NCRT <= 16 ? 1 : NCRT / 16;             // 16-channel slabs = lanes per pixel
    constexpr int RW = 32 / NS;                                // pixel rows per warp
    const Geo& g = a.g;
    const int RB = a.row_bytes;                                // packed row: pair (144*NS) or single tensor (80*NS)
    const int ROWS = a.TH + 2 * (g.p + a.roff);
    const int pw = radius_w(g);
    const bool fold = g.wsw == 1;                              // folded 1-D signal: rows continue into neighbour columns
    const int w0 = blockIdx.x * 4, h0 = blockIdx.y * a.TH, u = blockIdx.z;
    const int NSTAGES = g.wsw + min(3, g.W - 1 - w0);          // no stages for centre columns past the image
    CA_PIPE_PROLOGUE(false)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int slab = lane % NS, lrow = lane / NS;              // this lane's channel slab and row inside the warp
    const int lr = (lt >> 5) * RW + lrow, h = h0 + lr;         // row inside the tile, image row
    const bool active = h < g.H;
    // Values of A are staged for CH = min(ws, 32) window rows at a time, per centre column r in
    // slot r (one shared slot when folded: a stage then pairs with a single column), as
    // [tile row][CHS] with tile row = warp row (plain) or warp row + row inside the chunk
    // (transposed: the CSR row of the streamed pixel).  Two buffers per warp: the next piece is
    // copied while the current one is used.
    const int CH = min(g.ws, kRunChunk), CHS = CH | 1;
    const int TRW = RW + (TRANS ? CH - 1 : 0);
    const int nslots = fold ? 1 : 4;
    const int buf_floats = nslots * TRW * CHS;
    const int nch = (g.ws + CH - 1) / CH;                      // pieces per stage
    // 2-D windows that fit one piece: source and tile offsets of every staged element are the same
    // for all stages and centre columns up to the column base; they come from two tables
    const bool tabled = nch == 1 && !fold;
    float* wbase = reinterpret_cast<float*>(smem_al + (size_t)a.nstages * a.stage_bytes) +
                   (size_t)warp * (2 * buf_floats + (tabled ? 2 * RW * CH : 0));
    const int hw0 = h0 + (lt >> 5) * RW;                       // first image row of this warp
    const float* nzu = a.cs0 + (int64_t)u * g.Np * g.K;
    const int rows_here = hw0 >= g.H ? 0 : min(RW, g.H - hw0);
    const int X = axis_len(g);
    int* tsrc = reinterpret_cast<int*>(wbase + 2 * buf_floats);
    int* tdst = tsrc + RW * CH;
    if (tabled) {
        for (int idx = lane; idx < RW * g.ws; idx += 32) {
            const int wr = idx / g.ws, e = idx - wr * g.ws;
            if (!TRANS) {
                int posh = e + run_rot(hw0 + wr, g.H, g.p, g.ws);
                posh -= (posh >= g.ws) ? g.ws : 0;
                tsrc[idx] = (hw0 + wr) * g.K + posh;
                tdst[idx] = wr * CHS + e;
            } else {
                const int tr = wr + e;
                int hj = (hw0 + tr - g.p) % g.H;
                hj += (hj < 0) ? g.H : 0;
                tsrc[idx] = hj * g.K + axis_pos(g.p - e, hj, g.H, g.p, g.ws);
                tdst[idx] = tr * CHS + e;
            }
        }
        __syncwarp();
    }

    // starts the copies for piece c of stage s into buffer tb
    auto fetch_piece = [&](int s, int c, int tb) {
        const int mask = stage_mask<4>(s, pw);
        const int wc = stage_column(g, w0, s);
        const int d0 = c * CH, len = min(CH, g.ws - d0);
        float* tbuf = wbase + tb * buf_floats;
        if (hw0 >= g.H) { cp_async_commit(); return; }                 // warp past the image: nothing to stage
        const int row0 = lane / len, e0 = lane - row0 * len;           // first element of this lane
        const int drow = 32 / len, de = 32 - drow * len;               // step of 32 elements
#pragma unroll 1
        for (int r = 0; r < 4; ++r) {
            if (!((mask >> r) & 1) || w0 + r >= g.W) continue;
            float* dst = tbuf + (fold ? 0 : r) * TRW * CHS;
            if (tabled) {
                const int posw = TRANS ? axis_pos(r + pw - s, wc, g.W, pw, g.wsw)
                                       : axis_pos(s - pw - r, w0 + r, g.W, pw, g.wsw);
                const float* src = nzu + (int64_t)g.H * (TRANS ? wc : w0 + r) * g.K + posw * g.ws;
                const int n = (TRANS ? RW : rows_here) * g.ws;
#pragma unroll 4
                for (int idx = lane; idx < n; idx += 32) cp_async4(dst + tdst[idx], src + tsrc[idx]);
            } else if (!TRANS) {
                const int posw = axis_pos(s - pw - r, w0 + r, g.W, pw, g.wsw);
                const float* src = nzu + ((int64_t)g.H * (w0 + r) + hw0) * g.K + posw * g.ws;
                const int n = rows_here * len;
                int row = row0, e = e0;                                    // element idx = row*len + e
                for (int idx = lane; idx < n; idx += 32) {
                    int posh = d0 + e + run_rot(axis_coord(g, hw0 + row, w0 + r), X, g.p, g.ws);
                    posh -= (posh >= g.ws) ? g.ws : 0;
                    cp_async4(dst + row * CHS + e, src + (int64_t)row * g.K + posh);
                    row += drow;
                    e += de;
                    if (e >= len) { e -= len; ++row; }
                }
            } else {
                // entry (tile row tr, e) belongs to warp row tr - e: the CSR row of the streamed pixel
                // (column wc, image row hw0 + d0 + tr - p), at the position of offset p - (d0 + e)
                const int posw = axis_pos(r + pw - s, wc, g.W, pw, g.wsw);
                const int n = RW * len;
                int wr = row0, e = e0;                                     // warp row, row inside the chunk
                for (int idx = lane; idx < n; idx += 32) {
                    const int tr = wr + e;
                    int hj = hw0 + d0 + tr - g.p;
                    int64_t rowidx;                                         // CSR row inside the unit
                    int x;
                    if (fold) {
                        x = (g.H * wc + hj) % X;
                        x += (x < 0) ? X : 0;
                        rowidx = x;
                    } else {
                        hj += (hj < 0) ? g.H : 0;                          // here ws > 32, so H > 32 > the tile's
                        hj -= (hj >= g.H) ? g.H : 0;                       // overhang: two subtractions suffice
                        hj -= (hj >= g.H) ? g.H : 0;
                        x = hj;
                        rowidx = hj + (int64_t)g.H * wc;
                    }
                    const int posh = axis_pos(g.p - d0 - e, x, X, g.p, g.ws);
                    cp_async4(dst + tr * CHS + e, nzu + rowidx * g.K + posw * g.ws + posh);
                    wr += drow;
                    e += de;
                    if (e >= len) { e -= len; ++wr; }
                }
            }
        }
        cp_async_commit();
    };

    u64 acc[4][8];
    float asum[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        asum[r] = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[r][i] = zero2();
    }
    fetch_piece(s_begin, 0, 0);
    int piece = 0;                                             // pieces consumed so far (buffer = piece & 1)

    CA_PIPE_LOOP({
        const int mask = stage_mask<4>(s, pw);
        const uint32_t rowbase = smem_u32(pipe.vec(buf)) + (lr + a.roff) * RB;
        for (int c = 0; c < nch; ++c, ++piece) {
            const int d0 = c * CH, len = min(CH, g.ws - d0);
            if (c + 1 < nch) {
                fetch_piece(s, c + 1, (piece + 1) & 1);
                cp_async_wait<1>();
            } else if (s + 1 < s_end) {
                fetch_piece(s + 1, 0, (piece + 1) & 1);
                cp_async_wait<1>();
            } else {
                cp_async_wait<0>();
            }
            __syncwarp();
            const float* tile = wbase + (piece & 1) * buf_floats;
            // operands of window row d0 + e: the streamed vector and the four values of A, fetched
            // one row ahead of the FMAs that use them
            auto fetch_row = [&](int e, u64 (&vv)[8], float (&aa)[4]) {
                lds_slab16<NS>(rowbase + (d0 + e) * RB, a.which, slab, vv);
                const float* ap = tile + (lrow + (TRANS ? e : 0)) * CHS + e;
#pragma unroll
                for (int r = 0; r < 4; ++r) aa[r] = ((mask >> r) & 1) ? ap[(fold ? 0 : r) * TRW * CHS] : 0.f;
            };
            u64 vn[8];
            float an[4];
            fetch_row(0, vn, an);
#pragma unroll 2
            for (int e = 0; e < len; ++e) {
                u64 v2[8];
                float av[4];
#pragma unroll
                for (int i = 0; i < 8; ++i) v2[i] = vn[i];
#pragma unroll
                for (int r = 0; r < 4; ++r) av[r] = an[r];
                if (e + 1 < len) fetch_row(e + 1, vn, an);
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    if ((mask >> r) & 1) {
                        asum[r] += av[r];
                        const u64 a2 = pack2(av[r], av[r]);
#pragma unroll
                        for (int i = 0; i < 8; ++i) acc[r][i] = fma2(a2, v2[i], acc[r][i]);
                    }
                }
            }
            __syncwarp();
        }
    })

    if (a.c0) {
        u64 ctr[4][8];
        load_centre<CPE, 4, NCRT>(a.c0, g, u, h, w0, active, 1.f, ctr, 16 * slab);
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const u64 ns = pack2(-asum[r], -asum[r]);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[r][i] = fma2(ns, ctr[r][i], acc[r][i]);
        }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float x, y;
            unpack2(acc[r][i], x, y);
            store_centre<CPE, NCRT>(a.o0, g, u, h, w0, active, r, i, a.scale * x + ca_poison, a.scale * y + ca_poison, 16 * slab);
        }
}

// =====================================================================
// Backward, query-owned: dq.  The s chain starts at -L (log2 domain) and the
// dP chain at -D, so P = 2^chain and dS = P * chain'.
// =====================================================================
// MODE 0: softmax, P = 2^chain.  MODE 1: 1.5-entmax, g = max(chain, 0) with the chain = s/2 - tau, dS = g*(dP - D).
// MODE 2: the entmax pre-pass: only num += g*dP and den += g (in aux and sumds), D = num/den.
// The same query-owned sweep serves the entmax forward, which has no dy: MODE 3 the row maximum of s/2 (in aux);
// MODE 4 one step of the threshold search: with t = chain = s/2 - tau, the sum of max(t, 0) (sumds), of its
// square (aux), the size of the support {t > 0}, its smallest member and the largest t outside (ex[0..2]);
// MODE 5 the apply: dq (here y) += max(chain, 0)^2 * v.
template <bool DIST, int MASK, int NQ, int MODE, int NS = 1>
__device__ __forceinline__ void dq_stage(uint32_t rowbase, int ws, int rm, float sl2, const u64 (&q)[NQ][8],
                                         const u64 (&dy)[NQ][8], u64 (&dq)[NQ][8], const u64 (&nL2)[NQ],
                                         const u64 (&nD2)[NQ], const float (&bq)[NQ], float (&sumds)[NQ],
                                         float (&aux)[NQ], float (&ex)[NQ][3], int slab = 0) {
#pragma unroll 2      // two keys in flight: the second key's loads overlap the first key's FMAs
    for (int di = 0; di < ws; ++di) {
        const uint32_t a0 = rowbase + di * (kRowBytes * NS);
        float dp[NQ];
        if (MODE <= 2) {
            u64 v2[8];
            lds_slab16<NS>(a0, 1, slab, v2);
#pragma unroll
            for (int r = 0; r < NQ; ++r)
                if (CA_ON(r)) {
                    u64 t = nD2[r];                               // (-D, 0)
#pragma unroll
                    for (int i = 0; i < 8; ++i) t = fma2(dy[r][i], v2[i], t);
                    dp[r] = lane_sum<NS>(hsum2(t));              // -D sits on slab 0 only; rm is warp-uniform
                }
        }
        u64 k2[8];
        lds_slab16<NS>(a0, 0, slab, k2);
        float bk = 0.f;
        if (DIST) {
            u64 n = zero2();
#pragma unroll
            for (int i = 0; i < 8; ++i) n = fma2(k2[i], k2[i], n);
            bk = -0.5f * sl2 * hsum2(n);
        }
#pragma unroll
        for (int r = 0; r < NQ; ++r)
            if (CA_ON(r)) {
                u64 t = nL2[r];                                   // (-L, 0), log2 domain
                if (DIST) t = add2(t, pack2(bq[r] + bk, 0.f));
#pragma unroll
                for (int i = 0; i < 8; ++i) t = fma2(q[r][i], k2[i], t);
                const float chain = lane_sum<NS>(hsum2(t));
                if (MODE == 3) {
                    aux[r] = fmaxf(aux[r], chain);
                } else if (MODE == 4) {
                    const bool in = chain > 0.f;
                    const float tp = fmaxf(chain, 0.f);
                    sumds[r] += tp;
                    aux[r] = fmaf(tp, tp, aux[r]);
                    ex[r][0] += in ? 1.f : 0.f;
                    ex[r][1] = fminf(ex[r][1], in ? chain : INFINITY);
                    ex[r][2] = fmaxf(ex[r][2], in ? -INFINITY : chain);
                } else if (MODE == 5) {
                    u64 v2[8];
                    lds_slab16<NS>(a0, 1, slab, v2);
                    const float tp = fmaxf(chain, 0.f);
                    const float w = tp * tp;
                    const u64 w2 = pack2(w, w);
#pragma unroll
                    for (int i = 0; i < 8; ++i) dq[r][i] = fma2(w2, v2[i], dq[r][i]);
                } else if (MODE == 2) {
                    const float gg = fmaxf(chain, 0.f);
                    aux[r] = fmaf(gg, dp[r], aux[r]);
                    sumds[r] += gg;
                } else {
                    const float ds = (MODE == 0 ? fast_exp2(chain) : fmaxf(chain, 0.f)) * dp[r];
                    if (DIST) sumds[r] += ds;
                    const u64 d2 = pack2(ds, ds);
#pragma unroll
                    for (int i = 0; i < 8; ++i) dq[r][i] = fma2(d2, k2[i], dq[r][i]);
                }
            }
    }
}

template <bool DIST, int CPE, int NQ, int MODE, int NCRT = 16>
__global__ void __launch_bounds__(128, (NQ <= 2 ? 3 : 2)) dq_tiled_kernel(TileArgs a, const __grid_constant__ CUtensorMap mv,
                                                          const __grid_constant__ CUtensorMap msc) {
    constexpr int NS = NCRT <= 16 ? 1 : NCRT / 16;
    const Geo& g = a.g;
    const int ROWS = a.TH + 2 * (g.p + a.roff);
    const int NSTAGES = g.wsw + NQ - 1;
    const int w0 = blockIdx.x * NQ, h0 = blockIdx.y * a.TH, u = blockIdx.z;
    const float sl2 = MODE ? 0.5f * a.scale : a.scale * kLog2e;     // entmax: the chain is s/2 - tau
    bool settled[NQ];                                               // MODE 4: rows whose threshold is final
    if (MODE == 4) {
        // a block whose rows all have their final threshold leaves before any barrier or copy exists
        // (launched without a stage split and for one-slab units: thread = row)
        const int hh = h0 + (int)threadIdx.x;
        bool mine = true;
#pragma unroll
        for (int r = 0; r < NQ; ++r) {
            settled[r] = true;
            if (hh < g.H && w0 + r < g.W) settled[r] = __ldg(a.cs1 + (int64_t)u * g.Np + hh + g.H * (w0 + r)) != 0.f;
            mine = mine && settled[r];
        }
        if (__syncthreads_and(mine)) return;
    }
    CA_PIPE_PROLOGUE(false)
    const int slab = NS == 1 ? 0 : (lt % NS);
    const int lr = NS == 1 ? lt : (lt >> 5) * (32 / NS) + (lt & 31) / NS, h = h0 + lr;
    const bool active = h < g.H;

    u64 q[NQ][8], dy[NQ][8], dq[NQ][8];
    load_centre<CPE, NQ, NCRT>(a.c0, g, u, h, w0, active, sl2, q, 16 * slab);
    if (MODE <= 2) {
        load_centre<CPE, NQ, NCRT>(a.c1, g, u, h, w0, active, 1.f, dy, 16 * slab);
    } else {
#pragma unroll
        for (int r = 0; r < NQ; ++r)
#pragma unroll
            for (int i = 0; i < 8; ++i) dy[r][i] = zero2();
    }
    u64 nL2[NQ], nD2[NQ];
    float bq[NQ], sumds[NQ], aux[NQ], ex[NQ][3];
#pragma unroll
    for (int r = 0; r < NQ; ++r) {
        const bool ok = active && (w0 + r < g.W) && slab == 0;       // row scalars enter the lane sums once
        const int64_t o = (int64_t)u * g.Np + h + g.H * (w0 + r);
        nL2[r] = pack2((ok && MODE != 3) ? -__ldg(a.cs0 + o) * (MODE ? 1.f : kLog2e) : 0.f, 0.f);
        nD2[r] = pack2((ok && MODE <= 1) ? -__ldg(a.cs1 + o) : 0.f, 0.f);
        sumds[r] = 0.f;
        aux[r] = MODE == 3 ? -INFINITY : 0.f;
        ex[r][0] = 0.f;
        ex[r][1] = INFINITY;
        ex[r][2] = -INFINITY;
        bq[r] = 0.f;
        if (DIST) {
            u64 n = zero2();
#pragma unroll
            for (int i = 0; i < 8; ++i) n = fma2(q[r][i], q[r][i], n);
            bq[r] = -0.5f * hsum2(n) / sl2;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) dq[r][i] = zero2();
    }

    CA_PIPE_LOOP({
        const int mask = stage_mask<NQ>(s, radius_w(g));
        CA_MASK_SWITCH(((1 << NQ) - 1), mask, (dq_stage<DIST, MK, NQ, MODE, NS>(smem_u32(pipe.vec(buf)) + (lr + a.roff) * (kRowBytes * NS), g.ws, mask,
                                                     sl2, q, dy, dq, nL2, nD2, bq, sumds, aux, ex, slab)));
    })

    if (MODE == 3) {
        // first threshold of the search: tau >= max - 1 always
#pragma unroll
        for (int r = 0; r < NQ; ++r)
            if (active && slab == 0 && w0 + r < g.W)
                a.ostats[(int64_t)u * g.Np + h + g.H * (w0 + r)] = aux[r] - 1.f + ca_poison;
        return;
    }
    if (MODE == 4) {
        // the quadratic sum_S (t - d)^2 = 1 solved on the support S of the current tau; final when tau + d has
        // the same support and the step was short against the distances it was computed from
#pragma unroll
        for (int r = 0; r < NQ; ++r)
            if (active && slab == 0 && w0 + r < g.W && !settled[r]) {
                const int64_t o = (int64_t)u * g.Np + h + g.H * (w0 + r);
                const float n = ex[r][0], sa = sumds[r], sb = aux[r];
                float d = 0.f;
                bool same = true;
                if (n > 0.f) {
                    const float disc = fmaxf(fmaf(sa, sa, -n * (sb - 1.f)), 0.f);
                    d = (sa - sqrtf(disc)) / n;
                    same = (d >= 0.f ? d < ex[r][1] : d >= ex[r][2]) && d * n <= 0.5f * sa;
                    if (!same && a.iter >= 10) d = 0.5f * (sb - 1.f) / sa;     // late steps: Newton on the convex sum
                }
                float ntau, zero;
                unpack2(nL2[r], ntau, zero);
                a.ostats[o] = d - ntau + ca_poison;
                a.o1[o] = same ? 1.f : 0.f;
            }
        return;
    }
    if (MODE == 2) {
        // pre-pass of the entmax pullback: D = sum g*dP / sum g per query row (launched without a stage split)
#pragma unroll
        for (int r = 0; r < NQ; ++r)
            if (active && slab == 0 && w0 + r < g.W)
                a.ostats[(int64_t)u * g.Np + h + g.H * (w0 + r)] = (sumds[r] > 0.f ? aux[r] / sumds[r] : 0.f) + ca_poison;
        return;
    }
    if (a.nsplit == 2) {
        float* xch = reinterpret_cast<float*>(smem_al);
        if (part == 1) {
#pragma unroll
            for (int r = 0; r < NQ; ++r) {
                xch[(r * 17 + 16) * PT + lt] = sumds[r];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float x, y;
                    unpack2(dq[r][i], x, y);
                    xch[(r * 17 + 2 * i) * PT + lt] = x;
                    xch[(r * 17 + 2 * i + 1) * PT + lt] = y;
                }
            }
        }
        __syncthreads();
        if (part == 1) return;
#pragma unroll
        for (int r = 0; r < NQ; ++r) {
            sumds[r] += xch[(r * 17 + 16) * PT + lt];
#pragma unroll
            for (int i = 0; i < 8; ++i)
                dq[r][i] = add2(dq[r][i], pack2(xch[(r * 17 + 2 * i) * PT + lt], xch[(r * 17 + 2 * i + 1) * PT + lt]));
        }
    }
    // dq = scale * (sum ds*k - [distance] sum(ds) * q);  q registers hold q*scale*log2(e) (entmax: q*scale/2)
    const float qfac = MODE ? 2.f : kLn2;
    if (NS == 1) {
        CA_BF_DISPATCH(
            _Pragma("unroll")
            for (int r = 0; r < NQ; ++r) {
                _Pragma("unroll")
                for (int i = 0; i < 8; ++i) {
                    float x, y, qx, qy;
                    unpack2(dq[r][i], x, y);
                    unpack2(q[r][i], qx, qy);
                    if (MODE == 5) {
                        x += ca_poison;
                        y += ca_poison;
                    } else {
                        x = a.scale * x - (DIST ? sumds[r] * qx * qfac : 0.f) + ca_poison;
                        y = a.scale * y - (DIST ? sumds[r] * qy * qfac : 0.f) + ca_poison;
                    }
                    store_centre<CPE, NCRV, BF>(a.o0, g, u, h, w0, active, r, i, x, y);
                }
            })
    } else {
#pragma unroll
        for (int r = 0; r < NQ; ++r) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float x, y, qx, qy;
                unpack2(dq[r][i], x, y);
                unpack2(q[r][i], qx, qy);
                x = a.scale * x - (DIST ? sumds[r] * qx * qfac : 0.f) + ca_poison;
                y = a.scale * y - (DIST ? sumds[r] * qy * qfac : 0.f) + ca_poison;
                store_centre<CPE, NCRT>(a.o0, g, u, h, w0, active, r, i, x, y, 16 * slab);
            }
        }
    }
}

// =====================================================================
// Backward, key-owned: dk and dv of three key pixels per thread.  The stage
// rows carry (q | dy) of the query pixels plus their L and D.
// =====================================================================
template <bool DIST, int MASK, int NQ, bool ENT, int NS = 1>
__device__ __forceinline__ void dkdv_stage(uint32_t base, const float* Lb, const float* Db, int row0, int ws, int rm,
                                           float sl2, const u64 (&k)[NQ][8], const u64 (&v)[NQ][8], u64 (&dk)[NQ][8],
                                           u64 (&dv)[NQ][8], const float (&bk)[NQ], float (&sumds)[NQ], int slab = 0) {
#pragma unroll 1
    for (int di = 0; di < ws; ++di) {
        const int row = row0 + di;
        const uint32_t a0 = base + row * (kRowBytes * NS);
        // the row scalars enter the lane sums once: on slab 0
        const float nLj = (NS == 1 || slab == 0) ? -Lb[row] : 0.f, nDj = (NS == 1 || slab == 0) ? -Db[row] : 0.f;
        u64 y2[8];
        lds_slab16<NS>(a0, 1, slab, y2);
        float dp[NQ];
#pragma unroll
        for (int r = 0; r < NQ; ++r)
            if (CA_ON(r)) {
                u64 t = pack2(nDj, 0.f);
#pragma unroll
                for (int i = 0; i < 8; ++i) t = fma2(v[r][i], y2[i], t);
                dp[r] = lane_sum<NS>(hsum2(t));
            }
        u64 q2[8];
        lds_slab16<NS>(a0, 0, slab, q2);
        float bqj = 0.f;
        if (DIST) {
            u64 n = zero2();
#pragma unroll
            for (int i = 0; i < 8; ++i) n = fma2(q2[i], q2[i], n);
            bqj = -0.5f * sl2 * hsum2(n);
        }
#pragma unroll
        for (int r = 0; r < NQ; ++r)
            if (CA_ON(r)) {
                u64 t = pack2(DIST ? nLj + bk[r] + bqj : nLj, 0.f);
#pragma unroll
                for (int i = 0; i < 8; ++i) t = fma2(k[r][i], q2[i], t);
                const float chain = lane_sum<NS>(hsum2(t));
                float P, ds;
                if (!ENT) {
                    P = fast_exp2(chain);
                    ds = P * dp[r];
                } else {                                     // g = max(s/2 - tau, 0): P = g^2, dS = g*(dP - D)
                    const float gg = fmaxf(chain, 0.f);
                    P = gg * gg;
                    ds = gg * dp[r];
                }
                if (DIST) sumds[r] += ds;
                const u64 d2 = pack2(ds, ds), p2 = pack2(P, P);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    dk[r][i] = fma2(d2, q2[i], dk[r][i]);
                    dv[r][i] = fma2(p2, y2[i], dv[r][i]);
                }
            }
    }
}

template <bool DIST, int CPE, int NQ, bool ENT, int NCRT = 16>
__global__ void __launch_bounds__(128, (NQ <= 2 ? 3 : 2)) dkdv_tiled_kernel(TileArgs a, const __grid_constant__ CUtensorMap mv,
                                                            const __grid_constant__ CUtensorMap msc) {
    constexpr int NS = NCRT <= 16 ? 1 : NCRT / 16;
    const Geo& g = a.g;
    const int ROWS = a.TH + 2 * (g.p + a.roff);
    const int NSTAGES = g.wsw + NQ - 1;
    const int w0 = blockIdx.x * NQ, h0 = blockIdx.y * a.TH, u = blockIdx.z;
    const float sl2 = ENT ? 0.5f * a.scale : a.scale * kLog2e;      // entmax: the chain is s/2 - tau
    CA_PIPE_PROLOGUE(true)
    const int slab = NS == 1 ? 0 : (lt % NS);
    const int lr = NS == 1 ? lt : (lt >> 5) * (32 / NS) + (lt & 31) / NS, h = h0 + lr;
    const bool active = h < g.H;

    u64 k[NQ][8], v[NQ][8], dk[NQ][8], dv[NQ][8];
    load_centre<CPE, NQ, NCRT>(a.c0, g, u, h, w0, active, sl2, k, 16 * slab);
    load_centre<CPE, NQ, NCRT>(a.c1, g, u, h, w0, active, 1.f, v, 16 * slab);
    float bk[NQ], sumds[NQ];
#pragma unroll
    for (int r = 0; r < NQ; ++r) {
        sumds[r] = 0.f;
        bk[r] = 0.f;
        if (DIST) {
            u64 n = zero2();
#pragma unroll
            for (int i = 0; i < 8; ++i) n = fma2(k[r][i], k[r][i], n);
            bk[r] = -0.5f * hsum2(n) / sl2;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            dk[r][i] = zero2();
            dv[r][i] = zero2();
        }
    }

    CA_PIPE_LOOP({
        const int mask = stage_mask<NQ>(s, radius_w(g));
        CA_MASK_SWITCH(((1 << NQ) - 1), mask, (dkdv_stage<DIST, MK, NQ, ENT, NS>(smem_u32(pipe.vec(buf)), pipe.sc0(buf), pipe.sc1(buf),
                                                      lr + a.roff, g.ws, mask, sl2, k, v, dk, dv, bk, sumds, slab)));
    })

    if (a.nsplit == 2) {
        float* xch = reinterpret_cast<float*>(smem_al);
        if (part == 1) {
#pragma unroll
            for (int r = 0; r < NQ; ++r) {
                xch[(r * 33 + 32) * PT + lt] = sumds[r];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float x, y;
                    unpack2(dk[r][i], x, y);
                    xch[(r * 33 + 2 * i) * PT + lt] = x;
                    xch[(r * 33 + 2 * i + 1) * PT + lt] = y;
                    unpack2(dv[r][i], x, y);
                    xch[(r * 33 + 16 + 2 * i) * PT + lt] = x;
                    xch[(r * 33 + 17 + 2 * i) * PT + lt] = y;
                }
            }
        }
        __syncthreads();
        if (part == 1) return;
#pragma unroll
        for (int r = 0; r < NQ; ++r) {
            sumds[r] += xch[(r * 33 + 32) * PT + lt];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                dk[r][i] = add2(dk[r][i], pack2(xch[(r * 33 + 2 * i) * PT + lt], xch[(r * 33 + 2 * i + 1) * PT + lt]));
                dv[r][i] = add2(dv[r][i], pack2(xch[(r * 33 + 16 + 2 * i) * PT + lt], xch[(r * 33 + 17 + 2 * i) * PT + lt]));
            }
        }
    }
    // dk = scale * (sum ds*q - [distance] sum(ds) * k);  k registers hold k*scale*log2(e)
    if (NS == 1) {
        CA_BF_DISPATCH(
            _Pragma("unroll")
            for (int r = 0; r < NQ; ++r) {
                _Pragma("unroll")
                for (int i = 0; i < 8; ++i) {
                    float x, y, kx, ky, vx, vy;
                    unpack2(dk[r][i], x, y);
                    unpack2(k[r][i], kx, ky);
                    unpack2(dv[r][i], vx, vy);
                    x = a.scale * x - (DIST ? sumds[r] * kx * (ENT ? 2.f : kLn2) : 0.f) + ca_poison;
                    y = a.scale * y - (DIST ? sumds[r] * ky * (ENT ? 2.f : kLn2) : 0.f) + ca_poison;
                    store_centre<CPE, NCRV, BF>(a.o0, g, u, h, w0, active, r, i, x, y);
                    store_centre<CPE, NCRV, BF>(a.o1, g, u, h, w0, active, r, i, vx + ca_poison, vy + ca_poison);
                }
            })
    } else {
#pragma unroll
        for (int r = 0; r < NQ; ++r) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float x, y, kx, ky, vx, vy;
                unpack2(dk[r][i], x, y);
                unpack2(k[r][i], kx, ky);
                unpack2(dv[r][i], vx, vy);
                x = a.scale * x - (DIST ? sumds[r] * kx * (ENT ? 2.f : kLn2) : 0.f) + ca_poison;
                y = a.scale * y - (DIST ? sumds[r] * ky * (ENT ? 2.f : kLn2) : 0.f) + ca_poison;
                store_centre<CPE, NCRT>(a.o0, g, u, h, w0, active, r, i, x, y, 16 * slab);
                store_centre<CPE, NCRT>(a.o1, g, u, h, w0, active, r, i, vx + ca_poison, vy + ca_poison, 16 * slab);
            }
        }
    }
}

// =====================================================================
// Pack kernel: two tensors in the reference layout -> [unit][column][row'][32]
// with the circular halo along h unrolled, plus (optionally) the two scalar
// planes [2*unit + {0: stats*log2(e), 1: D}][column][row'].
// One thread per (row', column, unit, tensor) plus one per (row', column, unit) for the planes.
// =====================================================================
struct PackArgs {
    Geo g;
    int pp;                 // p' (even)
    int Hp;                 // padded rows per column: roundup4(H + 2p')
    int npairs;             // 1 or 2 tensor pairs
    int single;             // 1: rows hold one tensor (src[0]) in 20 words per slab instead of a pair in 36
    const float* src[4];    // pair j = (src[2j], src[2j+1])
    float* dst[2];
    float* planes;          // nullable
    const float* stats;     // with planes
    float stat_mul;         // plane 0 = stats * stat_mul: log2(e) for the softmax log-sum-exp, 1 for the entmax tau
    const float* Din;       // with planes: D given ...
    const float* y;         // ... or computed as dy . y
    const float* dy;
    float* Dout;            // nullable: D in the reference layout (interior rows)
};

template <int CPE, int NCRT, bool BF>
__device__ __forceinline__ void pack_body(const PackArgs& a) {
    constexpr int NS = NCRT <= 16 ? 1 : NCRT / 16;
    constexpr int NCR = NCRT;
    const Geo& g = a.g;
    const int rr = blockIdx.x * blockDim.x + threadIdx.x;
    const int w = blockIdx.y;
    // z slot: one per tensor copy and unit, plus one slot for the scalar planes
    const int nt = a.single ? 1 : 2;                      // tensors per packed row
    const int slots = nt * a.npairs + (a.planes ? 1 : 0);
    const int u = blockIdx.z / slots, slot = blockIdx.z % slots;
    if (rr >= a.Hp) return;
    const bool real_row = rr < g.H + 2 * a.pp;
    // source pixel of packed row rr: the halo rows wrap inside the column (2-D) or continue into the
    // neighbouring columns of a folded 1-D signal
    int pix = 0;
    if (real_row) {
        if (g.wsw == 1) {
            pix = (g.H * w + rr - a.pp) % g.Npk;
            if (pix < 0) pix += g.Npk;
        } else {
            pix = (rr - a.pp + g.H) % g.H + g.H * w;
        }
    }
    const int64_t orow = ((int64_t)u * g.Wk + w) * a.Hp + rr;
    if (slot < nt * a.npairs) {
        const int pair = slot / nt, t = slot % nt;
        const float* src = a.src[2 * pair + t];
        const int row_floats = (a.single ? kSingleFloats : kRowFloats) * NS;
        float4* dp = reinterpret_cast<float4*>(a.dst[pair] + orow * row_floats) + 4 * NS * t;
        // chunk-major: the NS slabs of a 4-channel chunk are adjacent, so each pass writes 16*NS
        // contiguous bytes
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            float4 vals[NS];
#pragma unroll
            for (int sl = 0; sl < NS; ++sl) {
                const int cc = 16 * sl + 4 * c;
                if (!real_row || cc >= NCR) {             // padding rows; channels past a narrow unit
                    vals[sl] = make_float4(0.f, 0.f, 0.f, 0.f);
                } else if (CPE == 1) {
                    const int64_t o = goff<1, NCR>(u, cc, g.Npk, pix);
                    vals[sl] = make_float4(ld_real<BF>(src, o), ld_real<BF>(src, o + g.Npk),
                                           ld_real<BF>(src, o + 2 * (int64_t)g.Npk),
                                           ld_real<BF>(src, o + 3 * (int64_t)g.Npk));
                } else {
                    const float2 lo = __ldg(reinterpret_cast<const float2*>(src + goff<2, NCR>(u, cc, g.Npk, pix)));
                    const float2 hi = __ldg(reinterpret_cast<const float2*>(src + goff<2, NCR>(u, cc + 2, g.Npk, pix)));
                    vals[sl] = make_float4(lo.x, lo.y, hi.x, hi.y);
                }
            }
#pragma unroll
            for (int sl = 0; sl < NS; ++sl) dp[c * NS + sl] = vals[sl];
        }
        if (t == nt - 1) {
#pragma unroll
            for (int sl = 0; sl < NS; ++sl) dp[4 * NS + sl] = make_float4(0.f, 0.f, 0.f, 0.f);    // padding
        }
        return;
    }
    float L = 0.f, D = 0.f;
    if (real_row) {
        const int64_t so = (int64_t)u * g.Npk + pix;
        L = __ldg(a.stats + so) * a.stat_mul;
        if (a.Din) {
            D = __ldg(a.Din + so);
        } else {
            constexpr int NC = NCR;                             // D = dy . y over all real channels of the unit
            float dyv[NC], yv[NC];
#pragma unroll
            for (int cc = 0; cc < NC; ++cc) {
                const int64_t o = goff<CPE, NCR>(u, cc, g.Npk, pix);
                dyv[cc] = ld_real<BF>(a.dy, o);
                yv[cc] = ld_real<BF>(a.y, o);
            }
#pragma unroll
            for (int cc = 0; cc < NC; ++cc) D = fmaf(dyv[cc], yv[cc], D);
            if (a.Dout && rr >= a.pp && rr < a.pp + g.H) a.Dout[so] = D;
        }
    }
    const int64_t plane = (int64_t)g.Wk * a.Hp;
    a.planes[(2 * (int64_t)u) * plane + (int64_t)w * a.Hp + rr] = L;
    a.planes[(2 * (int64_t)u + 1) * plane + (int64_t)w * a.Hp + rr] = D;
}

template <int CPE, int NCRT>
__global__ void __launch_bounds__(128) pack_kernel(PackArgs a) {
    if (CPE == 1 && a.g.bf16) pack_body<CPE, NCRT, true>(a);
    else pack_body<CPE, NCRT, false>(a);
}

// Pair packing for one-slab units (8 or 16 real channels) through shared memory: a block gathers 128
// packed rows of one (column, unit, pair) -- every thread the 2 x NCR channel values of its row, 32
// independent coalesced loads -- into a [128][36] tile, and the block writes the tile out as one contiguous
// run of 16-byte stores (consecutive lanes on consecutive addresses: full sectors), where the direct form
// above writes 64-byte pieces 144 bytes apart.  z slots: one per pair and unit, plus one for the planes.
template <int CPE, int NCRT, bool BF>
__device__ __forceinline__ void pack_rows_body(const PackArgs& a, float (*tile)[kRowFloats]) {
    const Geo& g = a.g;
    const int rr0 = blockIdx.x * 128, rr = rr0 + threadIdx.x;
    const int w = blockIdx.y;
    const int slots = a.npairs + (a.planes ? 1 : 0);
    const int u = blockIdx.z / slots, slot = blockIdx.z % slots;
    const bool in_rows = rr < a.Hp;
    const bool real_row = in_rows && rr < g.H + 2 * a.pp;
    int pix = 0;
    if (real_row) {
        if (g.wsw == 1) {
            pix = (g.H * w + rr - a.pp) % g.Npk;
            if (pix < 0) pix += g.Npk;
        } else {
            pix = (rr - a.pp + g.H) % g.H + g.H * w;
        }
    }
    if (slot < a.npairs) {
        float4 vals[8];
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            const float* src = a.src[2 * slot + t];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int cc = 4 * c;
                if (!real_row || cc >= NCRT) {
                    vals[4 * t + c] = make_float4(0.f, 0.f, 0.f, 0.f);
                } else if (CPE == 1) {
                    const int64_t o = goff<1, NCRT>(u, cc, g.Npk, pix);
                    vals[4 * t + c] = make_float4(ld_real<BF>(src, o), ld_real<BF>(src, o + g.Npk),
                                                  ld_real<BF>(src, o + 2 * (int64_t)g.Npk),
                                                  ld_real<BF>(src, o + 3 * (int64_t)g.Npk));
                } else {
                    const float2 lo = __ldg(reinterpret_cast<const float2*>(src + goff<2, NCRT>(u, cc, g.Npk, pix)));
                    const float2 hi = __ldg(reinterpret_cast<const float2*>(src + goff<2, NCRT>(u, cc + 2, g.Npk, pix)));
                    vals[4 * t + c] = make_float4(lo.x, lo.y, hi.x, hi.y);
                }
            }
        }
        float4* trow = reinterpret_cast<float4*>(tile[threadIdx.x]);
#pragma unroll
        for (int i = 0; i < 8; ++i) trow[i] = vals[i];
        trow[8] = make_float4(0.f, 0.f, 0.f, 0.f);                       // padding words
        __syncthreads();
        const int nrows = min(128, a.Hp - rr0);
        float4* out = reinterpret_cast<float4*>(a.dst[slot] + (((int64_t)u * g.Wk + w) * a.Hp + rr0) * kRowFloats);
        const float4* tin = reinterpret_cast<const float4*>(&tile[0][0]);
        for (int i = threadIdx.x; i < nrows * (kRowFloats / 4); i += 128) out[i] = tin[i];
        return;
    }
    if (!in_rows) return;
    float L = 0.f, D = 0.f;
    if (real_row) {
        const int64_t so = (int64_t)u * g.Npk + pix;
        L = __ldg(a.stats + so) * a.stat_mul;
        if (a.Din) {
            D = __ldg(a.Din + so);
        } else {
            float dyv[NCRT], yv[NCRT];
#pragma unroll
            for (int cc = 0; cc < NCRT; ++cc) {
                const int64_t o = goff<CPE, NCRT>(u, cc, g.Npk, pix);
                dyv[cc] = ld_real<BF>(a.dy, o);
                yv[cc] = ld_real<BF>(a.y, o);
            }
#pragma unroll
            for (int cc = 0; cc < NCRT; ++cc) D = fmaf(dyv[cc], yv[cc], D);
            if (a.Dout && rr >= a.pp && rr < a.pp + g.H) a.Dout[so] = D;
        }
    }
    const int64_t plane = (int64_t)g.Wk * a.Hp;
    a.planes[(2 * (int64_t)u) * plane + (int64_t)w * a.Hp + rr] = L;
    a.planes[(2 * (int64_t)u + 1) * plane + (int64_t)w * a.Hp + rr] = D;
}

template <int CPE, int NCRT>
__global__ void __launch_bounds__(128) pack_rows_kernel(PackArgs a) {
    __shared__ __align__(16) float tile[128][kRowFloats];
    if (CPE == 1 && a.g.bf16) pack_rows_body<CPE, NCRT, true>(a, tile);
    else pack_rows_body<CPE, NCRT, false>(a, tile);
}

// The same for units of NS = 2 or 4 slabs (32 / 64 real channels), Float32 or ComplexF32: a block gathers 128 / NS
// packed rows, thread (row, slab) the two 16-channel slabs of its row and slab (consecutive lanes on consecutive
// rows: coalesced planar loads), into a [128 / NS][36 * NS] tile in the packed order [tensor][4-channel chunk]
// [slab][4], and writes the tile out as one contiguous run.  The direct form writes 16 * NS-byte pieces 144 * NS
// bytes apart.  In the planes slot the NS threads of a row share the dy . y sum through the tile.
template <int CPE, int NCRT>
__global__ void __launch_bounds__(128) pack_rows_wide_kernel(PackArgs a) {
    constexpr int NS = NCRT / 16, RB = 128 / NS, RF = kRowFloats * NS;
    __shared__ __align__(16) float tile[RB][RF];
    const Geo& g = a.g;
    const int rl = threadIdx.x % RB, slab = threadIdx.x / RB;
    const int rr0 = blockIdx.x * RB, rr = rr0 + rl;
    const int w = blockIdx.y;
    const int slots = a.npairs + (a.planes ? 1 : 0);
    const int u = blockIdx.z / slots, slot = blockIdx.z % slots;
    const bool in_rows = rr < a.Hp;
    const bool real_row = in_rows && rr < g.H + 2 * a.pp;
    int pix = 0;
    if (real_row) {
        if (g.wsw == 1) {
            pix = (g.H * w + rr - a.pp) % g.Npk;
            if (pix < 0) pix += g.Npk;
        } else {
            pix = (rr - a.pp + g.H) % g.H + g.H * w;
        }
    }
    if (slot < a.npairs) {
        float4* trow = reinterpret_cast<float4*>(tile[rl]);
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            const float* src = a.src[2 * slot + t];
            float4 vals[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int cc = 16 * slab + 4 * c;
                if (!real_row) {
                    vals[c] = make_float4(0.f, 0.f, 0.f, 0.f);
                } else if (CPE == 1) {
                    const int64_t o = goff<1, NCRT>(u, cc, g.Npk, pix);
                    vals[c] = make_float4(__ldg(src + o), __ldg(src + o + g.Npk), __ldg(src + o + 2 * (int64_t)g.Npk),
                                          __ldg(src + o + 3 * (int64_t)g.Npk));
                } else {
                    const float2 lo = __ldg(reinterpret_cast<const float2*>(src + goff<2, NCRT>(u, cc, g.Npk, pix)));
                    const float2 hi = __ldg(reinterpret_cast<const float2*>(src + goff<2, NCRT>(u, cc + 2, g.Npk, pix)));
                    vals[c] = make_float4(lo.x, lo.y, hi.x, hi.y);
                }
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) trow[t * (4 * NS) + c * NS + slab] = vals[c];
        }
        trow[8 * NS + slab] = make_float4(0.f, 0.f, 0.f, 0.f);                 // padding words
        __syncthreads();
        const int nrows = min(RB, a.Hp - rr0);
        float4* out = reinterpret_cast<float4*>(a.dst[slot] + (((int64_t)u * g.Wk + w) * a.Hp + rr0) * RF);
        const float4* tin = reinterpret_cast<const float4*>(&tile[0][0]);
        for (int i = threadIdx.x; i < nrows * (RF / 4); i += 128) out[i] = tin[i];
        return;
    }
    // scalar planes: L and D = dy . y (or the given D); every thread sums its slab's 16 channels
    float part = 0.f;
    if (real_row && !a.Din) {
        float dyv[16], yv[16];
#pragma unroll
        for (int cc = 0; cc < 16; ++cc) {
            const int64_t o = goff<CPE, NCRT>(u, 16 * slab + cc, g.Npk, pix);
            dyv[cc] = __ldg(a.dy + o);
            yv[cc] = __ldg(a.y + o);
        }
#pragma unroll
        for (int cc = 0; cc < 16; ++cc) part = fmaf(dyv[cc], yv[cc], part);
    }
    tile[rl][slab] = part;
    __syncthreads();
    if (slab != 0 || !in_rows) return;
    float L = 0.f, D = 0.f;
    if (real_row) {
        const int64_t so = (int64_t)u * g.Npk + pix;
        L = __ldg(a.stats + so) * a.stat_mul;
        if (a.Din) {
            D = __ldg(a.Din + so);
        } else {
#pragma unroll
            for (int sl = 0; sl < NS; ++sl) D += tile[rl][sl];
            if (a.Dout && rr >= a.pp && rr < a.pp + g.H) a.Dout[so] = D;
        }
    }
    const int64_t plane = (int64_t)g.Wk * a.Hp;
    a.planes[(2 * (int64_t)u) * plane + (int64_t)w * a.Hp + rr] = L;
    a.planes[(2 * (int64_t)u + 1) * plane + (int64_t)w * a.Hp + rr] = D;
}

// ---------------------------------------------------------------- host side
struct Padded {
    int pp, Hp;
    size_t pair_floats;     // one packed tensor pair
    size_t single_floats;   // one packed single tensor
    size_t plane_floats;    // both scalar planes
};

int slabs_of(const Geo& g) { return g.cr <= 16 ? 1 : g.cr / 16; }

Padded padded_of(const Geo& g) {
    Padded P;
    P.pp = (g.p + 1) & ~1;
    P.Hp = (g.H + 2 * P.pp + 3) & ~3;
    P.pair_floats = (size_t)g.units * g.Wk * P.Hp * kRowFloats * slabs_of(g);
    P.single_floats = (size_t)g.units * g.Wk * P.Hp * kSingleFloats * slabs_of(g);
    P.plane_floats = (size_t)2 * g.units * g.Wk * P.Hp;
    return P;
}

bool tiled_shape_ok(const Geo& g) {
    // 16 real channels per unit, 8 zero-extended to 16 (half of the FMAs are then spent on zeros), or 32 / 64
    // (2 / 4 lanes per pixel; Float32 storage only)
    const bool chan = g.cr == 16 || g.cr == 8 || ((g.cr == 32 || g.cr == 64) && !g.bf16);
    return chan && (g.wsw == g.ws || g.wsw == 1) && g.ws >= 3 && g.H >= 16 && g.ws <= (g.wsw == 1 ? 127 : 63);
}

// The stand-alone operator kernels also take 8 (zero-extended), 32 or 64 real channels per unit
// (2 or 4 lanes per pixel for the wide ones).
bool tiled_operator_ok(const Geo& g) {
    return (g.cr == 8 || g.cr == 16 || g.cr == 32 || g.cr == 64) && (g.wsw == g.ws || g.wsw == 1) && g.ws >= 3 &&
           g.H >= 16 && g.ws <= (g.wsw == 1 ? 127 : 63) && g.Wk == g.W;
}

// The geometry the tiled kernels run on.  2-D problems are taken as they are.  A 1-D signal of
// length N (H = N, W = 1) is folded column-major into an Hf x (N / Hf) image: pixel n = h + Hf*w keeps
// its address, its window is the rows h-p..h+p of its own column, and the halo rows of the packed
// columns continue into the neighbouring columns (the pack kernel fills them by linear index), so
// the 2-D kernels run unchanged with a window that is one column wide.
bool fold_geo(const Geo& in, Geo* out) {
    *out = in;
    if (in.wsw == in.ws) return true;                      // 2-D
    if (in.wsw != 1 || in.Wk != in.W) return false;
    if (in.W != 1) return true;                            // already folded
    for (int hf : {128, 96, 64, 48, 32, 16}) {
        if (in.H % hf == 0 && in.H / hf >= 1) {
            out->H = hf;
            out->W = out->Wk = in.H / hf;
            return true;
        }
    }
    return false;
}

// Launch-shape overrides for tuning sessions.  Compiled out of the shipped library (the build
// never defines CA_TUNING): no launch reads the environment.
#ifdef CA_TUNING
int tune_int(const char* name, int dflt) {
    const char* v = getenv(name);
    return v && *v ? atoi(v) : dflt;
}
#else
inline int tune_int(const char*, int dflt) { return dflt; }
#endif

int launch_pack(const PackArgs& a, cudaStream_t st) {
    dim3 grid((a.Hp + 127) / 128, a.g.Wk, a.g.units * ((a.single ? 1 : 2) * a.npairs + (a.planes ? 1 : 0)));
    const int cr = a.g.cr;
    // beyond the grid limits (very long folded 1-D signals, very many units) the generic kernels run
    if (grid.y > 65535u || grid.z > 65535u) return CA_ERR_UNSUPPORTED;
    if (!a.single && cr <= 16) {
        // one-slab pairs: the shared-memory form (one z slot per pair instead of one per tensor)
        dim3 grid2(grid.x, grid.y, a.g.units * (a.npairs + (a.planes ? 1 : 0)));
        if (a.g.cpe == 1) {
            if (cr == 8) pack_rows_kernel<1, 8><<<grid2, 128, 0, st>>>(a);
            else pack_rows_kernel<1, 16><<<grid2, 128, 0, st>>>(a);
        } else {
            if (cr == 8) pack_rows_kernel<2, 8><<<grid2, 128, 0, st>>>(a);
            else pack_rows_kernel<2, 16><<<grid2, 128, 0, st>>>(a);
        }
        CA_CHECK_LAUNCH("pack kernel");
        return CA_OK;
    }
    if (!a.single && (cr == 32 || cr == 64) && !a.g.bf16) {
        // wide pairs: the shared-memory form with 128 / NS rows per block
        const int rb = 128 / (cr / 16);
        dim3 grid2((a.Hp + rb - 1) / rb, grid.y, a.g.units * (a.npairs + (a.planes ? 1 : 0)));
        if (a.g.cpe == 1) {
            if (cr == 32) pack_rows_wide_kernel<1, 32><<<grid2, 128, 0, st>>>(a);
            else pack_rows_wide_kernel<1, 64><<<grid2, 128, 0, st>>>(a);
        } else {
            if (cr == 32) pack_rows_wide_kernel<2, 32><<<grid2, 128, 0, st>>>(a);
            else pack_rows_wide_kernel<2, 64><<<grid2, 128, 0, st>>>(a);
        }
        CA_CHECK_LAUNCH("pack kernel");
        return CA_OK;
    }
#define CA_PACK(CPEV)                                                        \
    do {                                                                     \
        if (cr == 8) pack_kernel<CPEV, 8><<<grid, 128, 0, st>>>(a);          \
        else if (cr == 16) pack_kernel<CPEV, 16><<<grid, 128, 0, st>>>(a);   \
        else if (cr == 32) pack_kernel<CPEV, 32><<<grid, 128, 0, st>>>(a);   \
        else pack_kernel<CPEV, 64><<<grid, 128, 0, st>>>(a);                 \
    } while (0)
    if (a.g.cpe == 1) CA_PACK(1);
    else CA_PACK(2);
#undef CA_PACK
    CA_CHECK_LAUNCH("pack kernel");
    return CA_OK;
}

struct Launch {
    TileArgs a;
    CUtensorMap mv, msc;
    dim3 grid;
    int threads;
    size_t smem;
};

// SM count of the current device (cached per device ordinal).
int sm_count() {
    static std::atomic<int> cache[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    int n = cache[dev].load(std::memory_order_relaxed);
    if (!n) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cache[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

// Fills the launch geometry and the tensor maps of the packed pair (and of the
// scalar planes when given).  `nq` centre pixels per thread, `xch_floats` per
// thread for the merge of a split tile.  CTAs have at most 128 threads: four
// warps of rows, or two warps of rows times two stage groups on small grids.
int prepare(const Geo& g, const Padded& P, int nq, int xch_floats, const char* env_warps, const float* pair,
            const float* planes, Launch* L, bool allow_split = true, int max_warps = 4, int ns = 1,
            bool single = false, int stages = kStages) {
    const int rw = 32 / ns;                             // pixel rows per warp (ns lanes share a pixel)
    const int rf = (single ? kSingleFloats : kRowFloats) * ns, rb = rf * 4;
    int warps = (g.H + rw - 1) / rw;
    if (warps > max_warps) warps = max_warps;
    const long cols = (g.W + nq - 1) / nq;
    const long ctas4 = cols * ((g.H + rw * warps - 1) / (rw * warps)) * g.units;
    int nsplit = (ctas4 * warps < 6L * sm_count()) ? 2 : 1;
    nsplit = tune_int("CIRCATT_SPLIT", nsplit);
    if (!allow_split) nsplit = 1;
    if (nsplit == 2 && warps > 2) warps = 2;
    warps = tune_int(env_warps, warps);
    if (warps * nsplit > 4) warps = 4 / nsplit;
    TileArgs& a = L->a;
    a.g = g;
    a.status = status_word();
    a.wait_tries = kWaitTries;
    a.TH = rw * warps;
    a.roff = P.pp - g.p;
    a.nsplit = nsplit;
    a.row_bytes = rb;
    const int ROWS = a.TH + 2 * P.pp;
    if (ROWS > 256) { set_error("tile of %d rows exceeds the TMA box limit", ROWS); return CA_ERR_UNSUPPORTED; }
    const int sstride = (ROWS * 4 + 127) & ~127;
    const int vbytes = (ROWS * rb + 127) & ~127;
    a.stage_bytes = (vbytes + (planes ? 2 * sstride : 0) + 1023) & ~1023;
    L->grid = dim3((unsigned)cols, (g.H + a.TH - 1) / a.TH, g.units);
    L->threads = 32 * warps * nsplit;
    a.nstages = stages;
    size_t smem = (size_t)nsplit * stages * a.stage_bytes;
    const size_t xch = (size_t)xch_floats * 32 * warps * sizeof(float);
    if (nsplit == 2 && xch > smem) smem = xch;
    L->smem = smem + 1024;
    if (L->smem > 220 * 1024) return CA_ERR_UNSUPPORTED;     // window too large for the stage ring: generic kernels
    const uint64_t dims[4] = {(uint64_t)rf, (uint64_t)P.Hp, (uint64_t)g.Wk, (uint64_t)g.units};
    const uint64_t strides[3] = {(uint64_t)rb, (uint64_t)P.Hp * rb, (uint64_t)P.Hp * rb * g.Wk};
    const uint32_t box[4] = {(uint32_t)rf, (uint32_t)ROWS, 1, 1};
    int rc;
    if ((rc = encode_tensor_map(&L->mv, pair, 4, dims, strides, box, false))) return rc;
    if (planes) {
        const uint64_t sdims[3] = {(uint64_t)P.Hp, (uint64_t)g.Wk, (uint64_t)2 * g.units};
        const uint64_t sstr[2] = {(uint64_t)P.Hp * 4, (uint64_t)P.Hp * 4 * g.Wk};
        const uint32_t sbox[3] = {(uint32_t)ROWS, 1, 1};
        if ((rc = encode_tensor_map(&L->msc, planes, 3, sdims, sstr, sbox, false))) return rc;
    } else {
        L->msc = L->mv;
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

#define CA_LAUNCH_TILED(KERNEL, L, st)                                                \
    do {                                                                              \
        int rc__ = set_smem(KERNEL, (L).smem);                                        \
        if (rc__) return rc__;                                                        \
        KERNEL<<<(L).grid, (L).threads, (L).smem, st>>>((L).a, (L).mv, (L).msc);      \
        count_tiled_launch();                                                         \
    } while (0)

#define CA_DIST_CPE(KERNEL_T, dist, cpe, L, st)                                       \
    do {                                                                              \
        if ((cpe) == 1) {                                                             \
            if (dist) CA_LAUNCH_TILED((KERNEL_T<true, 1>), L, st);                    \
            else CA_LAUNCH_TILED((KERNEL_T<false, 1>), L, st);                        \
        } else {                                                                      \
            if (dist) CA_LAUNCH_TILED((KERNEL_T<true, 2>), L, st);                    \
            else CA_LAUNCH_TILED((KERNEL_T<false, 2>), L, st);                        \
        }                                                                             \
    } while (0)

#define CA_DIST_CPE_NQ(KERNEL_T, dist, cpe, NQV, XV, NCRV_, L, st)                    \
    do {                                                                              \
        if ((cpe) == 1) {                                                             \
            if (dist) CA_LAUNCH_TILED((KERNEL_T<true, 1, NQV, XV, NCRV_>), L, st);    \
            else CA_LAUNCH_TILED((KERNEL_T<false, 1, NQV, XV, NCRV_>), L, st);        \
        } else {                                                                      \
            if (dist) CA_LAUNCH_TILED((KERNEL_T<true, 2, NQV, XV, NCRV_>), L, st);    \
            else CA_LAUNCH_TILED((KERNEL_T<false, 2, NQV, XV, NCRV_>), L, st);        \
        }                                                                             \
    } while (0)

// Centre pixels per thread.  Large problems use the widest tile the registers allow (least
// shared-memory traffic per FMA); problems too small to fill the GPU use narrower tiles, which
// means more, shorter-lived warps.
int pick_nq(const Geo& g, int wide, int narrow, const char* env) {
    const long tasks = ((long)(g.W + wide - 1) / wide) * ((g.H + 31) / 32) * g.units;     // warps at the wide tile
    const int nq = tasks < 12L * sm_count() ? narrow : wide;
    return tune_int(env, nq);
}

// mode 0: softmax; 1: entmax; 2: entmax pre-pass (writes D, needs no D and no dq).  The entmax
// variants exist for four centre pixels per thread and run without a stage split.
int run_dq(const Geo& g, const Padded& P, float scale, int dist, const float* q, const float* dy, const float* stats,
           const float* D, const float* kv, float* dq, cudaStream_t st, int mode = 0, float* Dout = nullptr) {
    Launch L{};
    const int ns = slabs_of(g);
    if (ns > 1 && mode) return CA_ERR_UNSUPPORTED;             // the entmax variants exist for one-slab units
    if (mode >= 3) return CA_ERR_UNSUPPORTED;                  // the forward's sweeps go through run_entmax_fwd_sweep
    // two query columns per thread measured faster than four at every size for the softmax dq sweep of one-slab
    // units (160 registers, three blocks per SM, against 255 and two)
    const int nq = mode ? 4 : (ns > 1 ? (g.ws <= 9 ? 2 : 4) : tune_int("CIRCATT_DQ_NQ", 2));
    int rc = prepare(g, P, nq, 17 * nq, "CIRCATT_DQ_WARPS", kv, nullptr, &L, mode == 0 && ns == 1, 4, ns);
    if (rc) return rc;
    L.a.scale = scale; L.a.c0 = q; L.a.c1 = dy; L.a.cs0 = stats; L.a.cs1 = D; L.a.o0 = dq; L.a.ostats = Dout;
    if (ns == 2 && nq == 2) CA_DIST_CPE_NQ(dq_tiled_kernel, dist, g.cpe, 2, 0, 32, L, st);
    else if (ns == 2) CA_DIST_CPE_NQ(dq_tiled_kernel, dist, g.cpe, 4, 0, 32, L, st);
    else if (ns == 4 && nq == 2) CA_DIST_CPE_NQ(dq_tiled_kernel, dist, g.cpe, 2, 0, 64, L, st);
    else if (ns == 4) CA_DIST_CPE_NQ(dq_tiled_kernel, dist, g.cpe, 4, 0, 64, L, st);
    else if (mode == 2) CA_DIST_CPE_NQ(dq_tiled_kernel, dist, g.cpe, 4, 2, 16, L, st);
    else if (mode == 1) CA_DIST_CPE_NQ(dq_tiled_kernel, dist, g.cpe, 4, 1, 16, L, st);
    else if (nq == 2) CA_DIST_CPE_NQ(dq_tiled_kernel, dist, g.cpe, 2, 0, 16, L, st);
    else CA_DIST_CPE_NQ(dq_tiled_kernel, dist, g.cpe, 4, 0, 16, L, st);
    CA_CHECK_LAUNCH("tiled dq kernel");
    return CA_OK;
}

// One sweep of the entmax forward over the packed (k|v): mode 3 row maximum -> first threshold (tau),
// 4 one step of the threshold search (tau and `settled` updated in place), 5 y = sum max(s/2 - tau, 0)^2 v.
int run_entmax_fwd_sweep(const Geo& g, const Padded& P, float scale, int dist, const float* q, const float* kv,
                         float* tau, float* settled, float* y, int mode, int iter, cudaStream_t st) {
    Launch L{};
    if (slabs_of(g) > 1) return CA_ERR_UNSUPPORTED;
    int rc = prepare(g, P, 4, 17 * 4, "CIRCATT_DQ_WARPS", kv, nullptr, &L, false, 4, 1);
    if (rc) return rc;
    L.a.scale = scale; L.a.c0 = q; L.a.cs0 = tau; L.a.cs1 = settled; L.a.o0 = y; L.a.o1 = settled; L.a.ostats = tau;
    L.a.iter = iter;
    if (mode == 3) CA_DIST_CPE_NQ(dq_tiled_kernel, dist, g.cpe, 4, 3, 16, L, st);
    else if (mode == 4) CA_DIST_CPE_NQ(dq_tiled_kernel, dist, g.cpe, 4, 4, 16, L, st);
    else CA_DIST_CPE_NQ(dq_tiled_kernel, dist, g.cpe, 4, 5, 16, L, st);
    CA_CHECK_LAUNCH("tiled entmax forward sweep");
    return CA_OK;
}

int run_dkdv(const Geo& g, const Padded& P, float scale, int dist, const float* k, const float* v, const float* qdy,
             const float* planes, float* dk, float* dv, cudaStream_t st, bool entmax = false) {
    Launch L{};
    const int ns = slabs_of(g);
    if (ns > 1 && entmax) return CA_ERR_UNSUPPORTED;
    const int nq = 3;
    int rc = prepare(g, P, nq, 33 * nq, "CIRCATT_DKDV_WARPS", qdy, planes, &L, ns == 1, 4, ns);
    if (rc) return rc;
    L.a.scale = scale; L.a.c0 = k; L.a.c1 = v; L.a.o0 = dk; L.a.o1 = dv;
    if (ns == 2) CA_DIST_CPE_NQ(dkdv_tiled_kernel, dist, g.cpe, 3, false, 32, L, st);
    else if (ns == 4) CA_DIST_CPE_NQ(dkdv_tiled_kernel, dist, g.cpe, 3, false, 64, L, st);
    else if (entmax) CA_DIST_CPE_NQ(dkdv_tiled_kernel, dist, g.cpe, 3, true, 16, L, st);
    else CA_DIST_CPE_NQ(dkdv_tiled_kernel, dist, g.cpe, 3, false, 16, L, st);
    CA_CHECK_LAUNCH("tiled dk/dv kernel");
    return CA_OK;
}

}  // namespace

// ---------------------------------------------------------------- tensor maps
int encode_tensor_map(CUtensorMap* map, const float* base, int rank, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box, bool swizzle128) {
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
                    swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
        return CA_ERR_CUDA;
    }
    return CA_OK;
}

// ---------------------------------------------------------------- entry points of this file
size_t tiled_fwd_workspace(const Geo& gin) {
    Geo g;
    if (!fold_geo(gin, &g)) return 0;
    if (!tiled_shape_ok(g)) return 0;
    return (padded_of(g).pair_floats + (size_t)g.Np * g.units) * sizeof(float);
}

size_t tiled_bwd_stage_workspace(const Geo& gin) {
    Geo g;
    if (!fold_geo(gin, &g)) return 0;
    if (!tiled_shape_ok(g)) return 0;
    const Padded P = padded_of(g);
    return (P.pair_floats + P.plane_floats) * sizeof(float);
}

size_t tiled_bwd_workspace(const Geo& gin) {
    Geo g;
    if (!fold_geo(gin, &g)) return 0;
    if (!tiled_shape_ok(g)) return 0;
    const Padded P = padded_of(g);
    return (2 * P.pair_floats + P.plane_floats) * sizeof(float);
}

int tiled_stage_timeouts(int* count) {
    cudaError_t e = cudaMemcpyFromSymbol(count, g_stage_timeouts, sizeof(int));
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyFromSymbol(stage timeouts)");
    return CA_OK;
}

int tiled_emit_a(const Geo& g, float scale, int dist, const float* q, const float* stats, float* nz,
                 void* workspace, cudaStream_t st, bool single = false);

int tiled_attention_fwd(const Geo& gin, float scale, int dist, const float* q, const float* k, const float* v,
                        float* y, float* nz, float* stats, void* workspace, cudaStream_t st) {
    Geo g;
    if (!fold_geo(gin, &g)) return CA_ERR_UNSUPPORTED;
    if (!tiled_shape_ok(g) || (nz && g.Wk != g.W)) return CA_ERR_UNSUPPORTED;
    if (!workspace) { set_error("workspace of ca_attention_fwd_workspace() bytes is NULL"); return CA_ERR_NULL; }
    const Padded P = padded_of(g);
    float* kv = static_cast<float*>(workspace);
    if (nz && !stats) stats = kv + P.pair_floats;         // scratch statistics behind the packed pair
    PackArgs pa{};
    pa.g = g; pa.pp = P.pp; pa.Hp = P.Hp; pa.npairs = 1;
    pa.src[0] = k; pa.src[1] = v; pa.dst[0] = kv;
    int rc = launch_pack(pa, st);
    if (rc) return rc;
    Launch L{};
    const int ns = slabs_of(g);
    // four columns per thread, or two when the grid is small or the window is short (with ws <= 9 most
    // stages of a four-column tile pair with only some of its columns: measured 18 % faster at ws 7)
    const int nq = g.ws <= 9 ? tune_int("CIRCATT_FWD_NQ", 2) : (ns > 1 ? 4 : pick_nq(g, 4, 2, "CIRCATT_FWD_NQ"));
    if ((rc = prepare(g, P, nq, 18 * nq, "CIRCATT_FWD_WARPS", kv, nullptr, &L, ns == 1, 4, ns))) return rc;
    L.a.scale = scale; L.a.c0 = q; L.a.o0 = y; L.a.ostats = stats;
#define CA_FWD2(DCV, EX, NQV, NCRV_)                                                            \
    do {                                                                                 \
        if (g.cpe == 1) {                                                                \
            if (dist) CA_LAUNCH_TILED((fwd_tiled_kernel<DCV, true, 1, EX, NQV, NCRV_>), L, st); \
            else CA_LAUNCH_TILED((fwd_tiled_kernel<DCV, false, 1, EX, NQV, NCRV_>), L, st);     \
        } else {                                                                         \
            if (dist) CA_LAUNCH_TILED((fwd_tiled_kernel<DCV, true, 2, EX, NQV, NCRV_>), L, st); \
            else CA_LAUNCH_TILED((fwd_tiled_kernel<DCV, false, 2, EX, NQV, NCRV_>), L, st);     \
        }                                                                                \
    } while (0)
#define CA_FWD(DCV)                                                                      \
    do {                                                                                 \
        if (nq == 2) CA_FWD2(DCV, true, 2, 16);                                          \
        else CA_FWD2(DCV, true, 4, 16);                                                  \
    } while (0)
    // wide units: chunks of 7 or 5 keys where they divide the window, else chunks of four plus a tail
    if (ns == 2 && nq == 2 && g.ws % 7 == 0) CA_FWD2(7, true, 2, 32);
    else if (ns == 4 && nq == 2 && g.ws % 7 == 0) CA_FWD2(7, true, 2, 64);
    else if (ns == 2 && nq == 4 && g.ws % 7 == 0) CA_FWD2(7, true, 4, 32);       // windows 21, 35, 49, 63
    else if (ns == 4 && nq == 4 && g.ws % 7 == 0) CA_FWD2(7, true, 4, 64);
    else if (ns == 2 && nq == 4 && g.ws % 5 == 0) CA_FWD2(5, true, 4, 32);       // windows 15, 25, 45, 55
    else if (ns == 4 && nq == 4 && g.ws % 5 == 0) CA_FWD2(5, true, 4, 64);
    else if (ns == 2 && nq == 2) CA_FWD2(4, false, 2, 32);
    else if (ns == 2) CA_FWD2(4, false, 4, 32);
    else if (ns == 4 && nq == 2) CA_FWD2(4, false, 2, 64);
    else if (ns == 4) CA_FWD2(4, false, 4, 64);
    else if (g.ws % 7 == 0) CA_FWD(7);
    else if (g.ws % 5 == 0) CA_FWD(5);
    else if (g.ws % 3 == 0) CA_FWD(3);
    else if (nq == 2) CA_FWD2(4, false, 2, 16);
    else CA_FWD2(4, false, 4, 16);
#undef CA_FWD2
#undef CA_FWD
    CA_CHECK_LAUNCH("tiled forward kernel");
    if (nz) return tiled_emit_a(g, scale, dist, q, stats, nz, workspace, st);
    return CA_OK;
}

// A's values in CSR order from q, the packed (k|v) pair left in `workspace` by
// tiled_attention_fwd, and the row statistics.
int tiled_emit_a(const Geo& g, float scale, int dist, const float* q, const float* stats, float* nz,
                 void* workspace, cudaStream_t st, bool single) {
    if (!tiled_operator_ok(g)) return CA_ERR_UNSUPPORTED;
    const Padded P = padded_of(g);
    const int ns = slabs_of(g);
    Launch L{};
    // three copy stages, or two when that lets one more CTA reside on an SM
    const int ch = std::min(g.ws, kRunChunk), nslots = g.wsw == 1 ? 1 : 4;
    int rc = CA_OK;
    auto setup = [&](int stages) {
        L = Launch{};
        rc = prepare(g, P, 4, 0, "CIRCATT_FWD_WARPS", static_cast<const float*>(workspace), nullptr, &L, true, 4, ns,
                     single, stages);
        // per warp: staging tile, run rotations, offset table
        if (!rc) L.smem += (size_t)L.threads / 32 * (32 / ns) * (nslots * (ch + 1) + 4 + ch) * sizeof(float);
        return rc;
    };
    if (setup(kStages)) return rc;
    {
        const size_t per_sm = 227 * 1024, with3 = L.smem + 1024;          // + the driver's per-CTA reservation
        const size_t with2 = with3 - (size_t)L.a.nsplit * L.a.stage_bytes;
        const int want = tune_int("CIRCATT_EMIT_STAGES", 0);
        // the kernel's registers allow three CTAs per SM at most
        if (want == 2 || (want == 0 && std::min<size_t>(3, per_sm / with2) > std::min<size_t>(3, per_sm / with3)))
            if (setup(2)) return rc;
    }
    if (L.smem > 200 * 1024) return CA_ERR_UNSUPPORTED;
#define CA_EMIT(NSV)                                                                  \
    do {                                                                              \
        if (g.cpe == 1) {                                                             \
            if (dist) CA_LAUNCH_TILED((emit_a_tiled_kernel<true, 1, NSV>), L, st);    \
            else CA_LAUNCH_TILED((emit_a_tiled_kernel<false, 1, NSV>), L, st);        \
        } else {                                                                      \
            if (dist) CA_LAUNCH_TILED((emit_a_tiled_kernel<true, 2, NSV>), L, st);    \
            else CA_LAUNCH_TILED((emit_a_tiled_kernel<false, 2, NSV>), L, st);        \
        }                                                                             \
    } while (0)
    L.a.scale = scale; L.a.c0 = q; L.a.cs0 = stats; L.a.o0 = nz;
    if (g.cr == 8) CA_EMIT(8);
    else if (g.cr == 16) CA_EMIT(16);
    else if (g.cr == 32) CA_EMIT(32);
    else CA_EMIT(64);
#undef CA_EMIT
    CA_CHECK_LAUNCH("tiled A kernel");
    return CA_OK;
}

int tiled_attention_bwd_dq(const Geo& gin, float scale, int dist, const float* q, const float* k, const float* v,
                           const float* dy, const float* stats, const float* D, float* dq, void* workspace,
                           cudaStream_t st) {
    Geo g;
    if (!fold_geo(gin, &g)) return CA_ERR_UNSUPPORTED;
    if (!tiled_shape_ok(g)) return CA_ERR_UNSUPPORTED;
    if (!workspace) { set_error("workspace of ca_attention_bwd_stage_workspace() bytes is NULL"); return CA_ERR_NULL; }
    const Padded P = padded_of(g);
    float* kv = static_cast<float*>(workspace);
    PackArgs pa{};
    pa.g = g; pa.pp = P.pp; pa.Hp = P.Hp; pa.npairs = 1;
    pa.src[0] = k; pa.src[1] = v; pa.dst[0] = kv;
    int rc = launch_pack(pa, st);
    if (rc) return rc;
    return run_dq(g, P, scale, dist, q, dy, stats, D, kv, dq, st);
}

int tiled_attention_bwd_dkdv(const Geo& gin, float scale, int dist, const float* q, const float* k, const float* v,
                             const float* dy, const float* stats, const float* D, float* dk, float* dv,
                             void* workspace, cudaStream_t st) {
    Geo g;
    if (!fold_geo(gin, &g)) return CA_ERR_UNSUPPORTED;
    if (!tiled_shape_ok(g)) return CA_ERR_UNSUPPORTED;
    if (!workspace) { set_error("workspace of ca_attention_bwd_stage_workspace() bytes is NULL"); return CA_ERR_NULL; }
    const Padded P = padded_of(g);
    float* qdy = static_cast<float*>(workspace);
    float* planes = qdy + P.pair_floats;
    PackArgs pa{};
    pa.g = g; pa.pp = P.pp; pa.Hp = P.Hp; pa.npairs = 1;
    pa.src[0] = q; pa.src[1] = dy; pa.dst[0] = qdy;
    pa.planes = planes; pa.stats = stats; pa.stat_mul = kLog2e; pa.Din = D;
    int rc = launch_pack(pa, st);
    if (rc) return rc;
    return run_dkdv(g, P, scale, dist, k, v, qdy, planes, dk, dv, st);
}

// Helper stream (one per host thread and device) on which the dk/dv sweep of a small problem runs
// next to the dq sweep: neither fills the GPU alone.  It is forked from and joined
// back to the caller's stream with events, so the caller sees ordinary stream order.  The
// stream and its two events belong to the calling host thread, so callers on different threads
// (and streams) neither share them nor wait for each other.
struct ForkJoin {
    cudaStream_t side = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr;
};
static thread_local ForkJoin g_fork[64];

static ForkJoin* fork_join_for_current_device() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    ForkJoin& f = g_fork[dev];
    if (!f.side) {
        if (cudaStreamCreateWithFlags(&f.side, cudaStreamNonBlocking) != cudaSuccess ||
            cudaEventCreateWithFlags(&f.fork, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&f.join, cudaEventDisableTiming) != cudaSuccess) {
            f.side = nullptr;
            cudaGetLastError();
            return nullptr;
        }
    }
    return &f;
}

// Whole backward in three launches: pack (both pairs, D, planes), dq, dk/dv.
int tiled_attention_bwd(const Geo& gin, float scale, int dist, const float* q, const float* k, const float* v,
                        const float* y, const float* dy, const float* stats, float* D, float* dq, float* dk,
                        float* dv, void* workspace, const void* fwd_workspace, cudaStream_t st) {
    Geo g;
    if (!fold_geo(gin, &g)) return CA_ERR_UNSUPPORTED;
    if (!tiled_shape_ok(g) || g.Wk != g.W) return CA_ERR_UNSUPPORTED;
    if (!workspace) { set_error("workspace is NULL"); return CA_ERR_NULL; }
    const Padded P = padded_of(g);
    float* kv = static_cast<float*>(workspace);
    float* qdy = kv + P.pair_floats;
    float* planes = qdy + P.pair_floats;
    PackArgs pa{};
    pa.g = g; pa.pp = P.pp; pa.Hp = P.Hp;
    if (fwd_workspace) {
        // the forward of the same problem left its packed (k|v) at the start of its workspace: only
        // (q|dy) and the planes are packed here
        kv = const_cast<float*>(static_cast<const float*>(fwd_workspace));
        pa.npairs = 1;
        pa.src[0] = q; pa.src[1] = dy;
        pa.dst[0] = qdy;
    } else {
        pa.npairs = 2;
        pa.src[0] = k; pa.src[1] = v; pa.src[2] = q; pa.src[3] = dy;
        pa.dst[0] = kv; pa.dst[1] = qdy;
    }
    pa.planes = planes; pa.stats = stats; pa.stat_mul = kLog2e; pa.y = y; pa.dy = dy; pa.Dout = D;
    int rc = launch_pack(pa, st);
    if (rc) return rc;
    const bool small = (long)g.Np * g.units < 2048L * sm_count();      // fewer than ~4 CTAs per SM per sweep
    if (small && tune_int("CIRCATT_CONCURRENT", 1)) {
        ForkJoin* f = fork_join_for_current_device();
        if (f && cudaEventRecord(f->fork, st) == cudaSuccess && cudaStreamWaitEvent(f->side, f->fork, 0) == cudaSuccess) {
            rc = run_dkdv(g, P, scale, dist, k, v, qdy, planes, dk, dv, f->side);
            int rc2 = run_dq(g, P, scale, dist, q, dy, stats, D, kv, dq, st);
            cudaError_t e = cudaEventRecord(f->join, f->side);
            if (e == cudaSuccess) e = cudaStreamWaitEvent(st, f->join, 0);
            if (e != cudaSuccess) return cuda_fail(e, "joining the helper stream");
            return rc ? rc : rc2;
        }
        cudaGetLastError();
    }
    if ((rc = run_dq(g, P, scale, dist, q, dy, stats, D, kv, dq, st))) return rc;
    return run_dkdv(g, P, scale, dist, k, v, qdy, planes, dk, dv, st);
}

// Entmax-1.5 backward on the fused kernels.  Unlike the softmax, D = sum g*dP / sum g is not dy.y, so
// a pre-pass over the packed (k|v) computes it first: pack (k|v) -> pre-pass -> pack (q|dy) + planes
// (tau, D) -> dq and dk/dv.  `stats` holds tau.
int tiled_attention_bwd_entmax(const Geo& gin, float scale, int dist, const float* q, const float* k, const float* v,
                               const float* dy, const float* stats, float* D, float* dq, float* dk, float* dv,
                               void* workspace, cudaStream_t st) {
    Geo g;
    if (!fold_geo(gin, &g)) return CA_ERR_UNSUPPORTED;
    if (!tiled_shape_ok(g) || g.Wk != g.W || g.bf16) return CA_ERR_UNSUPPORTED;
    if (!workspace) { set_error("workspace is NULL"); return CA_ERR_NULL; }
    const Padded P = padded_of(g);
    float* kv = static_cast<float*>(workspace);
    float* qdy = kv + P.pair_floats;
    float* planes = qdy + P.pair_floats;
    PackArgs pa{};
    pa.g = g; pa.pp = P.pp; pa.Hp = P.Hp; pa.npairs = 1;
    pa.src[0] = k; pa.src[1] = v; pa.dst[0] = kv;
    int rc = launch_pack(pa, st);
    if (rc) return rc;
    if ((rc = run_dq(g, P, scale, dist, q, dy, stats, nullptr, kv, nullptr, st, 2, D))) return rc;
    PackArgs pb{};
    pb.g = g; pb.pp = P.pp; pb.Hp = P.Hp; pb.npairs = 1;
    pb.src[0] = q; pb.src[1] = dy; pb.dst[0] = qdy;
    pb.planes = planes; pb.stats = stats; pb.stat_mul = 1.f; pb.Din = D;
    if ((rc = launch_pack(pb, st))) return rc;
    if ((rc = run_dq(g, P, scale, dist, q, dy, stats, D, kv, dq, st, 1))) return rc;
    return run_dkdv(g, P, scale, dist, k, v, qdy, planes, dk, dv, st, true);
}

// The 1.5-entmax forward in flash mode without A-sized memory: the packed (k|v) is swept once for the row
// maxima, a fixed number of times for the thresholds (blocks whose rows are all final leave at once) and once
// for y.  `stats` (nullable) receives tau and doubles as the search's state; the `settled` plane and a tau plane
// for callers without `stats` live behind the pair in the workspace (tiled_fwd_entmax_workspace bytes).
size_t tiled_fwd_entmax_workspace(const Geo& gin) {
    Geo g;
    if (!fold_geo(gin, &g)) return 0;
    if (!tiled_shape_ok(g) || g.bf16 || slabs_of(g) > 1) return 0;
    return padded_of(g).pair_floats * sizeof(float) + 2 * (size_t)g.Np * g.units * sizeof(float);
}

int tiled_attention_fwd_entmax(const Geo& gin, float scale, int dist, const float* q, const float* k, const float* v,
                               float* y, float* stats, void* workspace, cudaStream_t st) {
    Geo g;
    if (!fold_geo(gin, &g)) return CA_ERR_UNSUPPORTED;
    if (!tiled_shape_ok(g) || g.Wk != g.W || g.bf16 || slabs_of(g) > 1) return CA_ERR_UNSUPPORTED;
    if (!workspace) return CA_ERR_UNSUPPORTED;
    const Padded P = padded_of(g);
    float* kv = static_cast<float*>(workspace);
    float* settled = kv + P.pair_floats;
    if (!stats) stats = settled + (size_t)g.Np * g.units;       // a caller that does not want tau
    PackArgs pa{};
    pa.g = g; pa.pp = P.pp; pa.Hp = P.Hp; pa.npairs = 1;
    pa.src[0] = k; pa.src[1] = v; pa.dst[0] = kv;
    int rc = launch_pack(pa, st);
    if (rc) return rc;
    cudaError_t e = cudaMemsetAsync(settled, 0, (size_t)g.Np * g.units * sizeof(float), st);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync");
    if ((rc = run_entmax_fwd_sweep(g, P, scale, dist, q, kv, stats, settled, nullptr, 3, 0, st))) return rc;
    // the support iteration ends after 3-5 steps on ordinary rows; the steps past the tenth are Newton steps,
    // which converge for every row
    for (int it = 0; it < kEntmaxFwdSteps; ++it)
        if ((rc = run_entmax_fwd_sweep(g, P, scale, dist, q, kv, stats, settled, nullptr, 4, it, st))) return rc;
    return run_entmax_fwd_sweep(g, P, scale, dist, q, kv, stats, settled, y, 5, 0, st);
}

// ---------------------------------------------------------------- stand-alone operators
size_t tiled_operator_workspace(const Geo& gin) {
    Geo g;
    if (!fold_geo(gin, &g)) return 0;
    if (!tiled_operator_ok(g)) return 0;
    return padded_of(g).single_floats * sizeof(float);
}

// Packs one tensor as single-tensor rows.
static int pack_single(const Geo& g, const Padded& P, const float* src, float* dst, cudaStream_t st) {
    PackArgs pa{};
    pa.g = g; pa.pp = P.pp; pa.Hp = P.Hp; pa.npairs = 1; pa.single = 1;
    pa.src[0] = src; pa.dst[0] = dst;
    return launch_pack(pa, st);
}

// Scaled similarity scores in CSR order: x indexes the row pixel, y the column pixel.
int tiled_similarity(const Geo& gin, float scale, int dist, const float* x, const float* y, float* nz,
                     void* workspace, cudaStream_t st) {
    Geo g;
    if (!fold_geo(gin, &g)) return CA_ERR_UNSUPPORTED;
    if (!workspace || !tiled_operator_workspace(g)) return CA_ERR_UNSUPPORTED;
    int rc = pack_single(g, padded_of(g), y, static_cast<float*>(workspace), st);
    if (rc) return rc;
    return tiled_emit_a(g, scale, dist, x, nullptr, nz, workspace, st, true);
}

static int run_apply(const Geo& g, const Padded& P, const float* nz, const float* packed,
                     const float* centre, float* out, float alpha, int transposed, cudaStream_t st) {
    Launch L{};
    const int ns = slabs_of(g);
    // 2-D, one slab: two warps of rows per CTA (smaller stages, more CTAs per SM); otherwise four
    int rc = prepare(g, P, 4, 0, "CIRCATT_APPLY_WARPS", packed, nullptr, &L, false, (ns == 1 && g.wsw != 1) ? 2 : 4, ns, true);
    if (rc) return rc;
    const int ch = std::min(g.ws, kRunChunk), chs = ch | 1;
    const int trw = 32 / ns + (transposed ? ch - 1 : 0);
    // per warp: two buffers and, for single-piece 2-D windows, the two offset tables
    const bool tabled = g.ws <= kRunChunk && g.wsw != 1;
    L.smem += (size_t)L.threads / 32 * (2 * (g.wsw == 1 ? 1 : 4) * trw * chs + (tabled ? 2 * (32 / ns) * ch : 0)) * sizeof(float);
    if (L.smem > 200 * 1024) {
        set_error("tiled apply: window %d with %d channels per unit needs %zu bytes of shared memory", g.ws, g.cr, L.smem);
        return CA_ERR_UNSUPPORTED;
    }
    L.a.scale = alpha; L.a.which = 0; L.a.c0 = centre; L.a.cs0 = nz; L.a.o0 = out;
#define CA_APPLY(NSV)                                                                     \
    do {                                                                                  \
        if (g.cpe == 1) {                                                                 \
            if (transposed) CA_LAUNCH_TILED((apply_tiled_kernel<1, true, NSV>), L, st);   \
            else CA_LAUNCH_TILED((apply_tiled_kernel<1, false, NSV>), L, st);             \
        } else {                                                                          \
            if (transposed) CA_LAUNCH_TILED((apply_tiled_kernel<2, true, NSV>), L, st);   \
            else CA_LAUNCH_TILED((apply_tiled_kernel<2, false, NSV>), L, st);             \
        }                                                                                 \
    } while (0)
    if (g.cr == 8) CA_APPLY(8);
    else if (g.cr == 16) CA_APPLY(16);
    else if (g.cr == 32) CA_APPLY(32);
    else CA_APPLY(64);
#undef CA_APPLY
    CA_CHECK_LAUNCH("tiled apply kernel");
    return CA_OK;
}

// out = alpha * (A (x) v) or alpha * (A^T (x) v) from the values of A in CSR order.
int tiled_apply(const Geo& gin, const float* nz, const float* v, float* out, float alpha, int transposed,
                void* workspace, cudaStream_t st) {
    Geo g;
    if (!fold_geo(gin, &g)) return CA_ERR_UNSUPPORTED;
    if (!workspace || !tiled_operator_workspace(g)) return CA_ERR_UNSUPPORTED;
    const Padded P = padded_of(g);
    float* packed = static_cast<float*>(workspace);
    int rc = pack_single(g, P, v, packed, st);
    if (rc) return rc;
    return run_apply(g, P, nz, packed, nullptr, out, alpha, transposed, st);
}

// Pullback of the similarity: dx[j] = scale * sum_i dS[j,i] y[i], dy[i] = scale * sum_j dS[j,i] x[j]
// (Distance: minus the sum of the dS involved times the pixel's own vector).
int tiled_similarity_bwd(const Geo& gin, float scale, int dist, const float* x, const float* y, const float* dS,
                         float* dx, float* dy, void* workspace, cudaStream_t st) {
    Geo g;
    if (!fold_geo(gin, &g)) return CA_ERR_UNSUPPORTED;
    if (!workspace || !tiled_operator_workspace(g)) return CA_ERR_UNSUPPORTED;
    const Padded P = padded_of(g);
    float* packed = static_cast<float*>(workspace);
    int rc;
    if (dx) {
        if ((rc = pack_single(g, P, y, packed, st))) return rc;
        if ((rc = run_apply(g, P, dS, packed, dist ? x : nullptr, dx, scale, 0, st))) return rc;
    }
    if (dy) {
        if ((rc = pack_single(g, P, x, packed, st))) return rc;
        if ((rc = run_apply(g, P, dS, packed, dist ? y : nullptr, dy, scale, 1, st))) return rc;
    }
    return CA_OK;
}


// ---------------------------------------------------------------- bounded-wait self test
// One CTA arms a stage barrier with more bytes than the single bulk copy it issues delivers, so the
// barrier never completes; the wait must run out after `tries` polls, the CTA must report through the
// same counter and status word as the tiled kernels and return.  Nothing faults and nothing spins
// without a limit; the copy itself lands (the thread polls its destination, again with a limit).
__device__ __align__(16) float g_probe_src[8] = {1.f, 2.f, 3.f, 4.f, 5.f, 6.f, 7.f, 8.f};

__global__ void __launch_bounds__(32) stage_timeout_probe_kernel(uint32_t tries, int* status, int* out) {
    __shared__ __align__(16) float dst[8];
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        dst[7] = 0.f;
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    __syncthreads();
    bool ok = true;
    if (threadIdx.x == 0) {
        mbar_arrive_expect_tx(&bar, 64);                      // 64 bytes expected ...
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], 32, [%2];"
                     ::"r"(smem_u32(dst)), "l"(g_probe_src), "r"(smem_u32(&bar)) : "memory");   // ... 32 delivered
        ok = mbar_wait(&bar, 0, tries);
        // the copy in flight gets a bounded chance to land before the CTA (and its shared memory) goes away
        for (uint32_t i = 0; i < (1u << 16) && *reinterpret_cast<volatile float*>(&dst[7]) != 8.f; ++i) {}
        if (!ok) {
            atomicAdd(&g_stage_timeouts, 1);
            if (status) atomicOr(status, 1);
        }
        if (out) *out = ok ? 0 : 1;
    }
}

int tiled_probe_stage_timeout(uint32_t tries, int* out, cudaStream_t st) {
    stage_timeout_probe_kernel<<<1, 32, 0, st>>>(tries, status_word(), out);
    CA_CHECK_LAUNCH("stage timeout probe kernel");
    return CA_OK;
}

}  // namespace ca
