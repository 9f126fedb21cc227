// C ABI of the circulant-attention library: argument checks and dispatch.
#include "common.cuh"
#include "rowops.cuh"
#include "window_generic.cuh"
#include "tiled.cuh"
#include "line.cuh"

#include <string.h>
#include <atomic>

namespace ca {

static thread_local char g_err[512] = "";
static thread_local int* g_status_word = nullptr;
int* status_word() { return g_status_word; }
static std::atomic<int64_t> g_launches{0};

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
static std::atomic<int64_t> g_tiled_launches{0};
void count_tiled_launch() { g_tiled_launches.fetch_add(1, std::memory_order_relaxed); }

// FP32 FMA peak probe: 16 independent packed-FMA chains per thread, registers only.
__global__ void __launch_bounds__(256) ffma_probe_kernel(int iters, float* __restrict__ sink) {
    unsigned long long acc[16];
    const float seed = 1.0f + 1e-6f * threadIdx.x;
    unsigned long long a, b;
    asm("mov.b64 %0, {%1, %2};" : "=l"(a) : "f"(seed), "f"(seed * 0.5f));
    asm("mov.b64 %0, {%1, %2};" : "=l"(b) : "f"(1e-7f), "f"(-1e-7f));
#pragma unroll
    for (int i = 0; i < 16; ++i) asm("mov.b64 %0, {%1, %2};" : "=l"(acc[i]) : "f"((float)i), "f"(0.5f * i));
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int i = 0; i < 16; ++i)
            asm volatile("fma.rn.f32x2 %0, %1, %0, %2;" : "+l"(acc[i]) : "l"(a), "l"(b));
    }
    float out = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        float x, y;
        asm("mov.b64 {%0, %1}, %2;" : "=f"(x), "=f"(y) : "l"(acc[i]));
        out += x + y;
    }
    sink[(size_t)blockIdx.x * blockDim.x + threadIdx.x] = out;
}

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
    set_error("%s: %s", what, cudaGetErrorString(e));
    return CA_ERR_CUDA;
}

int make_geo(const ca_desc* d, Geo* g, bool allow_band) {
    if (!d) { set_error("descriptor is NULL"); return CA_ERR_NULL; }
    if (d->ndim != 1 && d->ndim != 2) { set_error("ndim=%d: only 1 or 2 spatial dims are supported", d->ndim); return CA_ERR_BAD_DESC; }
    if (d->ws < 1 || d->ws % 2 != 1) { set_error("filter size M=%d must be odd.", d->ws); return CA_ERR_BAD_DESC; }
    if (d->H < d->ws) { set_error("spatial extent %d is smaller than the window %d", d->H, d->ws); return CA_ERR_BAD_DESC; }
    if (d->ndim == 1 && d->W != 1) { set_error("1-D signals must have W == 1 (got %d)", d->W); return CA_ERR_BAD_DESC; }
    if (d->channels < 1 || d->units < 1) { set_error("channels=%d units=%d must be positive", d->channels, d->units); return CA_ERR_BAD_DESC; }
    if (d->dtype != CA_F32 && d->dtype != CA_C64 && d->dtype != CA_BF16) { set_error("unknown dtype %d", d->dtype); return CA_ERR_BAD_DESC; }
    if (d->similarity != CA_DOT && d->similarity != CA_DISTANCE) { set_error("unknown similarity %d", d->similarity); return CA_ERR_BAD_DESC; }
    if (d->normalizer != CA_SOFTMAX && d->normalizer != CA_ENTMAX15) { set_error("unknown normalizer %d", d->normalizer); return CA_ERR_BAD_DESC; }
    const int p = (d->ws - 1) / 2;
    const bool band = d->Wk != 0 && d->Wk != d->W;
    if (band) {
        if (!allow_band) { set_error("band mode (Wk != W) is not supported by this entry point"); return CA_ERR_UNSUPPORTED; }
        if (d->ndim != 2) { set_error("band mode needs 2 spatial dims"); return CA_ERR_BAD_DESC; }
        if (d->wk_off < p || d->wk_off + d->W + p > d->Wk) {
            set_error("band mode: key-side tensor (Wk=%d, offset %d) does not cover the window of %d query columns", d->Wk, d->wk_off, d->W);
            return CA_ERR_BAD_DESC;
        }
    } else if (d->ndim == 2 && d->W < d->ws) {
        set_error("spatial extent %d is smaller than the window %d", d->W, d->ws);
        return CA_ERR_BAD_DESC;
    }
    g->H = d->H; g->W = d->W;
    g->Wk = band ? d->Wk : d->W;
    g->wk_off = band ? d->wk_off : 0;
    g->ws = d->ws; g->p = p;
    g->wsw = d->ndim == 2 ? d->ws : 1;
    g->K = g->ws * g->wsw;
    const int64_t np = (int64_t)d->H * d->W, npk = (int64_t)d->H * g->Wk;
    if (np > INT32_MAX / 2 || npk > INT32_MAX / 2) { set_error("more than 2^30 pixels per unit"); return CA_ERR_TOO_LARGE; }
    g->Np = (int)np; g->Npk = (int)npk;
    g->units = d->units;
    g->c = d->channels;
    g->cpe = d->dtype == CA_C64 ? 2 : 1;
    g->cr = g->c * g->cpe;
    g->bf16 = d->dtype == CA_BF16;
    if (d->units > 65535) { set_error("units=%d exceeds the grid limit 65535", d->units); return CA_ERR_TOO_LARGE; }
    return CA_OK;
}

// bfloat16 storage exists only in the fused tiled attention kernels.
static int no_bf16(const Geo& g, const char* what) {
    if (!g.bf16) return CA_OK;
    set_error("%s: bfloat16 storage is implemented by the fused attention kernels only "
              "(softmax, 16 channels per unit, a workspace given)", what);
    return CA_ERR_UNSUPPORTED;
}

static int pick_cmax(int cr) {
    for (int c : {4, 8, 16, 32, 64}) if (cr <= c) return c;
    return 0;
}

#define CA_DISPATCH_CMAX(cmax, cpe, CALL)                                           \
    do {                                                                            \
        if (cpe == 1) {                                                             \
            switch (cmax) {                                                         \
                case 4:  { constexpr int CM = 4;  constexpr int CP = 1; CALL; } break; \
                case 8:  { constexpr int CM = 8;  constexpr int CP = 1; CALL; } break; \
                case 16: { constexpr int CM = 16; constexpr int CP = 1; CALL; } break; \
                case 32: { constexpr int CM = 32; constexpr int CP = 1; CALL; } break; \
                default: { constexpr int CM = 64; constexpr int CP = 1; CALL; } break; \
            }                                                                       \
        } else {                                                                    \
            switch (cmax) {                                                         \
                case 4:  { constexpr int CM = 4;  constexpr int CP = 2; CALL; } break; \
                case 8:  { constexpr int CM = 8;  constexpr int CP = 2; CALL; } break; \
                case 16: { constexpr int CM = 16; constexpr int CP = 2; CALL; } break; \
                case 32: { constexpr int CM = 32; constexpr int CP = 2; CALL; } break; \
                default: { constexpr int CM = 64; constexpr int CP = 2; CALL; } break; \
            }                                                                       \
        }                                                                           \
    } while (0)

static int launch_similarity(const Geo& g, float scale, int dist, const float* x, const float* y,
                             float* nz, cudaStream_t st) {
    dim3 grid((g.Np + 127) / 128, g.units);
    if (g.cpe == 1) similarity_generic<1><<<grid, 128, 0, st>>>(g, scale, dist, x, y, nz);
    else similarity_generic<2><<<grid, 128, 0, st>>>(g, scale, dist, x, y, nz);
    CA_CHECK_LAUNCH("similarity kernel");
    return CA_OK;
}

static int launch_apply(const Geo& g, const float* nz, const float* v, const float* center, float* out,
                        float alpha, int transpose, int a_bcast, int v_bcast, cudaStream_t st) {
    ApplyArgs a{g, nz, v, center, out, alpha, transpose, a_bcast, v_bcast};
    if (g.cr > 65535) { set_error("more than 65535 real channels per unit"); return CA_ERR_TOO_LARGE; }
    dim3 grid((g.Np + 127) / 128, g.cr, g.units);
    if (g.cpe == 1) apply_generic<1><<<grid, 128, 0, st>>>(a);
    else apply_generic<2><<<grid, 128, 0, st>>>(a);
    CA_CHECK_LAUNCH("apply kernel");
    return CA_OK;
}

static int launch_row_normalize(int64_t rows, int K, int entmax, const float* s, float* p, float* stats,
                                cudaStream_t st) {
    const int64_t blocks = (rows * 32 + 255) / 256;
    if (blocks > INT32_MAX) { set_error("too many rows"); return CA_ERR_TOO_LARGE; }
    if (entmax) {
        if (K <= 64) row_entmax15_reg_kernel<2><<<(unsigned)blocks, 256, 0, st>>>(rows, K, s, p, stats);
        else if (K <= 128) row_entmax15_reg_kernel<4><<<(unsigned)blocks, 256, 0, st>>>(rows, K, s, p, stats);
        else if (K <= 256) row_entmax15_reg_kernel<8><<<(unsigned)blocks, 256, 0, st>>>(rows, K, s, p, stats);
        else if (K <= 512) row_entmax15_reg_kernel<16><<<(unsigned)blocks, 256, 0, st>>>(rows, K, s, p, stats);
        else row_entmax15_kernel<<<(unsigned)blocks, 256, 0, st>>>(rows, K, s, p, stats);
    }
    else row_softmax_kernel<<<(unsigned)blocks, 256, 0, st>>>(rows, K, s, p, stats);
    CA_CHECK_LAUNCH("row normalize kernel");
    return CA_OK;
}

static int launch_row_normalize_bwd(int64_t rows, int K, int entmax, const float* p, const float* dp, float* ds,
                                    cudaStream_t st) {
    const int64_t blocks = (rows * 32 + 255) / 256;
    if (blocks > INT32_MAX) { set_error("too many rows"); return CA_ERR_TOO_LARGE; }
    row_normalize_bwd_kernel<<<(unsigned)blocks, 256, 0, st>>>(rows, K, entmax, p, dp, ds);
    CA_CHECK_LAUNCH("row normalize pullback kernel");
    return CA_OK;
}

static int check_nnz(const Geo& g) {
    // the reference stores nnz as Int32 (src/circulant.jl:64,86)
    const int64_t nnz = (int64_t)g.Np * g.K;
    if (nnz > INT32_MAX) { set_error("Np*K = %lld entries per unit exceed Int32", (long long)nnz); return CA_ERR_TOO_LARGE; }
    return CA_OK;
}

static int elementwise_grid(int64_t n) {
    int64_t b = (n + 255) / 256;
    const int64_t cap = 148 * 16;
    return (int)(b < cap ? (b < 1 ? 1 : b) : cap);
}

}  // namespace ca

using namespace ca;

extern "C" {

int ca_version(void) { return 100; }

int64_t ca_probe_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int64_t ca_probe_tiled_launch_count(void) { return g_tiled_launches.load(std::memory_order_relaxed); }

int ca_probe_ffma(int32_t blocks, int32_t iters, float* sink, void* stream) {
    if (blocks < 1 || iters < 1) { set_error("blocks and iters must be positive"); return CA_ERR_BAD_DESC; }
    if (!sink) { set_error("sink is NULL"); return CA_ERR_NULL; }
    ffma_probe_kernel<<<blocks, 256, 0, as_stream(stream)>>>(iters, sink);
    CA_CHECK_LAUNCH("FFMA probe kernel");
    return CA_OK;
}

const char* ca_last_error(void) { return g_err; }

int ca_status_word(int32_t* device_word) {
    g_status_word = device_word;
    return CA_OK;
}

int ca_probe_stage_timeout(int32_t max_tries, int32_t* out, void* stream) {
    if (max_tries < 1 || max_tries > (1 << 20)) { set_error("max_tries must be in 1..2^20"); return CA_ERR_BAD_DESC; }
    return tiled_probe_stage_timeout((uint32_t)max_tries, out, as_stream(stream));
}

int ca_structure(int32_t H, int32_t W, int32_t ndim, int32_t ws, int64_t nbatch,
                 int32_t* rowptr, int32_t* colval, void* stream) {
    ca_desc d{};
    d.H = H; d.W = W; d.ndim = ndim; d.ws = ws; d.channels = 1; d.units = 1;
    Geo g;
    int rc = make_geo(&d, &g, false);
    if (rc) return rc;
    if (!rowptr || !colval) { set_error("rowptr/colval is NULL"); return CA_ERR_NULL; }
    if (nbatch < 1) { set_error("nbatch must be positive"); return CA_ERR_BAD_DESC; }
    if ((rc = check_nnz(g))) return rc;
    const int64_t n = (int64_t)g.Np * g.K;   // >= Np+1 because K >= 1... guard the 1x1 window
    const int64_t threads = n > g.Np + 1 ? n : g.Np + 1;
    structure_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, as_stream(stream)>>>(
        g.H, g.W, g.ws, g.wsw, nbatch, rowptr, colval);
    CA_CHECK_LAUNCH("structure kernel");
    return CA_OK;
}

size_t ca_operator_workspace(const ca_desc* d) {
    Geo g;
    if (make_geo(d, &g, false)) return 0;
    return tiled_operator_workspace(g);
}

int ca_similarity(const ca_desc* d, const void* x, const void* y, float* nz, void* workspace, void* stream) {
    Geo g;
    int rc = make_geo(d, &g, false);
    if (rc) return rc;
    if (!x || !y || !nz) { set_error("x/y/nz is NULL"); return CA_ERR_NULL; }
    if ((rc = no_bf16(g, "ca_similarity"))) return rc;
    if ((rc = check_nnz(g))) return rc;
    rc = tiled_similarity(g, d->scale, d->similarity == CA_DISTANCE, (const float*)x, (const float*)y, nz, workspace,
                          as_stream(stream));
    if (rc != CA_ERR_UNSUPPORTED) return rc;
    return launch_similarity(g, d->scale, d->similarity == CA_DISTANCE, (const float*)x, (const float*)y, nz,
                             as_stream(stream));
}

int ca_similarity_bwd(const ca_desc* d, const void* x, const void* y, const float* dS,
                      void* dx, void* dy, void* workspace, void* stream) {
    Geo g;
    int rc = make_geo(d, &g, false);
    if (rc) return rc;
    if (!x || !y || !dS) { set_error("x/y/dS is NULL"); return CA_ERR_NULL; }
    if ((rc = no_bf16(g, "ca_similarity_bwd"))) return rc;
    const bool dist = d->similarity == CA_DISTANCE;
    cudaStream_t st = as_stream(stream);
    rc = tiled_similarity_bwd(g, d->scale, dist, (const float*)x, (const float*)y, dS, (float*)dx, (float*)dy,
                              workspace, st);
    if (rc != CA_ERR_UNSUPPORTED) return rc;
    if (dx && (rc = launch_apply(g, dS, (const float*)y, dist ? (const float*)x : nullptr, (float*)dx,
                                 d->scale, 0, 0, 0, st))) return rc;
    if (dy && (rc = launch_apply(g, dS, (const float*)x, dist ? (const float*)y : nullptr, (float*)dy,
                                 d->scale, 1, 0, 0, st))) return rc;
    return CA_OK;
}

int ca_row_normalize(const ca_desc* d, const float* s, float* p, float* stats, void* stream) {
    Geo g;
    int rc = make_geo(d, &g, false);
    if (rc) return rc;
    if (!s || !p) { set_error("s/p is NULL"); return CA_ERR_NULL; }
    return launch_row_normalize((int64_t)g.Np * g.units, g.K, d->normalizer == CA_ENTMAX15, s, p, stats,
                                as_stream(stream));
}

int ca_row_normalize_bwd(const ca_desc* d, const float* p, const float* dp, float* ds, void* stream) {
    Geo g;
    int rc = make_geo(d, &g, false);
    if (rc) return rc;
    if (!p || !dp || !ds) { set_error("p/dp/ds is NULL"); return CA_ERR_NULL; }
    return launch_row_normalize_bwd((int64_t)g.Np * g.units, g.K, d->normalizer == CA_ENTMAX15, p, dp, ds,
                                    as_stream(stream));
}

int ca_apply(const ca_desc* d, const float* nz, const void* v, void* out,
             int32_t transpose, int32_t a_bcast, int32_t v_bcast, void* workspace, void* stream) {
    Geo g;
    int rc = make_geo(d, &g, false);
    if (rc) return rc;
    if (!nz || !v || !out) { set_error("nz/v/out is NULL"); return CA_ERR_NULL; }
    if ((rc = no_bf16(g, "ca_apply"))) return rc;
    if (!a_bcast && !v_bcast) {
        rc = tiled_apply(g, nz, (const float*)v, (float*)out, 1.f, transpose != 0, workspace, as_stream(stream));
        if (rc != CA_ERR_UNSUPPORTED) return rc;
    }
    return launch_apply(g, nz, (const float*)v, nullptr, (float*)out, 1.f, transpose, a_bcast, v_bcast,
                        as_stream(stream));
}

static size_t score_bytes(const Geo& g) {
    return (((size_t)g.Np * g.K * g.units * sizeof(float)) + 255) & ~(size_t)255;
}

// Attention as a chain of the tiled operators (similarity -> row normaliser -> apply, and the
// reference's own pullback chain of src/rrules.jl backwards) with the scores in scratch memory.
// Used where no fused kernel exists: entmax with A materialised or with wide units, and a cotangent on A.  The scratch is A-sized, so the chain is taken only while A fits Int32 indexing and 4 GiB.
static bool composed_path(const ca_desc* d, const Geo& g, bool backward = false, bool has_dA = false) {
    if (g.bf16 || g.Wk != g.W || !tiled_operator_workspace(g)) return false;
    // 1-D windows are long (the scores of a row do not stay in cache between the operators): the
    // backward of narrow units is faster on the generic kernels, which recompute instead
    if (backward && g.wsw == 1 && g.cr <= 16) return false;
    if ((int64_t)g.Np * g.K > INT32_MAX || score_bytes(g) > ((size_t)4 << 30)) return false;
    return d->normalizer == CA_ENTMAX15 || has_dA;
}

static std::atomic<int64_t> g_entmax_scratch_limit{(int64_t)256 << 20};

int64_t ca_entmax_scratch_limit(int64_t bytes) {
    if (bytes < 0) return g_entmax_scratch_limit.load(std::memory_order_relaxed);
    return g_entmax_scratch_limit.exchange(bytes, std::memory_order_relaxed);
}

// Flash-mode entmax forward on the repeated tiled sweeps instead of the operator chain: when the shape is
// covered and the chain's score buffer would exceed the limit (or cannot be indexed at all).
static bool entmax_fwd_on_sweeps(const Geo& g, bool want_nz) {
    if (want_nz || g.Wk != g.W || !tiled_fwd_entmax_workspace(g)) return false;
    if ((int64_t)g.Np * g.K > INT32_MAX) return true;
    return (int64_t)score_bytes(g) > g_entmax_scratch_limit.load(std::memory_order_relaxed);
}

size_t ca_attention_fwd_workspace(const ca_desc* d, int32_t want_nz) {
    Geo g;
    if (make_geo(d, &g, true)) return 0;
    if (!want_nz && line_shape_ok(g)) return 0;              // the 1-D kernels stage from the tensors themselves
    if (d->normalizer == CA_ENTMAX15) {
        const bool band = g.Wk != g.W;
        // flash mode on the fused sweeps: the packed (k|v) and one scalar plane, nothing A-sized
        if (entmax_fwd_on_sweeps(g, want_nz != 0)) return tiled_fwd_entmax_workspace(g);
        // otherwise: scores (unless they are written to nz) followed by the packed operand of the tiled operators
        return (want_nz ? 0 : score_bytes(g)) + (band ? 0 : tiled_operator_workspace(g));
    }
    if (composed_path(d, g)) return (want_nz ? 0 : score_bytes(g)) + tiled_operator_workspace(g);
    const bool band = g.Wk != g.W;
    return (want_nz && band) ? 0 : tiled_fwd_workspace(g);
}

int ca_attention_fwd(const ca_desc* d, const void* q, const void* k, const void* v,
                     void* y, float* nz, float* stats, void* workspace, void* stream) {
    Geo g;
    int rc = make_geo(d, &g, true);
    if (rc) return rc;
    if (!q || !k || !v || !y) { set_error("q/k/v/y is NULL"); return CA_ERR_NULL; }
    const bool band = g.Wk != g.W;
    if (nz && band) { set_error("band mode never materialises A"); return CA_ERR_UNSUPPORTED; }
    if (nz && (rc = check_nnz(g))) return rc;
    cudaStream_t st = as_stream(stream);
    const int dist = d->similarity == CA_DISTANCE;

    const bool ent = d->normalizer == CA_ENTMAX15;
    if (!nz) {
        // 1-D signals in flash mode: sliding-window kernels, softmax and entmax, no scratch
        rc = line_attention_fwd(g, d->scale, dist, ent, (const float*)q, (const float*)k, (const float*)v,
                                (float*)y, stats, st);
        if (rc != CA_ERR_UNSUPPORTED) return rc;
    }
    if (ent && (rc = no_bf16(g, "ca_attention_fwd with entmax"))) return rc;
    if (ent && workspace && entmax_fwd_on_sweeps(g, nz != nullptr)) {
        // 2-D (and wide 1-D) flash mode: repeated sweeps of the tiled kernels, the threshold search included
        rc = tiled_attention_fwd_entmax(g, d->scale, dist, (const float*)q, (const float*)k, (const float*)v,
                                        (float*)y, stats, workspace, st);
        if (rc != CA_ERR_UNSUPPORTED) return rc;
        // the workspace was sized for the sweeps (ca_attention_fwd_workspace follows the same rule), so the chain
        // below, which needs an A-sized buffer, must not run on it
        set_error("entmax forward: the fused sweeps do not cover this launch (grid limits); raise ca_entmax_scratch_limit to use the operator chain");
        return CA_ERR_UNSUPPORTED;
    }
    if (ent || (composed_path(d, g) && (nz || workspace))) {
        // scores -> row normaliser (threshold or log-sum-exp per row) -> apply; the scores live in
        // nz or in the workspace
        if (band) { set_error("entmax in band mode is not implemented"); return CA_ERR_UNSUPPORTED; }
        if ((rc = check_nnz(g))) return rc;
        float* sbuf = nz ? nz : (float*)workspace;
        if (!sbuf) { set_error("entmax without nz needs a workspace of ca_attention_fwd_workspace() bytes"); return CA_ERR_NULL; }
        void* opws = (workspace && tiled_operator_workspace(g))
                         ? (void*)((char*)workspace + (nz ? 0 : score_bytes(g))) : nullptr;
        rc = tiled_similarity(g, d->scale, dist, (const float*)q, (const float*)k, sbuf, opws, st);
        if (rc == CA_ERR_UNSUPPORTED)
            rc = launch_similarity(g, d->scale, dist, (const float*)q, (const float*)k, sbuf, st);
        if (rc) return rc;
        if ((rc = launch_row_normalize((int64_t)g.Np * g.units, g.K, ent, sbuf, sbuf, stats, st))) return rc;
        rc = tiled_apply(g, sbuf, (const float*)v, (float*)y, 1.f, 0, opws, st);
        if (rc != CA_ERR_UNSUPPORTED) return rc;
        return launch_apply(g, sbuf, (const float*)v, nullptr, (float*)y, 1.f, 0, 0, 0, st);
    }

    if (workspace) {
        rc = tiled_attention_fwd(g, d->scale, dist, (const float*)q, (const float*)k, (const float*)v,
                                 (float*)y, nz, stats, workspace, st);
        if (rc != CA_ERR_UNSUPPORTED) return rc;
    }

    if ((rc = no_bf16(g, "ca_attention_fwd on this shape"))) return rc;
    const int cmax = pick_cmax(g.cr);
    if (!cmax) { set_error("fused attention supports at most 64 real channels per unit (got %d); use similarity + normalize + apply", g.cr); return CA_ERR_UNSUPPORTED; }
    FwdArgs a{g, d->scale, dist, (const float*)q, (const float*)k, (const float*)v, (float*)y, nz, stats};
    dim3 grid((g.Np + 127) / 128, g.units);
    CA_DISPATCH_CMAX(cmax, g.cpe, (fwd_softmax_generic<CM, CP><<<grid, 128, 0, st>>>(a)));
    CA_CHECK_LAUNCH("fused forward kernel");
    return CA_OK;
}

static size_t d_bytes(const Geo& g) { return (((size_t)g.Npk * g.units * sizeof(float)) + 255) & ~(size_t)255; }

size_t ca_attention_bwd_workspace(const ca_desc* d, int32_t with_dA) {
    Geo g;
    if (make_geo(d, &g, false)) return 0;
    // D, then the larger of the two scratch layouts the shape can take (fused tiled kernels; operator chain)
    const size_t fused = tiled_bwd_workspace(g);
    const size_t chain = composed_path(d, g, true, with_dA != 0) ? 2 * score_bytes(g) + tiled_operator_workspace(g) : 0;
    return d_bytes(g) + (fused > chain ? fused : chain);
}

size_t ca_attention_bwd_stage_workspace(const ca_desc* d) {
    Geo g;
    if (make_geo(d, &g, true)) return 0;
    return d->normalizer == CA_SOFTMAX ? tiled_bwd_stage_workspace(g) : 0;
}

int ca_stage_timeouts(int32_t* count) {
    if (!count) { set_error("count is NULL"); return CA_ERR_NULL; }
    int c = 0;
    int rc = tiled_stage_timeouts(&c);
    *count = c;
    return rc;
}

int ca_attention_bwd_pre(const ca_desc* d, const void* q, const void* k, const void* v,
                         const void* y, const void* dy, const float* stats,
                         const float* nz, const float* dA, float* D, void* stream) {
    Geo g;
    if (!d) { set_error("descriptor is NULL"); return CA_ERR_NULL; }
    ca_desc dd = *d;
    // the softmax pre-pass without a cotangent on A is D = dy . y per pixel: it looks at no window, so a band
    // narrower than the window (legal for the band split, whose halos come from the neighbours) is accepted
    if (dd.normalizer == CA_SOFTMAX && !dA && dd.ws >= 1 && dd.ws % 2 == 1) dd.ws = 1;
    int rc = make_geo(&dd, &g, true);
    if (rc) return rc;
    if (!dy || !D) { set_error("dy/D is NULL"); return CA_ERR_NULL; }
    if ((rc = no_bf16(g, "ca_attention_bwd_pre"))) return rc;
    if (dA && !nz && d->normalizer == CA_SOFTMAX) { set_error("a cotangent on A needs the saved A (nz)"); return CA_ERR_NULL; }
    if (dA && g.Wk != g.W) { set_error("band mode never materialises A"); return CA_ERR_UNSUPPORTED; }
    cudaStream_t st = as_stream(stream);
    BwdArgs a{g, d->scale, d->similarity == CA_DISTANCE, d->normalizer == CA_ENTMAX15,
              (const float*)q, (const float*)k, (const float*)v, (const float*)y, (const float*)dy,
              stats, nz, dA, D, nullptr, nullptr, nullptr};
    dim3 grid((g.Np + 127) / 128, g.units);
    if (a.entmax) {
        if (!q || !k || !v || !stats) { set_error("q/k/v/stats is NULL"); return CA_ERR_NULL; }
        const int cmax = pick_cmax(g.cr);
        if (!cmax) { set_error("fused attention supports at most 64 real channels per unit (got %d)", g.cr); return CA_ERR_UNSUPPORTED; }
        CA_DISPATCH_CMAX(cmax, g.cpe, (bwd_query_generic<CM, CP, 1><<<grid, 128, 0, st>>>(a)));
    } else {
        if (!y) { set_error("y is NULL"); return CA_ERR_NULL; }
        if (g.cpe == 1) bwd_pre_softmax<1><<<grid, 128, 0, st>>>(a);
        else bwd_pre_softmax<2><<<grid, 128, 0, st>>>(a);
    }
    CA_CHECK_LAUNCH("backward pre-pass kernel");
    return CA_OK;
}

int ca_attention_bwd_dq(const ca_desc* d, const void* q, const void* k, const void* v,
                        const void* dy, const float* stats, const float* D, const float* dA,
                        void* dq, void* workspace, void* stream) {
    Geo g;
    int rc = make_geo(d, &g, true);
    if (rc) return rc;
    if (!q || !k || !v || !dy || !stats || !D || !dq) { set_error("a required pointer is NULL"); return CA_ERR_NULL; }
    if (dA && g.Wk != g.W) { set_error("band mode never materialises A"); return CA_ERR_UNSUPPORTED; }
    cudaStream_t st = as_stream(stream);
    const int dist = d->similarity == CA_DISTANCE, ent = d->normalizer == CA_ENTMAX15;
    if (!ent && !dA && workspace) {
        rc = tiled_attention_bwd_dq(g, d->scale, dist, (const float*)q, (const float*)k, (const float*)v,
                                    (const float*)dy, stats, D, (float*)dq, workspace, st);
        if (rc != CA_ERR_UNSUPPORTED) return rc;
    }
    if ((rc = no_bf16(g, "ca_attention_bwd_dq on this shape"))) return rc;
    const int cmax = pick_cmax(g.cr);
    if (!cmax) { set_error("fused attention supports at most 64 real channels per unit (got %d)", g.cr); return CA_ERR_UNSUPPORTED; }
    BwdArgs a{g, d->scale, dist, ent, (const float*)q, (const float*)k, (const float*)v, nullptr,
              (const float*)dy, stats, nullptr, dA, const_cast<float*>(D), (float*)dq, nullptr, nullptr};
    dim3 grid((g.Np + 127) / 128, g.units);
    CA_DISPATCH_CMAX(cmax, g.cpe, (bwd_query_generic<CM, CP, 0><<<grid, 128, 0, st>>>(a)));
    CA_CHECK_LAUNCH("backward dq kernel");
    return CA_OK;
}

int ca_attention_bwd_dkdv(const ca_desc* d, const void* q, const void* k, const void* v,
                          const void* dy, const float* stats, const float* D, const float* dA,
                          void* dk, void* dv, void* workspace, void* stream) {
    Geo g;
    int rc = make_geo(d, &g, true);
    if (rc) return rc;
    if (!q || !k || !v || !dy || !stats || !D || !dk || !dv) { set_error("a required pointer is NULL"); return CA_ERR_NULL; }
    if (dA && g.Wk != g.W) { set_error("band mode never materialises A"); return CA_ERR_UNSUPPORTED; }
    cudaStream_t st = as_stream(stream);
    const int dist = d->similarity == CA_DISTANCE, ent = d->normalizer == CA_ENTMAX15;
    if (!ent && !dA && workspace) {
        rc = tiled_attention_bwd_dkdv(g, d->scale, dist, (const float*)q, (const float*)k, (const float*)v,
                                      (const float*)dy, stats, D, (float*)dk, (float*)dv, workspace, st);
        if (rc != CA_ERR_UNSUPPORTED) return rc;
    }
    if ((rc = no_bf16(g, "ca_attention_bwd_dkdv on this shape"))) return rc;
    const int cmax = pick_cmax(g.cr);
    if (!cmax) { set_error("fused attention supports at most 64 real channels per unit (got %d)", g.cr); return CA_ERR_UNSUPPORTED; }
    BwdArgs a{g, d->scale, dist, ent, (const float*)q, (const float*)k, (const float*)v, nullptr,
              (const float*)dy, stats, nullptr, dA, const_cast<float*>(D), nullptr, (float*)dk, (float*)dv};
    dim3 grid((g.Np + 127) / 128, g.units);
    CA_DISPATCH_CMAX(cmax, g.cpe, (bwd_key_generic<CM, CP><<<grid, 128, 0, st>>>(a)));
    CA_CHECK_LAUNCH("backward dk/dv kernel");
    return CA_OK;
}

int ca_attention_bwd(const ca_desc* d, const void* q, const void* k, const void* v,
                     const void* y, const void* dy, const float* stats,
                     const float* nz, const float* dA,
                     void* dq, void* dk, void* dv, void* workspace, const void* fwd_workspace, void* stream) {
    Geo g;
    int rc = make_geo(d, &g, false);
    if (rc) return rc;
    if (!workspace) { set_error("workspace of ca_attention_bwd_workspace() bytes is NULL"); return CA_ERR_NULL; }
    float* D = (float*)workspace;
    if (!dA && line_shape_ok(g)) {
        const bool ent = d->normalizer == CA_ENTMAX15;
        if (!q || !k || !v || (!ent && !y) || !dy || !stats || !dq || !dk || !dv) { set_error("a required pointer is NULL"); return CA_ERR_NULL; }
        rc = line_attention_bwd(g, d->scale, d->similarity == CA_DISTANCE, ent, (const float*)q, (const float*)k,
                                (const float*)v, (const float*)y, (const float*)dy, stats, D, (float*)dq, (float*)dk,
                                (float*)dv, as_stream(stream));
        if (rc != CA_ERR_UNSUPPORTED) return rc;
    }
    if (d->normalizer == CA_ENTMAX15 && !dA && g.wsw != 1) {
        // fused kernels with the entmax weights recomputed from tau (no A-sized traffic).  2-D only: 1-D
        // signals took the sliding-tile kernels above; what is left of 1-D (wide units, windows under 5) is
        // shared-memory bound on the folded tiled kernels and runs the generic ones.
        if (!q || !k || !v || !dy || !stats || !dq || !dk || !dv) { set_error("a required pointer is NULL"); return CA_ERR_NULL; }
        rc = tiled_attention_bwd_entmax(g, d->scale, d->similarity == CA_DISTANCE, (const float*)q, (const float*)k,
                                        (const float*)v, (const float*)dy, stats, D, (float*)dq, (float*)dk,
                                        (float*)dv, (char*)workspace + d_bytes(g), as_stream(stream));
        if (rc != CA_ERR_UNSUPPORTED) return rc;
    }
    if (composed_path(d, g, true, dA != nullptr)) {
        // the pullback chain of src/rrules.jl:42-72 on the tiled operators:
        //   P (saved, or recomputed from q, k) ; dv = P^T dy ; dP = Re(dy . conj(v)) on the window (+ dA) ;
        //   dS = normaliser pullback ; (dq, dk) = similarity pullback
        if (!q || !k || !v || !dy || !dq || !dk || !dv) { set_error("a required pointer is NULL"); return CA_ERR_NULL; }
        cudaStream_t st = as_stream(stream);
        const int dist = d->similarity == CA_DISTANCE, ent = d->normalizer == CA_ENTMAX15;
        float* pbuf = (float*)((char*)workspace + d_bytes(g));
        float* dpbuf = (float*)((char*)pbuf + score_bytes(g));
        void* opws = (char*)dpbuf + score_bytes(g);
        const int64_t rows = (int64_t)g.Np * g.units, nnz = rows * g.K;
        auto chain = [&]() -> int {
            int r;
            const float* P = nz;
            if (!P) {
                if ((r = tiled_similarity(g, d->scale, dist, (const float*)q, (const float*)k, pbuf, opws, st))) return r;
                if ((r = launch_row_normalize(rows, g.K, ent, pbuf, pbuf, nullptr, st))) return r;
                P = pbuf;
            }
            if ((r = tiled_apply(g, P, (const float*)dy, (float*)dv, 1.f, 1, opws, st))) return r;
            if ((r = tiled_similarity(g, 1.f, 0, (const float*)dy, (const float*)v, dpbuf, opws, st))) return r;
            if (dA && (r = ca_axpby(nnz, 1.f, dpbuf, 1.f, dA, dpbuf, stream))) return r;
            if ((r = launch_row_normalize_bwd(rows, g.K, ent, P, dpbuf, dpbuf, st))) return r;
            return tiled_similarity_bwd(g, d->scale, dist, (const float*)q, (const float*)k, dpbuf, (float*)dq,
                                        (float*)dk, opws, st);
        };
        rc = chain();
        // a step of the chain that does not fit this window (shared memory of the transposed apply
        // at wide units and large windows) leaves the whole pullback to the generic kernels below,
        // which overwrite dq, dk and dv
        if (rc != CA_ERR_UNSUPPORTED) return rc;
    }
    if (d->normalizer == CA_SOFTMAX && !dA) {
        if (!q || !k || !v || !y || !dy || !stats || !dq || !dk || !dv) { set_error("a required pointer is NULL"); return CA_ERR_NULL; }
        rc = tiled_attention_bwd(g, d->scale, d->similarity == CA_DISTANCE, (const float*)q, (const float*)k,
                                 (const float*)v, (const float*)y, (const float*)dy, stats, D, (float*)dq,
                                 (float*)dk, (float*)dv, (char*)workspace + d_bytes(g), fwd_workspace, as_stream(stream));
        if (rc != CA_ERR_UNSUPPORTED) return rc;
    }
    if ((rc = no_bf16(g, "ca_attention_bwd on this shape"))) return rc;
    if ((rc = ca_attention_bwd_pre(d, q, k, v, y, dy, stats, nz, dA, D, stream))) return rc;
    if ((rc = ca_attention_bwd_dq(d, q, k, v, dy, stats, D, dA, dq, nullptr, stream))) return rc;
    return ca_attention_bwd_dkdv(d, q, k, v, dy, stats, D, dA, dk, dv, nullptr, stream);
}

int ca_axpby(int64_t n, float alpha, const float* x, float beta, const float* y, float* out, void* stream) {
    if (n < 0) { set_error("negative length"); return CA_ERR_BAD_DESC; }
    if (n == 0) return CA_OK;
    if (!x || !out || (beta != 0.f && !y)) { set_error("x/y/out is NULL"); return CA_ERR_NULL; }
    axpby_kernel<<<elementwise_grid((n + 3) / 4), 256, 0, as_stream(stream)>>>(n, alpha, x, beta, beta != 0.f ? y : nullptr, out);
    CA_CHECK_LAUNCH("axpby kernel");
    return CA_OK;
}

static int check_bcast(const char* what, int v1, int v2, int o1, int o2) {
    if ((v1 != 1 && v1 != o1) || (v2 != 1 && v2 != o2)) {
        set_error("%s batch dims (%d,%d) do not broadcast to (%d,%d)", what, v1, v2, o1, o2);
        return CA_ERR_BAD_DESC;
    }
    return CA_OK;
}

int ca_scale_batch(int64_t inner, int32_t o1, int32_t o2, const float* a, int32_t a1, int32_t a2,
                   const float* c, int32_t c1, int32_t c2, float* out, void* stream) {
    if (inner < 1 || o1 < 1 || o2 < 1 || o1 > 65535 || o2 > 65535) { set_error("bad extents"); return CA_ERR_BAD_DESC; }
    if (!a || !c || !out) { set_error("a/c/out is NULL"); return CA_ERR_NULL; }
    int rc;
    if ((rc = check_bcast("values", a1, a2, o1, o2)) || (rc = check_bcast("scale", c1, c2, o1, o2))) return rc;
    dim3 grid(elementwise_grid(inner), o1, o2);
    scale_batch_kernel<<<grid, 256, 0, as_stream(stream)>>>(inner, o1, o2, a, a1, a2, c, c1, c2, out);
    CA_CHECK_LAUNCH("scale kernel");
    return CA_OK;
}

int ca_dot_batch(int64_t inner, int32_t o1, int32_t o2, const float* x, int32_t x1, int32_t x2,
                 const float* y, int32_t y1, int32_t y2, float* out, void* stream) {
    if (inner < 1 || o1 < 1 || o2 < 1 || o1 > 65535 || o2 > 65535) { set_error("bad extents"); return CA_ERR_BAD_DESC; }
    if (!x || !out) { set_error("x/out is NULL"); return CA_ERR_NULL; }
    int rc;
    if ((rc = check_bcast("x", x1, x2, o1, o2))) return rc;
    if (y && (rc = check_bcast("y", y1, y2, o1, o2))) return rc;
    dim3 grid(o1, o2);
    dot_batch_kernel<<<grid, 1024, 0, as_stream(stream)>>>(inner, o1, x, x1, x2, y, y1, y2, out);
    CA_CHECK_LAUNCH("dot kernel");
    return CA_OK;
}

int ca_sum_batch(int64_t inner, int32_t b1, int32_t b2, int32_t sum1, int32_t sum2,
                 const float* in, float* out, void* stream) {
    if (inner < 1 || b1 < 1 || b2 < 1) { set_error("bad extents"); return CA_ERR_BAD_DESC; }
    if (!in || !out) { set_error("in/out is NULL"); return CA_ERR_NULL; }
    const int64_t total = inner * (sum1 ? 1 : b1) * (sum2 ? 1 : b2);
    sum_batch_kernel<<<elementwise_grid(total), 256, 0, as_stream(stream)>>>(inner, b1, b2, sum1, sum2, in, out);
    CA_CHECK_LAUNCH("batch sum kernel");
    return CA_OK;
}

int ca_sum_rows(const ca_desc* d, const float* nz, float* out, void* stream) {
    Geo g;
    int rc = make_geo(d, &g, false);
    if (rc) return rc;
    if (!nz || !out) { set_error("nz/out is NULL"); return CA_ERR_NULL; }
    const int64_t rows = (int64_t)g.Np * g.units;
    if ((rows * 32 + 255) / 256 > INT32_MAX) { set_error("too many rows"); return CA_ERR_TOO_LARGE; }
    sum_rows_kernel<<<(unsigned)((rows * 32 + 255) / 256), 256, 0, as_stream(stream)>>>(rows, g.K, nz, out);
    CA_CHECK_LAUNCH("row sum kernel");
    return CA_OK;
}

int ca_sum_cols(const ca_desc* d, const float* nz, float* out, void* stream) {
    Geo g;
    int rc = make_geo(d, &g, false);
    if (rc) return rc;
    if (!nz || !out) { set_error("nz/out is NULL"); return CA_ERR_NULL; }
    dim3 grid((g.Np + 127) / 128, g.units);
    sum_cols_kernel<<<grid, 128, 0, as_stream(stream)>>>(g, nz, out);
    CA_CHECK_LAUNCH("column sum kernel");
    return CA_OK;
}

}  // extern "C"
