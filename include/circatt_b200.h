/*
 * circatt_b200.h -- C ABI of the B200 (sm_100a) circulant-attention library.
 *
 * Every entry point replaces a piece of device work that the Julia package
 * CirculantAttention.jl (v1.0.1) performs through CUDA.jl codegen, cuSPARSE or
 * NNlib/cuDNN.  The citation on each declaration is the reference file:line
 * whose device work the entry point stands in for.
 *
 * Conventions
 *  - All pointers are DEVICE pointers into memory owned by the caller.  The
 *    library never allocates or frees caller-visible memory, never
 *    synchronises the device, and orders all its work on the stream it is
 *    given (`stream` is a cudaStream_t passed as void*; NULL = legacy
 *    default).  ca_attention_bwd may run one of its sweeps on an internal
 *    helper stream that is forked from and joined back to that stream with
 *    events, which is invisible to stream-ordered callers.
 *  - Dense tensors use the Julia column-major layout of the reference:
 *    element (h, w, ch, u) of a (H, W, c, units) array sits at
 *    h + H*(w + W*(ch + c*u)); 1-D signals have W = 1.  `units` is the merged
 *    head*batch dimension after the reference's `splitheads`
 *    (src/attention.jl:44): head index fastest.  CA_C64 tensors hold
 *    interleaved (re, im) float pairs.
 *  - Sparse values (`nz`) are float32 (also for complex inputs,
 *    src/array.jl:12-14, src/similarity.jl:139), laid out as the reference's
 *    nzVal: K = ws^ndim consecutive entries per row (query pixel), rows
 *    consecutive, units outermost: nz[k + K*(row + Np*u)].  Inside a row the
 *    entries are in ascending column order -- the order `cartesian_circulant`
 *    (src/circulant.jl:4-44) defines.
 *  - Every function returns CA_OK (0) or a negative ca_status; the text of the
 *    last failure on the calling thread is returned by ca_last_error().
 */
#ifndef CIRCATT_B200_H
#define CIRCATT_B200_H

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum ca_status {
    CA_OK = 0,
    CA_ERR_BAD_DESC = -1,      /* inconsistent descriptor (even window, extent < window, ...) */
    CA_ERR_UNSUPPORTED = -2,   /* legal but not implemented combination */
    CA_ERR_NULL = -3,          /* a required pointer is NULL */
    CA_ERR_CUDA = -4,          /* a CUDA runtime call or launch failed */
    CA_ERR_TOO_LARGE = -5,     /* a size exceeds a documented limit */
    CA_ERR_COMM = -6           /* NCCL is missing or an NCCL call failed */
} ca_status;

enum { CA_F32 = 0, CA_C64 = 1, CA_BF16 = 2 }; /* element type of dense tensors; CA_BF16 (storage only: all
                                              * arithmetic and A's values, statistics and scratch stay Float32)
                                              * is accepted by the fused attention entry points on the shapes
                                              * their tiled kernels cover, and has no reference counterpart */
enum { CA_DOT = 0, CA_DISTANCE = 1 };       /* src/similarity.jl:15,29 */
enum { CA_SOFTMAX = 0, CA_ENTMAX15 = 1 };   /* row normaliser; entmax has no reference counterpart */

/* Problem descriptor shared by the windowed kernels. */
typedef struct ca_desc {
    int32_t H;          /* fast spatial extent (Julia dim 1) */
    int32_t W;          /* slow spatial extent (Julia dim 2); 1 when ndim == 1 */
    int32_t ndim;       /* number of spatial dims: 1 or 2 */
    int32_t channels;   /* channels per unit (C / nheads), counted in elements of `dtype` */
    int32_t units;      /* independent head*batch units */
    int32_t ws;         /* odd window length; every spatial extent must be >= ws */
    int32_t dtype;      /* CA_F32, CA_C64 or CA_BF16 */
    int32_t similarity; /* CA_DOT or CA_DISTANCE */
    int32_t normalizer; /* CA_SOFTMAX or CA_ENTMAX15 */
    int32_t Wk;         /* band mode: columns of the key-side tensors (0 or W = circular wrap) */
    int32_t wk_off;     /* band mode: key-side column that holds query column 0 */
    float   scale;      /* factor applied to the raw similarity (1/sqrt(c) inside attention) */
} ca_desc;

/* Library version (major*10000 + minor*100 + patch). */
int ca_version(void);

/* Text of the last error raised on the calling thread ("" if none). */
const char* ca_last_error(void);

/* ---------------------------------------------------------------- structure
 * CSR structure of the circulant / BCCB pattern, 1-based Int32, replicated
 * `nbatch` times as the reference does with `repeat` (src/array.jl:9):
 *   rowptr[r + (Np+1)*b] = 1 + K*r           (src/circulant.jl:71-73, 93-95)
 *   colval[n + Np*K*b]   = column of entry n  (src/circulant.jl:46-62 -> :4-44)
 */
int ca_structure(int32_t H, int32_t W, int32_t ndim, int32_t ws, int64_t nbatch,
                 int32_t* rowptr, int32_t* colval, void* stream);

/* ---------------------------------------------------------------- operator workspace
 * Bytes of caller-owned scratch with which ca_similarity, ca_similarity_bwd and
 * ca_apply run on the tiled TMA kernels (2-D, 16 real channels per unit); 0 when
 * the shape is only covered by the generic kernels.  The three calls accept
 * workspace == NULL and then always use the generic kernels.  No reference
 * counterpart (the reference's operators allocate through CUDA.jl's pool). */
size_t ca_operator_workspace(const ca_desc* d);

/* ---------------------------------------------------------------- similarity
 * nz = scale * simfun(x[row pixel], y[column pixel]) for every stored entry.
 * Replaces circulant_similarity_kernel! (src/similarity.jl:55-103) and its
 * launcher (src/similarity.jl:36-53). */
int ca_similarity(const ca_desc* d, const void* x, const void* y, float* nz, void* workspace, void* stream);

/* Pullback of ca_similarity (src/rrules.jl:1-32):
 *   Dot:      dx = scale * dS Y               dy = scale * dS^T X
 *   Distance: dx = scale * (dS Y - rowsum(dS) X)   dy = scale * (dS^T X - colsum(dS) Y) */
int ca_similarity_bwd(const ca_desc* d, const void* x, const void* y, const float* dS,
                      void* dx, void* dy, void* workspace, void* stream);

/* ---------------------------------------------------------------- row normaliser
 * Row softmax (src/similarity.jl:105-126; NNlib.softmax! over each row's K
 * entries) or 1.5-entmax.  `p` may alias `s`.  `stats` (nullable, Np*units
 * floats) receives the row log-sum-exp (softmax) or threshold tau (entmax). */
int ca_row_normalize(const ca_desc* d, const float* s, float* p, float* stats, void* stream);

/* Pullback (src/rrules.jl:42-56 -> NNlib.∇softmax_data): ds = p*(dp - sum_row p*dp);
 * entmax: ds = g*(dp - sum g*dp / sum g), g = sqrt(p).  `ds` may alias `dp`. */
int ca_row_normalize_bwd(const ca_desc* d, const float* p, const float* dp, float* ds, void* stream);

/* ---------------------------------------------------------------- apply
 * out = A (x) v or A^T (x) v: the CUSPARSE.bmm! call sites of
 * src/batchedmul.jl:82-110 as used by circulant_attention!/
 * circulant_transposed_attention! (src/attention.jl:53-80).  Real A with a
 * CA_C64 v multiplies both parts (replaces the promotion copy of
 * src/batchedmul.jl:43-80).  a_bcast / v_bcast != 0 mean that A / v hold one
 * unit that is shared by all d->units outputs. */
int ca_apply(const ca_desc* d, const float* nz, const void* v, void* out,
             int32_t transpose, int32_t a_bcast, int32_t v_bcast, void* workspace, void* stream);

/* ---------------------------------------------------------------- fused attention
 * y = rownormalize(scale * simfun(q, k)) (x) v  in one pass
 * (circulant_attention, src/attention.jl:19-25; per-head via the merged unit
 * dimension, src/attention.jl:38-44).  `nz` (nullable) receives A's values in
 * CSR order; `stats` (nullable, Np*units floats) the per-row log-sum-exp /
 * entmax threshold needed by ca_attention_bwd.  `workspace` must hold
 * ca_attention_fwd_workspace() bytes (may be NULL when that is 0); the tiled
 * sm_100a kernels keep their packed copies of k and v there.  A NULL workspace
 * where one is needed selects the slower untiled kernels (softmax) or is an
 * error (entmax without nz). */
size_t ca_attention_fwd_workspace(const ca_desc* d, int32_t want_nz);
int ca_attention_fwd(const ca_desc* d, const void* q, const void* k, const void* v,
                     void* y, float* nz, float* stats, void* workspace, void* stream);

/* The same forward for callers that cannot allocate device memory (code that
 * runs inside somebody else's memory pool, fixed-budget real-time loops,
 * plugins that only ever receive pointers).  It has no counterpart in the
 * reference.  The workspace is a fixed array of ca_static_scratch_bytes()
 * (64 MiB) inside the library's device image: every GPU that loads the library
 * holds it until the process exits.  Problems whose workspace
 * (ca_attention_fwd_workspace) is larger are rejected with CA_ERR_TOO_LARGE.
 * All calls on a GPU share that array and it keeps the last call's contents,
 * so calls that overlap on the GPU race with each other; nothing in it needs
 * clearing between calls.  The first call on each device resolves the array's
 * address on the host; make it before beginning any stream capture.  The call
 * performs no cudaMalloc / cudaFree and calls no allocating library routine. */
size_t ca_static_scratch_bytes(void);
int ca_attention_fwd_static(const ca_desc* d, const void* q, const void* k, const void* v,
                            void* y, float* nz, float* stats, void* stream);

/* Gradient of the above (the composition of the reference's rrules for
 * similarity, softmax and apply: src/rrules.jl:1-72).  `dA` (nullable) is the
 * cotangent arriving on the returned A (CSR order); when it is given, `nz`
 * (the A saved by the forward) must be given as well.  `y` is the forward
 * output.  dq, dk, dv are overwritten.  Deterministic: no atomics.
 * `fwd_workspace` (nullable) is the workspace the matching ca_attention_fwd
 * call (same descriptor, same k and v) was given, left untouched since: the
 * tiled softmax kernels then stream the packed copy of (k, v) the forward left
 * there instead of packing k and v again.  The Julia counterpart is keeping a
 * forward intermediate alive inside the pullback closure (src/rrules.jl:44-55
 * keeps the softmax output that way).  The workspace size depends on whether
 * a cotangent on A will be passed (`with_dA`): that case runs the reference's
 * pullback chain on A-sized scratch. */
size_t ca_attention_bwd_workspace(const ca_desc* d, int32_t with_dA);
int ca_attention_bwd(const ca_desc* d, const void* q, const void* k, const void* v,
                     const void* y, const void* dy, const float* stats,
                     const float* nz, const float* dA,
                     void* dq, void* dk, void* dv, void* workspace, const void* fwd_workspace,
                     void* stream);

/* The three stages of ca_attention_bwd, exposed separately for the band-split
 * (multi-GPU) path, where D and the query-side halos are exchanged between
 * stages.  D holds one float per (query-side pixel, unit):
 *   softmax: D = dy . y + sum_k A_k dA_k      entmax: D = sum g dP / sum g.
 * In band mode (d->Wk = W + 2p) ca_attention_bwd_dq reads k, v with Wk columns,
 * and ca_attention_bwd_dkdv reads q, dy, stats, D with Wk columns.
 * `workspace` of the dq / dkdv stages (nullable: NULL selects the slower
 * untiled kernels) must hold ca_attention_bwd_stage_workspace() bytes. */
int ca_attention_bwd_pre(const ca_desc* d, const void* q, const void* k, const void* v,
                         const void* y, const void* dy, const float* stats,
                         const float* nz, const float* dA, float* D, void* stream);
size_t ca_attention_bwd_stage_workspace(const ca_desc* d);
int ca_attention_bwd_dq(const ca_desc* d, const void* q, const void* k, const void* v,
                        const void* dy, const float* stats, const float* D, const float* dA,
                        void* dq, void* workspace, void* stream);
int ca_attention_bwd_dkdv(const ca_desc* d, const void* q, const void* k, const void* v,
                          const void* dy, const float* stats, const float* D, const float* dA,
                          void* dk, void* dv, void* workspace, void* stream);

/* Failure reporting of the device-side waits.  Every wait in the library's
 * kernels (the shared-memory stage copies of the tiled kernels) is bounded.  A
 * thread block whose wait runs out stops computing, stores NaN instead of
 * results for its tile, bumps a per-device counter, and sets bit 0 of the
 * status word registered by the host thread that made the call.
 * ca_status_word registers a device int32 (zeroed by the caller) for all later
 * calls of the calling host thread (NULL: none); the caller reads it at its
 * own synchronisation points.  ca_stage_timeouts copies the counter of the
 * current device to the host (it synchronises the device: a diagnostic, not
 * for hot paths).  The reference has no counterpart: CUDA.jl kernels cannot
 * time out, they hang (src/similarity.jl:47-51 launches without any bound). */
int ca_status_word(int32_t* device_word);
int ca_stage_timeouts(int32_t* count);

/* The 1.5-entmax forward in flash mode (nz == NULL) has two routes on 2-D problems of 8 or 16 real channels
 * per unit: the operator chain (scores -> threshold -> apply) on an A-sized scratch buffer, which is the
 * faster one while that buffer is small, and repeated sweeps of the fused tiled kernels (row maximum, a few
 * steps of the threshold search, apply), which need only the packed (k|v) and two scalar planes.  The chain
 * is taken while its scratch stays within this limit (default 256 MiB); ca_attention_fwd_workspace follows
 * the same rule.  Sets the limit when `bytes` >= 0 and returns the previous one (process-wide). */
int64_t ca_entmax_scratch_limit(int64_t bytes);

/* ---------------------------------------------------------------- multi-GPU halo exchange
 * Band split of very large images (no counterpart in the reference, which is a
 * single-device package): one process per GPU owns a band of columns and needs
 * p = (ws-1)/2 columns of the key-side tensors from the ranks r-1 and r+1
 * (mod world: the circular wrap).  ca_comm_unique_id fills 128 bytes that rank 0
 * hands to the other ranks by any means; ca_comm_init joins the ring on the
 * current device (world == 1 needs no NCCL); ca_halo_exchange sends
 * `send_right` to rank r+1 and `send_left` to rank r-1 and receives the
 * neighbours' counterparts into `recv_left` / `recv_right` (nbytes each,
 * contiguous device buffers of the caller: gather the halo columns of all
 * tensors of one exchange into one message), ordered on `stream`.  NCCL is
 * bound at run time; CA_ERR_COMM reports a missing library or a failed call. */
int ca_comm_unique_id(void* id128);

/* Several strided device-to-device copies in ONE launch: job j copies `nchunks` pieces of `chunk_bytes` bytes,
 * `src_stride_bytes` apart at the source and `dst_stride_bytes` apart at the destination.  The halo columns
 * of a column-major (H, W, ...) tensor are such pieces (H*p elements per trailing index, H*W elements
 * apart), so one call gathers the outgoing halos of all tensors of an exchange into the two messages (and
 * copies the bands into their extended slabs), and a second one scatters the incoming halos.  `jobs` is a
 * HOST array of at most CA_MAX_CHUNK_JOBS entries (it is passed to the kernel by value). */
#define CA_MAX_CHUNK_JOBS 32
typedef struct ca_chunk_job {
    const void* src;
    void* dst;
    int64_t chunk_bytes;
    int64_t nchunks;
    int64_t src_stride_bytes;
    int64_t dst_stride_bytes;
} ca_chunk_job;
int ca_copy_chunks(const ca_chunk_job* jobs, int32_t njobs, void* stream);
int ca_comm_init(int32_t rank, int32_t world, const void* id128, void** comm);
int ca_comm_destroy(void* comm);
int ca_halo_exchange(void* comm, const void* send_left, const void* send_right,
                     void* recv_left, void* recv_right, size_t nbytes, void* stream);

/* ---------------------------------------------------------------- algebra on values
 * out[n,i,j] = alpha*x[n,i,j] + beta*y[n,i,j] over a flat length (X+Y, X-Y, c*X:
 * src/array.jl:66-81).  y may be NULL when beta == 0. */
int ca_axpby(int64_t n, float alpha, const float* x, float beta, const float* y,
             float* out, void* stream);

/* scale (src/array.jl:179-186): values of shape (inner, a1, a2) times c of shape
 * (c1, c2), each batch extent either 1 or the output's (o1, o2). */
int ca_scale_batch(int64_t inner, int32_t o1, int32_t o2,
                   const float* a, int32_t a1, int32_t a2,
                   const float* c, int32_t c1, int32_t c2,
                   float* out, void* stream);

/* out[i,j] = sum_n x[n,i,j]*y[n,i,j] (y NULL: sum of x) per batch slice, with the
 * same broadcasting rule.  Covers LinearAlgebra.dot (src/array.jl:83-85),
 * sum(A) (src/array.jl:162), sum(dims=(1,2)) (src/array.jl:151-154) and the
 * reduction inside the scale pullback (src/rrules.jl:105-108). */
int ca_dot_batch(int64_t inner, int32_t o1, int32_t o2,
                 const float* x, int32_t x1, int32_t x2,
                 const float* y, int32_t y1, int32_t y2,
                 float* out, void* stream);

/* Sum of values over batch dims (src/array.jl:132-149): in (inner, b1, b2) ->
 * out (inner, sum1 ? 1 : b1, sum2 ? 1 : b2). */
int ca_sum_batch(int64_t inner, int32_t b1, int32_t b2, int32_t sum1, int32_t sum2,
                 const float* in, float* out, void* stream);

/* Row sums (dims=2, src/array.jl:126-130) and column sums (dims=1,
 * src/array.jl:119-124; the reference does a transposed SpMM against ones).
 * out has Np*units floats. */
int ca_sum_rows(const ca_desc* d, const float* nz, float* out, void* stream);
int ca_sum_cols(const ca_desc* d, const float* nz, float* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CIRCATT_B200_H */
