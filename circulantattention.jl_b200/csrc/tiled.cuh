// Tiled sm_100a kernels for the hot shapes (declarations; see tiled.cu).
#pragma once
#include "common.cuh"

namespace ca {

// Workspace sizes in bytes; 0 when the shape is outside what the tiled kernels cover.
size_t tiled_fwd_workspace(const Geo& g);
size_t tiled_bwd_workspace(const Geo& g);        // whole backward (without D)
size_t tiled_bwd_stage_workspace(const Geo& g);  // one of the separately callable stages

// Each returns CA_ERR_UNSUPPORTED (without touching the error text) when the
// shape is outside what the tiled kernels cover; the caller then falls back
// to the generic kernels.
int tiled_attention_fwd(const Geo& g, float scale, int dist, const float* q, const float* k, const float* v,
                        float* y, float* nz, float* stats, void* workspace, cudaStream_t st);
int tiled_attention_bwd(const Geo& g, float scale, int dist, const float* q, const float* k, const float* v,
                        const float* y, const float* dy, const float* stats, float* D, float* dq, float* dk,
                        float* dv, void* workspace, const void* fwd_workspace, cudaStream_t st);
int tiled_attention_bwd_dq(const Geo& g, float scale, int dist, const float* q, const float* k, const float* v,
                           const float* dy, const float* stats, const float* D, float* dq, void* workspace,
                           cudaStream_t st);
int tiled_attention_bwd_dkdv(const Geo& g, float scale, int dist, const float* q, const float* k, const float* v,
                             const float* dy, const float* stats, const float* D, float* dk, float* dv,
                             void* workspace, cudaStream_t st);
// The 1.5-entmax backward (stats = tau); workspace of tiled_bwd_workspace bytes.
int tiled_attention_bwd_entmax(const Geo& g, float scale, int dist, const float* q, const float* k, const float* v,
                               const float* dy, const float* stats, float* D, float* dq, float* dk, float* dv,
                               void* workspace, cudaStream_t st);
// The 1.5-entmax forward in flash mode (y and stats = tau) by repeated sweeps over the packed (k|v): no
// A-sized memory.  One-slab units only; workspace of tiled_fwd_entmax_workspace bytes (0: shape not covered).
size_t tiled_fwd_entmax_workspace(const Geo& g);
int tiled_attention_fwd_entmax(const Geo& g, float scale, int dist, const float* q, const float* k, const float* v,
                               float* y, float* stats, void* workspace, cudaStream_t st);
// Copies the count of stage-copy timeouts to the host (synchronises the device).
int tiled_stage_timeouts(int* count);
// Launches the one-CTA self test of the bounded stage wait (`out`: nullable device int, 1 = the wait ran out).
int tiled_probe_stage_timeout(uint32_t tries, int* out, cudaStream_t st);

// Stand-alone operators on the tiled kernels.  `workspace` holds one packed
// tensor pair (tiled_operator_workspace bytes, 0 when the shape is not covered).
size_t tiled_operator_workspace(const Geo& g);
int tiled_similarity(const Geo& g, float scale, int dist, const float* x, const float* y, float* nz,
                     void* workspace, cudaStream_t st);
int tiled_apply(const Geo& g, const float* nz, const float* v, float* out, float alpha, int transposed,
                void* workspace, cudaStream_t st);
int tiled_similarity_bwd(const Geo& g, float scale, int dist, const float* x, const float* y, const float* dS,
                         float* dx, float* dy, void* workspace, cudaStream_t st);

}  // namespace ca
