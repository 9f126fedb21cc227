// Tiled sm_100a kernels for the hot shapes (declarations; see tiled.cu).
#pragma once
#include "common.cuh"

namespace ca {

// Each returns CA_ERR_UNSUPPORTED (without touching the error text) when the
// shape is outside what the tiled kernels cover; the caller then falls back
// to the generic kernels.
int tiled_attention_fwd(const Geo& g, float scale, int dist, const float* q, const float* k, const float* v,
                        float* y, float* nz, float* stats, cudaStream_t st);
int tiled_attention_bwd_dq(const Geo& g, float scale, int dist, const float* q, const float* k, const float* v,
                           const float* dy, const float* stats, const float* D, float* dq, cudaStream_t st);
int tiled_attention_bwd_dkdv(const Geo& g, float scale, int dist, const float* q, const float* k, const float* v,
                             const float* dy, const float* stats, const float* D, float* dk, float* dv,
                             cudaStream_t st);
int tiled_apply(const Geo& g, const float* nz, const float* v, float* out, cudaStream_t st);

}  // namespace ca
