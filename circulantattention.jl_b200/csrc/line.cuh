// Fused attention kernels for 1-D signals (declarations; see line.cu).
#pragma once
#include "common.cuh"

namespace ca {

// 1-D signals of at most 16 real channels per unit with a window of 5 to 511, Float32 or ComplexF32.
bool line_shape_ok(const Geo& g);

// Flash-mode forward (y and the row statistic: log-sum-exp, or the entmax threshold), no scratch memory.
// CA_ERR_UNSUPPORTED (error text untouched) outside line_shape_ok.
int line_attention_fwd(const Geo& g, float scale, int dist, int entmax, const float* q, const float* k,
                       const float* v, float* y, float* stats, cudaStream_t st);
// Backward without a cotangent on A; D (Np * units floats) is scratch.  y is read for softmax only.
int line_attention_bwd(const Geo& g, float scale, int dist, int entmax, const float* q, const float* k,
                       const float* v, const float* y, const float* dy, const float* stats, float* D, float* dq,
                       float* dk, float* dv, cudaStream_t st);

}  // namespace ca
