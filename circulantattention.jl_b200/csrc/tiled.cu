#include "tiled.cuh"

namespace ca {

int tiled_attention_fwd(const Geo&, float, int, const float*, const float*, const float*, float*, float*, float*,
                        cudaStream_t) { return CA_ERR_UNSUPPORTED; }
int tiled_attention_bwd_dq(const Geo&, float, int, const float*, const float*, const float*, const float*,
                           const float*, const float*, float*, cudaStream_t) { return CA_ERR_UNSUPPORTED; }
int tiled_attention_bwd_dkdv(const Geo&, float, int, const float*, const float*, const float*, const float*,
                             const float*, const float*, float*, float*, cudaStream_t) { return CA_ERR_UNSUPPORTED; }
int tiled_apply(const Geo&, const float*, const float*, float*, cudaStream_t) { return CA_ERR_UNSUPPORTED; }

}  // namespace ca
