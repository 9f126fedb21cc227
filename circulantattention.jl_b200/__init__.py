"""B200-native circulant attention behind the API of CirculantAttention.jl.

The package is a thin host layer: `api` mirrors the reference's Julia methods,
`ops` calls the C ABI of `libcircatt_b200.so` (hand-written sm_100a kernels in
`csrc/`), `jl` provides Julia-shaped column-major tensors, `parallel` shards
the work over GPUs, and `graphs` records calls into CUDA graphs.  There is no CPU or PyTorch fallback.
"""
from . import graphs, jl, ops, parallel  # noqa: F401
from .graphs import capture  # noqa: F401
from ._lib import CircAttError, LIB_PATH, lib  # noqa: F401
from .api import (  # noqa: F401
    AbstractSimilarity, BatchedTranspose, Circulant, LazyAdjacency, CuSparseArrayCSR, DistanceSimilarity, DotSimilarity,
    ENTMAX15, SOFTMAX, Otimes, batched_adjoint, batched_mul, batched_transpose, cat, circulant,
    circulant_adjacency, circulant_adjacency_, circulant_attention, circulant_attention_,
    circulant_mh_adjacency, circulant_mh_attention, circulant_mh_transposed_attention, mix_otimes,
    circulant_similarity, circulant_similarity_, circulant_transposed_attention,
    circulant_transposed_attention_, dot, entmax15, kernel_length, otimes, scale, softmax, softmax_,
    spatial_dims, spatial_size, splitheads, sum,
)
