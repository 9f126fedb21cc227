// Shared host/device helpers of the circulant-attention kernels (sm_100a).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include "../../include/circatt_b200.h"
#include "../../include/circatt_b200_probe.h"

namespace ca {

// ---------------------------------------------------------------- errors
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

// Device word registered by the calling host thread with ca_status_word (NULL: none).
int* status_word();

void count_launch();
void count_tiled_launch();     // launches of the TMA-tiled kernels only (tests use it to see which path ran)

#define CA_CHECK_LAUNCH(what)                                        \
    do {                                                             \
        ca::count_launch();                                          \
        cudaError_t e__ = cudaGetLastError();                        \
        if (e__ != cudaSuccess) return ca::cuda_fail(e__, what);     \
    } while (0)

// ---------------------------------------------------------------- geometry
// Window geometry in pixel units.  The query side has H x W pixels; the key
// side has H x Wk pixels.  With Wk == W the window wraps circularly along both
// axes; in band mode (Wk = W + 2p, wk_off = p) the key-side tensors already
// hold the neighbouring columns, so only the fast axis wraps.
struct Geo {
    int H, W, Wk, wk_off;
    int ws, p;
    int wsw;      // window extent along w: ws in 2-D, 1 in 1-D
    int K;        // entries per row: ws * wsw
    int Np, Npk;  // pixels on the query side / key side
    int units;
    int c;        // channels per unit in elements
    int cpe;      // floats per element: 1 (f32) or 2 (c64)
    int cr;       // real channels per unit: c * cpe
    int bf16;     // dense tensors are stored as bfloat16 (cpe == 1); arithmetic stays Float32
};

__host__ __device__ inline int wrap_axis(int x, int X) {
    x += (x < 0) ? X : 0;
    x -= (x >= X) ? X : 0;
    return x;
}

// Position of window offset d (in [-p, p]) inside the ascending-column run of a
// row whose own coordinate on that axis is x (axis length X).  Border rows are
// rotated so that wrapped columns keep the run sorted, which is what the
// circshift_index calls of the reference (src/circulant.jl:11-15, 30-39) do.
__host__ __device__ inline int axis_pos(int d, int x, int X, int p, int ws) {
    if (x < p) {
        int t = d + x;
        return t < 0 ? t + ws : t;
    }
    if (x >= X - p) {
        int t = d + x - X;
        return t < 0 ? t + ws : t;
    }
    return d + p;
}

int make_geo(const ca_desc* d, Geo* g, bool allow_band);

static inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

// ---------------------------------------------------------------- device math
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

}  // namespace ca
