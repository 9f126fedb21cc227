// Multi-GPU halo exchange of the band split through the C ABI: NCCL point-to-point sends between a rank
// and its two neighbours on the ring of bands (the modulo of the ring is the circular wrap of the
// window).  One process per GPU.  NCCL is bound at run time (dlopen of libnccl.so.2), so that the
// library loads on hosts without NCCL and shares the copy a host program (PyTorch, CUDA.jl's NCCL.jl)
// has already loaded; the single-rank case needs no NCCL at all.
//
// Incoming halos land in the caller's own receive buffers; the kernels then read local memory only.
#include "common.cuh"

#include <dlfcn.h>
#include <string.h>
#include <nccl.h>
#include <algorithm>
#include <mutex>

namespace ca {
namespace {

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

// Several strided copies in one launch: job j copies nchunks pieces of chunk_bytes from src (pieces
// src_stride_bytes apart) to dst (dst_stride_bytes apart).  Block (x, j) walks the 32 KB segments x, x + gridDim.x,
// ... of job j's pieces; 16-byte accesses when every address of the job allows them.
struct ChunkJobs {
    ca_chunk_job job[CA_MAX_CHUNK_JOBS];
    int n;
};

constexpr int64_t kChunkSegment = 32 * 1024;      // bytes one block copies at a time

__global__ void __launch_bounds__(256) copy_chunks_kernel(const __grid_constant__ ChunkJobs jobs) {
    const ca_chunk_job& b = jobs.job[blockIdx.y];
    const char* src = static_cast<const char*>(b.src);
    char* dst = static_cast<char*>(b.dst);
    const bool wide = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst) | (uintptr_t)b.chunk_bytes |
                        (uintptr_t)b.src_stride_bytes | (uintptr_t)b.dst_stride_bytes) & 15) == 0;
    const bool words = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst) | (uintptr_t)b.chunk_bytes |
                         (uintptr_t)b.src_stride_bytes | (uintptr_t)b.dst_stride_bytes) & 3) == 0;
    // work items: (piece, 32 KB segment of the piece)
    const int64_t segs = (b.chunk_bytes + kChunkSegment - 1) / kChunkSegment;
    const int64_t items = b.nchunks * segs;
    for (int64_t it = blockIdx.x; it < items; it += gridDim.x) {
        const int64_t c = it / segs, sg = it - c * segs;
        const int64_t begin = sg * kChunkSegment;
        const int64_t len = min(kChunkSegment, b.chunk_bytes - begin);
        const char* s = src + c * b.src_stride_bytes + begin;
        char* d = dst + c * b.dst_stride_bytes + begin;
        if (wide) {
            const int64_t n = len >> 4;
            for (int64_t i = threadIdx.x; i < n; i += blockDim.x)
                reinterpret_cast<uint4*>(d)[i] = __ldg(reinterpret_cast<const uint4*>(s) + i);
        } else if (words) {
            const int64_t n = len >> 2;
            for (int64_t i = threadIdx.x; i < n; i += blockDim.x)
                reinterpret_cast<uint32_t*>(d)[i] = __ldg(reinterpret_cast<const uint32_t*>(s) + i);
        } else {
            for (int64_t i = threadIdx.x; i < len; i += blockDim.x) d[i] = s[i];
        }
    }
}

std::mutex g_nccl_mutex;
NcclApi g_nccl;

template <typename F>
bool bind(void* h, const char* name, F* out) {
    *out = reinterpret_cast<F>(dlsym(h, name));
    return *out != nullptr;
}

// Binds NCCL on first use.  Returns CA_OK or CA_ERR_COMM with the error text set.
int nccl_api(NcclApi** api) {
    std::lock_guard<std::mutex> lock(g_nccl_mutex);
    if (!g_nccl.handle) {
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) { set_error("NCCL is not available: %s", dlerror()); return CA_ERR_COMM; }
        NcclApi a;
        a.handle = h;
        if (!bind(h, "ncclGetUniqueId", &a.GetUniqueId) || !bind(h, "ncclCommInitRank", &a.CommInitRank) ||
            !bind(h, "ncclCommDestroy", &a.CommDestroy) || !bind(h, "ncclSend", &a.Send) ||
            !bind(h, "ncclRecv", &a.Recv) || !bind(h, "ncclGroupStart", &a.GroupStart) ||
            !bind(h, "ncclGroupEnd", &a.GroupEnd) || !bind(h, "ncclGetErrorString", &a.GetErrorString)) {
            set_error("libnccl lacks a required symbol");
            return CA_ERR_COMM;
        }
        g_nccl = a;
    }
    *api = &g_nccl;
    return CA_OK;
}

int nccl_fail(NcclApi* api, ncclResult_t r, const char* what) {
    set_error("%s: %s", what, api->GetErrorString(r));
    return CA_ERR_COMM;
}

struct Comm {
    int rank = 0, world = 1;
    ncclComm_t nccl = nullptr;     // NULL for a single rank
};

}  // namespace
}  // namespace ca

using namespace ca;

extern "C" {

int ca_comm_unique_id(void* id128) {
    if (!id128) { set_error("id buffer is NULL"); return CA_ERR_NULL; }
    static_assert(sizeof(ncclUniqueId) == 128, "NCCL unique ids are 128 bytes");
    NcclApi* api;
    int rc = nccl_api(&api);
    if (rc) return rc;
    ncclResult_t r = api->GetUniqueId(static_cast<ncclUniqueId*>(id128));
    if (r != ncclSuccess) return nccl_fail(api, r, "ncclGetUniqueId");
    return CA_OK;
}

int ca_comm_init(int32_t rank, int32_t world, const void* id128, void** comm) {
    if (!comm) { set_error("comm is NULL"); return CA_ERR_NULL; }
    *comm = nullptr;
    if (world < 1 || rank < 0 || rank >= world) { set_error("bad rank %d of %d", rank, world); return CA_ERR_BAD_DESC; }
    Comm* c = new Comm;
    c->rank = rank;
    c->world = world;
    if (world > 1) {
        if (!id128) { delete c; set_error("unique id is NULL"); return CA_ERR_NULL; }
        NcclApi* api;
        int rc = nccl_api(&api);
        if (rc) { delete c; return rc; }
        ncclUniqueId id;
        memcpy(&id, id128, sizeof(id));
        ncclResult_t r = api->CommInitRank(&c->nccl, world, id, rank);      // binds to the current device
        if (r != ncclSuccess) { delete c; return nccl_fail(api, r, "ncclCommInitRank"); }
    }
    *comm = c;
    return CA_OK;
}

int ca_comm_destroy(void* comm) {
    if (!comm) return CA_OK;
    Comm* c = static_cast<Comm*>(comm);
    int rc = CA_OK;
    if (c->nccl) {
        NcclApi* api;
        rc = nccl_api(&api);
        if (!rc) {
            ncclResult_t r = api->CommDestroy(c->nccl);
            if (r != ncclSuccess) rc = nccl_fail(api, r, "ncclCommDestroy");
        }
    }
    delete c;
    return rc;
}

int ca_copy_chunks(const ca_chunk_job* jobs, int32_t njobs, void* stream) {
    if (njobs < 0 || njobs > CA_MAX_CHUNK_JOBS) { set_error("njobs=%d outside 0..%d", njobs, CA_MAX_CHUNK_JOBS); return CA_ERR_BAD_DESC; }
    if (njobs == 0) return CA_OK;
    if (!jobs) { set_error("jobs is NULL"); return CA_ERR_NULL; }
    ChunkJobs pack{};
    int64_t most = 0;
    for (int j = 0; j < njobs; ++j) {
        const ca_chunk_job& b = jobs[j];
        if (b.chunk_bytes < 0 || b.nchunks < 0) { set_error("job %d has a negative size", j); return CA_ERR_BAD_DESC; }
        if (b.chunk_bytes > 0 && b.nchunks > 0 && (!b.src || !b.dst)) { set_error("job %d has a NULL buffer", j); return CA_ERR_NULL; }
        pack.job[j] = b;
        most = std::max(most, b.nchunks * ((b.chunk_bytes + kChunkSegment - 1) / kChunkSegment));
    }
    pack.n = njobs;
    if (most == 0) return CA_OK;
    const dim3 grid((unsigned)std::min<int64_t>(most, 148 * 8), (unsigned)njobs);
    copy_chunks_kernel<<<grid, 256, 0, as_stream(stream)>>>(pack);
    CA_CHECK_LAUNCH("chunk copy kernel");
    return CA_OK;
}

int ca_halo_exchange(void* comm, const void* send_left, const void* send_right, void* recv_left, void* recv_right,
                     size_t nbytes, void* stream) {
    if (!comm) { set_error("comm is NULL"); return CA_ERR_NULL; }
    if (nbytes == 0) return CA_OK;
    if (!send_left || !send_right || !recv_left || !recv_right) { set_error("a halo buffer is NULL"); return CA_ERR_NULL; }
    Comm* c = static_cast<Comm*>(comm);
    cudaStream_t st = as_stream(stream);
    if (c->world == 1) {
        // the band is the whole image: its halos are its own wrapped columns
        cudaError_t e = cudaMemcpyAsync(recv_left, send_right, nbytes, cudaMemcpyDeviceToDevice, st);
        if (e == cudaSuccess) e = cudaMemcpyAsync(recv_right, send_left, nbytes, cudaMemcpyDeviceToDevice, st);
        if (e != cudaSuccess) return cuda_fail(e, "halo copy");
        return CA_OK;
    }
    NcclApi* api;
    int rc = nccl_api(&api);
    if (rc) return rc;
    const int left = (c->rank + c->world - 1) % c->world, right = (c->rank + 1) % c->world;
    ncclResult_t r = api->GroupStart();
    if (r != ncclSuccess) return nccl_fail(api, r, "ncclGroupStart");
    // with two ranks both neighbours are the same peer: sends and receives pair up in issue order
    ncclResult_t r1 = api->Send(send_right, nbytes, ncclChar, right, c->nccl, st);
    ncclResult_t r2 = api->Send(send_left, nbytes, ncclChar, left, c->nccl, st);
    ncclResult_t r3 = api->Recv(recv_left, nbytes, ncclChar, left, c->nccl, st);
    ncclResult_t r4 = api->Recv(recv_right, nbytes, ncclChar, right, c->nccl, st);
    r = api->GroupEnd();
    for (ncclResult_t x : {r1, r2, r3, r4, r})
        if (x != ncclSuccess) return nccl_fail(api, x, "halo exchange (ncclSend / ncclRecv)");
    return CA_OK;
}

}  // extern "C"
