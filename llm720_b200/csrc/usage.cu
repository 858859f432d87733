// Expert-usage histogram on the device.  Replaces the tracker's per-step loop
// of the reference (llm/utils/experts/tracking.py:96-100: the [B,S,H,k] index
// tensor is copied to the host and every element increments a Python Counter)
// with one pass of atomic increments over the ids where they already are.
#include <cstdio>

#include "common.cuh"
#include "kernels.h"

namespace peer { void set_global_error(const char* msg); }

namespace {

__global__ void usage_histogram_kernel(const int64_t* __restrict__ ids, int64_t n, unsigned long long* __restrict__ counts,
                                       int64_t num_experts, unsigned long long* __restrict__ dropped) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const int64_t id = ids[i];
        if (id >= 0 && id < num_experts) atomicAdd(counts + id, 1ULL);
        else if (dropped) atomicAdd(dropped, 1ULL);       // never dereferenced: counted instead
    }
}

}  // namespace

extern "C" int peer_usage_histogram(const int64_t* ids, int64_t n_ids, int64_t* counts, int64_t num_experts,
                                    int64_t* dropped, void* stream) {
    if (n_ids == 0) return PEER_OK;
    if (!ids || !counts || n_ids < 0 || num_experts <= 0) {
        peer::set_global_error("peer_usage_histogram: null pointer or non-positive size");
        return PEER_ERR_INVALID_ARG;
    }
    int64_t blocks = (n_ids + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    usage_histogram_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        ids, n_ids, reinterpret_cast<unsigned long long*>(counts), num_experts,
        reinterpret_cast<unsigned long long*>(dropped));
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        char buf[256];
        snprintf(buf, sizeof buf, "peer_usage_histogram: %s", cudaGetErrorString(e));
        peer::set_global_error(buf);
        return PEER_ERR_CUDA;
    }
    return PEER_OK;
}
