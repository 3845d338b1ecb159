// MultiHeadCacheAttention for callers that have no way to hand over a workspace.
//
// pplb200_mhca_forward needs caller-allocated scratch (work counter, tile prefix sums, fp32 split
// partials).  Some callers cannot provide it: an operator that is invoked outside its engine's
// device context has no tmp-buffer pool to borrow from, and a serving process that has already
// committed all device memory to the KV cache (or that forbids raw cudaMalloc next to its own
// caching allocator) cannot safely allocate one either.  For them the scratch lives in a fixed
// array in the library's own device image.  Nothing in this file, or in anything it calls,
// allocates or frees device memory.
#include <cuda_runtime.h>
#include <stdio.h>

#include <mutex>

#include "launch.h"

namespace {

constexpr uint64_t kStaticScratchBytes = 32ull << 20;  // 32 MiB per GPU that loads the library

// Lives in every context that loads this library until the process exits.  In HOST code this name
// is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
void* g_scratch_ptr[kMaxDevices] = {};
bool g_scratch_known[kMaxDevices] = {};

// Device address of the array on the CURRENT device, looked up once per device.
int static_scratch_address(void** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        (void)cudaGetLastError();
        fprintf(stderr, "[ppl_nn_b200] RC_DEVICE_RUNTIME_ERROR: no current CUDA device\n");
        return PPLB200_DEVICE_RUNTIME_ERROR;
    }
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_scratch_known[dev]) {
        void* ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess || ptr == nullptr) {
            (void)cudaGetLastError();
            fprintf(stderr, "[ppl_nn_b200] RC_DEVICE_RUNTIME_ERROR: cudaGetSymbolAddress(static scratch): %s\n",
                    cudaGetErrorString(e));
            return PPLB200_DEVICE_RUNTIME_ERROR;
        }
        g_scratch_ptr[dev] = ptr;
        g_scratch_known[dev] = true;
    }
    *out = g_scratch_ptr[dev];
    return PPLB200_SUCCESS;
}

}  // namespace

extern "C" {

uint64_t pplb200_static_scratch_bytes(void) {
    return kStaticScratchBytes;
}

int pplb200_mhca_forward_noalloc(const pplb200_attn_params* p, const void* query, const void* current_key,
                                 const void* current_value, const int64_t* seqstarts, const int64_t* kvstarts,
                                 const int64_t* cachestarts, const int64_t* start_pos, void* cache, void* scale,
                                 void* attn_output, void* stream) {
    uint64_t need = 0;
    int rc = pplb200_mhca_workspace_size(p, &need);  // validates the params as well
    if (rc != PPLB200_SUCCESS) {
        return rc;
    }
    if (need > kStaticScratchBytes) {
        fprintf(stderr,
                "[ppl_nn_b200] RC_OUT_OF_MEMORY: this call needs %llu bytes of scratch but the built-in scratch "
                "holds %llu; use pplb200_mhca_forward with a caller-allocated workspace\n",
                static_cast<unsigned long long>(need), static_cast<unsigned long long>(kStaticScratchBytes));
        return PPLB200_OUT_OF_MEMORY;
    }
    void* scratch = nullptr;
    rc = static_scratch_address(&scratch);
    if (rc != PPLB200_SUCCESS) {
        return rc;
    }
    // The kernels receive the looked-up device address.  The planning kernel of every call resets the
    // work counter and the status word; everything else in the scratch is written before it is read.
    return pplb200_mhca_forward(p, query, current_key, current_value, seqstarts, kvstarts, cachestarts, start_pos,
                                cache, scale, scratch, kStaticScratchBytes, attn_output, stream);
}

int pplb200_static_scratch_status(void* stream, uint32_t* status) {
    if (!status) {
        return PPLB200_NOT_FOUND;
    }
    void* scratch = nullptr;
    const int rc = static_scratch_address(&scratch);
    if (rc != PPLB200_SUCCESS) {
        return rc;
    }
    return pplb200_mhca_device_status(scratch, stream, status);
}

}  // extern "C"
