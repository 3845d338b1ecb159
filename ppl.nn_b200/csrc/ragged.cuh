// Device helpers shared by the token-streaming kernels (append, gather, rotary embedding): the warp-wide
// lookup of the sequence that owns a token, and the walk over (token, chunk of 32 groups) work items.
#pragma once

#include "common.cuh"

namespace pplb200 {

// The segment b in [0, n) that holds x: starts[b] <= x < starts[b + 1] (starts has n + 1 non-decreasing
// entries and starts[0] <= x < starts[n]); the largest such b, so empty segments are skipped.  All 32
// lanes call it with the same arguments: each round probes 32 pivots at once, so 1024 segments take two
// dependent loads instead of ten.
__device__ __forceinline__ int32_t warp_find_segment(const int64_t* __restrict__ starts, int32_t n, int64_t x,
                                                     int lane) {
    int32_t lo = 0, hi = n;  // answer in [lo, hi)
    while (hi - lo > 1) {
        const int32_t step = (hi - lo + 31) >> 5;
        const int64_t piv = static_cast<int64_t>(lo) + static_cast<int64_t>(lane + 1) * step;
        const bool le = piv < hi && starts[piv] <= x;  // true for a prefix of the lanes
        const int c = __popc(__ballot_sync(0xffffffffu, le));
        const int64_t nlo = static_cast<int64_t>(lo) + static_cast<int64_t>(c) * step;
        hi = nlo + step < hi ? static_cast<int32_t>(nlo + step) : hi;
        lo = static_cast<int32_t>(nlo);
    }
    return lo;
}

constexpr int kChunks = 4;  // 32-group chunks per warp item: 2 KB of fp16 in flight per warp during the lookup

// Work items of a warp: (token, run of kChunks chunks of 32 groups), walked without divisions in the loop.
struct WarpItems {
    int64_t tok;
    int32_t chunk;
    int64_t step_tok;
    int32_t step_chunk;
    int32_t chunks_per_token;

    __device__ __forceinline__ explicit WarpItems(int32_t groups_per_token, int32_t chunks_per_item = kChunks) {
        chunks_per_token = (groups_per_token + 32 * chunks_per_item - 1) / (32 * chunks_per_item);  // items per token
        const int64_t warp_id = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
        const int64_t warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
        tok = warp_id / chunks_per_token;
        chunk = static_cast<int32_t>(warp_id - tok * chunks_per_token);
        step_tok = warps / chunks_per_token;
        step_chunk = static_cast<int32_t>(warps - step_tok * chunks_per_token);
    }
    __device__ __forceinline__ void next() {
        tok += step_tok;
        chunk += step_chunk;
        if (chunk >= chunks_per_token) {
            chunk -= chunks_per_token;
            ++tok;
        }
    }
};

// head_dim is 64 or 128, so a head has 8 or 16 groups: shifts instead of divisions
__device__ __forceinline__ void split_group(int32_t g, int32_t groups_per_tensor_row, int group_shift, int& kv,
                                            int& head, int& grp) {
    kv = g >= groups_per_tensor_row ? 1 : 0;
    const int32_t r2 = g - kv * groups_per_tensor_row;
    head = r2 >> group_shift;
    grp = r2 & ((1 << group_shift) - 1);
}

}  // namespace pplb200
