// KeyValueCache kernels: INT8 group quantise-and-append, and the dequantising gather that produces
// the operator's key/value outputs.  Both are pure streaming kernels (HBM-bound, a few MB per call):
// one thread owns one quantisation group of 8 channels = one 128-bit load of halves, one 64-bit
// store of codes and one 16-bit store of the scale, so a warp moves 512 B in and 320 B out fully
// coalesced.
#include "common.cuh"
#include "launch.h"

namespace pplb200 {

// the segment b in [0, n) that holds x: starts[b] <= x < starts[b + 1]   (starts has n + 1
// non-decreasing entries and starts[0] <= x < starts[n])
__device__ __forceinline__ int64_t find_segment(const int64_t* __restrict__ starts, int64_t n, int64_t x) {
    int64_t lo = 0, hi = n;  // answer in [lo, hi)
    while (hi - lo > 1) {
        const int64_t mid = (lo + hi) >> 1;
        if (starts[mid] <= x) {
            lo = mid;
        } else {
            hi = mid;
        }
    }
    return lo;  // the largest b with starts[b] <= x, so empty segments are skipped
}

__global__ void __launch_bounds__(256)
kv_append_i8g8_kernel(const __half* __restrict__ cur_k, const __half* __restrict__ cur_v,
                      const int64_t* __restrict__ seqstarts, const int64_t* __restrict__ cachestarts,
                      const int64_t* __restrict__ start_pos, int8_t* __restrict__ cache, __half* __restrict__ scale,
                      CacheGeom geom, int64_t batch, int64_t total_tokens, int num_kv_heads, int head_dim) {
    const int groups_per_head = head_dim >> 3;
    const int64_t groups_per_tensor_row = static_cast<int64_t>(num_kv_heads) * groups_per_head;
    const int64_t groups_per_token = 2 * groups_per_tensor_row;
    const int64_t total = total_tokens * groups_per_token;
    for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t tok = idx / groups_per_token;
        const int64_t r = idx - tok * groups_per_token;
        const int kv = r >= groups_per_tensor_row ? 1 : 0;
        const int64_t r2 = r - kv * groups_per_tensor_row;
        const int head = static_cast<int>(r2 / groups_per_head);
        const int grp = static_cast<int>(r2 - static_cast<int64_t>(head) * groups_per_head);

        const __half* src = (kv ? cur_v : cur_k) + (tok * num_kv_heads + head) * head_dim + grp * 8;
        const uint4 in = *reinterpret_cast<const uint4*>(src);

        uint2 codes;
        __half s16;
        quant_group8(in, codes, s16);

        const int64_t b = find_segment(seqstarts, batch, tok);
        const int64_t row = cache_row(geom, cachestarts, b, start_pos[b] + (tok - seqstarts[b]));
        const int64_t off = cache_offset(geom, row, kv, head);
        *reinterpret_cast<uint2*>(cache + off + grp * 8) = codes;
        scale[(off >> 3) + grp] = s16;
    }
}

__global__ void __launch_bounds__(256)
kv_gather_dequant_kernel(const int64_t* __restrict__ kvstarts, const int64_t* __restrict__ cachestarts,
                         const int8_t* __restrict__ cache, const __half* __restrict__ scale,
                         __half* __restrict__ key_out, __half* __restrict__ value_out, CacheGeom geom, int64_t batch,
                         int64_t total_kv, int num_kv_heads, int head_dim) {
    const int groups_per_head = head_dim >> 3;
    const int64_t groups_per_tensor_row = static_cast<int64_t>(num_kv_heads) * groups_per_head;
    const int64_t groups_per_token = 2 * groups_per_tensor_row;
    const int64_t total = total_kv * groups_per_token;
    for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t j = idx / groups_per_token;
        const int64_t r = idx - j * groups_per_token;
        const int kv = r >= groups_per_tensor_row ? 1 : 0;
        const int64_t r2 = r - kv * groups_per_tensor_row;
        const int head = static_cast<int>(r2 / groups_per_head);
        const int grp = static_cast<int>(r2 - static_cast<int64_t>(head) * groups_per_head);

        const int64_t b = find_segment(kvstarts, batch, j);
        const int64_t row = cache_row(geom, cachestarts, b, j - kvstarts[b]);
        const int64_t off = cache_offset(geom, row, kv, head);
        const uint2 codes = *reinterpret_cast<const uint2*>(cache + off + grp * 8);
        const float s = __half2float(scale[(off >> 3) + grp]);

        uint4 out;
        __half2* o2 = reinterpret_cast<__half2*>(&out);
        const uint32_t w[2] = {codes.x, codes.y};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c0 = static_cast<int8_t>((w[i >> 1] >> (16 * (i & 1))) & 0xffu);
            const int c1 = static_cast<int8_t>((w[i >> 1] >> (16 * (i & 1) + 8)) & 0xffu);
            o2[i] = __floats2half2_rn(static_cast<float>(c0) * s, static_cast<float>(c1) * s);
        }
        __half* dst = (kv ? value_out : key_out) + (j * num_kv_heads + head) * head_dim + grp * 8;
        *reinterpret_cast<uint4*>(dst) = out;
    }
}

static int grid_for(int64_t work_items, int threads, int sm_count) {
    int64_t blocks = (work_items + threads - 1) / threads;
    const int64_t cap = static_cast<int64_t>(sm_count) * 16;  // grid-stride beyond 16 resident waves of CTAs
    if (blocks > cap) {
        blocks = cap;
    }
    return blocks < 1 ? 1 : static_cast<int>(blocks);
}

int launch_kv_append(const pplb200_attn_params& p, const CacheGeom& geom, const void* cur_k, const void* cur_v,
                     const int64_t* seqstarts, const int64_t* cachestarts, const int64_t* start_pos, void* cache,
                     void* scale, int sm_count, cudaStream_t stream) {
    if (p.total_tokens <= 0) {
        return PPLB200_SUCCESS;
    }
    const int64_t work = p.total_tokens * 2 * p.num_kv_heads * (p.head_dim / 8);
    const int grid = grid_for(work, 256, sm_count);
    KernelTimer timer(PPLB200_KERNEL_APPEND, stream);
    kv_append_i8g8_kernel<<<grid, 256, 0, stream>>>(
        static_cast<const __half*>(cur_k), static_cast<const __half*>(cur_v), seqstarts, cachestarts, start_pos,
        static_cast<int8_t*>(cache), static_cast<__half*>(scale), geom, p.batch, p.total_tokens, p.num_kv_heads,
        p.head_dim);
    return check_launch("kv_append_i8g8_kernel");
}

int launch_kv_gather_dequant(const pplb200_attn_params& p, const CacheGeom& geom, const int64_t* kvstarts,
                             const int64_t* cachestarts, const void* cache, const void* scale, int64_t total_kv,
                             void* key_out, void* value_out, int sm_count, cudaStream_t stream) {
    if (total_kv <= 0) {
        return PPLB200_SUCCESS;
    }
    const int64_t work = total_kv * 2 * p.num_kv_heads * (p.head_dim / 8);
    const int grid = grid_for(work, 256, sm_count);
    kv_gather_dequant_kernel<<<grid, 256, 0, stream>>>(
        kvstarts, cachestarts, static_cast<const int8_t*>(cache), static_cast<const __half*>(scale),
        static_cast<__half*>(key_out), static_cast<__half*>(value_out), geom, p.batch, total_kv, p.num_kv_heads,
        p.head_dim);
    return check_launch("kv_gather_dequant_kernel");
}

}  // namespace pplb200
