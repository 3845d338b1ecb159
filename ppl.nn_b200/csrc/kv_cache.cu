// KeyValueCache kernels: INT8 group quantise-and-append, and the dequantising gather that produces
// the operator's key/value outputs.  Both are pure streaming kernels (HBM-bound).  A warp owns 32
// consecutive quantisation groups of ONE token, kChunks times over: a lane's group is one 128-bit load of
// halves, one 64-bit store of codes and one 16-bit store of the scale, so each chunk moves 512 B in and
// 320 B out fully coalesced.  The sequence that owns the token is looked up once per warp item, by all
// lanes together, while the item's kChunks loads are in flight.
#include "common.cuh"
#include "launch.h"
#include "ragged.cuh"

namespace pplb200 {

// FAST: every warp item lies wholly inside the K part or the V part of a token row (the row of one tensor is
// a multiple of 32 * kChunks groups) and a cache row holds K and V of all heads back to back.  The source
// and destination of an item are then one base address per warp plus the lane's offset: no bounds tests,
// no per-lane choice between the two tensors, no group index arithmetic.
template <bool FAST>
__global__ void __launch_bounds__(256)
kv_append_i8g8_kernel(const __half* __restrict__ cur_k, const __half* __restrict__ cur_v,
                      const int64_t* __restrict__ seqstarts, const int64_t* __restrict__ cachestarts,
                      const int64_t* __restrict__ start_pos, int8_t* __restrict__ cache, __half* __restrict__ scale,
                      CacheGeom geom, int32_t batch, int32_t first_seq, int64_t total_tokens, int64_t max_tokens,
                      uint32_t* __restrict__ status, int num_kv_heads, int head_dim) {
    grid_launch_dependents();
    grid_dependency_wait();
    // tokens of the sequences before first_seq are not this launch's business (the decode kernel appends the
    // new tokens of the decode sequences itself)
    const int64_t tok_begin = first_seq > 0 ? seqstarts[first_seq] : 0;
    total_tokens -= tok_begin;
    cur_k += tok_begin * num_kv_heads * head_dim;
    cur_v += tok_begin * num_kv_heads * head_dim;
    const int lane = threadIdx.x & 31;
    const int group_shift = head_dim == 128 ? 4 : 3;
    const int32_t groups_per_tensor_row = num_kv_heads << group_shift;
    const int32_t groups_per_token = 2 * groups_per_tensor_row;
    const int32_t row_elems = num_kv_heads * head_dim;  // one token row of K (or V)
    // a cache row that holds K and V of all heads back to back: the offset of a group is its index
    const bool dense_row = geom.stride_h == head_dim && geom.stride_kv == row_elems;
    if constexpr (FAST) {
        const int32_t items_per_tensor = groups_per_tensor_row / (32 * kChunks);
        for (WarpItems it(groups_per_token); it.tok < total_tokens; it.next()) {
            const bool is_v = it.chunk >= items_per_tensor;  // warp-uniform
            const int32_t g0 = it.chunk * (32 * kChunks);    // first group of the item within the token row
            const __half* src = (is_v ? cur_v : cur_k) + it.tok * row_elems +
                                (g0 - (is_v ? groups_per_tensor_row : 0)) * 8 + lane * 8;
            uint4 in[kChunks];
#pragma unroll
            for (int c = 0; c < kChunks; ++c) {
                in[c] = *reinterpret_cast<const uint4*>(src + c * 256);
            }
            const int64_t tok = it.tok + tok_begin;
            const int32_t b = warp_find_segment(seqstarts, batch, tok, lane);
            const int64_t row = cache_row(geom, cachestarts, b, start_pos[b] + (tok - seqstarts[b]));
            if (!cache_row_ok(row, max_tokens)) {  // a wrong index tensor: flag it and leave the cache alone
                if (lane == 0 && status != nullptr) {
                    atomicOr(status, kDevRowOutOfRange);
                }
                continue;
            }
            const int64_t row_off = row * geom.stride_s + geom.layer_idx * geom.stride_l + static_cast<int64_t>(g0) * 8;
            int8_t* c_dst = cache + row_off + lane * 8;
            __half* s_dst = scale + (row_off >> 3) + lane;
#pragma unroll
            for (int c = 0; c < kChunks; ++c) {
                uint2 codes;
                __half s16;
                quant_group8(in[c], codes, s16);
                *reinterpret_cast<uint2*>(c_dst + c * 256) = codes;
                s_dst[c * 32] = s16;
            }
        }
    } else {
        for (WarpItems it(groups_per_token); it.tok < total_tokens; it.next()) {
            // the payload loads go out before the lookups, which then overlap with them; the 64-bit part of every
            // address is formed once per token, the rest is 32-bit arithmetic on the group index
            const __half* k_tok = cur_k + it.tok * row_elems;
            const __half* v_tok = cur_v + it.tok * row_elems;
            uint4 in[kChunks];
#pragma unroll
            for (int c = 0; c < kChunks; ++c) {
                const int32_t g = (it.chunk * kChunks + c) * 32 + lane;
                in[c] = make_uint4(0u, 0u, 0u, 0u);
                if (g < groups_per_token) {
                    // groups of a token row are laid out exactly like its channels: group r2 = channels 8 r2 ..
                    const bool is_v = g >= groups_per_tensor_row;
                    const int32_t r2 = g - (is_v ? groups_per_tensor_row : 0);
                    in[c] = *reinterpret_cast<const uint4*>((is_v ? v_tok : k_tok) + r2 * 8);
                }
            }
            const int64_t tok = it.tok + tok_begin;
            const int32_t b = warp_find_segment(seqstarts, batch, tok, lane);
            const int64_t row = cache_row(geom, cachestarts, b, start_pos[b] + (tok - seqstarts[b]));
            if (!cache_row_ok(row, max_tokens)) {  // a wrong index tensor: flag it and leave the cache alone
                if (lane == 0 && status != nullptr) {
                    atomicOr(status, kDevRowOutOfRange);
                }
                continue;
            }
            const int64_t row_off = row * geom.stride_s + geom.layer_idx * geom.stride_l;
            int8_t* c_row = cache + row_off;
            __half* s_row = scale + (row_off >> 3);
#pragma unroll
            for (int c = 0; c < kChunks; ++c) {
                const int32_t g = (it.chunk * kChunks + c) * 32 + lane;
                uint2 codes;
                __half s16;
                quant_group8(in[c], codes, s16);
                if (g < groups_per_token) {
                    int64_t off = static_cast<int64_t>(g) * 8;  // K then V of all heads back to back (layout 0)
                    if (!dense_row) {
                        int kv, head, grp;
                        split_group(g, groups_per_tensor_row, group_shift, kv, head, grp);
                        off = kv * geom.stride_kv + head * geom.stride_h + grp * 8;
                    }
                    *reinterpret_cast<uint2*>(c_row + off) = codes;
                    s_row[off >> 3] = s16;
                }
            }
        }
    }
}

__global__ void __launch_bounds__(256)
kv_gather_dequant_kernel(const int64_t* __restrict__ kvstarts, const int64_t* __restrict__ cachestarts,
                         const int8_t* __restrict__ cache, const __half* __restrict__ scale,
                         __half* __restrict__ key_out, __half* __restrict__ value_out, CacheGeom geom, int32_t batch,
                         int64_t total_kv, int64_t max_tokens, int num_kv_heads, int head_dim) {
    const int lane = threadIdx.x & 31;
    const int group_shift = head_dim == 128 ? 4 : 3;
    const int32_t groups_per_tensor_row = num_kv_heads << group_shift;
    const int32_t groups_per_token = 2 * groups_per_tensor_row;
    for (WarpItems it(groups_per_token); it.tok < total_kv; it.next()) {
        const int64_t j = it.tok;
        const int32_t b = warp_find_segment(kvstarts, batch, j, lane);
        const int64_t row = cache_row(geom, cachestarts, b, j - kvstarts[b]);
        const bool row_ok = cache_row_ok(row, max_tokens);  // a row outside the cache reads as zeros
        uint2 codes[kChunks];
        uint16_t sbits[kChunks];
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
            const int32_t g = (it.chunk * kChunks + c) * 32 + lane;
            codes[c] = make_uint2(0u, 0u);
            sbits[c] = 0;
            if (g < groups_per_token && row_ok) {
                int kv, head, grp;
                split_group(g, groups_per_tensor_row, group_shift, kv, head, grp);
                const int64_t off = cache_offset(geom, row, kv, head);
                codes[c] = *reinterpret_cast<const uint2*>(cache + off + grp * 8);
                sbits[c] = reinterpret_cast<const uint16_t*>(scale)[(off >> 3) + grp];
            }
        }
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
            const int32_t g = (it.chunk * kChunks + c) * 32 + lane;
            if (g >= groups_per_token) {
                continue;
            }
            int kv, head, grp;
            split_group(g, groups_per_tensor_row, group_shift, kv, head, grp);
            const float sf = __half2float(__ushort_as_half(sbits[c]));
            uint4 out;
            __half2* o2 = reinterpret_cast<__half2*>(&out);
            const uint32_t w[2] = {codes[c].x, codes[c].y};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int c0 = static_cast<int8_t>((w[i >> 1] >> (16 * (i & 1))) & 0xffu);
                const int c1 = static_cast<int8_t>((w[i >> 1] >> (16 * (i & 1) + 8)) & 0xffu);
                o2[i] = __floats2half2_rn(static_cast<float>(c0) * sf, static_cast<float>(c1) * sf);
            }
            __half* dst = (kv ? value_out : key_out) + (j * num_kv_heads + head) * head_dim + grp * 8;
            *reinterpret_cast<uint4*>(dst) = out;
        }
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
                     void* scale, int64_t first_seq, uint32_t* status, int sm_count, cudaStream_t stream) {
    // sequences before first_seq are decode sequences with one token each, so this many tokens remain
    const int64_t tokens = p.total_tokens - first_seq;
    if (tokens <= 0 || first_seq >= p.batch) {
        return PPLB200_SUCCESS;
    }
    const int64_t items_per_token = (2 * p.num_kv_heads * (p.head_dim / 8) + 32 * kChunks - 1) / (32 * kChunks);
    const int grid = grid_for(tokens * items_per_token * 32, 256, sm_count);  // a warp per item
    KernelTimer timer(PPLB200_KERNEL_APPEND, stream);
    const int64_t groups_per_tensor_row = static_cast<int64_t>(p.num_kv_heads) * (p.head_dim / 8);
    const bool fast = groups_per_tensor_row % (32 * kChunks) == 0 && geom.stride_h == p.head_dim &&
                      geom.stride_kv == static_cast<int64_t>(p.num_kv_heads) * p.head_dim;
    auto kernel = fast ? kv_append_i8g8_kernel<true> : kv_append_i8g8_kernel<false>;
    launch_dependent(kernel, dim3(grid), dim3(256), 0, stream, static_cast<const __half*>(cur_k),
                     static_cast<const __half*>(cur_v), seqstarts, cachestarts, start_pos, static_cast<int8_t*>(cache),
                     static_cast<__half*>(scale), geom, static_cast<int32_t>(p.batch), static_cast<int32_t>(first_seq),
                     p.total_tokens, p.max_tokens, status, p.num_kv_heads, p.head_dim);
    return check_launch("kv_append_i8g8_kernel");
}

int launch_kv_gather_dequant(const pplb200_attn_params& p, const CacheGeom& geom, const int64_t* kvstarts,
                             const int64_t* cachestarts, const void* cache, const void* scale, int64_t total_kv,
                             void* key_out, void* value_out, int sm_count, cudaStream_t stream) {
    if (total_kv <= 0) {
        return PPLB200_SUCCESS;
    }
    const int64_t items_per_token = (2 * p.num_kv_heads * (p.head_dim / 8) + 32 * kChunks - 1) / (32 * kChunks);
    const int grid = grid_for(total_kv * items_per_token * 32, 256, sm_count);  // a warp per item
    kv_gather_dequant_kernel<<<grid, 256, 0, stream>>>(
        kvstarts, cachestarts, static_cast<const int8_t*>(cache), static_cast<const __half*>(scale),
        static_cast<__half*>(key_out), static_cast<__half*>(value_out), geom, static_cast<int32_t>(p.batch), total_kv,
        p.max_tokens, p.num_kv_heads, p.head_dim);
    return check_launch("kv_gather_dequant_kernel");
}

}  // namespace pplb200
