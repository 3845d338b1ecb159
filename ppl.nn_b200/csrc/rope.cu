// Rotary position embedding for ragged batches (opmx.dynamic_batching.RotaryPositionEmbedding), alone and
// fused with the INT8 quantise-and-append of the KV cache.  HBM-bound streaming kernels with the same work
// split as the append kernel: a warp owns chunks of 32 groups of 8 channels of ONE token.
//
// Convention (the reference keeps the arithmetic in an external library; this is the restatement used by
// the CPU oracle as well): channel pairs (2j, 2j+1), j < rotary_dim / 2, are rotated by the angle
//   pos_eff * inv_freq[j],   inv_freq[j] = theta_eff ^ (-2j / rotary_dim)   (evaluated in double, kept as float)
//   pos = start_pos[b] + index of the token in its sequence
//   scaling none:    pos_eff = pos,                   theta_eff = theta
//   scaling linear:  pos_eff = pos / scaling_factor,  theta_eff = theta
//   scaling dynamic: pos_eff = pos; with L = start_pos[b] + seqlen[b] > max_position_embeddings:
//                    theta_eff = theta * (scaling_factor * L / max_position_embeddings - (scaling_factor - 1))
//                                        ^ (rotary_dim / (rotary_dim - 2))
// in float: angle = pos_eff * inv_freq[j], (sin, cos) = sincosf(angle),
//   out[2j] = x[2j] * cos - x[2j+1] * sin,   out[2j+1] = x[2j] * sin + x[2j+1] * cos,  rounded to fp16 once.
// A pair never straddles a group of 8 channels, which is what makes the fusion with the group quantiser a
// register-only affair: the fused kernel quantises the fp16-rounded rotated key, so its cache rows are
// bit-identical to running the two operators one after the other.
#include <math.h>

#include "common.cuh"
#include "launch.h"
#include "ragged.cuh"

namespace pplb200 {

namespace {

struct RopeDev {
    const float* table;     // [rows][rotary_dim / 2] inverse frequencies; rows = batch (dynamic) or 1
    int32_t table_per_seq;  // 1: one row per sequence
    int32_t half_rot;       // rotary_dim / 2
    int32_t linear;         // divide the position by scaling_factor
    float scaling_factor;
};

// One row of inverse frequencies per sequence (dynamic scaling) or a single row.
__global__ void rope_table_kernel(const int64_t* __restrict__ seqstarts, const int64_t* __restrict__ start_pos,
                                  float* __restrict__ table, int32_t rows, int32_t half_rot, int32_t dynamic,
                                  double theta, double scaling_factor, int32_t max_position_embeddings) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int32_t row = blockIdx.x;
    if (row >= rows) {
        return;
    }
    double theta_eff = theta;
    if (dynamic) {
        const double len = static_cast<double>(start_pos[row] + (seqstarts[row + 1] - seqstarts[row]));
        if (len > static_cast<double>(max_position_embeddings)) {
            const double rot = 2.0 * half_rot;
            theta_eff = theta * pow(scaling_factor * len / max_position_embeddings - (scaling_factor - 1.0), rot / (rot - 2.0));
        }
    }
    for (int32_t j = threadIdx.x; j < half_rot; j += blockDim.x) {
        table[static_cast<int64_t>(row) * half_rot + j] =
            static_cast<float>(pow(theta_eff, -2.0 * j / (2.0 * half_rot)));
    }
}

constexpr int kRopeChunks = 8;  // chunks of 32 groups per warp item: the sines and cosines are shared by all of them

// A lane always works on the same group of channels of whatever head it is looking at (32 is a multiple
// of the groups per head), so the four (sin, cos) pairs of its channels are computed once per token.
struct LaneRotation {
    float sn[4], cs[4];
    bool on[4];
    __device__ __forceinline__ void init(int grp, float pos_eff, const float* __restrict__ inv_freq, int half_rot) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int j = grp * 4 + i;  // pair index inside the head
            on[i] = j < half_rot;
            sn[i] = 0.0f;
            cs[i] = 1.0f;
            if (on[i]) {
                sincosf(__fmul_rn(pos_eff, inv_freq[j]), &sn[i], &cs[i]);
            }
        }
    }
    __device__ __forceinline__ uint4 apply(uint4 in) const {
        const __half2* h2 = reinterpret_cast<const __half2*>(&in);
        uint4 out = in;
        __half2* o2 = reinterpret_cast<__half2*>(&out);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (on[i]) {
                const float2 x = __half22float2(h2[i]);
                const float a = __fsub_rn(__fmul_rn(x.x, cs[i]), __fmul_rn(x.y, sn[i]));
                const float b = __fadd_rn(__fmul_rn(x.x, sn[i]), __fmul_rn(x.y, cs[i]));
                o2[i] = __floats2half2_rn(a, b);
            }
        }
        return out;
    }
};

struct RopeArgs {
    const __half* query;
    const __half* key;
    const __half* value;        // fused only
    __half* rotated_query;
    __half* rotated_key;        // may be null in the fused kernel: the rotated key then exists in the cache only
    const int64_t* seqstarts;
    const int64_t* start_pos;
    const int64_t* cachestarts;  // fused only
    int8_t* cache;               // fused only
    __half* scale;               // fused only
    CacheGeom geom;              // fused only
    RopeDev rope;
    int32_t batch;
    int64_t total_tokens;
    int64_t max_tokens;          // fused only: rows of the cache
    int32_t num_heads;
    int32_t num_kv_heads;
    int32_t head_dim;
    int32_t bypass_key;
};

// FUSED = false: groups of a token = [query heads | key heads]; rotate and store.
// FUSED = true:  groups of a token = [query heads | key heads | value heads]; the key groups are rotated,
//                rounded to fp16 (stored if rotated_key is given), quantised and appended; the value groups are
//                quantised and appended.
template <bool FUSED>
__global__ void __launch_bounds__(256) rope_kernel(const RopeArgs a) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int lane = threadIdx.x & 31;
    const int group_shift = a.head_dim == 128 ? 4 : 3;
    const int32_t q_groups = a.num_heads << group_shift;
    const int32_t k_groups = a.num_kv_heads << group_shift;
    const int32_t groups_per_token = q_groups + k_groups + (FUSED ? k_groups : 0);
    const int grp = lane & ((1 << group_shift) - 1);  // the same for every chunk: 32 is a multiple of the groups per head
    for (WarpItems it(groups_per_token, kRopeChunks); it.tok < a.total_tokens; it.next()) {
        uint4 in[kRopeChunks];
#pragma unroll
        for (int c = 0; c < kRopeChunks; ++c) {
            const int32_t g = (it.chunk * kRopeChunks + c) * 32 + lane;
            in[c] = make_uint4(0u, 0u, 0u, 0u);
            if (g < groups_per_token) {
                const __half* src;
                if (g < q_groups) {
                    src = a.query + (it.tok * q_groups + g) * 8;
                } else if (g < q_groups + k_groups) {
                    src = a.key + (it.tok * k_groups + (g - q_groups)) * 8;
                } else {
                    src = a.value + (it.tok * k_groups + (g - q_groups - k_groups)) * 8;
                }
                in[c] = *reinterpret_cast<const uint4*>(src);
            }
        }
        const int32_t b = warp_find_segment(a.seqstarts, a.batch, it.tok, lane);
        const int64_t pos = a.start_pos[b] + (it.tok - a.seqstarts[b]);
        float pos_eff = static_cast<float>(pos);
        if (a.rope.linear) {
            pos_eff = __fdiv_rn(pos_eff, a.rope.scaling_factor);
        }
        const float* inv_freq = a.rope.table + (a.rope.table_per_seq ? static_cast<int64_t>(b) * a.rope.half_rot : 0);
        int64_t row = 0;
        bool row_ok = false;  // a row outside the cache (a wrong index tensor) is not written
        if (FUSED) {
            row = cache_row(a.geom, a.cachestarts, b, pos);
            row_ok = cache_row_ok(row, a.max_tokens);
        }
        LaneRotation rotn;
        rotn.init(grp, pos_eff, inv_freq, a.rope.half_rot);
#pragma unroll
        for (int c = 0; c < kRopeChunks; ++c) {
            const int32_t g = (it.chunk * kRopeChunks + c) * 32 + lane;
            if (g >= groups_per_token) {
                continue;
            }
            if (g < q_groups) {
                const uint4 r = rotn.apply(in[c]);
                *reinterpret_cast<uint4*>(a.rotated_query + (it.tok * q_groups + g) * 8) = r;
                continue;
            }
            const bool is_key = g < q_groups + k_groups;
            const int32_t gk = g - q_groups - (is_key ? 0 : k_groups);
            uint4 r = in[c];
            if (is_key) {
                if (!a.bypass_key) {
                    r = rotn.apply(in[c]);
                }
                if (a.rotated_key && (a.rotated_key != a.key || !a.bypass_key)) {
                    *reinterpret_cast<uint4*>(a.rotated_key + (it.tok * k_groups + gk) * 8) = r;
                }
            }
            if (FUSED && row_ok) {
                uint2 codes;
                __half s16;
                quant_group8(r, codes, s16);
                const int64_t off = cache_offset(a.geom, row, is_key ? 0 : 1, gk >> group_shift);
                *reinterpret_cast<uint2*>(a.cache + off + grp * 8) = codes;
                a.scale[(off >> 3) + grp] = s16;
            }
        }
    }
}

int grid_for_items(int64_t tokens, int32_t groups_per_token, int sm_count) {
    const int64_t items_per_token = (groups_per_token + 32 * kRopeChunks - 1) / (32 * kRopeChunks);
    int64_t blocks = (tokens * items_per_token * 32 + 255) / 256;
    const int64_t cap = static_cast<int64_t>(sm_count) * 16;
    blocks = blocks > cap ? cap : blocks;
    return blocks < 1 ? 1 : static_cast<int>(blocks);
}

}  // namespace

uint64_t rope_workspace_bytes(const pplb200_rope_params& p) {
    const int rot = p.rotary_dim == 0 ? p.head_dim : p.rotary_dim;
    const int64_t rows = p.scaling_type == 2 ? (p.batch > 0 ? p.batch : 1) : 1;
    return (static_cast<uint64_t>(rows) * (rot / 2) * 4 + 255) / 256 * 256;
}

int launch_rope(const pplb200_rope_params& p, const pplb200_attn_params* append, const CacheGeom* geom,
                const void* query, const void* key, const void* value, const int64_t* seqstarts,
                const int64_t* start_pos, const int64_t* cachestarts, void* workspace, void* rotated_query,
                void* rotated_key, void* cache, void* scale, int sm_count, cudaStream_t stream) {
    if (p.total_tokens <= 0 || p.batch <= 0) {
        return PPLB200_SUCCESS;
    }
    const int rot = p.rotary_dim == 0 ? p.head_dim : p.rotary_dim;
    const int32_t rows = p.scaling_type == 2 ? static_cast<int32_t>(p.batch) : 1;
    float* table = static_cast<float*>(workspace);
    launch_dependent(rope_table_kernel, dim3(static_cast<unsigned>(rows)), dim3(64), 0, stream, seqstarts, start_pos, table,
                     rows, static_cast<int32_t>(rot / 2), static_cast<int32_t>(p.scaling_type == 2 ? 1 : 0),
                     static_cast<double>(p.theta), static_cast<double>(p.scaling_factor), p.max_position_embeddings);
    int rc = check_launch("rope_table_kernel");
    if (rc != PPLB200_SUCCESS) {
        return rc;
    }
    RopeArgs a;
    memset(&a, 0, sizeof(a));
    a.query = static_cast<const __half*>(query);
    a.key = static_cast<const __half*>(key);
    a.value = static_cast<const __half*>(value);
    a.rotated_query = static_cast<__half*>(rotated_query);
    a.rotated_key = static_cast<__half*>(rotated_key);
    a.seqstarts = seqstarts;
    a.start_pos = start_pos;
    a.cachestarts = cachestarts;
    a.cache = static_cast<int8_t*>(cache);
    a.scale = static_cast<__half*>(scale);
    if (geom) {
        a.geom = *geom;
    }
    a.rope.table = table;
    a.rope.table_per_seq = p.scaling_type == 2 ? 1 : 0;
    a.rope.half_rot = rot / 2;
    a.rope.linear = p.scaling_type == 1 ? 1 : 0;
    a.rope.scaling_factor = p.scaling_factor;
    a.batch = static_cast<int32_t>(p.batch);
    a.total_tokens = p.total_tokens;
    a.num_heads = p.num_heads;
    a.num_kv_heads = p.num_kv_heads;
    a.head_dim = p.head_dim;
    a.bypass_key = p.bypass_key;
    a.max_tokens = append ? append->max_tokens : 0;
    const int32_t groups = (p.num_heads + p.num_kv_heads * (append ? 2 : 1)) * (p.head_dim / 8);
    const int grid = grid_for_items(p.total_tokens, groups, sm_count);
    KernelTimer timer(PPLB200_KERNEL_APPEND, stream);
    if (append) {
        launch_dependent(rope_kernel<true>, dim3(grid), dim3(256), 0, stream, a);
    } else {
        launch_dependent(rope_kernel<false>, dim3(grid), dim3(256), 0, stream, a);
    }
    return check_launch("rope_kernel");
}

}  // namespace pplb200
