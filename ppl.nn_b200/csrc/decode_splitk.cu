// Split-k decode attention over the INT8 KV cache (one query token per sequence, GQA).
//
// The kernel is HBM-bound: per (token, kv head) it must read head_dim code bytes and head_dim/8 fp16
// scales for K and for V (320 B at head_dim 128) and does 4*group*head_dim flops on them.
//
// Shape of the computation
//   * The unit of work is a TILE: 16 consecutive tokens of one (sequence, kv head [, octet of query
//     heads]) pair, called a segment.  All tiles of the batch form one sequence ordered by (sequence,
//     head, position).  A planning kernel turns the device-side lengths into a prefix sum of tile
//     counts and cuts the sequence into ranges of equal size, one per resident warp ("stream-k"): every
//     warp streams the same number of tiles no matter how ragged the batch is.  A range may start or
//     end in the middle of a segment; such pieces go to the workspace as fp32 partials (at most two
//     per range) and a second-pass kernel merges them.  Pieces that cover a whole segment are written
//     as fp16 output directly.
//   * The heads are dealt round-robin into `head_lanes` (8, 4, 2 or 1) classes; the 8 warps of a CTA take
//     the same range of different classes, i.e. adjacent heads of the same token rows, so that in the
//     token-major cache layout the CTA streams 8 x 128 contiguous bytes per row (with fewer classes
//     the remaining warps take the next ranges of the same class).  Where it pays (see
//     want_lockstep) the warps that share a range also meet at a named barrier after every tile, which
//     keeps their requests to neighbouring addresses together in time.
//   * Every warp is an independent worker with its own 2-stage pipeline.  Per tile (5 KB at head_dim
//     128) one lane issues two bulk-tensor (TMA) copies, K codes and V codes, and all lanes together
//     copy the two small scale tiles with one 16-byte cp.async each (a TMA copy costs the warp tens
//     of issue slots whatever its size, which is too much for a 512-byte tile); everything completes
//     on one mbarrier; the pipeline runs across segment boundaries without draining.  The only
//     block-level synchronisation is the hand-out of the next range.
//   * Per tile the warp computes S^T[16 tokens x 8 heads] = K[16 x Dh] * Q^T with mma.m16n8k16
//     (tokens are the M dimension, the up-to-8 query heads of the group the N dimension),
//     dequantising K in registers: a byte permute builds the half 1024+u from each code byte, a
//     subtract gives the code exactly, a multiply applies the group scale.  Softmax runs in fp32 in the
//     exp2 domain with a lazily updated reference maximum; P^T is transposed between lanes with
//     movmatrix and O^T[Dh x 8 heads] += V^T * P^T follows, with V dequantised the same way (two
//     tokens are interleaved into one half2 by a permute).
//
//   * The append of the decode sequences' new tokens is part of this kernel: the new token of a sequence is
//     row kvlen-1, which lies in the LAST tile of each of its segments.  The warp that holds that tile reads
//     the head's 2 x head_dim halves of current_key/current_value, quantises them (one group of 8 per lane),
//     stores codes and scales to the cache row and overwrites the row in its own staged copy of the tile,
//     which the bulk copy may have read before or while the row was being written.  A decode step therefore
//     needs no separate append launch.
//
// Every wait on an mbarrier is bounded; on a timeout the warp records a status code, stops issuing copies
// and waiting, finishes (with wrong numbers, flagged) and drains the copies it still has in flight before
// the kernel returns, instead of hanging.
#include <cuda.h>
#include <stdlib.h>

#include <cub/block/block_scan.cuh>

#include "common.cuh"
#include "launch.h"
#include "tensor_map.h"

namespace pplb200 {

namespace {

// Tuning knobs (compile-time).  Measured on B200 with the LLaMA-2-7B decode workload: throughput in the
// token-major cache layout grows with the number of resident warps (each warp's row sequence is served
// by few DRAM banks at a time), not with the depth of its pipeline, so 16 warps x 2 stages per SM beat
// 12 x 3 and 8 x 4 at equal bytes in flight; 128 registers per thread is what 16 warps allow.  The 16
// warps are 2 CTAs of 8: eight head lanes per CTA read 1 KB of every token row together, 3-10 % faster
// than 4 CTAs of 4 on every workload and cache layout tried, and within 2 % of 1 CTA of 16.
#ifndef PPLB200_DECODE_WARPS
#define PPLB200_DECODE_WARPS 8
#endif
#ifndef PPLB200_DECODE_STAGES
#define PPLB200_DECODE_STAGES 2
#endif
#ifndef PPLB200_DECODE_CTAS
#define PPLB200_DECODE_CTAS 2
#endif

#ifndef PPLB200_DECODE_KRESID
#define PPLB200_DECODE_KRESID 1  // second MMA with the rounding remainders of the dequantised keys (see dequant_k_word)
#endif
#ifndef PPLB200_DECODE_OVERSUB_DEFAULT
#define PPLB200_DECODE_OVERSUB_DEFAULT 1
#endif

constexpr int kTileTok = 16;
constexpr int kStages = PPLB200_DECODE_STAGES;
constexpr int kWarps = PPLB200_DECODE_WARPS;
constexpr int kThreads = kWarps * 32;
constexpr int kCtasPerSm = PPLB200_DECODE_CTAS;
constexpr int kMinRangeTiles = 8;  // never cut the work finer than 128 tokens per range
constexpr float kNegBig = -1.0e30f;
constexpr float kRescaleSlack = 8.0f;  // the reference maximum may lag by up to 2^8 before a rescale

template <int DH>
struct Traits {
    static constexpr int kCodeBytes = kTileTok * DH;
    static constexpr int kScaleBytes = kTileTok * (DH / 8) * 2;
    static constexpr int kStageBytes = 2 * kCodeBytes + 2 * kScaleBytes;
    static constexpr int kWarpBytes = kStages * kStageBytes;
    static constexpr int kSmemBytes = kWarps * kWarpBytes + 1024;  // + slack to align the base to 1 KB
    static constexpr int kKRegs = DH / 16;                         // 32-bit code words per thread per K row
    static constexpr int kVRegs = DH / 32;                         // 32-bit code words per thread per V row
    static constexpr int kMTiles = DH / 16;                        // 16-channel output tiles
};

// Header of the decode region of the workspace, written by the planning kernel.
struct PlanHeader {
    uint32_t status;        // device status word (first word of the workspace)
    int32_t counter;        // next range to hand out
    int32_t range_tiles;    // R: tiles per range (uniform mode)
    int32_t num_ranges;
    int64_t total_tiles;    // tiles of one head class: (num_vheads / head_lanes) * sum_b tiles_b
    int32_t per_segment;    // 1: ranges are whole segments (split-k off), 0: uniform ranges
    int32_t reserved;
};

struct DecodeArgs {
    const __half* q;
    __half* out;
    const int64_t* seqstarts;
    const int64_t* cachestarts;
    const int64_t* start_pos;
    PlanHeader* hdr;
    const int32_t* tile_prefix;  // [decoding_batches + 1] prefix sum of tiles per sequence
    float* part_ml;              // [slots][8][2]
    float* part_o;               // [slots][8][DH]
    CacheGeom geom;
    int64_t max_kvlen;
    int32_t decoding_batches;
    int32_t num_heads;
    int32_t group;
    int32_t octets;
    int32_t head_lanes;   // head classes = warps of a CTA that share a range
    int32_t class_heads;  // virtual heads per class: num_vheads / head_lanes
    int32_t layer_idx;
    int32_t lockstep;     // 1: the warps that share a range synchronise after every tile
    CacheMapOrder order;
    const __half* scale;  // the scale tensor (copied with cp.async, addressed with the cache strides / 8)
    int64_t max_tokens;
    float scale_log2;
    // Fused append (cur_k != nullptr): the warp that streams the LAST tile of a (sequence, kv head) segment
    // quantises that head's slice of the sequence's new token, stores it to its cache row and patches its own
    // shared-memory copy of the tile with the same codes and scales.
    const __half* cur_k;
    const __half* cur_v;
    int8_t* cache;
    int32_t num_kv_heads;
    MaskDev mask;  // the optional attn_mask input (kernel instances with MASK only)
};

// Order of the four outer dimensions of the cache tensor maps (see CacheMapOrder), as a template
// parameter so that the coordinates of a copy cost nothing to assemble in the two standard layouts.
constexpr int kOrderRowLast = 0;   // (head, k|v, layer, row): cache_layout 0
constexpr int kOrderRowFirst = 1;  // (row, head, k|v, layer): cache_layout 3
constexpr int kOrderGeneric = 2;   // anything else: positions looked up at run time

// One head's tile of `kTileTok` cache rows -> shared memory at `dst` (a shared-space address).
template <int ORDER>
__device__ __forceinline__ void tma_load_cache_tile(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                                    const CacheMapOrder& od, int row, int head, int kv, int layer) {
    int c1, c2, c3, c4;
    if constexpr (ORDER == kOrderRowLast) {
        c1 = head; c2 = kv; c3 = layer; c4 = row;
    } else if constexpr (ORDER == kOrderRowFirst) {
        c1 = row; c2 = head; c3 = kv; c4 = layer;
    } else {
        int c[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int pos = i + 1;
            c[i] = od.pos_row == pos ? row : (od.pos_head == pos ? head : (od.pos_kv == pos ? kv : layer));
        }
        c1 = c[0]; c2 = c[1]; c3 = c[2]; c4 = c[3];
    }
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
        : "memory");
}

// 16- or 8-byte asynchronous copy global -> shared; `src_bytes` < BYTES zero-fills the rest.
template <int BYTES>
__device__ __forceinline__ void cp_async(uint32_t dst, const void* src, uint32_t src_bytes) {
    if constexpr (BYTES == 16) {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
    } else {
        asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
    }
}
// The executing thread's earlier cp.async copies arrive on the mbarrier when they have landed.
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}

// ------------------------------------------------------------------------------------------
// Planning kernel (one CTA): tiles per decode sequence -> exclusive prefix sum, the longest
// sequence, and from them the range size; resets the work counter and the status word.
// ------------------------------------------------------------------------------------------
constexpr int kPlanThreads = 512;

__global__ void __launch_bounds__(kPlanThreads)
decode_plan_kernel(const int64_t* __restrict__ seqstarts, const int64_t* __restrict__ start_pos,
                   int32_t decoding_batches, int32_t class_heads, int64_t max_kvlen, int32_t split_k_mode,
                   int32_t workers, int32_t max_ranges, int32_t static_ranges, PlanHeader* __restrict__ hdr,
                   int32_t* __restrict__ tile_prefix) {
    using Scan = cub::BlockScan<int32_t, kPlanThreads>;
    __shared__ typename Scan::TempStorage tmp;
    __shared__ int32_t carry;
    __shared__ int32_t longest;
    grid_launch_dependents();
    grid_dependency_wait();  // the workspace may still be read by the previous call's kernels
    if (threadIdx.x == 0) {
        carry = 0;
        longest = 1;
        hdr->status = 0;
        hdr->counter = static_ranges;  // the main kernel's CTAs take ranges [0, static_ranges) without asking
    }
    __syncthreads();
    for (int32_t base = 0; base < decoding_batches; base += kPlanThreads) {
        const int32_t b = base + threadIdx.x;
        int32_t n = 0;
        if (b < decoding_batches) {
            int64_t kvlen = start_pos[b] + (seqstarts[b + 1] - seqstarts[b]);
            if (kvlen > max_kvlen) {
                kvlen = max_kvlen;
                atomicOr(&hdr->status, kDevLengthClamped);
            }
            if (kvlen < 1) {
                kvlen = 1;  // an empty sequence still owns one (fully masked) tile so that its output is written
            }
            n = static_cast<int32_t>((kvlen + kTileTok - 1) / kTileTok);
            atomicMax(&longest, n);
        }
        int32_t excl, total;
        Scan(tmp).ExclusiveSum(n, excl, total);
        const int32_t c = carry;
        if (b < decoding_batches) {
            tile_prefix[b] = c + excl;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            carry = c + total;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        tile_prefix[decoding_batches] = carry;
        const int64_t total = static_cast<int64_t>(carry) * class_heads;
        hdr->total_tiles = total;
        if (split_k_mode == 0) {
            hdr->per_segment = 1;
            hdr->range_tiles = 0;
            hdr->num_ranges = decoding_batches * class_heads;
        } else {
            int64_t r = (total + workers - 1) / workers;  // equal share per resident warp of the class
            r = r < kMinRangeTiles ? kMinRangeTiles : r;
            if (split_k_mode == 2) {
                const int64_t half = (longest + 1) / 2;  // "always": the longest sequence is cut at least once
                r = r < half ? r : half;
                r = r < 1 ? 1 : r;
            }
            int64_t nr = (total + r - 1) / r;
            if (nr > max_ranges) {  // cannot happen for lengths within max_kvlen; keep the partial slots in bounds
                r = (total + max_ranges - 1) / max_ranges;
                nr = (total + r - 1) / r;
            }
            hdr->per_segment = 0;
            hdr->range_tiles = static_cast<int32_t>(r);
            hdr->num_ranges = static_cast<int32_t>(nr);
        }
    }
}

// ------------------------------------------------------------------------------------------
// Main kernel
// ------------------------------------------------------------------------------------------

// lo += low half of ph, hi += high half of ph: the fp16 values widened exactly, one mixed-precision add each
__device__ __forceinline__ void add_halves_to_floats(float& lo, float& hi, uint32_t ph) {
    asm("{\n"
        ".reg .b16 h0, h1;\n"
        "mov.b32 {h0, h1}, %2;\n"
        "add.rn.f32.f16 %0, h0, %0;\n"
        "add.rn.f32.f16 %1, h1, %1;\n"
        "}\n"
        : "+f"(lo), "+f"(hi)
        : "r"(ph));
}

// K codes word -> two half2 (channels 0,1 and 2,3 of the word), scaled: k = fp16(code * scale).  The product
// of a 7-bit code and an 11-bit scale does not fit fp16; its rounding error, 2^-11 relative per element, is the
// largest error of the whole kernel on keys with outlier channels (scores with a wide range: a pair of
// competing tokens then shifts weight by 1e-3).  So the error itself is kept: e = fma(code, scale, -k) is the
// exact remainder code * scale - k (the rounding error of a product is representable), and a second MMA adds
// e . q to the same accumulator, which makes the scores those of the exactly dequantised keys.
__device__ __forceinline__ void dequant_k_word(uint32_t w, __half2 s2, uint32_t& lo, uint32_t& hi, uint32_t& elo,
                                               uint32_t& ehi) {
    const uint32_t x = w ^ 0x80808080u;
    const __half2 c_lo = biased_bytes_to_half2<0x5140u>(x), c_hi = biased_bytes_to_half2<0x5342u>(x);
    const __half2 k_lo = __hmul2(c_lo, s2), k_hi = __hmul2(c_hi, s2);
    lo = h2_as_u32(k_lo);
    hi = h2_as_u32(k_hi);
#if PPLB200_DECODE_KRESID
    elo = h2_as_u32(__hfma2(c_lo, s2, __hneg2(k_lo)));
    ehi = h2_as_u32(__hfma2(c_hi, s2, __hneg2(k_hi)));
#else
    elo = ehi = 0u;
#endif
}

// V codes words of two tokens (same 4 channels) -> four half2 {token A, token B}, one per channel.
__device__ __forceinline__ void dequant_v_pair(uint32_t wa, uint32_t wb, __half2 s2, uint32_t (&h)[4]) {
    const uint32_t x = prmt(wa, wb, 0x5140u) ^ 0x80808080u;  // a0 b0 a1 b1
    const uint32_t y = prmt(wa, wb, 0x7362u) ^ 0x80808080u;  // a2 b2 a3 b3
    h[0] = h2_as_u32(__hmul2(biased_bytes_to_half2<0x5140u>(x), s2));
    h[1] = h2_as_u32(__hmul2(biased_bytes_to_half2<0x5342u>(x), s2));
    h[2] = h2_as_u32(__hmul2(biased_bytes_to_half2<0x5140u>(y), s2));
    h[3] = h2_as_u32(__hmul2(biased_bytes_to_half2<0x5342u>(y), s2));
}

// The new token of decode sequence b (query row `tok`, position `pos` = kvlen - 1) for kv head `kvh`: one
// lane per quantisation group (K groups first, then V groups) quantises 8 halves, stores codes and scale to
// the cache row and overwrites row pos % 16 of the staged tile at `st`, whose bulk copy has completed.
template <int DH>
__device__ __forceinline__ void append_token_into_tile(const DecodeArgs& a, uint32_t st, int lane, int64_t tok,
                                                       int kvh, int32_t b, int32_t pos) {
    using T = Traits<DH>;
    constexpr int kGroups = DH / 8;  // quantisation groups of one head row
    if (lane < 2 * kGroups) {
        const int kv = lane / kGroups;  // 0: key, 1: value
        const int grp = lane - kv * kGroups;
        const __half* src = (kv ? a.cur_v : a.cur_k) + (tok * a.num_kv_heads + kvh) * DH + grp * 8;
        uint2 codes;
        __half s16;
        quant_group8(*reinterpret_cast<const uint4*>(src), codes, s16);
        const int64_t row = cache_row(a.geom, a.cachestarts, b, pos);
        if (row >= 0 && row < a.max_tokens) {
            const int64_t off = cache_offset(a.geom, row, kv, kvh) + grp * 8;
            *reinterpret_cast<uint2*>(a.cache + off) = codes;
            const_cast<__half*>(a.scale)[off >> 3] = s16;
        } else if (grp == 0) {
            atomicOr(&a.hdr->status, kDevRowOutOfRange);
        }
        const int r = pos & (kTileTok - 1);
        uint32_t caddr = st + kv * T::kCodeBytes + r * DH;
        if constexpr (DH == 128) {
            caddr += (((grp >> 1) ^ (r & 7)) << 4) + ((grp & 1) << 3);  // 16-byte chunks swizzled by the row
        } else {
            caddr += grp * 8;
        }
        asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(caddr), "r"(codes.x), "r"(codes.y) : "memory");
        const uint32_t saddr = st + 2 * T::kCodeBytes + kv * T::kScaleBytes + r * (kGroups * 2) + grp * 2;
        asm volatile("st.shared.u16 [%0], %1;" ::"r"(saddr), "h"(__half_as_ushort(s16)) : "memory");
    }
    fence_proxy_async_smem();  // the stage is refilled by a bulk copy after these generic-proxy writes
    __syncwarp();
}

// Position in the tile sequence of one head class: sequence b, class-local head index vc (the virtual
// head, i.e. kv head x octet of query heads, is vc * head_lanes + class), tile index within the
// segment, tiles per segment of this sequence, first cache row of the sequence and the kv head.
struct Cursor {
    int32_t b, vc, tile, n;
    int32_t row_base;
    int32_t kvh;
};

// KDOT (one query head per kv head, no mask): the scores come from integer dot products instead of the
// tensor cores.  With a single query head the MMA's eight columns hold one useful number, while its A
// operand still wants every key dequantised to fp16 (21 instructions per 8 codes with the remainder).  The
// query row is instead quantised once per piece to int16 with one fp32 scale per 8-channel group
// (|error| <= 2^-16 of the group's largest element), and a group's partial score is dp2a(codes, q) -- exact in
// int32 -- times the key scale times the query scale: 8 instructions per 8 codes and keys that are exact by
// construction.  V, the softmax bookkeeping and the output go through the MMA as before.
template <int DH, int ORDER, bool MASK, bool KDOT>
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
decode_splitk_kernel(const __grid_constant__ CUtensorMap tmap_codes, const DecodeArgs a) {
    using T = Traits<DH>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[kWarps * kStages];
    __shared__ int32_t s_base;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2;
    const int t = lane & 3;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kWarps * kStages; ++i) {
            mbar_init(&full_bar[i], 33);  // lane 0's expect_tx arrival + one cp.async arrival per lane
        }
        mbar_fence_init();
        tma_prefetch_desc(&tmap_codes);
    }
    __syncthreads();
    grid_dependency_wait();  // from here on: the plan, and the cache rows the append kernel wrote
    // The merge kernel may be scheduled from here on: the plan is complete and visible, so the merge kernel can
    // read the plan and work out its segments ahead of its own wait for this grid.
    grid_launch_dependents();

    // shared-space addresses of this warp's stage ring (1 KB aligned for the 128-byte swizzle) and barriers
    const uint32_t wsm = ((smem_u32(smem_raw) + 1023u) & ~1023u) + warp * T::kWarpBytes;
    const uint32_t wbar = smem_u32(full_bar + warp * kStages);
    // per-thread byte offsets into a stage, fixed for the whole kernel
    //   K rows g and g+8: the thread's channel slab (two 16-byte chunks at Dh 128, swizzled by the row);
    //   V rows 2t, 2t+1 (+8): the thread's channel slab (one chunk, swizzled by the row)
    uint32_t k_off, ks_off, v_off_a, v_off_b, vs_off;
    if constexpr (DH == 128) {
        k_off = g * 128 + (((2 * t) ^ g) << 4);
        ks_off = 2 * T::kCodeBytes + g * 32 + t * 8;
        v_off_a = T::kCodeBytes + (2 * t) * 128 + ((g ^ (2 * t)) << 4);
        v_off_b = T::kCodeBytes + (2 * t + 1) * 128 + ((g ^ (2 * t + 1)) << 4);
        vs_off = 2 * T::kCodeBytes + T::kScaleBytes + (2 * t) * 32 + g * 4;
    } else {
        k_off = g * 64 + t * 16;
        ks_off = 2 * T::kCodeBytes + g * 16 + t * 4;
        v_off_a = T::kCodeBytes + (2 * t) * 64 + g * 8;
        v_off_b = v_off_a + 64;
        vs_off = 2 * T::kCodeBytes + T::kScaleBytes + (2 * t) * 16 + g * 2;
    }

    // scale tiles: lane l copies bytes [l * DH/8, (l + 1) * DH/8) of the tile, i.e. half a scale row
    constexpr int kScaleCopy = DH / 8;  // 16 or 8 bytes per lane
    const int64_t scale_row_bytes = a.geom.stride_s / 4;  // cache stride / 8 elements * 2 bytes
    const int64_t scale_lane_off = (lane >> 1) * scale_row_bytes + (lane & 1) * kScaleCopy;
    const int64_t scale_kv_bytes = a.geom.stride_kv / 4;
    const uint32_t scale_dst_off = 2 * T::kCodeBytes + lane * kScaleCopy;
    const char* scale_layer = reinterpret_cast<const char*>(a.scale) + a.layer_idx * (a.geom.stride_l / 4);
    const int64_t scale_head_bytes = a.geom.stride_h / 4;

    uint32_t c_stage = 0, c_phase = 0;  // consume position in the stage ring
    uint32_t i_stage = 0;               // issue position in the stage ring
    bool wait_dead = false;             // set after the first timed-out wait: stop waiting and issuing, just finish
    int32_t dead_inflight = 0;          // tiles issued but not yet seen complete when the warp gave up ...
    uint32_t dead_stage = 0, dead_phase = 0;  // ... and the ring position of the first of them

    const int nvc = a.class_heads;
    const int cls = warp % a.head_lanes;             // head class of this warp
    const int sub = warp / a.head_lanes;             // which of the CTA's consecutive ranges it takes
    const int ranges_per_cta = kWarps / a.head_lanes;
    const int32_t DB = a.decoding_batches;
    const int32_t num_ranges = a.hdr->num_ranges;
    const int32_t range_tiles = a.hdr->range_tiles;
    const int32_t per_segment = a.hdr->per_segment;
    const int64_t total_tiles = a.hdr->total_tiles;
    const bool paged = a.geom.cache_mode != 0;
    const int page_shift = (a.geom.page_size & (a.geom.page_size - 1)) == 0 ? 31 - __clz(a.geom.page_size) : -1;
    const int octets = a.octets;
    const int head_lanes = a.head_lanes;
    const bool lockstep = a.lockstep != 0;
    const int layer = a.layer_idx;
    const int32_t max_rows = static_cast<int32_t>(a.max_tokens);
    const int64_t scale_tile_bytes = kTileTok * scale_row_bytes;
    // paged mode: a tile starts a page when its token offset has no bits below the page size (page sizes that
    // are not powers of two look the page up for every tile)
    const uint32_t page_mask = page_shift >= 0 ? static_cast<uint32_t>(a.geom.page_size) - 1u : 0u;

    constexpr int32_t kBadRow = -(1 << 30);  // row_base of a sequence whose cachestarts entry is not a cache row
    auto load_seq = [&](Cursor& c) {  // per-sequence fields
        c.n = a.tile_prefix[c.b + 1] - a.tile_prefix[c.b];
        c.row_base = 0;
        if (!paged) {
            const int64_t cs = a.cachestarts[c.b];
            c.row_base = (cs >= 0 && cs < a.max_tokens) ? static_cast<int32_t>(cs) : kBadRow;
        }
    };
    auto set_head = [&](Cursor& c) { c.kvh = octets == 1 ? c.vc * head_lanes + cls : (c.vc * head_lanes + cls) / octets; };
    auto advance = [&](Cursor& c, int32_t by) {
        // moves within the segment or to the start of the next one (by never crosses two boundaries)
        c.tile += by;
        if (c.tile >= c.n) {
            c.tile = 0;
            if (++c.vc == nvc) {
                c.vc = 0;
                ++c.b;
                if (c.b < DB) {
                    load_seq(c);
                }
            }
            set_head(c);
        }
    };

    for (bool first_round = true;; first_round = false) {
        // The first ranges are dealt statically, one batch per CTA (with one range per resident warp, the
        // usual plan, that is all of them: no atomic and no barrier ahead of the first loads); the counter,
        // which the planning kernel starts behind the static batches, hands out the rest.
        int32_t base = static_cast<int32_t>(blockIdx.x) * ranges_per_cta;
        if (!first_round) {
            __syncthreads();  // everyone has read the previous s_base
            if (threadIdx.x == 0) {
                s_base = atomicAdd(&a.hdr->counter, ranges_per_cta);
            }
            __syncthreads();
            base = s_base;
        }
        const int32_t r = base + sub;
        if (base >= num_ranges) {
            break;  // uniform for the CTA
        }
        if (r >= num_ranges) {
            continue;
        }
        // ---- the range [lo, hi) of the class's tile sequence and the segment it starts in ----
        int64_t lo, hi;
        Cursor cc;
        if (per_segment) {
            cc.b = r / nvc;
            cc.vc = r - cc.b * nvc;
            cc.tile = 0;
            load_seq(cc);
            lo = static_cast<int64_t>(a.tile_prefix[cc.b]) * nvc + static_cast<int64_t>(cc.vc) * cc.n;
            hi = lo + cc.n;
        } else {
            lo = static_cast<int64_t>(r) * range_tiles;
            hi = lo + range_tiles;
            hi = hi > total_tiles ? total_tiles : hi;
            // largest b with tile_prefix[b] * nvc <= lo.  All lanes search together, 32 pivots per round: a
            // thousand sequences take two dependent loads instead of ten, which is microseconds at the start
            // of a kernel that only runs for tens of them.
            int32_t l = 0, h = DB;
            while (h - l > 1) {
                const int32_t step = (h - l + 31) >> 5;
                const int32_t piv = l + (lane + 1) * step;
                const bool le = piv < h && static_cast<int64_t>(a.tile_prefix[piv]) * nvc <= lo;  // true for a prefix of the lanes
                const int32_t c = __popc(__ballot_sync(0xffffffffu, le));
                l += c * step;
                h = l + step < h ? l + step : h;
            }
            cc.b = l;
            load_seq(cc);
            const int64_t rem = lo - static_cast<int64_t>(a.tile_prefix[l]) * nvc;
            cc.vc = static_cast<int32_t>(rem / cc.n);
            cc.tile = static_cast<int32_t>(rem - static_cast<int64_t>(cc.vc) * cc.n);
        }
        set_head(cc);
        Cursor ic = cc;                                // issue cursor: runs up to kStages tiles ahead
        int32_t to_issue = static_cast<int32_t>(hi - lo);  // tiles of the range not yet issued
        int32_t to_consume = to_issue;

        // Position of the next tile to issue, kept incrementally: its first cache row (negative: not a cache
        // row) and this lane's source address in the scale tensor.  Both are worked out in full where a new
        // segment or, in paged mode, a new page begins; inside a run of consecutive rows a tile adds 16 rows.
        int32_t i_row = 0;
        const char* i_src = nullptr;
        auto locate = [&]() {
            const int tok = ic.tile * kTileTok;
            int32_t row = ic.row_base + tok;  // kBadRow + tok stays negative
            if (paged) {  // the page table row of the sequence gives the first cache row of every page
                const uint32_t page = page_shift >= 0 ? static_cast<uint32_t>(tok) >> page_shift
                                                      : static_cast<uint32_t>(tok) / static_cast<uint32_t>(a.geom.page_size);
                row = kBadRow;
                if (page < static_cast<uint32_t>(a.geom.cachestart_stride_b)) {
                    const int64_t first = a.cachestarts[ic.b * a.geom.cachestart_stride_b + page];
                    if (first >= 0 && first < a.max_tokens) {
                        row = static_cast<int32_t>(first) + (tok - static_cast<int>(page) * a.geom.page_size);
                    }
                }
            }
            i_row = row;
            i_src = scale_layer + (row >= 0 ? row : 0) * scale_row_bytes + ic.kvh * scale_head_bytes + scale_lane_off;
        };
        auto issue_one = [&]() {
            // A tile whose first row is not a cache row (a wrong index tensor) is flagged and read as zeros:
            // the scale copies read nothing and the bulk copies start past the last row, which zero-fills.
            int32_t row = i_row;
            if (row < 0 || row >= max_rows) {
                if (lane == 0) {
                    atomicOr(&a.hdr->status, kDevRowOutOfRange);
                }
                row = max_rows;
            }
            const uint32_t st = wsm + i_stage * T::kStageBytes;
            const uint32_t bar = wbar + i_stage * 8;
            {
                // scales: every lane copies its half row of the K tile and of the V tile
                const uint32_t nbytes = (row + (lane >> 1)) < max_rows ? kScaleCopy : 0;  // rows past the cache: zeros
                cp_async<kScaleCopy>(st + scale_dst_off, i_src, nbytes);
                cp_async<kScaleCopy>(st + scale_dst_off + T::kScaleBytes, i_src + scale_kv_bytes, nbytes);
                cp_async_arrive(bar);
            }
            if (lane == 0) {
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar),
                             "r"(2 * T::kCodeBytes)
                             : "memory");
                tma_load_cache_tile<ORDER>(st, &tmap_codes, bar, a.order, row, ic.kvh, 0, layer);
                tma_load_cache_tile<ORDER>(st + T::kCodeBytes, &tmap_codes, bar, a.order, row, ic.kvh, 1, layer);
            }
            __syncwarp();
            i_stage = (i_stage + 1 == kStages) ? 0 : i_stage + 1;
            --to_issue;
            // next tile: same segment and (paged) same page -> 16 rows on; otherwise locate it afresh
            if (++ic.tile < ic.n && !(paged && (static_cast<uint32_t>(ic.tile * kTileTok) & page_mask) == 0u)) {
                i_row += kTileTok;
                i_src += scale_tile_bytes;
            } else {
                if (ic.tile >= ic.n) {
                    ic.tile -= 1;
                    advance(ic, 1);
                }
                if (ic.b < DB) {
                    locate();
                }
            }
        };
        locate();
        if (wait_dead) {
            to_issue = 0;  // a warp that has given up runs through its remaining ranges without copies
        }
        for (int i = 0; i < kStages && to_issue > 0; ++i) {
            issue_one();
        }

        bool first_piece = true;
        while (to_consume > 0) {
            // ---- one piece: the part of segment (cc.b, cc.vc) that lies inside the range ----
            const int32_t t_first = cc.tile;
            const int32_t t_end = (cc.n - t_first) <= to_consume ? cc.n : t_first + to_consume;
            const int32_t b = cc.b;
            const int vh = cc.vc * head_lanes + cls;
            const int kvh = cc.kvh;
            const int oct = vh - kvh * octets;
            const int64_t qtok = a.seqstarts[b];
            const int64_t seqlen = a.seqstarts[b + 1] - qtok;
            int64_t kvlen64 = a.start_pos[b] + seqlen;
            // the new token is appended by the piece that holds the segment's last tile (never for a clamped or
            // empty sequence: the first is flagged by the planning kernel, the second has no token)
            const bool append_here = a.cur_k != nullptr && t_end == cc.n && seqlen >= 1 && kvlen64 <= a.max_kvlen;
            kvlen64 = kvlen64 > a.max_kvlen ? a.max_kvlen : kvlen64;
            const int32_t kvlen = static_cast<int32_t>(kvlen64);

            // KDOT: this lane's quarter of the query row as int16 pairs, one scale per group of 8 channels
            int32_t qi[KDOT ? DH / 8 : 1];
            float qs[KDOT ? DH / 32 : 1];
            if constexpr (KDOT) {
                const __half* qp = a.q + (qtok * a.num_heads + kvh) * DH + t * (DH / 4);
#pragma unroll
                for (int gi = 0; gi < DH / 32; ++gi) {
                    const uint4 v = *reinterpret_cast<const uint4*>(qp + 8 * gi);
                    const __half2* h2 = reinterpret_cast<const __half2*>(&v);
                    float2 f[4];
                    float amax = 0.0f;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        f[i] = __half22float2(h2[i]);
                        amax = max3_nan(amax, fabsf(f[i].x), fabsf(f[i].y));  // a NaN or infinite query element
                        // must reach the scores (0 * inf below), as it does through the MMA
                    }
                    const float inv = amax > 0.0f ? 32767.0f / amax : 0.0f;
                    qs[gi] = amax * (1.0f / 32767.0f);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int lo = __float2int_rn(f[i].x * inv), hi = __float2int_rn(f[i].y * inv);
                        qi[4 * gi + i] = static_cast<int32_t>((static_cast<uint32_t>(lo) & 0xffffu) | (static_cast<uint32_t>(hi) << 16));
                    }
                }
            }
            // Q fragments (B operand: k = channel, n = query head of the group)
            uint32_t qf[T::kKRegs][2];
            if constexpr (!KDOT) {
                const int hq_in_group = oct * 8 + g;
                if (hq_in_group < a.group) {
                    const __half* qp = a.q + (qtok * a.num_heads + kvh * a.group + hq_in_group) * DH + t * (DH / 4);
#pragma unroll
                    for (int i = 0; i < T::kKRegs / 2; ++i) {
                        const uint4 v = *reinterpret_cast<const uint4*>(qp + 8 * i);
                        qf[2 * i][0] = v.x;
                        qf[2 * i][1] = v.y;
                        qf[2 * i + 1][0] = v.z;
                        qf[2 * i + 1][1] = v.w;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < T::kKRegs; ++i) {
                        qf[i][0] = 0u;
                        qf[i][1] = 0u;
                    }
                }
            }
            float o[T::kMTiles][4];
#pragma unroll
            for (int i = 0; i < T::kMTiles; ++i) {
                o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
            }
            float m0 = kNegBig, m1 = kNegBig, l0 = 0.0f, l1 = 0.0f;
            // growth thresholds of the lazy maximum in the units of the scores as they are compared (see below)
            const float inv_sc = MASK ? 1.0f : 1.0f / a.scale_log2;
            float thr0 = (kNegBig + kRescaleSlack) * inv_sc, thr1 = thr0;
            // attn_mask rows of this thread's two query heads (2t, 2t+1 of the octet): element [kv position]
            const __half* mrow0 = nullptr;
            const __half* mrow1 = nullptr;
            int64_t mask_room = 0;  // columns of the mask from this sequence's position 0 on
            if constexpr (MASK) {
                const int64_t col0 = a.mask.kvstarts[b];
                mask_room = a.mask.cols - col0;
                const __half* base = a.mask.data + qtok * a.mask.cols + col0;
                const int h0 = oct * 8 + 2 * t;
                if (h0 < a.group) {
                    mrow0 = base + static_cast<int64_t>(kvh * a.group + h0) * a.mask.head_stride;
                }
                if (h0 + 1 < a.group) {
                    mrow1 = base + static_cast<int64_t>(kvh * a.group + h0 + 1) * a.mask.head_stride;
                }
                if (mask_room < kvlen && lane == 0) {
                    atomicOr(&a.hdr->status, kDevMaskOutOfRange);
                }
            }

            for (int32_t tile = t_first; tile < t_end; ++tile) {
                // the common case is one try (it parks the warp until the tile has landed, up to the hint); a warp
                // that has given up before falls through without waiting
                if (!mbar_try_wait_hint(wbar + c_stage * 8, c_phase, PPLB200_WAIT_HINT_NS) && !wait_dead) {
                    if (!mbar_wait_bounded(reinterpret_cast<uint64_t*>(full_bar + warp * kStages + c_stage), c_phase)) {
                        // Give up: no further copies are issued and no further waits are made; the tiles already
                        // issued (this one included) are waited for once more, briefly, before the kernel returns.
                        wait_dead = true;
                        dead_inflight = (to_consume - (tile - t_first)) - to_issue;
                        dead_stage = c_stage;
                        dead_phase = c_phase;
                        to_issue = 0;
                        if (lane == 0) {
                            atomicOr(&a.hdr->status, kDevTmaTimeout);
                        }
                    }
                }
                const uint32_t st = wsm + c_stage * T::kStageBytes;
                const int nvalid = kvlen - tile * kTileTok;  // >= 16 except in the last tile of the sequence
                if (append_here && tile == cc.n - 1) {
                    append_token_into_tile<DH>(a, st, lane, qtok + seqlen - 1, kvh, b, kvlen - 1);
                }

                // ---------------- S^T = K * Q^T ----------------
                float sacc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                {
                    uint32_t wa[T::kKRegs], wb[T::kKRegs];          // rows g and g+8, this thread's channel slab
                    uint32_t sa[T::kKRegs / 4], sb[T::kKRegs / 4];  // packed group scales (2 halves per word)
                    const uint32_t ka = st + k_off;
                    if constexpr (DH == 128) {
                        const uint4 a0 = lds128(ka);
                        const uint4 a1 = lds128(ka ^ 16u);
                        const uint4 b0 = lds128(ka + 1024u);
                        const uint4 b1 = lds128((ka ^ 16u) + 1024u);
                        wa[0] = a0.x; wa[1] = a0.y; wa[2] = a0.z; wa[3] = a0.w;
                        wa[4] = a1.x; wa[5] = a1.y; wa[6] = a1.z; wa[7] = a1.w;
                        wb[0] = b0.x; wb[1] = b0.y; wb[2] = b0.z; wb[3] = b0.w;
                        wb[4] = b1.x; wb[5] = b1.y; wb[6] = b1.z; wb[7] = b1.w;
                        const uint2 s_a = lds64(st + ks_off);
                        const uint2 s_b = lds64(st + ks_off + 256u);
                        sa[0] = s_a.x; sa[1] = s_a.y;
                        sb[0] = s_b.x; sb[1] = s_b.y;
                    } else {
                        const uint4 a0 = lds128(ka);
                        const uint4 b0 = lds128(ka + 512u);
                        wa[0] = a0.x; wa[1] = a0.y; wa[2] = a0.z; wa[3] = a0.w;
                        wb[0] = b0.x; wb[1] = b0.y; wb[2] = b0.z; wb[3] = b0.w;
                        sa[0] = lds32(st + ks_off);
                        sb[0] = lds32(st + ks_off + 128u);
                    }
                    if constexpr (KDOT) {
                        // rows g and g+8 against the one query head: per group an exact integer dot product,
                        // scaled by key scale x query scale; the quad then adds up its four quarter rows
                        float acc_a = 0.0f, acc_b = 0.0f;
#pragma unroll
                        for (int gi = 0; gi < DH / 32; ++gi) {
                            int da = 0, db = 0;
#pragma unroll
                            for (int w = 0; w < 2; ++w) {
                                const int rr = 2 * gi + w;
                                da = __dp2a_lo(qi[2 * rr], static_cast<int>(wa[rr]), da);
                                da = __dp2a_hi(qi[2 * rr + 1], static_cast<int>(wa[rr]), da);
                                db = __dp2a_lo(qi[2 * rr], static_cast<int>(wb[rr]), db);
                                db = __dp2a_hi(qi[2 * rr + 1], static_cast<int>(wb[rr]), db);
                            }
                            const float2 fa = __half22float2(u32_as_h2(sa[gi >> 1])), fb = __half22float2(u32_as_h2(sb[gi >> 1]));
                            acc_a = fmaf(__int2float_rn(da), ((gi & 1) ? fa.y : fa.x) * qs[gi], acc_a);
                            acc_b = fmaf(__int2float_rn(db), ((gi & 1) ? fb.y : fb.x) * qs[gi], acc_b);
                        }
                        acc_a += __shfl_xor_sync(0xffffffffu, acc_a, 1);
                        acc_b += __shfl_xor_sync(0xffffffffu, acc_b, 1);
                        acc_a += __shfl_xor_sync(0xffffffffu, acc_a, 2);
                        acc_b += __shfl_xor_sync(0xffffffffu, acc_b, 2);
                        sacc[0] = acc_a;  // token g
                        sacc[2] = acc_b;  // token g + 8
                    } else {
#pragma unroll
                    for (int rr = 0; rr < T::kKRegs; ++rr) {
                        // word rr holds channels 4rr..4rr+3 of the slab: quantisation group rr/2 of the slab
                        const __half2 pa = u32_as_h2(sa[rr >> 2]), pb = u32_as_h2(sb[rr >> 2]);
                        const __half2 s2a = (rr & 2) ? __high2half2(pa) : __low2half2(pa);
                        const __half2 s2b = (rr & 2) ? __high2half2(pb) : __low2half2(pb);
                        uint32_t a0, a1, a2, a3, e0, e1, e2, e3;
                        dequant_k_word(wa[rr], s2a, a0, a2, e0, e2);
                        dequant_k_word(wb[rr], s2b, a1, a3, e1, e3);
                        mma_m16n8k16_f16f32(sacc, a0, a1, a2, a3, qf[rr][0], qf[rr][1]);
#if PPLB200_DECODE_KRESID
                        mma_m16n8k16_f16f32(sacc, e0, e1, e2, e3, qf[rr][0], qf[rr][1]);
#endif
                    }
                    }
                }

                // ---------------- softmax (exp2 domain, lazy reference maximum) ----------------
                // Raw scores: token g / g+8, heads 2t / 2t+1.  Without a mask they stay unscaled: the growth test
                // compares them with thresholds kept in raw units (thr = (m + slack) / scale, updated only when the
                // reference maximum moves), and scale and maximum enter the exponent through one FMA.
                uint32_t pb0, pb1;  // P^T as the B operand of the second MMA: k = token, n = head
                if constexpr (KDOT) {
                    // one head: every lane of quad g holds the raw scores of tokens g and g + 8
                    float s_lo = sacc[0], s_hi = sacc[2];
                    if (nvalid < kTileTok) {  // rows past the end of the sequence weigh nothing
                        s_lo = g < nvalid ? s_lo : -INFINITY;
                        s_hi = g + 8 < nvalid ? s_hi : -INFINITY;
                    }
                    const float sc = a.scale_log2;
                    float lm = fmaxf(s_lo, s_hi);
                    if (__any_sync(0xffffffffu, lm > thr0)) {
#pragma unroll
                        for (int off = 4; off <= 16; off <<= 1) {
                            lm = fmaxf(lm, __shfl_xor_sync(0xffffffffu, lm, off));
                        }
                        const float n0 = fmaxf(m0, lm * sc);
                        const float r0 = ex2_approx(m0 - n0);
                        m0 = n0;
                        thr0 = (m0 + kRescaleSlack) * inv_sc;
                        l0 *= r0;
#pragma unroll
                        for (int i = 0; i < T::kMTiles; ++i) {
                            o[i][0] *= r0;
                            o[i][1] *= r0;
                            o[i][2] *= r0;
                            o[i][3] *= r0;
                        }
                    }
                    // the normaliser sums the fp16-rounded weights, the very numbers the MMA consumes
                    const uint32_t ph = h2_as_u32(__floats2half2_rn(ex2_approx(fmaf(s_lo, sc, -m0)), ex2_approx(fmaf(s_hi, sc, -m0))));
                    float l_hi = 0.0f;
                    add_halves_to_floats(l0, l_hi, ph);
                    l0 += l_hi;
                    // B fragment of lane (g', t'): tokens 2t', 2t'+1 and 2t'+8, 2t'+9 of head g' -- the one real head
                    // is g' = 0; the other columns get the same weights and their outputs are never stored
                    const uint32_t x = __shfl_sync(0xffffffffu, ph, 8 * t), y = __shfl_sync(0xffffffffu, ph, 8 * t + 4);
                    pb0 = prmt(x, y, 0x5410u);
                    pb1 = prmt(x, y, 0x7632u);
                } else {
                    float s0 = sacc[0], s1 = sacc[1], s2 = sacc[2], s3 = sacc[3];
                    if constexpr (MASK) {  // additive mask on the scaled scores (exp2 domain: times log2 e)
                        constexpr float kLog2e = 1.4426950408889634f;
                        s0 *= a.scale_log2;
                        s1 *= a.scale_log2;
                        s2 *= a.scale_log2;
                        s3 *= a.scale_log2;
                        const int64_t p0 = static_cast<int64_t>(tile) * kTileTok + g, p1 = p0 + 8;
                        const bool in0 = p0 < kvlen && p0 < mask_room, in1 = p1 < kvlen && p1 < mask_room;
                        if (mrow0) {
                            if (in0) s0 = fmaf(__half2float(mrow0[p0]), kLog2e, s0);
                            if (in1) s2 = fmaf(__half2float(mrow0[p1]), kLog2e, s2);
                        }
                        if (mrow1) {
                            if (in0) s1 = fmaf(__half2float(mrow1[p0]), kLog2e, s1);
                            if (in1) s3 = fmaf(__half2float(mrow1[p1]), kLog2e, s3);
                        }
                        // +inf or NaN in a mask would poison the running maximum: such entries count as "masked out"
                        s0 = s0 < 3.0e38f ? s0 : -INFINITY;
                        s1 = s1 < 3.0e38f ? s1 : -INFINITY;
                        s2 = s2 < 3.0e38f ? s2 : -INFINITY;
                        s3 = s3 < 3.0e38f ? s3 : -INFINITY;
                    }
                    // Rows past the end of the sequence score -inf: weight 0 against the (always finite) reference
                    // maximum, also where no row of the tile is left (an empty sequence, or a mask that removes every
                    // real token of the tile).
                    constexpr float kOut = -INFINITY;
                    if (nvalid < kTileTok) {  // only the last tile of a sequence has rows past its end
                        if (g >= nvalid) {
                            s0 = kOut;
                            s1 = kOut;
                        }
                        if (g + 8 >= nvalid) {
                            s2 = kOut;
                            s3 = kOut;
                        }
                    }
                    const float sc = MASK ? 1.0f : a.scale_log2;  // what is left to apply to s0..s3
                    {
                        float lm0 = fmaxf(s0, s2), lm1 = fmaxf(s1, s3);
                        const bool need = (lm0 > thr0) || (lm1 > thr1);
                        if (__any_sync(0xffffffffu, need)) {
    #pragma unroll
                            for (int off = 4; off <= 16; off <<= 1) {
                                lm0 = fmaxf(lm0, __shfl_xor_sync(0xffffffffu, lm0, off));
                                lm1 = fmaxf(lm1, __shfl_xor_sync(0xffffffffu, lm1, off));
                            }
                            const float n0 = fmaxf(m0, lm0 * sc), n1 = fmaxf(m1, lm1 * sc);
                            const float r0 = ex2_approx(m0 - n0), r1 = ex2_approx(m1 - n1);
                            m0 = n0;
                            m1 = n1;
                            thr0 = (m0 + kRescaleSlack) * inv_sc;
                            thr1 = (m1 + kRescaleSlack) * inv_sc;
                            l0 *= r0;
                            l1 *= r1;
    #pragma unroll
                            for (int i = 0; i < T::kMTiles; ++i) {
                                o[i][0] *= r0;
                                o[i][1] *= r1;
                                o[i][2] *= r0;
                                o[i][3] *= r1;
                            }
                        }
                    }
                    const float p0 = ex2_approx(fmaf(s0, sc, -m0)), p1 = ex2_approx(fmaf(s1, sc, -m1));
                    const float p2 = ex2_approx(fmaf(s2, sc, -m0)), p3 = ex2_approx(fmaf(s3, sc, -m1));
                    // The MMA consumes P rounded to fp16, so the normaliser sums the SAME rounded values: a
                    // rounding of p then cancels between numerator and denominator (exactly so when one token
                    // dominates), which keeps the output within one fp16 ulp of an fp32 evaluation.
                    const __half2 ph01 = __floats2half2_rn(p0, p1), ph23 = __floats2half2_rn(p2, p3);
                    add_halves_to_floats(l0, l1, h2_as_u32(ph01));
                    add_halves_to_floats(l0, l1, h2_as_u32(ph23));
                    // P^T as the B operand of the second MMA: k = token, n = head
                    pb0 = movmatrix_trans(h2_as_u32(ph01));
                    pb1 = movmatrix_trans(h2_as_u32(ph23));
                }

                // ---------------- O^T += V^T * P^T ----------------
                {
                    uint32_t va[T::kVRegs], vb[T::kVRegs], vcw[T::kVRegs], vd[T::kVRegs];
                    uint32_t sca, scb, scc, scd;  // scales of the thread's channel groups, per token
                    if constexpr (DH == 128) {
                        const uint4 xa = lds128(st + v_off_a);
                        const uint4 xb = lds128(st + v_off_b);
                        const uint4 xc = lds128(st + v_off_a + 1024u);
                        const uint4 xd = lds128(st + v_off_b + 1024u);
                        va[0] = xa.x; va[1] = xa.y; va[2] = xa.z; va[3] = xa.w;
                        vb[0] = xb.x; vb[1] = xb.y; vb[2] = xb.z; vb[3] = xb.w;
                        vcw[0] = xc.x; vcw[1] = xc.y; vcw[2] = xc.z; vcw[3] = xc.w;
                        vd[0] = xd.x; vd[1] = xd.y; vd[2] = xd.z; vd[3] = xd.w;
                        sca = lds32(st + vs_off);
                        scb = lds32(st + vs_off + 32u);
                        scc = lds32(st + vs_off + 256u);
                        scd = lds32(st + vs_off + 288u);
                    } else {
                        const uint2 xa = lds64(st + v_off_a);
                        const uint2 xb = lds64(st + v_off_b);
                        const uint2 xc = lds64(st + v_off_a + 512u);
                        const uint2 xd = lds64(st + v_off_b + 512u);
                        va[0] = xa.x; va[1] = xa.y;
                        vb[0] = xb.x; vb[1] = xb.y;
                        vcw[0] = xc.x; vcw[1] = xc.y;
                        vd[0] = xd.x; vd[1] = xd.y;
                        sca = lds16(st + vs_off);
                        scb = lds16(st + vs_off + 16u);
                        scc = lds16(st + vs_off + 128u);
                        scd = lds16(st + vs_off + 144u);
                    }
                    if (nvalid < kTileTok) {
                        // rows past the end of the sequence hold other data (or nothing): their scales may be
                        // anything, and 0 * NaN would poison the accumulator even though P is exactly 0 there
                        sca = 2 * t < nvalid ? sca : 0u;
                        scb = 2 * t + 1 < nvalid ? scb : 0u;
                        scc = 2 * t + 8 < nvalid ? scc : 0u;
                        scd = 2 * t + 9 < nvalid ? scd : 0u;
                    }
#pragma unroll
                    for (int q = 0; q < T::kVRegs; ++q) {
                        // word q holds channels 4q..4q+3 of the thread's slab: group q/2 of the slab
                        const uint32_t sel = (q & 2) ? 0x7632u : 0x5410u;
                        const __half2 s_ab = u32_as_h2(prmt(sca, scb, sel));
                        const __half2 s_cd = u32_as_h2(prmt(scc, scd, sel));
                        uint32_t hab[4], hcd[4];
                        dequant_v_pair(va[q], vb[q], s_ab, hab);
                        dequant_v_pair(vcw[q], vd[q], s_cd, hcd);
                        mma_m16n8k16_f16f32(o[2 * q], hab[0], hab[1], hcd[0], hcd[1], pb0, pb1);
                        mma_m16n8k16_f16f32(o[2 * q + 1], hab[2], hab[3], hcd[2], hcd[3], pb0, pb1);
                    }
                }

                if (lockstep) {  // the warps that share this range (same tile count) meet after every tile
                    asm volatile("bar.sync %0, %1;" ::"r"(1 + sub), "r"(head_lanes * 32) : "memory");
                }
                __syncwarp();  // every lane has read this stage: it may be refilled
                if (++c_stage == kStages) {
                    c_stage = 0;
                    c_phase ^= 1u;
                }
                if (to_issue > 0) {  // never after the warp has given up
                    issue_one();
                }
            }

            // ---------------- end of the piece: write fp16 output or an fp32 partial ----------------
            if constexpr (KDOT) {  // columns 1.. of the fragments are copies of head 0's
                m1 = m0;
                l1 = l0;
            }
#pragma unroll
            for (int off = 4; off <= 16; off <<= 1) {
                l0 += __shfl_xor_sync(0xffffffffu, l0, off);
                l1 += __shfl_xor_sync(0xffffffffu, l1, off);
            }
            const bool complete = (t_first == 0) && (t_end == cc.n);
            // a range holds at most two partial pieces: its first piece (slot 0) and, if a different one, its
            // last piece (slot 1)
            const int64_t slot =
                (static_cast<int64_t>(r) * head_lanes + cls) * 2 + ((t_first > 0 || first_piece) ? 0 : 1);
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int h8 = 2 * t + hh;
                const int hq_in_group = oct * 8 + h8;
                if (hq_in_group >= a.group) {
                    continue;
                }
                const float lsum = hh ? l1 : l0;
                if (complete) {
                    const float inv = lsum > 0.0f ? 1.0f / lsum : 0.0f;
                    __half* dst = a.out + (qtok * a.num_heads + kvh * a.group + hq_in_group) * DH + (DH / 8) * g;
#pragma unroll
                    for (int jj = 0; jj < T::kMTiles / 4; ++jj) {
                        uint4 v;
                        v.x = h2_as_u32(__floats2half2_rn(o[4 * jj][hh] * inv, o[4 * jj][hh + 2] * inv));
                        v.y = h2_as_u32(__floats2half2_rn(o[4 * jj + 1][hh] * inv, o[4 * jj + 1][hh + 2] * inv));
                        v.z = h2_as_u32(__floats2half2_rn(o[4 * jj + 2][hh] * inv, o[4 * jj + 2][hh + 2] * inv));
                        v.w = h2_as_u32(__floats2half2_rn(o[4 * jj + 3][hh] * inv, o[4 * jj + 3][hh + 2] * inv));
                        *reinterpret_cast<uint4*>(dst + 8 * jj) = v;
                    }
                } else {
                    float* dst = a.part_o + (slot * 8 + h8) * DH + (DH / 8) * g;
#pragma unroll
                    for (int jj = 0; jj < T::kMTiles / 2; ++jj) {
                        *reinterpret_cast<float4*>(dst + 4 * jj) =
                            make_float4(o[2 * jj][hh], o[2 * jj][hh + 2], o[2 * jj + 1][hh], o[2 * jj + 1][hh + 2]);
                    }
                    if (g == 0) {
                        a.part_ml[(slot * 8 + h8) * 2] = hh ? m1 : m0;
                        a.part_ml[(slot * 8 + h8) * 2 + 1] = lsum;
                    }
                }
            }
            to_consume -= t_end - t_first;
            first_piece = false;
            advance(cc, t_end - t_first);
        }
    }
    if (wait_dead) {
        // Copies that were in flight when the warp gave up may still land in this CTA's shared memory: give
        // each of them one more bounded wait (from the ring position recorded then) before the CTA may exit.
        for (int32_t i = 0; i < dead_inflight && i < kStages; ++i) {
            mbar_wait_bounded(reinterpret_cast<uint64_t*>(full_bar + warp * kStages + dead_stage), dead_phase);
            if (++dead_stage == kStages) {
                dead_stage = 0;
                dead_phase ^= 1u;
            }
        }
    }
}

// ------------------------------------------------------------------------------------------
// Second pass: merge the fp32 partials of segments that were cut by range boundaries.  One warp per
// (sequence, query head).
// ------------------------------------------------------------------------------------------
template <int DH>
__global__ void __launch_bounds__(256)
decode_reduce_kernel(const PlanHeader* __restrict__ hdr, const int32_t* __restrict__ tile_prefix,
                     const float* __restrict__ part_ml, const float* __restrict__ part_o,
                     const int64_t* __restrict__ seqstarts, __half* __restrict__ out, int32_t decoding_batches,
                     int32_t num_heads, int32_t group, int32_t octets, int32_t head_lanes, int32_t class_heads) {
    grid_launch_dependents();
    // The plan (header, tile prefix sums) was complete before the decode grid let this grid be scheduled, so
    // the segment geometry is worked out first; only the partials need the decode grid to have finished.
    const int64_t wg = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (hdr->per_segment || wg >= static_cast<int64_t>(decoding_batches) * num_heads) {
        return;  // split-k off (every segment was written whole), or no such (sequence, head)
    }
    const int32_t b = static_cast<int32_t>(wg / num_heads);
    const int32_t qh = static_cast<int32_t>(wg - static_cast<int64_t>(b) * num_heads);
    const int32_t kvh = qh / group;
    const int32_t hq = qh - kvh * group;
    const int32_t vh = kvh * octets + (hq >> 3);
    const int32_t h8 = hq & 7;
    const int64_t R = hdr->range_tiles;
    const int32_t n = tile_prefix[b + 1] - tile_prefix[b];
    const int32_t cls = vh % head_lanes;
    const int32_t vc = vh / head_lanes;
    const int64_t seg_lo = static_cast<int64_t>(tile_prefix[b]) * class_heads + static_cast<int64_t>(vc) * n;
    const int64_t seg_hi = seg_lo + n;
    const int64_t r_first = seg_lo / R;
    const int64_t r_last = (seg_hi - 1) / R;
    if (r_first == r_last) {
        return;  // the segment lies inside one range and was written whole
    }
    grid_dependency_wait();  // the partials of the decode grid
    auto slot_of = [&](int64_t rr) -> int64_t {
        // the piece is the range's first piece unless the segment starts strictly inside the range
        const int64_t s = (rr == r_first && seg_lo > rr * R) ? 1 : 0;
        return ((rr * head_lanes + cls) * 2 + s) * 8 + h8;
    };
    float mx = kNegBig;
    for (int64_t rr = r_first + lane; rr <= r_last; rr += 32) {
        mx = fmaxf(mx, part_ml[slot_of(rr) * 2]);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    }
    // Up to 32 pieces at a time: lane i works out the weight and the slot of piece i, then the warp walks
    // the pieces four at a time so that the loads of four partial rows are in flight together.
    constexpr int kPer = DH / 32;
    float acc[kPer];
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
        acc[i] = 0.0f;
    }
    float den = 0.0f;
    for (int64_t base = r_first; base <= r_last; base += 32) {
        const int64_t rr = base + lane;
        const bool valid = rr <= r_last;
        const int64_t my_slot = valid ? slot_of(rr) : 0;
        float w = 0.0f;
        if (valid) {
            const float2 ml = *reinterpret_cast<const float2*>(part_ml + my_slot * 2);
            w = ex2_approx(ml.x - mx);
            den += w * ml.y;
        }
        const int cnt = static_cast<int>(r_last - base + 1 < 32 ? r_last - base + 1 : 32);
        for (int j = 0; j < cnt; j += 4) {
            float wj[4];
            float v[4][kPer];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                wj[u] = __shfl_sync(0xffffffffu, w, (j + u) & 31);
                const int64_t sl = __shfl_sync(0xffffffffu, my_slot, (j + u) & 31);
                const float* po = part_o + sl * DH + lane * kPer;
#pragma unroll
                for (int i = 0; i < kPer; ++i) {
                    v[u][i] = 0.0f;
                }
                if (j + u < cnt) {  // nothing is read past the last piece: unwritten slots may hold anything
                    if constexpr (kPer == 4) {
                        const float4 t4 = *reinterpret_cast<const float4*>(po);
                        v[u][0] = t4.x; v[u][1] = t4.y; v[u][2] = t4.z; v[u][3] = t4.w;
                    } else {
                        const float2 t2 = *reinterpret_cast<const float2*>(po);
                        v[u][0] = t2.x; v[u][1] = t2.y;
                    }
                } else {
                    wj[u] = 0.0f;
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
#pragma unroll
                for (int i = 0; i < kPer; ++i) {
                    acc[i] += wj[u] * v[u][i];
                }
            }
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        den += __shfl_xor_sync(0xffffffffu, den, off);
    }
    const float inv = den > 0.0f ? 1.0f / den : 0.0f;
    __half* dst = out + (seqstarts[b] * num_heads + qh) * DH + lane * kPer;
    if constexpr (kPer == 4) {
        uint2 o2;
        o2.x = h2_as_u32(__floats2half2_rn(acc[0] * inv, acc[1] * inv));
        o2.y = h2_as_u32(__floats2half2_rn(acc[2] * inv, acc[3] * inv));
        *reinterpret_cast<uint2*>(dst) = o2;
    } else {
        *reinterpret_cast<__half2*>(dst) = __floats2half2_rn(acc[0] * inv, acc[1] * inv);
    }
}

uint64_t align_up_u64(uint64_t x, uint64_t a) {
    return (x + a - 1) / a * a;
}

}  // namespace

// ------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------
int decode_oversubscription();
int make_decode_plan(const pplb200_attn_params& p, int sm_count, DecodePlan* plan) {
    DecodePlan& d = *plan;
    const int64_t DB = p.decoding_batches;
    const int group = p.num_heads / p.num_kv_heads;
    d.octets = (group + 7) / 8;
    d.num_vheads = static_cast<int64_t>(p.num_kv_heads) * d.octets;
    d.head_lanes = 1;
    for (int hl = kWarps; hl > 1; hl >>= 1) {  // the largest power of two <= kWarps that divides the head count
        if (d.num_vheads % hl == 0) {
            d.head_lanes = hl;
            break;
        }
    }
    d.class_heads = d.num_vheads / d.head_lanes;
    d.grid = static_cast<int64_t>(sm_count) * kCtasPerSm;
    // Ranges per resident warp of a class.  More than one trades extra split partials for a shorter tail
    // (ranges are handed out dynamically, so warps that fall behind take fewer of them).
    d.workers = d.grid * (kWarps / d.head_lanes) * decode_oversubscription();
    // upper bound of the number of ranges (per class) the planning kernel may create
    if (p.split_k_mode == 0 || DB == 0) {
        d.max_ranges = DB * d.class_heads;
        d.partial_slots = 0;
    } else {
        d.max_ranges = d.workers;
        if (p.split_k_mode == 2 && 2 * DB * d.class_heads + 1 > d.max_ranges) {
            d.max_ranges = 2 * DB * d.class_heads + 1;
        }
        d.partial_slots = 2 * d.max_ranges * d.head_lanes;
    }
    uint64_t off = 0;
    d.off_header = off;  // the status word is the first word of the header
    off = 256;
    d.off_tile_prefix = off;
    off = align_up_u64(off + static_cast<uint64_t>(DB + 1) * 4, 256);
    d.off_part_ml = off;
    off = align_up_u64(off + static_cast<uint64_t>(d.partial_slots) * 8 * 2 * 4, 256);
    d.off_part_o = off;
    off = align_up_u64(off + static_cast<uint64_t>(d.partial_slots) * 8 * p.head_dim * 4, 256);
    d.bytes = off;
    return PPLB200_SUCCESS;
}

int decode_oversubscription() {
    const char* e = getenv("PPLB200_DECODE_OVERSUB");  // tuning only; read per call so that a sweep can change it
    const int n = e ? atoi(e) : 0;
    return (n >= 1 && n <= 16) ? n : PPLB200_DECODE_OVERSUB_DEFAULT;
}

// PPLB200_DECODE_KDOT=0 sends one-head-per-kv-head batches through the tensor-core scores as well (A/B
// measurements only; read per call).
static bool decode_kdot_enabled() {
    const char* e = getenv("PPLB200_DECODE_KDOT");
    return !(e && e[0] == '0');
}

static int map_order_kind(const CacheMapOrder& od) {
    if (od.pos_head == 1 && od.pos_kv == 2 && od.pos_layer == 3 && od.pos_row == 4) {
        return kOrderRowLast;
    }
    if (od.pos_row == 1 && od.pos_head == 2 && od.pos_kv == 3 && od.pos_layer == 4) {
        return kOrderRowFirst;
    }
    return kOrderGeneric;
}

template <int DH, int ORDER, bool MASK, bool KDOT>
static int launch_main(const CUtensorMap& tm_codes, const DecodeArgs& a, int64_t grid, cudaStream_t stream) {
    using T = Traits<DH>;
    // the attribute belongs to the (kernel, device) pair: remembered per template instance and device
    static bool attr_set_on[kMaxDevices] = {};
    int dev_id = 0;
    if (cudaGetDevice(&dev_id) != cudaSuccess || dev_id < 0 || dev_id >= kMaxDevices) {
        return PPLB200_DEVICE_RUNTIME_ERROR;
    }
    bool& attr_set = attr_set_on[dev_id];
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(decode_splitk_kernel<DH, ORDER, MASK, KDOT>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, T::kSmemBytes);
        if (e != cudaSuccess) {
            fprintf(stderr, "[ppl_nn_b200] cudaFuncSetAttribute(decode_splitk_kernel): %s\n", cudaGetErrorString(e));
            return PPLB200_DEVICE_RUNTIME_ERROR;
        }
        attr_set = true;
    }
    {
        KernelTimer timer(PPLB200_KERNEL_DECODE, stream);
        launch_dependent(decode_splitk_kernel<DH, ORDER, MASK, KDOT>, dim3(static_cast<unsigned>(grid)), dim3(kThreads),
                         T::kSmemBytes, stream, tm_codes, a);
    }
    return check_launch("decode_splitk_kernel");
}

// Whether the warps that share a range run in lockstep (a barrier per tile).  Measured on B200, 8 head
// lanes: with a multi-layer token-major cache or the head-major layout the lockstep raises the decode
// bandwidth by 5-7 % (6.25 -> 6.57 TB/s with 8 layers, 6.25 -> 6.69 TB/s head-major, LLaMA-2-7B decode
// workload); where the token rows of the layer lie back to back (one layer, token-major) it costs 3-4 %.
// PPLB200_DECODE_LOCKSTEP=0|1 in the environment overrides the rule (tuning only).
static bool want_lockstep(const pplb200_attn_params& p, const DecodePlan& plan) {
    if (plan.head_lanes <= 1) {
        return false;
    }
    static const int forced = [] {
        const char* e = getenv("PPLB200_DECODE_LOCKSTEP");
        return (e && (e[0] == '0' || e[0] == '1')) ? e[0] - '0' : -1;
    }();
    if (forced >= 0) {
        return forced == 1;
    }
    const bool rows_back_to_back = p.cache_stride_s == 2 * static_cast<int64_t>(p.num_kv_heads) * p.head_dim;
    return !rows_back_to_back;
}

template <int DH>
static int launch_decode_dh(const pplb200_attn_params& p, const CacheGeom& geom, const DecodePlan& plan,
                            const void* query, const void* append_key, const void* append_value,
                            const int64_t* seqstarts, const int64_t* cachestarts, const int64_t* start_pos,
                            void* cache, void* scale, const MaskDev& mask, void* workspace, void* attn_output,
                            cudaStream_t stream) {
    static_assert(sizeof(PlanHeader) <= 256, "the header must fit in front of the prefix sums");
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    PlanHeader* hdr = reinterpret_cast<PlanHeader*>(ws + plan.off_header);
    int32_t* tile_prefix = reinterpret_cast<int32_t*>(ws + plan.off_tile_prefix);

    CUtensorMap tm_codes;
    CacheMapOrder order;
    int rc = make_cache_tensor_map(p, cache, kTileTok, &tm_codes, &order);
    if (rc != PPLB200_SUCCESS) {
        return rc;
    }

    // never more CTAs than there can be ranges
    int64_t grid = plan.grid;
    const int64_t per_cta = kWarps / plan.head_lanes;
    if ((plan.max_ranges + per_cta - 1) / per_cta < grid) {
        grid = (plan.max_ranges + per_cta - 1) / per_cta;
    }
    launch_dependent(decode_plan_kernel, dim3(1), dim3(kPlanThreads), 0, stream, seqstarts, start_pos,
                     static_cast<int32_t>(p.decoding_batches), static_cast<int32_t>(plan.class_heads), p.max_kvlen,
                     p.split_k_mode, static_cast<int32_t>(plan.workers), static_cast<int32_t>(plan.max_ranges),
                     static_cast<int32_t>(grid * per_cta), hdr, tile_prefix);
    rc = check_launch("decode_plan_kernel");
    if (rc != PPLB200_SUCCESS) {
        return rc;
    }

    DecodeArgs a;
    a.q = static_cast<const __half*>(query);
    a.out = static_cast<__half*>(attn_output);
    a.seqstarts = seqstarts;
    a.cachestarts = cachestarts;
    a.start_pos = start_pos;
    a.hdr = hdr;
    a.tile_prefix = tile_prefix;
    a.part_ml = reinterpret_cast<float*>(ws + plan.off_part_ml);
    a.part_o = reinterpret_cast<float*>(ws + plan.off_part_o);
    a.geom = geom;
    a.max_kvlen = p.max_kvlen;
    a.decoding_batches = static_cast<int32_t>(p.decoding_batches);
    a.num_heads = p.num_heads;
    a.group = p.num_heads / p.num_kv_heads;
    a.octets = plan.octets;
    a.head_lanes = plan.head_lanes;
    a.class_heads = static_cast<int32_t>(plan.class_heads);
    a.layer_idx = p.layer_idx;
    a.lockstep = want_lockstep(p, plan) ? 1 : 0;
    a.order = order;
    a.scale = static_cast<const __half*>(scale);
    a.max_tokens = p.max_tokens;
    a.scale_log2 = 1.4426950408889634f / sqrtf(static_cast<float>(DH));
    a.cur_k = static_cast<const __half*>(append_key);
    a.cur_v = static_cast<const __half*>(append_value);
    a.cache = static_cast<int8_t*>(cache);
    a.num_kv_heads = p.num_kv_heads;
    a.mask = mask;

    if (a.mask.data != nullptr) {  // the mask path need not be the fastest: one instance, run-time coordinate order
        rc = launch_main<DH, kOrderGeneric, true, false>(tm_codes, a, grid, stream);
    } else if (a.group == 1 && decode_kdot_enabled()) {  // one query head per kv head: integer-dot scores
        switch (map_order_kind(order)) {
            case kOrderRowLast: rc = launch_main<DH, kOrderRowLast, false, true>(tm_codes, a, grid, stream); break;
            case kOrderRowFirst: rc = launch_main<DH, kOrderRowFirst, false, true>(tm_codes, a, grid, stream); break;
            default: rc = launch_main<DH, kOrderGeneric, false, true>(tm_codes, a, grid, stream); break;
        }
    } else {
        switch (map_order_kind(order)) {
            case kOrderRowLast: rc = launch_main<DH, kOrderRowLast, false, false>(tm_codes, a, grid, stream); break;
            case kOrderRowFirst: rc = launch_main<DH, kOrderRowFirst, false, false>(tm_codes, a, grid, stream); break;
            default: rc = launch_main<DH, kOrderGeneric, false, false>(tm_codes, a, grid, stream); break;
        }
    }
    if (rc != PPLB200_SUCCESS) {
        return rc;
    }
    if (p.split_k_mode != 0) {
        const int64_t warps = p.decoding_batches * p.num_heads;
        const unsigned blocks = static_cast<unsigned>((warps + 7) / 8);
        launch_dependent(decode_reduce_kernel<DH>, dim3(blocks), dim3(256), 0, stream,
                         static_cast<const PlanHeader*>(hdr), static_cast<const int32_t*>(tile_prefix),
                         static_cast<const float*>(a.part_ml), static_cast<const float*>(a.part_o), seqstarts, a.out,
                         a.decoding_batches, p.num_heads, a.group, a.octets, a.head_lanes, a.class_heads);
        rc = check_launch("decode_reduce_kernel");
    }
    return rc;
}

int launch_decode(const pplb200_attn_params& p, const CacheGeom& geom, const DecodePlan& plan, const void* query,
                  const void* append_key, const void* append_value, const int64_t* seqstarts,
                  const int64_t* cachestarts, const int64_t* start_pos, void* cache, void* scale, const MaskDev& mask,
                  void* workspace, void* attn_output, cudaStream_t stream) {
    if (p.decoding_batches <= 0) {
        return PPLB200_SUCCESS;
    }
    if ((append_key == nullptr) != (append_value == nullptr)) {
        return PPLB200_INVALID_VALUE;
    }
    if (p.head_dim == 128) {
        return launch_decode_dh<128>(p, geom, plan, query, append_key, append_value, seqstarts, cachestarts, start_pos,
                                     cache, scale, mask, workspace, attn_output, stream);
    }
    if (p.head_dim == 64) {
        return launch_decode_dh<64>(p, geom, plan, query, append_key, append_value, seqstarts, cachestarts, start_pos,
                                    cache, scale, mask, workspace, attn_output, stream);
    }
    return PPLB200_UNSUPPORTED;
}

}  // namespace pplb200
