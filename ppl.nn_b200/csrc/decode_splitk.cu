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
//   * Every warp is an independent worker with its own TMA pipeline: one lane issues four bulk-tensor
//     copies per tile (K codes, V codes, K scales, V scales; 5 KB at head_dim 128) that complete on
//     an mbarrier; the pipeline runs across segment boundaries without draining.  There is no
//     block-level synchronisation after start-up.
//   * Per tile the warp computes S^T[16 tokens x 8 heads] = K[16 x Dh] * Q^T with mma.m16n8k16
//     (tokens are the M dimension, the up-to-8 query heads of the group the N dimension),
//     dequantising K in registers: a byte permute builds the half 1024+u from each code byte, a
//     subtract gives the code exactly, a multiply applies the group scale.  Softmax runs in fp32 in the
//     exp2 domain with a lazily updated reference maximum; P^T is transposed between lanes with
//     movmatrix and O^T[Dh x 8 heads] += V^T * P^T follows, with V dequantised the same way (two
//     tokens are interleaved into one half2 by a permute).
//
// Every wait on an mbarrier is bounded; on a timeout the warp records a status code, stops
// waiting and finishes (with wrong numbers, flagged) instead of hanging.
#include <cuda.h>

#include <cub/block/block_scan.cuh>

#include "common.cuh"
#include "launch.h"
#include "tensor_map.h"

namespace pplb200 {

namespace {

constexpr int kTileTok = 16;
constexpr int kStages = 4;
constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
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
    static constexpr bool kSwizzle = (DH == 128);                  // 128-byte rows use the 128B TMA swizzle
    static_assert(8 * DH * 4 + 64 <= kWarpBytes, "merge buffer must fit in the warp's stage buffers");
};

struct DecodeArgs {
    const __half* q;
    __half* out;
    const int64_t* seqstarts;
    const int64_t* cachestarts;
    const int64_t* start_pos;
    uint32_t* status;
    int32_t* counter;
    const int32_t* split_starts;
    float* part_ml;
    float* part_o;
    CacheGeom geom;
    int64_t chunk_tokens;
    int64_t max_kvlen;
    int32_t decoding_batches;
    int32_t num_heads;
    int32_t num_kv_heads;
    int32_t group;
    int32_t octets;
    int32_t head_warps;
    int32_t token_warps;
    int32_t num_hsets;
    int32_t layer_idx;
    CacheMapOrder order;
    float scale_log2;
};

// One head's tile of `kTileTok` cache rows, through a map whose outer dimensions are ordered by
// stride (see CacheMapOrder).
__device__ __forceinline__ void tma_load_cache_tile(void* dst, const CUtensorMap* map, uint64_t* bar,
                                                    const CacheMapOrder& od, int row, int head, int kv, int layer) {
    int c[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int pos = i + 1;
        c[i] = od.pos_row == pos ? row : (od.pos_head == pos ? head : (od.pos_kv == pos ? kv : layer));
    }
    tma_load_5d(dst, map, bar, 0, c[0], c[1], c[2], c[3]);
}

// ------------------------------------------------------------------------------------------
// Planning kernel: split counts per decode sequence -> exclusive prefix sum; resets the work
// counter and the status word.  One CTA.
// ------------------------------------------------------------------------------------------
constexpr int kPlanThreads = 512;

__global__ void __launch_bounds__(kPlanThreads)
decode_plan_kernel(const int64_t* __restrict__ seqstarts, const int64_t* __restrict__ start_pos,
                   int32_t decoding_batches, int64_t chunk_tokens, int64_t max_kvlen,
                   int32_t* __restrict__ split_starts, int32_t* __restrict__ counter, uint32_t* __restrict__ status,
                   int reset_status) {
    using Scan = cub::BlockScan<int32_t, kPlanThreads>;
    __shared__ typename Scan::TempStorage tmp;
    __shared__ int32_t carry;
    if (threadIdx.x == 0) {
        carry = 0;
        *counter = 0;
        if (reset_status) {
            *status = 0;
        }
    }
    __syncthreads();
    for (int32_t base = 0; base < decoding_batches; base += kPlanThreads) {
        const int32_t b = base + threadIdx.x;
        int32_t n = 0;
        if (b < decoding_batches) {
            int64_t kvlen = start_pos[b] + (seqstarts[b + 1] - seqstarts[b]);
            if (kvlen > max_kvlen) {
                kvlen = max_kvlen;
                atomicOr(status, kDevLengthClamped);
            }
            if (kvlen < 1) {
                kvlen = 1;  // an empty sequence still owns one (empty) split so that its output is written
            }
            n = static_cast<int32_t>((kvlen + chunk_tokens - 1) / chunk_tokens);
        }
        int32_t excl, total;
        Scan(tmp).ExclusiveSum(n, excl, total);
        const int32_t c = carry;
        if (b < decoding_batches) {
            split_starts[b] = c + excl;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            carry = c + total;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        split_starts[decoding_batches] = carry;
    }
}

// ------------------------------------------------------------------------------------------
// Main kernel
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 lds128(const uint8_t* p) {
    return *reinterpret_cast<const uint4*>(p);
}

// K codes word -> two half2 (channels 0,1 and 2,3 of the word), scaled.
__device__ __forceinline__ void dequant_k_word(uint32_t w, __half2 s2, uint32_t& lo, uint32_t& hi) {
    const uint32_t x = w ^ 0x80808080u;
    lo = h2_as_u32(__hmul2(biased_bytes_to_half2<0x5140u>(x), s2));
    hi = h2_as_u32(__hmul2(biased_bytes_to_half2<0x5342u>(x), s2));
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

template <int DH>
__global__ void __launch_bounds__(kThreads, 2)
decode_splitk_kernel(const __grid_constant__ CUtensorMap tmap_codes, const __grid_constant__ CUtensorMap tmap_scales,
                     const DecodeArgs a) {
    using T = Traits<DH>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t full_bar[kWarps * kStages];
    __shared__ int32_t s_item;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2;
    const int t = lane & 3;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kWarps * kStages; ++i) {
            mbar_init(&full_bar[i], 1);
        }
        mbar_fence_init();
        tma_prefetch_desc(&tmap_codes);
        tma_prefetch_desc(&tmap_scales);
    }
    __syncthreads();

    uint8_t* wsm = smem + warp * T::kWarpBytes;
    uint64_t* wbar = full_bar + warp * kStages;
    uint32_t tiles_done = 0;  // tiles this warp has consumed so far: selects stage and barrier parity
    bool wait_dead = false;   // set after the first timed-out wait: stop waiting, just finish

    const int HW = a.head_warps;
    const int TW = a.token_warps;
    const int head_sub = warp % HW;
    const int tw = warp / HW;

    const int32_t total_splits = a.split_starts[a.decoding_batches];
    const int64_t total_items = static_cast<int64_t>(total_splits) * a.num_hsets;

    for (;;) {
        if (threadIdx.x == 0) {
            s_item = atomicAdd(a.counter, 1);
        }
        __syncthreads();
        const int64_t item = s_item;
        if (item >= total_items) {
            break;
        }
        const int hset = static_cast<int>(item % a.num_hsets);
        const int32_t j = static_cast<int32_t>(item / a.num_hsets);
        // sequence that owns global split j: largest b with split_starts[b] <= j
        int32_t lo = 0, hi = a.decoding_batches;
        while (hi - lo > 1) {
            const int32_t mid = (lo + hi) >> 1;
            if (a.split_starts[mid] <= j) {
                lo = mid;
            } else {
                hi = mid;
            }
        }
        const int32_t b = lo;
        const int32_t first_split = a.split_starts[b];
        const int32_t nsplits = a.split_starts[b + 1] - first_split;
        const int32_t split = j - first_split;
        const int64_t qtok = a.seqstarts[b];
        int64_t kvlen = a.start_pos[b] + (a.seqstarts[b + 1] - qtok);
        kvlen = kvlen > a.max_kvlen ? a.max_kvlen : kvlen;
        const int64_t t0 = static_cast<int64_t>(split) * a.chunk_tokens;
        int64_t t1 = t0 + a.chunk_tokens;
        t1 = t1 > kvlen ? kvlen : t1;
        const int32_t ntiles = t1 > t0 ? static_cast<int32_t>((t1 - t0 + kTileTok - 1) / kTileTok) : 0;
        const int32_t my_n = ntiles > tw ? (ntiles - tw + TW - 1) / TW : 0;

        const int vhead = hset * HW + head_sub;
        const int kvh = vhead / a.octets;
        const int oct = vhead - kvh * a.octets;

        // ---- Q fragments (B operand: k = channel, n = query head of the group) ----
        uint32_t qf[T::kKRegs][2];
        {
            const int hq_in_group = oct * 8 + g;
            if (hq_in_group < a.group) {
                const __half* qp =
                    a.q + (qtok * a.num_heads + kvh * a.group + hq_in_group) * DH + t * (DH / 4);
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

        const uint32_t base_seq = tiles_done;
        auto issue = [&](int32_t local_idx) {
            const int64_t tok = t0 + static_cast<int64_t>(tw + local_idx * TW) * kTileTok;
            const int row = static_cast<int>(cache_row(a.geom, a.cachestarts, b, tok));
            const uint32_t stage = (base_seq + local_idx) % kStages;
            uint8_t* st = wsm + stage * T::kStageBytes;
            uint64_t* bar = &wbar[stage];
            mbar_arrive_expect_tx(bar, T::kStageBytes);
            tma_load_cache_tile(st, &tmap_codes, bar, a.order, row, kvh, 0, a.layer_idx);
            tma_load_cache_tile(st + T::kCodeBytes, &tmap_codes, bar, a.order, row, kvh, 1, a.layer_idx);
            tma_load_cache_tile(st + 2 * T::kCodeBytes, &tmap_scales, bar, a.order, row, kvh, 0, a.layer_idx);
            tma_load_cache_tile(st + 2 * T::kCodeBytes + T::kScaleBytes, &tmap_scales, bar, a.order, row, kvh, 1,
                                a.layer_idx);
        };

        if (lane == 0) {
            const int32_t npre = my_n < kStages ? my_n : kStages;
            for (int32_t i = 0; i < npre; ++i) {
                issue(i);
            }
        }

        for (int32_t i = 0; i < my_n; ++i) {
            const uint32_t seq = base_seq + i;
            const uint32_t stage = seq % kStages;
            if (!wait_dead) {
                if (!mbar_wait_bounded(&wbar[stage], (seq / kStages) & 1u)) {
                    wait_dead = true;
                    if (lane == 0) {
                        atomicOr(a.status, kDevTmaTimeout);
                    }
                }
            }
            const uint8_t* st = wsm + stage * T::kStageBytes;
            const uint8_t* kc = st;
            const uint8_t* vc = st + T::kCodeBytes;
            const uint8_t* ks = st + 2 * T::kCodeBytes;
            const uint8_t* vs = ks + T::kScaleBytes;
            const int64_t tok0 = t0 + static_cast<int64_t>(tw + i * TW) * kTileTok;
            const int nvalid = (t1 - tok0) < kTileTok ? static_cast<int>(t1 - tok0) : kTileTok;

            // ---------------- S^T = K * Q^T ----------------
            float sacc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            {
                uint32_t wa[T::kKRegs], wb[T::kKRegs];  // rows g and g+8, this thread's channel slab
                uint32_t sa[T::kKRegs / 4], sb[T::kKRegs / 4];  // packed group scales (2 halves per word)
                if constexpr (DH == 128) {
                    const uint4 a0 = lds128(kc + g * 128 + (((2 * t) ^ g) << 4));
                    const uint4 a1 = lds128(kc + g * 128 + (((2 * t + 1) ^ g) << 4));
                    const uint4 b0 = lds128(kc + (g + 8) * 128 + (((2 * t) ^ g) << 4));
                    const uint4 b1 = lds128(kc + (g + 8) * 128 + (((2 * t + 1) ^ g) << 4));
                    wa[0] = a0.x; wa[1] = a0.y; wa[2] = a0.z; wa[3] = a0.w;
                    wa[4] = a1.x; wa[5] = a1.y; wa[6] = a1.z; wa[7] = a1.w;
                    wb[0] = b0.x; wb[1] = b0.y; wb[2] = b0.z; wb[3] = b0.w;
                    wb[4] = b1.x; wb[5] = b1.y; wb[6] = b1.z; wb[7] = b1.w;
                    const uint2 s_a = *reinterpret_cast<const uint2*>(ks + g * 32 + t * 8);
                    const uint2 s_b = *reinterpret_cast<const uint2*>(ks + (g + 8) * 32 + t * 8);
                    sa[0] = s_a.x; sa[1] = s_a.y;
                    sb[0] = s_b.x; sb[1] = s_b.y;
                } else {
                    const uint4 a0 = lds128(kc + g * 64 + t * 16);
                    const uint4 b0 = lds128(kc + (g + 8) * 64 + t * 16);
                    wa[0] = a0.x; wa[1] = a0.y; wa[2] = a0.z; wa[3] = a0.w;
                    wb[0] = b0.x; wb[1] = b0.y; wb[2] = b0.z; wb[3] = b0.w;
                    sa[0] = *reinterpret_cast<const uint32_t*>(ks + g * 16 + t * 4);
                    sb[0] = *reinterpret_cast<const uint32_t*>(ks + (g + 8) * 16 + t * 4);
                }
#pragma unroll
                for (int r = 0; r < T::kKRegs; ++r) {
                    // word r holds channels 4r..4r+3 of the slab: quantisation group r/2 of the slab
                    const uint32_t sel = (r & 2) ? 0x3232u : 0x1010u;
                    const __half2 s2a = u32_as_h2(prmt(sa[r >> 2], 0u, sel));
                    const __half2 s2b = u32_as_h2(prmt(sb[r >> 2], 0u, sel));
                    uint32_t a0, a1, a2, a3;
                    dequant_k_word(wa[r], s2a, a0, a2);
                    dequant_k_word(wb[r], s2b, a1, a3);
                    mma_m16n8k16_f16f32(sacc, a0, a1, a2, a3, qf[r][0], qf[r][1]);
                }
            }

            // ---------------- softmax (exp2 domain, lazy reference maximum) ----------------
            float s0 = sacc[0] * a.scale_log2;  // token g,   head 2t
            float s1 = sacc[1] * a.scale_log2;  // token g,   head 2t+1
            float s2 = sacc[2] * a.scale_log2;  // token g+8, head 2t
            float s3 = sacc[3] * a.scale_log2;  // token g+8, head 2t+1
            if (g >= nvalid) {
                s0 = kNegBig;
                s1 = kNegBig;
            }
            if (g + 8 >= nvalid) {
                s2 = kNegBig;
                s3 = kNegBig;
            }
            {
                float lm0 = fmaxf(s0, s2), lm1 = fmaxf(s1, s3);
                const bool need = (lm0 > m0 + kRescaleSlack) || (lm1 > m1 + kRescaleSlack);
                if (__any_sync(0xffffffffu, need)) {
#pragma unroll
                    for (int off = 4; off <= 16; off <<= 1) {
                        lm0 = fmaxf(lm0, __shfl_xor_sync(0xffffffffu, lm0, off));
                        lm1 = fmaxf(lm1, __shfl_xor_sync(0xffffffffu, lm1, off));
                    }
                    const float n0 = fmaxf(m0, lm0), n1 = fmaxf(m1, lm1);
                    const float r0 = ex2_approx(m0 - n0), r1 = ex2_approx(m1 - n1);
                    m0 = n0;
                    m1 = n1;
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
            const float p0 = ex2_approx(s0 - m0), p1 = ex2_approx(s1 - m1);
            const float p2 = ex2_approx(s2 - m0), p3 = ex2_approx(s3 - m1);
            l0 += p0 + p2;
            l1 += p1 + p3;
            // P^T as the B operand of the second MMA: k = token, n = head
            const uint32_t pb0 = movmatrix_trans(h2_as_u32(__floats2half2_rn(p0, p1)));
            const uint32_t pb1 = movmatrix_trans(h2_as_u32(__floats2half2_rn(p2, p3)));

            // ---------------- O^T += V^T * P^T ----------------
            {
                const int ta = 2 * t, tb = 2 * t + 1, tc = 2 * t + 8, td = 2 * t + 9;
                uint32_t va[T::kVRegs], vb[T::kVRegs], vcw[T::kVRegs], vd[T::kVRegs];
                uint32_t sca, scb, scc, scd;  // scales of the thread's channel groups, per token
                if constexpr (DH == 128) {
                    const uint4 xa = lds128(vc + ta * 128 + ((g ^ (ta & 7)) << 4));
                    const uint4 xb = lds128(vc + tb * 128 + ((g ^ (tb & 7)) << 4));
                    const uint4 xc = lds128(vc + tc * 128 + ((g ^ (tc & 7)) << 4));
                    const uint4 xd = lds128(vc + td * 128 + ((g ^ (td & 7)) << 4));
                    va[0] = xa.x; va[1] = xa.y; va[2] = xa.z; va[3] = xa.w;
                    vb[0] = xb.x; vb[1] = xb.y; vb[2] = xb.z; vb[3] = xb.w;
                    vcw[0] = xc.x; vcw[1] = xc.y; vcw[2] = xc.z; vcw[3] = xc.w;
                    vd[0] = xd.x; vd[1] = xd.y; vd[2] = xd.z; vd[3] = xd.w;
                    sca = *reinterpret_cast<const uint32_t*>(vs + ta * 32 + g * 4);
                    scb = *reinterpret_cast<const uint32_t*>(vs + tb * 32 + g * 4);
                    scc = *reinterpret_cast<const uint32_t*>(vs + tc * 32 + g * 4);
                    scd = *reinterpret_cast<const uint32_t*>(vs + td * 32 + g * 4);
                } else {
                    const uint2 xa = *reinterpret_cast<const uint2*>(vc + ta * 64 + g * 8);
                    const uint2 xb = *reinterpret_cast<const uint2*>(vc + tb * 64 + g * 8);
                    const uint2 xc = *reinterpret_cast<const uint2*>(vc + tc * 64 + g * 8);
                    const uint2 xd = *reinterpret_cast<const uint2*>(vc + td * 64 + g * 8);
                    va[0] = xa.x; va[1] = xa.y;
                    vb[0] = xb.x; vb[1] = xb.y;
                    vcw[0] = xc.x; vcw[1] = xc.y;
                    vd[0] = xd.x; vd[1] = xd.y;
                    sca = *reinterpret_cast<const uint16_t*>(vs + ta * 16 + g * 2);
                    scb = *reinterpret_cast<const uint16_t*>(vs + tb * 16 + g * 2);
                    scc = *reinterpret_cast<const uint16_t*>(vs + tc * 16 + g * 2);
                    scd = *reinterpret_cast<const uint16_t*>(vs + td * 16 + g * 2);
                }
                if (nvalid < kTileTok) {
                    // rows past the end of the split hold other data (or nothing): their scales may be
                    // anything, and 0 * NaN would poison the accumulator even though P is exactly 0 there
                    sca = ta < nvalid ? sca : 0u;
                    scb = tb < nvalid ? scb : 0u;
                    scc = tc < nvalid ? scc : 0u;
                    scd = td < nvalid ? scd : 0u;
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

            __syncwarp();
            if (lane == 0 && i + kStages < my_n) {
                issue(i + kStages);
            }
        }
        tiles_done += static_cast<uint32_t>(my_n);

        // ---------------- merge the warps of this item and write ----------------
        {
#pragma unroll
            for (int off = 4; off <= 16; off <<= 1) {
                l0 += __shfl_xor_sync(0xffffffffu, l0, off);
                l1 += __shfl_xor_sync(0xffffffffu, l1, off);
            }
            float* wo = reinterpret_cast<float*>(wsm);  // [8 heads][DH], then max[8], sum[8]
#pragma unroll
            for (int jt = 0; jt < T::kMTiles; ++jt) {
                const int ch = (DH / 8) * g + 2 * jt;
                wo[(2 * t) * DH + ch] = o[jt][0];
                wo[(2 * t + 1) * DH + ch] = o[jt][1];
                wo[(2 * t) * DH + ch + 1] = o[jt][2];
                wo[(2 * t + 1) * DH + ch + 1] = o[jt][3];
            }
            if (g == 0) {
                wo[8 * DH + 2 * t] = m0;
                wo[8 * DH + 2 * t + 1] = m1;
                wo[8 * DH + 8 + 2 * t] = l0;
                wo[8 * DH + 8 + 2 * t + 1] = l1;
            }
        }
        __syncthreads();
        for (int e = threadIdx.x; e < HW * 8 * DH; e += kThreads) {
            const int hs = e / (8 * DH);
            const int r = e - hs * (8 * DH);
            const int h8 = r / DH;
            const int ch = r - h8 * DH;
            const int vh = hset * HW + hs;
            const int kvh_e = vh / a.octets;
            const int hq_in_group = (vh - kvh_e * a.octets) * 8 + h8;
            if (hq_in_group >= a.group) {
                continue;
            }
            float mx = kNegBig;
            for (int w = hs; w < kWarps; w += HW) {
                const float* src = reinterpret_cast<const float*>(smem + w * T::kWarpBytes);
                mx = fmaxf(mx, src[8 * DH + h8]);
            }
            float acc = 0.0f, den = 0.0f;
            for (int w = hs; w < kWarps; w += HW) {
                const float* src = reinterpret_cast<const float*>(smem + w * T::kWarpBytes);
                const float wgt = ex2_approx(src[8 * DH + h8] - mx);
                acc += wgt * src[h8 * DH + ch];
                den += wgt * src[8 * DH + 8 + h8];
            }
            const int qhead = kvh_e * a.group + hq_in_group;
            if (nsplits == 1) {
                const float v = den > 0.0f ? acc / den : 0.0f;
                a.out[(qtok * a.num_heads + qhead) * DH + ch] = __float2half_rn(v);
            } else {
                const int64_t slot = static_cast<int64_t>(first_split + split) * a.num_heads + qhead;
                a.part_o[slot * DH + ch] = acc;
                if (ch == 0) {
                    a.part_ml[slot * 2] = mx;
                    a.part_ml[slot * 2 + 1] = den;
                }
            }
        }
        // the stage buffers were read and written through the generic proxy; order that before the
        // bulk-tensor copies of the next item land in them
        fence_proxy_async_smem();
        __syncthreads();
    }
}

// ------------------------------------------------------------------------------------------
// Second pass: merge the fp32 partials of sequences that were split.  One warp per
// (sequence, query head).
// ------------------------------------------------------------------------------------------
template <int DH>
__global__ void __launch_bounds__(256)
decode_reduce_kernel(const int32_t* __restrict__ split_starts, const float* __restrict__ part_ml,
                     const float* __restrict__ part_o, const int64_t* __restrict__ seqstarts,
                     __half* __restrict__ out, int32_t decoding_batches, int32_t num_heads) {
    const int64_t wg = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wg >= static_cast<int64_t>(decoding_batches) * num_heads) {
        return;
    }
    const int32_t b = static_cast<int32_t>(wg / num_heads);
    const int32_t qh = static_cast<int32_t>(wg - static_cast<int64_t>(b) * num_heads);
    const int32_t first = split_starts[b];
    const int32_t ns = split_starts[b + 1] - first;
    if (ns <= 1) {
        return;
    }
    float mx = kNegBig;
    for (int32_t s = lane; s < ns; s += 32) {
        mx = fmaxf(mx, part_ml[(static_cast<int64_t>(first + s) * num_heads + qh) * 2]);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    }
    constexpr int kPer = DH / 32;
    float acc[kPer];
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
        acc[i] = 0.0f;
    }
    float den = 0.0f;
    for (int32_t s = 0; s < ns; ++s) {
        const int64_t slot = static_cast<int64_t>(first + s) * num_heads + qh;
        const float w = ex2_approx(part_ml[slot * 2] - mx);
        den += w * part_ml[slot * 2 + 1];
        const float* po = part_o + slot * DH + lane * kPer;
#pragma unroll
        for (int i = 0; i < kPer; ++i) {
            acc[i] += w * po[i];
        }
    }
    const float inv = den > 0.0f ? 1.0f / den : 0.0f;
    __half* dst = out + (seqstarts[b] * num_heads + qh) * DH + lane * kPer;
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
        dst[i] = __float2half_rn(acc[i] * inv);
    }
}

uint64_t align_up_u64(uint64_t x, uint64_t a) {
    return (x + a - 1) / a * a;
}

}  // namespace

// ------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------
int make_decode_plan(const pplb200_attn_params& p, int sm_count, DecodePlan* plan) {
    DecodePlan& d = *plan;
    const int64_t DB = p.decoding_batches;
    const int group = p.num_heads / p.num_kv_heads;
    d.octets = (group + 7) / 8;
    d.num_vheads = static_cast<int64_t>(p.num_kv_heads) * d.octets;
    d.head_warps = (d.num_vheads % 4 == 0) ? 4 : ((d.num_vheads % 2 == 0) ? 2 : 1);
    d.token_warps = kWarps / d.head_warps;
    d.num_hsets = d.num_vheads / d.head_warps;

    const int64_t slots = static_cast<int64_t>(sm_count) * 2;
    const int64_t max_kv = p.max_kvlen > 0 ? p.max_kvlen : 1;
    const int64_t whole = (max_kv + 63) / 64 * 64;
    int64_t chunk = whole;
    if (p.split_k_mode != 0 && DB > 0) {
        // Bound the largest work item to ~1/16 of a CTA slot's share of the (upper bound of the) work,
        // but keep splits long enough that their fp32 partials stay a small fraction of the traffic.
        const int64_t min_chunk = group >= 4 ? 512 : 256;
        int64_t target = DB * d.num_hsets * max_kv / (slots * 16);
        target = (target + 63) / 64 * 64;
        chunk = target < min_chunk ? min_chunk : target;
        if (p.split_k_mode == 2) {
            const int64_t half = ((max_kv + 1) / 2 + 63) / 64 * 64;
            chunk = chunk < half ? chunk : half;
        }
        chunk = chunk > whole ? whole : chunk;
        chunk = chunk < 64 ? 64 : chunk;
    }
    d.chunk_tokens = chunk;
    d.max_splits = (max_kv + chunk - 1) / chunk;
    const int64_t items_ub = DB * d.max_splits * d.num_hsets;
    d.grid = items_ub < slots ? items_ub : slots;
    if (d.grid < 1) {
        d.grid = 1;
    }

    uint64_t off = 0;
    d.off_status = off;
    d.off_counter = off + 4;
    off = 256;
    d.off_split_starts = off;
    off = align_up_u64(off + static_cast<uint64_t>(DB + 1) * 4, 256);
    const uint64_t slots_ub = d.max_splits > 1 ? static_cast<uint64_t>(DB) * d.max_splits * p.num_heads : 0;
    d.off_part_ml = off;
    off = align_up_u64(off + slots_ub * 2 * 4, 256);
    d.off_part_o = off;
    off = align_up_u64(off + slots_ub * p.head_dim * 4, 256);
    d.bytes = off;
    return PPLB200_SUCCESS;
}

template <int DH>
static int launch_decode_dh(const pplb200_attn_params& p, const CacheGeom& geom, const DecodePlan& plan,
                            const void* query, const int64_t* seqstarts, const int64_t* cachestarts,
                            const int64_t* start_pos, const void* cache, const void* scale, void* workspace,
                            void* attn_output, cudaStream_t stream) {
    using T = Traits<DH>;
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    uint32_t* status = reinterpret_cast<uint32_t*>(ws + plan.off_status);
    int32_t* counter = reinterpret_cast<int32_t*>(ws + plan.off_counter);
    int32_t* split_starts = reinterpret_cast<int32_t*>(ws + plan.off_split_starts);

    CUtensorMap tm_codes, tm_scales;
    CacheMapOrder order;
    int rc = make_cache_tensor_maps(p, cache, scale, kTileTok, &tm_codes, &tm_scales, &order);
    if (rc != PPLB200_SUCCESS) {
        return rc;
    }

    decode_plan_kernel<<<1, kPlanThreads, 0, stream>>>(seqstarts, start_pos, static_cast<int32_t>(p.decoding_batches),
                                                       plan.chunk_tokens, p.max_kvlen, split_starts, counter, status,
                                                       1);
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
    a.status = status;
    a.counter = counter;
    a.split_starts = split_starts;
    a.part_ml = reinterpret_cast<float*>(ws + plan.off_part_ml);
    a.part_o = reinterpret_cast<float*>(ws + plan.off_part_o);
    a.geom = geom;
    a.chunk_tokens = plan.chunk_tokens;
    a.max_kvlen = p.max_kvlen;
    a.decoding_batches = static_cast<int32_t>(p.decoding_batches);
    a.num_heads = p.num_heads;
    a.num_kv_heads = p.num_kv_heads;
    a.group = p.num_heads / p.num_kv_heads;
    a.octets = plan.octets;
    a.head_warps = plan.head_warps;
    a.token_warps = plan.token_warps;
    a.num_hsets = static_cast<int32_t>(plan.num_hsets);
    a.layer_idx = p.layer_idx;
    a.order = order;
    a.scale_log2 = 1.4426950408889634f / sqrtf(static_cast<float>(DH));

    static bool attr_set = false;  // per template instance; setting it twice is harmless
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(decode_splitk_kernel<DH>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             T::kSmemBytes);
        if (e != cudaSuccess) {
            fprintf(stderr, "[ppl_nn_b200] cudaFuncSetAttribute(decode_splitk_kernel): %s\n", cudaGetErrorString(e));
            return PPLB200_DEVICE_RUNTIME_ERROR;
        }
        attr_set = true;
    }
    {
        KernelTimer timer(PPLB200_KERNEL_DECODE, stream);
        decode_splitk_kernel<DH><<<static_cast<unsigned>(plan.grid), kThreads, T::kSmemBytes, stream>>>(
            tm_codes, tm_scales, a);
    }
    rc = check_launch("decode_splitk_kernel");
    if (rc != PPLB200_SUCCESS) {
        return rc;
    }
    if (plan.max_splits > 1) {
        const int64_t warps = p.decoding_batches * p.num_heads;
        const unsigned blocks = static_cast<unsigned>((warps + 7) / 8);
        decode_reduce_kernel<DH><<<blocks, 256, 0, stream>>>(split_starts, a.part_ml, a.part_o, seqstarts, a.out,
                                                             a.decoding_batches, p.num_heads);
        rc = check_launch("decode_reduce_kernel");
    }
    return rc;
}

int launch_decode(const pplb200_attn_params& p, const CacheGeom& geom, const DecodePlan& plan, const void* query,
                  const int64_t* seqstarts, const int64_t* cachestarts, const int64_t* start_pos, const void* cache,
                  const void* scale, void* workspace, void* attn_output, cudaStream_t stream) {
    if (p.decoding_batches <= 0) {
        return PPLB200_SUCCESS;
    }
    if (p.head_dim == 128) {
        return launch_decode_dh<128>(p, geom, plan, query, seqstarts, cachestarts, start_pos, cache, scale, workspace,
                                     attn_output, stream);
    }
    if (p.head_dim == 64) {
        return launch_decode_dh<64>(p, geom, plan, query, seqstarts, cachestarts, start_pos, cache, scale, workspace,
                                    attn_output, stream);
    }
    return PPLB200_UNSUPPORTED;
}

}  // namespace pplb200
