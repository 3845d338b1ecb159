// Device-side helpers shared by the sm_100a kernels: PTX wrappers for mbarrier, bulk-tensor (TMA)
// copies, warp-level MMA, byte permutes, and the INT8 group quantiser.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace pplb200 {

// ------------------------------------------------------------------------------------------
// Device status word (first 4 bytes of the workspace).  Kernels OR a code into it when a bounded
// wait gives up; they never spin forever.
// ------------------------------------------------------------------------------------------
constexpr uint32_t kDevOk = 0;
constexpr uint32_t kDevTmaTimeout = 1;
constexpr uint32_t kDevMmaTimeout = 2;
constexpr uint32_t kDevLengthClamped = 4;   // a sequence was longer than max_kvlen / max_seqlen and was clamped
constexpr uint32_t kDevRowOutOfRange = 8;   // an index tensor named a cache row outside [0, max_tokens): access skipped

constexpr uint32_t kDevMaskOutOfRange = 16;  // attn_mask is narrower than kvstarts needs: the missing entries read as 0

// Time budget of ONE bounded wait in every kernel of the library, in SM clock cycles: about 100 ms at
// 2 GHz, four orders of magnitude beyond any legitimate copy or MMA latency.  A wait that exhausts it
// records a status code; the waiting thread then stops waiting altogether, so a stuck kernel ends after
// roughly one budget per warp that waits, not one per wait.
constexpr long long kWaitBudgetCycles = 200000000LL;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ------------------------------------------------------------------------------------------
// mbarrier
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
    // make the initialised barriers visible to the async proxy (TMA / tcgen05 completions)
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}

// try_wait with a suspend-time hint: the hardware may park the thread for up to `hint_ns` and wakes
// it as soon as the phase completes, so a waiting warp does not burn issue slots by polling.
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar_addr, uint32_t parity, uint32_t hint_ns) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(bar_addr), "r"(parity), "r"(hint_ns)
        : "memory");
    return done != 0;
}

#ifndef PPLB200_WAIT_HINT_NS
#define PPLB200_WAIT_HINT_NS 20000
#endif

// Bounded wait.  Returns false when kWaitBudgetCycles ran out; the caller records a status code and
// carries on with whatever is in shared memory; nothing hangs.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity,
                                                  long long budget = kWaitBudgetCycles) {
    const uint32_t addr = smem_u32(bar);
    if (mbar_try_wait_hint(addr, parity, PPLB200_WAIT_HINT_NS)) {
        return true;
    }
    const long long t0 = clock64();
    for (;;) {
        if (mbar_try_wait_hint(addr, parity, PPLB200_WAIT_HINT_NS)) {
            return true;
        }
        if (clock64() - t0 > budget) {
            return false;
        }
    }
}

// Programmatic dependent launch (see launch_dependent in launch.h).  wait: everything the preceding grids
// of the stream wrote is visible after it (a no-op for a grid launched the ordinary way).
// launch_dependents: the next grid of the stream may be scheduled from here on.
__device__ __forceinline__ void grid_dependency_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void grid_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ------------------------------------------------------------------------------------------
// TMA: tiled bulk-tensor loads, global -> shared, completion on an mbarrier.  No multicast.
// The innermost coordinate must address a 16-byte boundary (callers only ever pass 0 there).
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const void* tmap, uint64_t* bar, int c0, int c1,
                                            int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(smem_dst)),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const void* tmap, uint64_t* bar, int c0, int c1,
                                            int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(smem_dst)),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

__device__ __forceinline__ void tma_load_5d(void* smem_dst, const void* tmap, uint64_t* bar, int c0, int c1,
                                            int c2, int c3, int c4) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(smem_u32(smem_dst)),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
        : "memory");
}

__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// ------------------------------------------------------------------------------------------
// Warp-level tensor-core MMA (used by the bandwidth-bound decode kernel, where the tile shape is
// 16 tokens x 8 heads and a CTA-wide tcgen05 tile would not fit the problem).
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_m16n8k16_f16f32(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                    uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 8x8 b16 transpose across the warp: lane (g,t) passes row g, columns 2t,2t+1 and receives
// row g, columns 2t,2t+1 of the transposed matrix.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) {
    return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) {
    return *reinterpret_cast<__half2*>(&u);
}

// Two biased bytes -> half2 of the signed codes.  `x` holds codes XOR 0x80 (i.e. code + 128 as an
// unsigned byte).  0x6400 | u is the half 1024 + u, so subtracting 1152 yields the code, exactly.
template <uint32_t SEL>
__device__ __forceinline__ __half2 biased_bytes_to_half2(uint32_t x) {
    const uint32_t h = prmt(x, 0x64646464u, SEL);
    return __hsub2(u32_as_h2(h), u32_as_h2(0x64806480u));
}

// ------------------------------------------------------------------------------------------
// INT8 group quantiser: 8 halves -> 8 codes + one fp16 scale.
//   a = max|x|, s16 = fp16_rn(a / 127.0f), c = s == 0 ? 0 : clamp(rint(x / float(s16)), -127, 127)
// IEEE division and round-half-even throughout: the file must be compiled without fast-math so
// that codes and scales are reproducible bit for bit on any IEEE host.
//
// The eight divisions are not carried out one by one.  q' = x * (1/s) lies within 4e-5 of fl(x/s)
// whenever |q'| <= 128, so if q' is further than that from every half-integer, rint(q') IS
// rint(fl(x/s)); only elements that close to a rounding boundary (a few in ten thousand), and
// anything non-finite, take the true division.  The rounding itself is the add-and-subtract of
// 1.5 * 2^23, which is round-half-even in the default rounding mode and leaves the integer in the
// low mantissa bits.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ int quant_code_exact(float v, float s) {
    float q = rintf(__fdiv_rn(v, s));
    if (!(q >= -127.0f)) {
        q = -127.0f;  // NaN as well
    }
    if (q > 127.0f) {
        q = 127.0f;
    }
    return static_cast<int>(q);
}

// NaN-propagating three-way maximum / minimum (a NaN among the operands must fail the range test below)
__device__ __forceinline__ float max3_nan(float a, float b, float c) {
    float d;
    asm("max.NaN.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float min3_nan(float a, float b, float c) {
    float d;
    asm("min.NaN.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

__device__ __forceinline__ void quant_group8(const uint4 in, uint2& codes, __half& scale16) {
    const __half2* h2 = reinterpret_cast<const __half2*>(&in);
    float2 v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[i] = __half22float2(h2[i]);
    }
    float a = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        a = fmaxf(a, fmaxf(fabsf(v[i].x), fabsf(v[i].y)));  // fmaxf drops a NaN operand, like `if (m > a) a = m`
    }
    // fp16_rn(fl(a / 127)) without the division: a is an fp16 number, and for every one of them the product
    // with fl(1/127), even with that constant an ulp off either way, rounds to the same fp16 value as the
    // IEEE quotient (the quotient never comes closer than 2^-19, relatively, to the midpoint of two fp16
    // numbers; checked exhaustively over all 31 745 non-negative halves).
    scale16 = __float2half_rn(__fmul_rn(a, 1.0f / 127.0f));
    const float s = __half2float(scale16);
    uint32_t w[2] = {0u, 0u};
    if (s != 0.0f) {
        constexpr float kMagic = 12582912.0f;  // 1.5 * 2^23
        // 1 ulp off at most (rcp.approx): q' is then within 127.1 * (2^-23 + 2^-24 + 2^-24) = 3e-5 of fl(x/s)
        float r;
        asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(s));
        uint32_t ub[8];
        float d[8];
        // two elements per instruction (packed fp32, each half rounded like the scalar operation)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 qf = __fmul2_rn(v[i], make_float2(r, r));
            const float2 u = __fadd2_rn(qf, make_float2(kMagic, kMagic));
            const float2 t = __fadd2_rn(u, make_float2(-kMagic, -kMagic));   // rint(qf) for |qf| < 2^22
            const float2 e = __ffma2_rn(t, make_float2(-1.0f, -1.0f), qf);  // qf - t, exact
            ub[2 * i] = __float_as_uint(u.x);  // low mantissa byte = the code in two's complement
            ub[2 * i + 1] = __float_as_uint(u.y);
            d[2 * i] = e.x;
            d[2 * i + 1] = e.y;
        }
        // With s a NORMAL half, s >= (a/127)(1 - 2^-11), hence |x/s| <= 127.07: no code can need the clamp.
        // A subnormal scale can be far below a/127; such groups (|x| < 0.008 throughout) take the exact path,
        // and so does a group with an element within 1e-4 of a rounding boundary or a NaN (an infinite x or s).
        const float d_hi = max3_nan(max3_nan(d[0], d[1], d[2]), max3_nan(d[3], d[4], d[5]), max3_nan(d[6], d[7], d[7]));
        const float d_lo = min3_nan(min3_nan(d[0], d[1], d[2]), min3_nan(d[3], d[4], d[5]), min3_nan(d[6], d[7], d[7]));
        const bool all_safe = s >= 6.103515625e-05f && d_hi < 0.4999f && d_lo > -0.4999f;
        if (!all_safe) {  // rare (about one group in a thousand): redo the group with true divisions
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                ub[2 * i] = static_cast<uint32_t>(quant_code_exact(v[i].x, s));
                ub[2 * i + 1] = static_cast<uint32_t>(quant_code_exact(v[i].y, s));
            }
        }
        w[0] = prmt(prmt(ub[0], ub[1], 0x0040u), prmt(ub[2], ub[3], 0x0040u), 0x5410u);
        w[1] = prmt(prmt(ub[4], ub[5], 0x0040u), prmt(ub[6], ub[7], 0x0040u), 0x5410u);
    }
    codes = make_uint2(w[0], w[1]);
}

// Cache geometry shared by all kernels: element offset of channel 0 of (row, kv, head) in `cache`;
// the scale tensor uses the same strides divided by 8.
struct CacheGeom {
    int64_t stride_s, stride_l, stride_h, stride_kv;  // elements of `cache`
    int64_t layer_idx;
    int64_t cachestart_stride_b;
    int32_t cache_mode;
    int32_t page_size;
};

// Cache row of position `pos` of sequence b, or -1 when the page table has no such page.  The result still
// has to be checked against [0, max_tokens) by the caller (cache_row_ok): the index tensors come from outside.
__device__ __forceinline__ int64_t cache_row(const CacheGeom& g, const int64_t* __restrict__ cachestarts, int64_t b,
                                             int64_t pos) {
    if (g.cache_mode == 0) {
        const int64_t first = cachestarts[b];
        return (first < 0 || pos < 0) ? -1 : first + pos;
    }
    // positions and page sizes are below 2^31 (checked on the host), so the division is a 32-bit one
    const uint32_t p = static_cast<uint32_t>(pos);
    const uint32_t page = p / static_cast<uint32_t>(g.page_size);
    if (pos < 0 || static_cast<int64_t>(page) >= g.cachestart_stride_b) {
        return -1;
    }
    const int64_t first = cachestarts[b * g.cachestart_stride_b + page];
    return first < 0 ? -1 : first + (p - page * static_cast<uint32_t>(g.page_size));
}

__device__ __forceinline__ bool cache_row_ok(int64_t row, int64_t max_tokens) {
    return row >= 0 && row < max_tokens;
}

// The optional attn_mask input on the device: additive fp16, [rows, cols] or [heads, rows, cols]; the element
// for query token q (row of the query tensor), head h and kv position j of sequence b is
// data[h * head_stride + q * cols + kvstarts[b] + j].  data == nullptr: no mask.
struct MaskDev {
    const __half* data;
    const int64_t* kvstarts;
    int64_t cols;
    int64_t head_stride;  // rows * cols, or 0 when one mask serves every head
};

__device__ __forceinline__ int64_t cache_offset(const CacheGeom& g, int64_t row, int kv, int head) {
    return row * g.stride_s + g.layer_idx * g.stride_l + kv * g.stride_kv + head * g.stride_h;
}

}  // namespace pplb200
