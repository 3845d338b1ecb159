// Causal prefill attention for the ragged batch tail (sequences [decoding_batches, batch)), as a
// dense contraction on the 5th-generation tensor cores: tcgen05.mma with TMEM accumulators, operands
// staged in shared memory by TMA (no multicast), fp16 inputs, fp32 accumulation.
//
// The unit of work is a 128-row query tile of one (sequence, query head).  The CTAs are persistent: two
// per SM (so that one CTA's MMAs run under the other's softmax), each drawing tiles from a global counter
// until none is left.  TMEM, the barriers and the stage rings live for the whole kernel; their phases run
// on from tile to tile, so the loads and the first Q K^T of the next tile are under way while the softmax
// threads finish the current one (a fresh CTA per tile cost 6.3 us of launch, set-up, load latency and
// epilogue per tile against ~1 us per 64-row kv block):
//   warp 0      draws and decodes tiles (one ahead) and hands them to the other roles through a ring in
//               shared memory; TMA producer: the Q tile, then K tiles (3-stage ring) and V tiles (2-stage
//               ring) of 64 rows each
//   warp 1      allocates TMEM (256 columns) and issues the MMAs: S = Q K^T into a 64-column TMEM buffer
//               (both operands in shared memory), then O += P V with P read from TMEM (the A operand)
//               and V from shared memory; completion is reported to mbarriers with tcgen05.commit
//   warps 2..5  128 softmax threads, one query row each (TMEM lane = row): read S once with tcgen05.ld
//               (the buffer is handed back to the MMA warp straight away), causal mask on diagonal
//               tiles only, running maximum in the exp2 domain (the O accumulator is rescaled in TMEM
//               only when the maximum grew by more than 2^8), write P as packed fp16 into one of two
//               TMEM buffers with tcgen05.st, so that the next tile's softmax does not wait for this
//               tile's P V, and finally divide O by the row sum and store fp16 rows (O is handed back to
//               the MMA warp as soon as it is in registers).  The row sum adds the fp16-rounded P values,
//               the very numbers the numerator uses.
// Both the producer and the MMA warp run warp-uniform code (every lane waits, an elected lane issues).
// K/V come from this call's fp16 current_key/current_value (the default), or, with
// enable_cache_prefill, from an fp16 staging copy of the INT8 cache rows (history included) that a
// dequantising gather writes into the workspace first.
//
// Every mbarrier wait is bounded.  When one gives up, the CTA sets an abort flag that all its other
// waits observe, records a status code, drains its own outstanding copies (bounded as well), frees its
// TMEM and returns.
#include <cuda.h>
#include <stdio.h>

#include <cub/block/block_scan.cuh>

#include "common.cuh"
#include "launch.h"
#include "ragged.cuh"
#include "tensor_map.h"

#ifndef PPLB200_PREFILL_WAIT
#define PPLB200_PREFILL_WAIT mbar_test_wait
#endif

namespace pplb200 {

namespace {

constexpr int kBlockM = 128;    // query rows per CTA
constexpr int kBlockN = 64;     // kv rows per block
constexpr int kThreads = 192;   // 6 warps
constexpr int kKStages = 3;
constexpr int kVStages = 2;
constexpr int kCtasPerSm = 2;
constexpr int kTileRing = 4;      // tile indices in flight between the producer and the other roles
constexpr int kCounterWord = 16;  // the tile counter is this many 32-bit words after the status word
constexpr float kNegBig = -1.0e30f;
constexpr float kRescaleSlack = 8.0f;

template <int DH>
struct PTraits {
    static constexpr int kColBlocks = DH / 64;                   // 64-element (128-byte) swizzled column blocks
    static constexpr int kQBlockBytes = kBlockM * 128;           // one [128 rows][64 halves] block of Q
    static constexpr int kKVBlockBytes = kBlockN * 128;          // one [64 rows][64 halves] block of K or V
    static constexpr int kQBytes = kColBlocks * kQBlockBytes;
    static constexpr int kKVBytes = kColBlocks * kKVBlockBytes;  // one K (or V) tile
    static constexpr int kBarrierBytes = 512;
    // The same for every head size (the Dh = 128 figure), so that never more than two CTAs share an SM
    // and the two 256-column TMEM allocations always fit.
    static constexpr int kSmemBytes = 32768 + (kKStages + kVStages) * (kBlockN * 256) + kBarrierBytes;
    static constexpr uint32_t kPCols = kBlockN / 2;              // packed fp16: two kv columns per TMEM column
    // TMEM columns: S (64) | P0 | P1 | O (128)
    static constexpr uint32_t kColS = 0, kColP = kBlockN, kColO = kColP + 2 * kPCols;
    static constexpr uint32_t kTmemCols = 256;
};

struct PrefillArgs {
    __half* out;
    const int64_t* seqstarts;
    const int64_t* start_pos;
    const int64_t* stage_starts;  // kv_mode 1: first staging row of each prefill sequence
    const int64_t* kvstarts;      // kv_mode 2: first K/V row of each sequence (a tensor of its own)
    uint32_t* status;
    int* tile_counter;  // next tile to hand out; zeroed before every launch
    int64_t max_seqlen;
    int32_t decoding_batches;
    int32_t prefill_batches;
    int32_t q_tiles;    // query tiles per sequence in the tile index space
    int32_t total_tiles;  // q_tiles * prefill_batches * num_heads
    int32_t seq_major;  // grid order
    int32_t num_heads;
    int32_t group;
    int32_t kv_mode;    // 0: K/V are this call's rows (same indexing as Q); 1: staged cache rows; 2: own K/V tensor
    int32_t is_causal;  // query row i sees kv positions <= (kvlen - seqlen) + i; otherwise all of them
    // head_rows > 0 (the un-cached operator on a batch of one-token sequences): a work unit is one
    // (sequence, kv head), and the head_rows query heads of that kv group are the ROWS of its tile, so K and V
    // of a sequence are read once per kv head instead of once per query head.  Unit pb = b * kv_heads + kvh;
    // its query rows are rows pb * head_rows .. of the query tensor seen as [tokens * heads, 1, Dh].
    int32_t head_rows;
    int32_t kv_heads;
    int64_t max_kvlen;
    float scale_log2;
    MaskDev mask;      // the optional attn_mask input (kernel instances with MASK only)
    float mask_scale;  // sqrt(head_dim): a mask value in units of the raw (unscaled) scores
};

// One unit of work: a 128-row query tile of one head, as decoded by the producer warp and handed to the
// other roles through shared memory.  head < 0: no more tiles.
struct Tile {
    int head, kvh, n_kv, rows_valid;
    int64_t q_row0, kv_row0, kvlen;
    int64_t first_row_last;  // last kv position visible to row 0 of the tile (negative: rows that see nothing)
    int64_t mask_col0;       // attn_mask column of kv position 0 of the tile's kv range (MASK instances)
};

struct Barriers {
    uint64_t q_full;
    uint64_t q_empty;     // the last Q K^T of a tile has completed: Q may be overwritten with the next tile's
    uint64_t o_free;      // the epilogue holds O in registers: the next tile may overwrite it
    uint64_t k_full[kKStages];
    uint64_t v_full[kVStages];
    uint64_t k_empty[kKStages];
    uint64_t v_empty[kVStages];
    uint64_t s_full;
    uint64_t s_free;
    uint64_t p_full[2];   // one per P buffer, so that a waiter can never be lapped
    uint64_t pv_done[2];  // P V of the tile that used P buffer 0 / 1 has completed
    uint64_t tile_full[kTileRing];  // the producer has published a tile index in tile_ring[e]
    uint64_t tile_free[kTileRing];  // the MMA warp and the softmax threads have read tile_ring[e]
    Tile tile_ring[kTileRing];
    uint32_t tmem_slot;
    int abort_word;
};
static_assert(sizeof(Barriers) <= 512, "barrier block");

// ---- tcgen05 wrappers ---------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)),
                 "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
// D[tmem] (+)= A[smem] * B[smem], M = 128, K = 16, fp16 inputs, fp32 accumulate
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]: the A operand (128 rows x 16 halves, two per column) read from TMEM
__device__ __forceinline__ void tc_mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                              uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
// l += lo(ph) + hi(ph), the two fp16 values widened exactly
__device__ __forceinline__ void add_half2_to_float(float& l, uint32_t ph) {
    asm("{\n"
        ".reg .b16 h0, h1;\n"
        "mov.b32 {h0, h1}, %1;\n"
        "add.rn.f32.f16 %0, h0, %0;\n"
        "add.rn.f32.f16 %0, h1, %0;\n"
        "}\n"
        : "+f"(l)
        : "r"(ph));
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
        "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// 256-bit store (32-byte aligned address)
__device__ __forceinline__ void st_global_v8(void* p, const uint32_t (&r)[8]) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(r[0]), "r"(r[1]), "r"(r[2]),
                 "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}

__device__ __forceinline__ void tmem_wait_ld() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptors (descriptor version 1, sm_100).
//   K-major operand, 128-byte swizzle ([rows][64 halves] blocks): lbo is unused (16), sbo = 1024 (8 rows
//   of 128 bytes).
//   MN-major operand, 128-byte swizzle (V as [kv rows][64 channels]): lbo = bytes between 64-channel
//   blocks, sbo = 1024 (8 kv rows of 128 bytes).
//   No swizzle: 8 x 8-half core matrices of 128 contiguous bytes, lbo / sbo apart along K / along N.
// Descriptors are built once as (low word, high word); stepping through a tile only adds to the low word
// (the start address in 16-byte units), which stays in uniform registers in warp-uniform code.
__device__ __forceinline__ uint32_t desc_lo(uint32_t saddr, uint32_t lbo_bytes) {
    return ((saddr & 0x3ffffu) >> 4) | (((lbo_bytes >> 4) & 0x3fffu) << 16);
}
__device__ __forceinline__ constexpr uint32_t desc_hi(uint32_t sbo_bytes, uint32_t layout) {
    return ((sbo_bytes >> 4) & 0x3fffu) | (1u << 14) | (layout << 29);
}
__device__ __forceinline__ uint64_t desc_join(uint32_t lo, uint32_t hi) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
    return d;
}
// One lane of a converged warp; the code around it stays warp-uniform.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "elect.sync _|p, 0xffffffff;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

// Instruction descriptor for kind::f16: fp16 A and B, fp32 D, M = 128.
__host__ __device__ constexpr uint32_t instr_desc_f16(int n, bool b_mn_major) {
    return (1u << 4) |                                 // D format: F32
           (0u << 7) | (0u << 10) |                    // A, B format: F16
           (0u << 15) | ((b_mn_major ? 1u : 0u) << 16) |  // A K-major; B K- or MN-major
           (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(kBlockM >> 4) << 24);
}

// Non-blocking test of an mbarrier phase.  The waits below poll with it: the blocking form
// (mbarrier.try_wait) parks the thread, and a parked thread was measured to resume a few hundred cycles
// after the phase had completed, which is as long as some of the pipeline stages here.
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}

// Bounded wait that also gives up as soon as another thread of the CTA has given up.  The common case,
// a phase that has completed already, costs one test; the polling loop is kept out of line.
__device__ __noinline__ bool wait_or_abort_slow(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                                uint32_t* status, uint32_t code) {
    const long long t0 = clock64();
    for (uint32_t i = 0;; i += 4) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (PPLB200_PREFILL_WAIT(bar, parity)) {
                return true;
            }
        }
        if ((i & 255u) == 252u) {
            if (*abort_flag) {
                return false;
            }
            if (clock64() - t0 > kWaitBudgetCycles) {
                break;
            }
        }
    }
    *abort_flag = 1;
    atomicOr(status, code);
    return false;
}
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                              uint32_t* status, uint32_t code) {
    if (PPLB200_PREFILL_WAIT(bar, parity)) {
        return true;
    }
    return wait_or_abort_slow(bar, parity, abort_flag, status, code);
}

template <int DH, bool MASK>
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                       const __grid_constant__ CUtensorMap tm_v, const PrefillArgs a) {
    using T = PTraits<DH>;
    // No static shared memory in this kernel: the dynamic window then starts on a 1 KB boundary, which the
    // 128-byte swizzle needs.  Checked below; a kernel that finds it otherwise reports it and returns.
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + T::kQBytes;
    uint8_t* sV = sK + kKStages * T::kKVBytes;
    Barriers& bars = *reinterpret_cast<Barriers*>(sV + kVStages * T::kKVBytes);
    volatile int* abort_flag = &bars.abort_word;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if ((smem_u32(smem) & 1023u) != 0u) {
        if (threadIdx.x == 0) {
            atomicOr(a.status, kDevTmaTimeout);
        }
        return;  // uniform for the CTA, before any barrier or TMEM allocation
    }

    // ---- setup (once per CTA; the CTA then works through tiles handed out by a global counter) ----
    if (threadIdx.x == 0) {
        bars.abort_word = 0;
        mbar_init(&bars.q_full, 1);
        mbar_init(&bars.q_empty, 1);
        for (int s = 0; s < kKStages; ++s) {
            mbar_init(&bars.k_full[s], 1);
            mbar_init(&bars.k_empty[s], 1);
        }
        for (int s = 0; s < kVStages; ++s) {
            mbar_init(&bars.v_full[s], 1);
            mbar_init(&bars.v_empty[s], 1);
        }
        mbar_init(&bars.s_full, 1);
        mbar_init(&bars.s_free, 128);
        mbar_init(&bars.o_free, 128);
        for (int e = 0; e < kTileRing; ++e) {
            mbar_init(&bars.tile_full[e], 1);
            mbar_init(&bars.tile_free[e], 129);  // 128 softmax threads + one lane of the MMA warp
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars.p_full[i], 128);
            mbar_init(&bars.pv_done[i], 1);
        }
        mbar_fence_init();
        tma_prefetch_desc(&tm_q);
        tma_prefetch_desc(&tm_k);
        tma_prefetch_desc(&tm_v);
    }
    if (warp == 1) {
        tmem_alloc(&bars.tmem_slot, T::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = bars.tmem_slot;

    // ---- which tile ----
    // Two orders of the tile index, both with the heads of one query tile adjacent (they share K/V in L2):
    //   tile-major      t = (qt_rev * prefill_batches + pb) * num_heads + head: the latest (longest)
    //                   query tile of every sequence first, then the ones before them; best balance
    //   sequence-major  t = (pb * q_tiles + qt_rev) * num_heads + head: the CTAs in flight work on
    //                   one or two sequences, whose K/V then stay in L2
    // The producer warp draws tile indices from the global counter, decodes them, drops those beyond their
    // sequence's length and publishes the others through a small ring in shared memory; the MMA warp and the
    // softmax threads read them there (head -1: no more tiles).  A tile that sees no kv position is zero-filled by
    // the softmax threads and ignored by the other two roles.
    auto decode_tile = [&](int t, Tile& ti) -> bool {
        int qt_rev, pb;
        if (a.seq_major) {
            const int per_seq = a.q_tiles * a.num_heads;
            pb = t / per_seq;
            const int rem = t - pb * per_seq;
            qt_rev = rem / a.num_heads;
            ti.head = rem - qt_rev * a.num_heads;
        } else {
            const int per_rev = a.prefill_batches * a.num_heads;
            qt_rev = t / per_rev;
            const int rem = t - qt_rev * per_rev;
            pb = rem / a.num_heads;
            ti.head = rem - pb * a.num_heads;
        }
        int b = a.decoding_batches + pb;
        int kvh_of_unit = -1;
        int64_t seq0, seqlen;
        if (a.head_rows > 0) {
            b = pb / a.kv_heads;
            kvh_of_unit = pb - b * a.kv_heads;
            seq0 = static_cast<int64_t>(pb) * a.head_rows;
            seqlen = a.head_rows;
        } else {
            seq0 = a.seqstarts[b];
            seqlen = a.seqstarts[b + 1] - seq0;
        }
        if (seqlen > a.max_seqlen) {
            seqlen = a.max_seqlen;
            if (lane == 0 && qt_rev == 0 && ti.head == 0) {  // only the producer warp decodes tiles
                atomicOr(a.status, kDevLengthClamped);
            }
        }
        const int n_qt = static_cast<int>((seqlen + kBlockM - 1) / kBlockM);
        if (qt_rev >= n_qt) {
            return false;
        }
        const int qt = n_qt - 1 - qt_rev;  // longest (latest) query tiles first
        ti.kvh = kvh_of_unit >= 0 ? kvh_of_unit : ti.head / a.group;
        const int64_t i0 = static_cast<int64_t>(qt) * kBlockM;
        ti.rows_valid = (seqlen - i0) < kBlockM ? static_cast<int>(seqlen - i0) : kBlockM;
        // kv rows of the sequence, how many there are, and how many of them precede query row 0 (hist)
        int64_t kv_row0 = seq0, kvlen = seqlen, hist = 0;
        if (a.kv_mode == 1) {
            hist = a.start_pos[b];
            kvlen = hist + seqlen;
            kv_row0 = a.stage_starts[pb];
        } else if (a.kv_mode == 2) {
            kv_row0 = a.kvstarts[b];
            kvlen = a.kvstarts[b + 1] - kv_row0;
            kvlen = kvlen > a.max_kvlen ? a.max_kvlen : kvlen;
            hist = kvlen - seqlen;  // causal masks are aligned to the END of the kv range
        }
        int64_t kv_visible = a.is_causal ? hist + i0 + ti.rows_valid : kvlen;  // kv positions the last valid row may see
        kv_visible = kv_visible > kvlen ? kvlen : kv_visible;
        ti.n_kv = kv_visible > 0 ? static_cast<int>((kv_visible + kBlockN - 1) / kBlockN) : 0;
        ti.q_row0 = seq0 + i0;
        ti.kv_row0 = kv_row0;
        ti.kvlen = kvlen;
        // last kv position visible to row 0 of the tile, and whether rows of this tile see nothing at all
        // (causal, more query rows than kv rows)
        ti.first_row_last = a.is_causal ? hist + i0 : kvlen - 1;
        ti.mask_col0 = 0;
        if constexpr (MASK) {
            // mask columns count kv positions of the sequence; with K/V taken from this call's rows (kv_mode 0)
            // kv row 0 is the sequence's first NEW token, position start_pos[b]
            ti.mask_col0 = a.mask.kvstarts[b] + (a.kv_mode == 0 ? a.start_pos[b] : 0);
        }
        return true;
    };
    const int total_tiles = a.total_tiles;
    // reader side of the ring: entry n of this CTA, or false after a timeout / abort
    auto next_tile = [&](int n, Tile& ti, bool one_lane_arrives) -> bool {
        const int e = n % kTileRing;
        if (!wait_or_abort(&bars.tile_full[e], (n / kTileRing) & 1, abort_flag, a.status, kDevTmaTimeout)) {
            return false;
        }
        ti = bars.tile_ring[e];
        if (one_lane_arrives) {
            __syncwarp();  // every lane has read the entry
            if (lane == 0) {
                mbar_arrive(&bars.tile_free[e]);
            }
        } else {
            mbar_arrive(&bars.tile_free[e]);
        }
        return true;
    };

    if (warp == 0) {
        // =========================== TMA producer ===========================
        // The whole warp runs the loop (waits are warp-uniform); an elected lane issues the copies.  A K
        // stage is free again as soon as its Q K^T has completed, a V stage once its P V has; the copies are
        // issued in the order in which those completions arrive: K(i), then V(i-1).  The stage rings and
        // their phases run on across tiles; Q is reloaded once the last Q K^T of the previous tile is done.
        bool ok = true;
        int tiles_done = 0, kc = 0, vc = 0;  // tiles with work so far; K and V copies issued so far
        int published = 0;
        // Draws the next tile that somebody needs, publishes it (or the end marker) and returns whether there
        // was one.  Costs an atomic and two dependent global loads, so it is called one tile ahead.
        auto fetch = [&](Tile& out) -> bool {
            for (;;) {
                int t = 0;
                if (lane == 0) {
                    t = atomicAdd(a.tile_counter, 1);
                }
                t = __shfl_sync(0xffffffffu, t, 0);
                const bool last = t >= total_tiles;
                if (!last && !decode_tile(t, out)) {
                    continue;  // beyond the end of its sequence: nobody needs it
                }
                if (last) {
                    out.head = -1;
                }
                const int e = published % kTileRing;
                if (published >= kTileRing) {
                    ok = wait_or_abort(&bars.tile_free[e], ((published / kTileRing) - 1) & 1, abort_flag, a.status, kDevMmaTimeout);
                    if (!ok) {
                        return false;
                    }
                }
                if (lane == 0) {
                    bars.tile_ring[e] = out;
                    mbar_arrive(&bars.tile_full[e]);
                }
                __syncwarp();
                ++published;
                return !last;
            }
        };
        Tile ti, nxt;
        bool have = fetch(ti);
        while (ok && have) {
            if (ti.n_kv == 0) {  // zero-filled by the softmax threads
                have = fetch(ti);
                continue;
            }
            bool fetched = false, have_next = false;
            if (tiles_done > 0) {
                ok = wait_or_abort(&bars.q_empty, (tiles_done - 1) & 1, abort_flag, a.status, kDevMmaTimeout);
                if (!ok) {
                    break;
                }
            }
            if (elect_one()) {
                mbar_arrive_expect_tx(&bars.q_full, T::kQBytes);
#pragma unroll
                for (int cb = 0; cb < T::kColBlocks; ++cb) {
                    tma_load_3d(sQ + cb * T::kQBlockBytes, &tm_q, &bars.q_full, cb * 64, ti.head, static_cast<int>(ti.q_row0));
                }
            }
            __syncwarp();
            ++tiles_done;
            for (int i = 0; ok && i <= ti.n_kv; ++i) {
                if (i == kKStages) {
                    // every stage of this tile's rings is on its way: now look up the next tile
                    have_next = fetch(nxt);
                    fetched = true;
                    if (!ok) {
                        break;
                    }
                }
                if (i < ti.n_kv) {
                    const int s = kc % kKStages;
                    if (kc >= kKStages) {
                        ok = wait_or_abort(&bars.k_empty[s], ((kc / kKStages) - 1) & 1, abort_flag, a.status, kDevMmaTimeout);
                        if (!ok) {
                            break;
                        }
                    }
                    if (elect_one()) {
                        const int row = static_cast<int>(ti.kv_row0 + static_cast<int64_t>(i) * kBlockN);
                        mbar_arrive_expect_tx(&bars.k_full[s], T::kKVBytes);
#pragma unroll
                        for (int cb = 0; cb < T::kColBlocks; ++cb) {
                            tma_load_3d(sK + s * T::kKVBytes + cb * T::kKVBlockBytes, &tm_k, &bars.k_full[s], cb * 64, ti.kvh, row);
                        }
                    }
                    __syncwarp();
                    ++kc;
                }
                if (i > 0) {
                    const int s = vc % kVStages;
                    if (vc >= kVStages) {
                        ok = wait_or_abort(&bars.v_empty[s], ((vc / kVStages) - 1) & 1, abort_flag, a.status, kDevMmaTimeout);
                        if (!ok) {
                            break;
                        }
                    }
                    if (elect_one()) {
                        const int row = static_cast<int>(ti.kv_row0 + static_cast<int64_t>(i - 1) * kBlockN);
                        mbar_arrive_expect_tx(&bars.v_full[s], T::kKVBytes);
#pragma unroll
                        for (int cb = 0; cb < T::kColBlocks; ++cb) {
                            tma_load_3d(sV + s * T::kKVBytes + cb * T::kKVBlockBytes, &tm_v, &bars.v_full[s], cb * 64, ti.kvh, row);
                        }
                    }
                    __syncwarp();
                    ++vc;
                }
            }
            if (ok && !fetched) {
                have_next = fetch(nxt);
            }
            ti = nxt;
            have = have_next;
        }
        if (*abort_flag) {
            // drain: every copy this warp issued must have landed before the CTA may exit
            if (tiles_done > 0) {
                mbar_wait_bounded(&bars.q_full, (tiles_done - 1) & 1);
            }
            for (int j = kc > kKStages ? kc - kKStages : 0; j < kc; ++j) {
                mbar_wait_bounded(&bars.k_full[j % kKStages], (j / kKStages) & 1);
            }
            for (int j = vc > kVStages ? vc - kVStages : 0; j < vc; ++j) {
                mbar_wait_bounded(&bars.v_full[j % kVStages], (j / kVStages) & 1);
            }
        }
    } else if (warp == 1) {
        // =========================== MMA issuer ===========================
        // Warp-uniform as well: all lanes wait, an elected lane issues.  Operand descriptors are built once.
        constexpr uint32_t idesc_qk = instr_desc_f16(kBlockN, false);
        constexpr uint32_t idesc_pv = instr_desc_f16(DH, true);
        constexpr uint32_t hi_sw128 = desc_hi(1024, 2);  // 128-byte swizzle, 8-row groups 1024 bytes apart
        const uint32_t q_lo = desc_lo(smem_u32(sQ), 16);
        const uint32_t k_lo = desc_lo(smem_u32(sK), 16);
        const uint32_t v_lo = desc_lo(smem_u32(sV), T::kKVBlockBytes);  // MN-major: 64-channel blocks lbo apart
        const uint32_t d_s = tmem_base + T::kColS, d_o = tmem_base + T::kColO, a_p = tmem_base + T::kColP;
        bool ok = true;
        int tiles_done = 0, kc = 0, vc = 0;  // tiles with work so far; Q K^T and P V issued so far (all tiles)
        for (int n = 0; ok; ++n) {
            Tile ti;
            if (!next_tile(n, ti, true) || ti.head < 0) {
                break;
            }
            if (ti.n_kv == 0) {
                continue;
            }
            ok = wait_or_abort(&bars.q_full, tiles_done & 1, abort_flag, a.status, kDevTmaTimeout);
            for (int j = 0; ok && j <= ti.n_kv; ++j) {
                if (j < ti.n_kv) {
                    // S = Q K(j)^T as soon as K(j) has landed and the softmax threads hold the previous scores in
                    // registers (the previous scores may be the last ones of the tile before)
                    const int s = kc % kKStages;
                    ok = wait_or_abort(&bars.k_full[s], (kc / kKStages) & 1, abort_flag, a.status, kDevTmaTimeout) &&
                         (kc == 0 || wait_or_abort(&bars.s_free, (kc - 1) & 1, abort_flag, a.status,
                                                       kDevMmaTimeout));
                    if (!ok) {
                        break;
                    }
                    tc_fence_after();
                    if (elect_one()) {
                        const uint32_t ks_lo = k_lo + s * (T::kKVBytes >> 4);
#pragma unroll
                        for (int cb = 0; cb < T::kColBlocks; ++cb) {
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                tc_mma_f16(d_s, desc_join(q_lo + cb * (T::kQBlockBytes >> 4) + 2 * k, hi_sw128),
                                           desc_join(ks_lo + cb * (T::kKVBlockBytes >> 4) + 2 * k, hi_sw128), idesc_qk,
                                           (cb | k) ? 1u : 0u);
                            }
                        }
                        tc_commit(&bars.s_full);
                        tc_commit(&bars.k_empty[s]);
                        if (j == ti.n_kv - 1) {
                            tc_commit(&bars.q_empty);  // the tile's last read of Q
                        }
                    }
                    __syncwarp();
                    ++kc;
                }
                if (j > 0) {
                    // O += P(j-1) V(j-1)
                    const int jp = j - 1;
                    const int s = vc % kVStages;
                    // V landed long ago; testing it first keeps it off the path from "P is ready" to the issue
                    ok = wait_or_abort(&bars.v_full[s], (vc / kVStages) & 1, abort_flag, a.status, kDevTmaTimeout) &&
                         wait_or_abort(&bars.p_full[vc & 1], (vc >> 1) & 1, abort_flag, a.status, kDevMmaTimeout);
                    if (ok && jp == 0 && tiles_done > 0) {
                        // the first P V of a tile overwrites O: the previous tile's epilogue must have read it
                        ok = wait_or_abort(&bars.o_free, (tiles_done - 1) & 1, abort_flag, a.status, kDevMmaTimeout);
                    }
                    if (!ok) {
                        break;
                    }
                    tc_fence_after();
                    if (elect_one()) {
                        const uint32_t vs_lo = v_lo + s * (T::kKVBytes >> 4);
                        const uint32_t pa = a_p + (vc & 1) * T::kPCols;
#pragma unroll
                        for (int ks = 0; ks < kBlockN / 16; ++ks) {
                            // P: kv index 16 ks = TMEM column 8 ks of the buffer (two halves per column);
                            // V: MN-major, kv rows 16 ks .. 16 ks + 15 (2048 bytes) of every 64-channel block
                            tc_mma_f16_ts(d_o, pa + 8 * ks, desc_join(vs_lo + ks * (2048 >> 4), hi_sw128), idesc_pv,
                                          (jp | ks) ? 1u : 0u);
                        }
                        tc_commit(&bars.v_empty[s]);
                        tc_commit(&bars.pv_done[vc & 1]);
                    }
                    __syncwarp();
                    ++vc;
                }
            }
            ++tiles_done;
        }
    } else {
        // =========================== softmax / epilogue ===========================
        const int lane_group = warp & 3;          // TMEM lanes this warp may touch: 32 * (warp % 4) ..
        const int r = lane_group * 32 + lane;     // query row of this thread within the tile
        const uint32_t t_lane = static_cast<uint32_t>(lane_group * 32) << 16;
        const uint32_t t_s = tmem_base + t_lane + T::kColS;
        const uint32_t t_o = tmem_base + t_lane + T::kColO;
        const uint32_t t_p = tmem_base + t_lane + T::kColP;
        const float sc = a.scale_log2;
        bool ok = true;
        int pc = 0;  // score tiles consumed = P tiles produced so far (all tiles of this CTA)
        for (int n = 0; ok; ++n) {
            Tile ti;
            if (!next_tile(n, ti, false) || ti.head < 0) {
                break;
            }
            const int head = ti.head, rows_valid = ti.rows_valid, n_kv = ti.n_kv;
            const int64_t q_row0 = ti.q_row0, kvlen = ti.kvlen, first_row_last = ti.first_row_last;
            const bool dead_rows = first_row_last < 0;
            if (n_kv == 0) {
                // nothing visible to any row of the tile: zeros
                for (int idx = threadIdx.x - 64; idx < rows_valid * (DH / 8); idx += 128) {
                    const int rr = idx / (DH / 8), c = idx - rr * (DH / 8);
                    *reinterpret_cast<uint4*>(a.out + ((q_row0 + rr) * a.num_heads + head) * DH + c * 8) = make_uint4(0u, 0u, 0u, 0u);
                }
                continue;
            }
            float m_ref = kNegBig, l_sum = 0.0f;
            for (int j = 0; ok && j < n_kv; ++j, ++pc) {
                // This tile's P buffer is free once the P V of the tile before the previous one has completed.  That
                // happened long before the scores of this tile arrive, so the test comes first and costs nothing
                // on the path from "S is ready" to the exponentials.
                if (pc >= 2) {
                    ok = wait_or_abort(&bars.pv_done[pc & 1], ((pc - 2) >> 1) & 1, abort_flag, a.status, kDevMmaTimeout);
                    if (!ok) {
                        break;
                    }
                }
                ok = wait_or_abort(&bars.s_full, pc & 1, abort_flag, a.status, kDevMmaTimeout);
                if (!ok) {
                    break;
                }
                tc_fence_after();
                float sv[kBlockN];
                {
                    uint32_t v[kBlockN / 32][32];
#pragma unroll
                    for (int c = 0; c < kBlockN / 32; ++c) {
                        tmem_ld32(t_s + 32 * c, v[c]);
                    }
                    tmem_wait_ld();
#pragma unroll
                    for (int c = 0; c < kBlockN / 32; ++c) {
#pragma unroll
                        for (int e = 0; e < 32; ++e) {
                            sv[32 * c + e] = __uint_as_float(v[c][e]);
                        }
                    }
                }
                // S is in registers: the MMA warp may overwrite the buffer with a later block's scores
                tc_fence_before();
                mbar_arrive(&bars.s_free);
                // columns of this tile that row r may see: col <= limit.  Only tiles that reach past the first
                // row's horizon or past the end of the kv range need the mask (uniform for the CTA).  Unless the
                // tile has rows that see nothing at all (handled below), column 0 of tile 0 is visible to every
                // row, so m_ref is a real score from the first tile on.
                // Score of a position the row may not see.  Without attn_mask a large negative FINITE number does:
                // every row sees column 0 of its first tile, so its reference maximum is a real score before any
                // such entry is exponentiated.  With a mask a row may see nothing at all; the entries are then
                // -inf, which exponentiates to 0 against the (always finite) reference maximum.
                constexpr float kOut = MASK ? -INFINITY : kNegBig;
                if constexpr (MASK) {
                    // additive mask, one fp16 per (query row, kv position); entries that the mask tensor does not
                    // hold read as 0 and are reported; +inf / NaN entries count as masked out
                    const int64_t col = ti.mask_col0 + static_cast<int64_t>(j) * kBlockN;
                    const int64_t room = a.mask.cols - col;
                    const int64_t vis = kvlen - static_cast<int64_t>(j) * kBlockN;
                    if (room < vis && room < kBlockN && r == 0) {
                        atomicOr(a.status, kDevMaskOutOfRange);
                    }
                    if (r < rows_valid) {
                        const __half* mrow = a.mask.data + static_cast<int64_t>(head) * a.mask.head_stride +
                                             (q_row0 + r) * a.mask.cols + col;
#pragma unroll
                        for (int e = 0; e < kBlockN; ++e) {
                            if (e < room && e < vis) {
                                const float t = fmaf(__half2float(mrow[e]), a.mask_scale, sv[e]);
                                sv[e] = t < 3.0e38f ? t : kOut;
                            }
                        }
                    }
                }
                const int64_t tile_hi = static_cast<int64_t>(j + 1) * kBlockN - 1;
                if (tile_hi > first_row_last || tile_hi >= kvlen) {
                    int64_t lim64 = (a.is_causal ? first_row_last + r : kvlen - 1);
                    lim64 = lim64 > kvlen - 1 ? kvlen - 1 : lim64;
                    lim64 -= static_cast<int64_t>(j) * kBlockN;
                    const int limit = lim64 > kBlockN ? kBlockN : (lim64 < -1 ? -1 : static_cast<int>(lim64));
#pragma unroll
                    for (int e = 0; e < kBlockN; ++e) {
                        sv[e] = e <= limit ? sv[e] : kOut;
                    }
                }
                float mx0 = fmax3(sv[0], sv[1], sv[2]), mx1 = fmax3(sv[3], sv[4], sv[5]);
#pragma unroll
                for (int e = 6; e + 3 < kBlockN; e += 4) {
                    mx0 = fmax3(mx0, sv[e], sv[e + 1]);
                    mx1 = fmax3(mx1, sv[e + 2], sv[e + 3]);
                }
                float mx = fmax3(mx0, mx1, fmaxf(sv[kBlockN - 2], sv[kBlockN - 1]));
                mx *= sc;  // sc > 0, so the maximum commutes with the scaling
                const bool grow = mx > m_ref + kRescaleSlack;
                if (__any_sync(0xffffffffu, grow)) {
                    const float m_new = grow ? mx : m_ref;
                    const float f = ex2_approx(m_ref - m_new);
                    m_ref = m_new;
                    l_sum *= f;
                    if (j > 0) {
                        // O may be touched once the previous tile's P V has completed
                        ok = wait_or_abort(&bars.pv_done[(pc - 1) & 1], ((pc - 1) >> 1) & 1, abort_flag, a.status, kDevMmaTimeout);
                        if (!ok) {
                            break;
                        }
                        tc_fence_after();
#pragma unroll
                        for (int c = 0; c < DH / 32; ++c) {
                            uint32_t v[32];
                            tmem_ld32(t_o + c * 32, v);
                            tmem_wait_ld();
#pragma unroll
                            for (int e = 0; e < 32; ++e) {
                                v[e] = __float_as_uint(__uint_as_float(v[e]) * f);
                            }
                            tmem_st32(t_o + c * 32, v);
                        }
                        tmem_wait_st();
                    }
                }
                // P = exp2(s * scale - m_ref) as packed fp16 into TMEM: column c of the buffer = kv columns 2c, 2c+1
                // a row that sees no kv position at all gets zero weights (exp2(-inf)), hence a zero output row
                const float neg_m = (dead_rows && first_row_last + r < 0) ? -INFINITY : -m_ref;
                const uint32_t t_pb = t_p + (pc & 1) * T::kPCols;
#pragma unroll
                for (int q = 0; q < kBlockN / 32; ++q) {
                    uint32_t pk[16];
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        // two scores per packed fp32 FMA (measured +1 %; exponentials of fp16 pairs in one
                        // special-function operation were also tried: no gain, and fp16 arguments cost accuracy)
                        const float2 x = __ffma2_rn(make_float2(sv[32 * q + 2 * e], sv[32 * q + 2 * e + 1]),
                                                    make_float2(sc, sc), make_float2(neg_m, neg_m));
                        pk[e] = h2_as_u32(__floats2half2_rn(ex2_approx(x.x), ex2_approx(x.y)));
                        add_half2_to_float(l_sum, pk[e]);
                    }
                    tmem_st16(t_pb + 16 * q, pk);
                }
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(&bars.p_full[pc & 1]);
            }
            // ---- epilogue: O / l -> fp16 rows ----
            if (ok) {
                ok = wait_or_abort(&bars.pv_done[(pc - 1) & 1], ((pc - 1) >> 1) & 1, abort_flag, a.status, kDevMmaTimeout);
            }
            if (ok) {
                tc_fence_after();
                const float inv = l_sum > 0.0f ? 1.0f / l_sum : 0.0f;
                __half* dst = a.out + ((q_row0 + r) * a.num_heads + head) * DH;
#pragma unroll
                for (int c = 0; c < DH / 64; ++c) {
                    uint32_t v[2][32];  // 64 columns per round: two loads in flight
                    tmem_ld32(t_o + c * 64, v[0]);
                    tmem_ld32(t_o + c * 64 + 32, v[1]);
                    tmem_wait_ld();
                    if (c == DH / 64 - 1) {
                        // O is in registers: the MMA warp may start the next tile's accumulation
                        tc_fence_before();
                        mbar_arrive(&bars.o_free);
                    }
                    if (r < rows_valid) {
                        // a thread owns a whole row, so a warp's store touches 32 rows: 32-byte stores fill whole
                        // sectors and halve the number of scattered requests
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
#pragma unroll
                            for (int q = 0; q < 2; ++q) {
                                uint32_t o[8];
#pragma unroll
                                for (int e = 0; e < 8; ++e) {
                                    o[e] = h2_as_u32(__floats2half2_rn(__uint_as_float(v[h][16 * q + 2 * e]) * inv,
                                                                       __uint_as_float(v[h][16 * q + 2 * e + 1]) * inv));
                                }
                                st_global_v8(dst + c * 64 + h * 32 + q * 16, o);
                            }
                        }
                    }
                }
            }
        }
    }

    // ---- teardown ----
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, T::kTmemCols);
    }
}

// Prefix sum of the (tile-padded) kv lengths of the prefill sequences: first staging row of each.  One CTA.
constexpr int kStagePlanThreads = 256;
__global__ void __launch_bounds__(kStagePlanThreads)
prefill_stage_plan_kernel(const int64_t* __restrict__ seqstarts, const int64_t* __restrict__ start_pos,
                          int32_t decoding_batches, int32_t prefill_batches, int64_t max_kvlen,
                          int64_t* __restrict__ stage_starts) {
    using Scan = cub::BlockScan<int64_t, kStagePlanThreads>;
    __shared__ typename Scan::TempStorage tmp;
    __shared__ int64_t carry;
    if (threadIdx.x == 0) {
        carry = 0;
    }
    __syncthreads();
    for (int32_t base = 0; base < prefill_batches; base += kStagePlanThreads) {
        const int32_t i = base + threadIdx.x;
        int64_t rows = 0;
        if (i < prefill_batches) {
            const int32_t b = decoding_batches + i;
            int64_t n = start_pos[b] + (seqstarts[b + 1] - seqstarts[b]);
            n = n > max_kvlen ? max_kvlen : (n < 0 ? 0 : n);
            rows = (n + kBlockN - 1) / kBlockN * kBlockN;
        }
        int64_t excl, total;
        Scan(tmp).ExclusiveSum(rows, excl, total);
        const int64_t c = carry;
        if (i < prefill_batches) {
            stage_starts[i] = c + excl;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            carry = c + total;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        stage_starts[prefill_batches] = carry;
    }
}

// Dequantise the cache rows of the prefill sequences (history and this call's tokens) into fp16 staging
// tensors [rows, Hkv, Dh]; the pad rows up to the next multiple of the kv tile are zeroed.  Same streaming
// shape as the KeyValueCache gather: a warp owns runs of 32 consecutive quantisation groups of one staging
// row (8 code bytes in and 16 bytes out per lane, coalesced) and looks the owning sequence up once per run.
__global__ void __launch_bounds__(256)
prefill_stage_dequant_kernel(const int64_t* __restrict__ seqstarts, const int64_t* __restrict__ start_pos,
                             const int64_t* __restrict__ cachestarts, const int64_t* __restrict__ stage_starts,
                             const int8_t* __restrict__ cache, const __half* __restrict__ scale,
                             __half* __restrict__ k_stage, __half* __restrict__ v_stage, CacheGeom geom,
                             int32_t decoding_batches, int32_t prefill_batches, int64_t max_kvlen, int64_t max_tokens,
                             uint32_t* __restrict__ status, int num_kv_heads, int head_dim) {
    const int lane = threadIdx.x & 31;
    const int group_shift = head_dim == 128 ? 4 : 3;
    const int32_t groups_per_tensor_row = num_kv_heads << group_shift;
    const int32_t groups_per_token = 2 * groups_per_tensor_row;
    const int64_t total_rows = stage_starts[prefill_batches];
    for (WarpItems it(groups_per_token); it.tok < total_rows; it.next()) {
        const int64_t row = it.tok;
        const int32_t i = warp_find_segment(stage_starts, prefill_batches, row, lane);
        const int32_t b = decoding_batches + i;
        const int64_t pos = row - stage_starts[i];
        int64_t kvlen = start_pos[b] + (seqstarts[b + 1] - seqstarts[b]);
        kvlen = kvlen > max_kvlen ? max_kvlen : kvlen;
        int64_t crow = -1;
        if (pos < kvlen) {
            crow = cache_row(geom, cachestarts, b, pos);
            if (!cache_row_ok(crow, max_tokens)) {  // a wrong index tensor: flagged, read as zeros
                if (lane == 0) {
                    atomicOr(status, kDevRowOutOfRange);
                }
                crow = -1;
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
            uint4 out = make_uint4(0u, 0u, 0u, 0u);
            if (crow >= 0) {
                const int64_t off = cache_offset(geom, crow, kv, head);
                const uint2 codes = *reinterpret_cast<const uint2*>(cache + off + grp * 8);
                const float sf = __half2float(scale[(off >> 3) + grp]);
                __half2* o2 = reinterpret_cast<__half2*>(&out);
                const uint32_t w[2] = {codes.x, codes.y};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int c0 = static_cast<int8_t>((w[e >> 1] >> (16 * (e & 1))) & 0xffu);
                    const int c1 = static_cast<int8_t>((w[e >> 1] >> (16 * (e & 1) + 8)) & 0xffu);
                    o2[e] = __floats2half2_rn(static_cast<float>(c0) * sf, static_cast<float>(c1) * sf);
                }
            }
            __half* dst = (kv ? v_stage : k_stage) + (row * num_kv_heads + head) * head_dim + grp * 8;
            *reinterpret_cast<uint4*>(dst) = out;
        }
    }
}

uint64_t align256(uint64_t x) {
    return (x + 255) / 256 * 256;
}

}  // namespace

int make_prefill_plan(const pplb200_attn_params& p, PrefillPlan* plan) {
    plan->prefill_batches = p.batch - p.decoding_batches;
    plan->q_tiles_per_seq = (p.max_seqlen + kBlockM - 1) / kBlockM;
    plan->kv_rows_bound = 0;
    plan->off_kv_stage = 0;
    plan->off_stage_starts = 0;
    plan->bytes = 0;
    if (plan->prefill_batches > 0 && p.enable_cache_prefill) {
        const int64_t per_seq = (p.max_kvlen + kBlockN - 1) / kBlockN * kBlockN;
        plan->kv_rows_bound = plan->prefill_batches * per_seq;
        plan->off_stage_starts = 0;
        plan->off_kv_stage = align256(static_cast<uint64_t>(plan->prefill_batches + 1) * 8);
        const uint64_t one = align256(static_cast<uint64_t>(plan->kv_rows_bound) * p.num_kv_heads * p.head_dim * 2);
        plan->bytes = plan->off_kv_stage + 2 * one;
    }
    return PPLB200_SUCCESS;
}

// Tensor maps + launch for one configuration of the kernel: Q rows [q_rows, Hq, Dh], K/V rows [kv_rows, Hkv, Dh].
template <int DH>
static int launch_attention_core(const void* query, const void* k_src, const void* v_src, int64_t q_rows, int64_t kv_rows,
                                 int num_heads, int num_kv_heads, int64_t q_tiles_per_seq, PrefillArgs a,
                                 cudaStream_t stream) {
    using T = PTraits<DH>;
    // tensor maps: {Dh, heads, rows} with a box of one head's [tile rows][64 halves], 128-byte swizzle
    CUtensorMap tm_q, tm_k, tm_v;
    const uint64_t dq[3] = {static_cast<uint64_t>(DH), static_cast<uint64_t>(num_heads), static_cast<uint64_t>(q_rows)};
    const uint64_t sq[2] = {static_cast<uint64_t>(DH) * 2, static_cast<uint64_t>(num_heads) * DH * 2};
    const uint32_t box[3] = {64, 1, kBlockM};
    const uint32_t box_kv[3] = {64, 1, kBlockN};
    int rc = encode_tensor_map(&tm_q, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, query, dq, sq, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != PPLB200_SUCCESS) {
        return rc;
    }
    const uint64_t dk[3] = {static_cast<uint64_t>(DH), static_cast<uint64_t>(num_kv_heads),
                            static_cast<uint64_t>(kv_rows)};
    const uint64_t sk[2] = {static_cast<uint64_t>(DH) * 2, static_cast<uint64_t>(num_kv_heads) * DH * 2};
    rc = encode_tensor_map(&tm_k, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, k_src, dk, sk, box_kv, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != PPLB200_SUCCESS) {
        return rc;
    }
    rc = encode_tensor_map(&tm_v, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, v_src, dk, sk, box_kv, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != PPLB200_SUCCESS) {
        return rc;
    }

    if ((reinterpret_cast<uintptr_t>(a.out) & 31u) != 0) {
        fprintf(stderr, "[ppl_nn_b200] attn_output must be 32-byte aligned\n");
        return PPLB200_INVALID_VALUE;
    }
    a.q_tiles = static_cast<int32_t>(q_tiles_per_seq);
    // K and V of everything this call may read against half of a 126 MB L2
    a.seq_major = static_cast<uint64_t>(kv_rows) * num_kv_heads * DH * 4 > (64ull << 20) ? 1 : 0;
    a.num_heads = num_heads;
    a.group = a.head_rows > 0 ? 1 : num_heads / num_kv_heads;
    a.scale_log2 = 1.4426950408889634f / sqrtf(static_cast<float>(DH));

    a.mask_scale = sqrtf(static_cast<float>(DH));
    const bool masked = a.mask.data != nullptr;
    auto kernel = masked ? prefill_tcgen05_kernel<DH, true> : prefill_tcgen05_kernel<DH, false>;

    // the attribute belongs to the (kernel, device) pair: remembered per template instance and device
    static bool attr_set_on[2][kMaxDevices] = {};
    int dev_id = 0;
    if (cudaGetDevice(&dev_id) != cudaSuccess || dev_id < 0 || dev_id >= kMaxDevices) {
        return PPLB200_DEVICE_RUNTIME_ERROR;
    }
    bool& attr_set = attr_set_on[masked ? 1 : 0][dev_id];
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             T::kSmemBytes);
        if (e != cudaSuccess) {
            fprintf(stderr, "[ppl_nn_b200] cudaFuncSetAttribute(prefill_tcgen05_kernel): %s\n", cudaGetErrorString(e));
            return PPLB200_DEVICE_RUNTIME_ERROR;
        }
        attr_set = true;
    }
    const int64_t tiles = q_tiles_per_seq * a.prefill_batches * num_heads;
    if (tiles > 0x7fffffff - (1 << 20)) {  // the counter runs past the last tile by one draw per CTA
        return PPLB200_UNSUPPORTED;
    }
    a.total_tiles = static_cast<int32_t>(tiles);
    a.tile_counter = reinterpret_cast<int*>(a.status + kCounterWord);
    if (cudaMemsetAsync(a.tile_counter, 0, 4, stream) != cudaSuccess) {
        (void)cudaGetLastError();
        return PPLB200_DEVICE_RUNTIME_ERROR;
    }
    // persistent CTAs: two per SM, drawing tiles from the counter
    int sm_count = 0;
    if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev_id) != cudaSuccess || sm_count <= 0) {
        (void)cudaGetLastError();
        return PPLB200_DEVICE_RUNTIME_ERROR;
    }
    const int64_t resident = static_cast<int64_t>(sm_count) * kCtasPerSm;
    const dim3 grid(static_cast<unsigned>(tiles < resident ? tiles : resident));
    {
        KernelTimer timer(PPLB200_KERNEL_PREFILL, stream);
        kernel<<<grid, kThreads, T::kSmemBytes, stream>>>(tm_q, tm_k, tm_v, a);
    }
    return check_launch("prefill_tcgen05_kernel");
}

template <int DH>
static int launch_prefill_dh(const pplb200_attn_params& p, const CacheGeom& geom, const PrefillPlan& plan,
                             const void* query, const void* cur_k, const void* cur_v, const int64_t* seqstarts,
                             const int64_t* cachestarts, const int64_t* start_pos, const void* cache, const void* scale,
                             const MaskDev& mask, void* region, uint32_t* status, void* attn_output,
                             cudaStream_t stream) {
    const void* k_src = cur_k;
    const void* v_src = cur_v;
    int64_t kv_rows = p.total_tokens;
    const int64_t* stage_starts = nullptr;
    int rc;
    if (p.enable_cache_prefill) {
        uint8_t* base = static_cast<uint8_t*>(region);
        int64_t* ss = reinterpret_cast<int64_t*>(base + plan.off_stage_starts);
        const uint64_t one = align256(static_cast<uint64_t>(plan.kv_rows_bound) * p.num_kv_heads * p.head_dim * 2);
        __half* ks = reinterpret_cast<__half*>(base + plan.off_kv_stage);
        __half* vs = reinterpret_cast<__half*>(base + plan.off_kv_stage + one);
        prefill_stage_plan_kernel<<<1, kStagePlanThreads, 0, stream>>>(
            seqstarts, start_pos, static_cast<int32_t>(p.decoding_batches), static_cast<int32_t>(plan.prefill_batches),
            p.max_kvlen, ss);
        rc = check_launch("prefill_stage_plan_kernel");
        if (rc != PPLB200_SUCCESS) {
            return rc;
        }
        // a warp per run of 32 * kChunks groups of a staging row; grid-stride beyond 16 CTAs per SM
        const int64_t items_per_row = (2 * p.num_kv_heads * (p.head_dim / 8) + 32 * kChunks - 1) / (32 * kChunks);
        int64_t blocks = (plan.kv_rows_bound * items_per_row * 32 + 255) / 256;
        blocks = blocks > 148 * 16 ? 148 * 16 : (blocks < 1 ? 1 : blocks);
        prefill_stage_dequant_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
            seqstarts, start_pos, cachestarts, ss, static_cast<const int8_t*>(cache), static_cast<const __half*>(scale),
            ks, vs, geom, static_cast<int32_t>(p.decoding_batches), static_cast<int32_t>(plan.prefill_batches),
            p.max_kvlen, p.max_tokens, status, p.num_kv_heads, p.head_dim);
        rc = check_launch("prefill_stage_dequant_kernel");
        if (rc != PPLB200_SUCCESS) {
            return rc;
        }
        k_src = ks;
        v_src = vs;
        kv_rows = plan.kv_rows_bound;
        stage_starts = ss;
    }

    PrefillArgs a = {};
    a.out = static_cast<__half*>(attn_output);
    a.seqstarts = seqstarts;
    a.start_pos = start_pos;
    a.stage_starts = stage_starts;
    a.kvstarts = nullptr;
    a.status = status;
    a.max_seqlen = p.max_seqlen;
    a.max_kvlen = p.max_kvlen;
    a.decoding_batches = static_cast<int32_t>(p.decoding_batches);
    a.prefill_batches = static_cast<int32_t>(plan.prefill_batches);
    a.kv_mode = p.enable_cache_prefill ? 1 : 0;
    a.is_causal = p.is_causal ? 1 : 0;  // the attribute is passed through, as the reference passes it
    a.mask = mask;
    return launch_attention_core<DH>(query, k_src, v_src, p.total_tokens, kv_rows, p.num_heads, p.num_kv_heads,
                                     plan.q_tiles_per_seq, a, stream);
}

// The un-cached operator: every sequence of the batch through the same kernel, K/V from their own tensors.
int launch_mha(int num_heads, int num_kv_heads, int head_dim, int is_causal, int64_t batch, int64_t max_seqlen,
               int64_t max_kvlen, int64_t total_q, int64_t total_kv, const void* query, const void* key,
               const void* value, const int64_t* seqstarts, const int64_t* kvstarts, const MaskDev& mask,
               uint32_t* status_word, void* attn_output, cudaStream_t stream) {
    if (batch <= 0 || max_seqlen <= 0 || total_q <= 0) {
        return PPLB200_SUCCESS;
    }
    PrefillArgs a = {};
    a.out = static_cast<__half*>(attn_output);
    a.seqstarts = seqstarts;
    a.start_pos = nullptr;
    a.stage_starts = nullptr;
    a.kvstarts = kvstarts;
    a.status = status_word;
    a.max_seqlen = max_seqlen;
    a.max_kvlen = max_kvlen;
    a.decoding_batches = 0;
    a.prefill_batches = static_cast<int32_t>(batch);
    a.kv_mode = 2;
    a.is_causal = is_causal ? 1 : 0;
    a.mask = mask;
    int64_t q_tiles = (max_seqlen + kBlockM - 1) / kBlockM;
    const int64_t kv_rows = total_kv > 0 ? total_kv : 1;  // a tensor map needs a non-empty extent
    int64_t q_rows = total_q;
    int q_heads = num_heads;
    const int group = num_heads / num_kv_heads;
    if (max_seqlen == 1 && total_q == batch && group > 1 && group <= kBlockM && mask.data == nullptr &&
        batch * num_kv_heads < (1 << 30)) {
        // every sequence has exactly one query token: the heads of a kv group become the rows of a tile (a
        // single row sees every kv position, causal or not)
        a.head_rows = group;
        a.kv_heads = num_kv_heads;
        a.prefill_batches = static_cast<int32_t>(batch * num_kv_heads);
        a.is_causal = 0;
        a.max_seqlen = group;
        q_tiles = 1;
        q_rows = total_q * num_heads;
        q_heads = 1;
    }
    if (head_dim == 128) {
        return launch_attention_core<128>(query, key, value, q_rows, kv_rows, q_heads, num_kv_heads, q_tiles, a, stream);
    }
    if (head_dim == 64) {
        return launch_attention_core<64>(query, key, value, q_rows, kv_rows, q_heads, num_kv_heads, q_tiles, a, stream);
    }
    return PPLB200_UNSUPPORTED;
}

int launch_prefill(const pplb200_attn_params& p, const CacheGeom& geom, const PrefillPlan& plan, const void* query,
                   const void* cur_k, const void* cur_v, const int64_t* seqstarts, const int64_t* cachestarts,
                   const int64_t* start_pos, const void* cache, const void* scale, const MaskDev& mask,
                   void* workspace_region, uint32_t* status_word, void* attn_output, cudaStream_t stream) {
    if (plan.prefill_batches <= 0 || plan.q_tiles_per_seq <= 0) {
        return PPLB200_SUCCESS;
    }
    if (p.head_dim == 128) {
        return launch_prefill_dh<128>(p, geom, plan, query, cur_k, cur_v, seqstarts, cachestarts, start_pos, cache,
                                      scale, mask, workspace_region, status_word, attn_output, stream);
    }
    if (p.head_dim == 64) {
        return launch_prefill_dh<64>(p, geom, plan, query, cur_k, cur_v, seqstarts, cachestarts, start_pos, cache, scale,
                                     mask, workspace_region, status_word, attn_output, stream);
    }
    return PPLB200_UNSUPPORTED;
}

}  // namespace pplb200
