/*
 * CPU baseline for the decode part of the INT8-KV cache attention path, shaped like the
 * reference's own CPU route.  TEST AND BENCHMARK INFRASTRUCTURE ONLY: it is timed next to the CUDA
 * path as a reported baseline and is never part of the product path.
 *
 * ppl.nn has no CPU implementation of its cache-attention operators.  What its x86 engine can run
 * for the same mathematics is, per sequence, the ONNX sub-graph
 *     MatMul(Q, K^T) -> Mul(1/sqrt(head_dim)) -> Softmax(axis=-1) -> MatMul(P, V)
 * in fp32 over the ALREADY DEQUANTISED cache:
 *     MatMul   src/ppl/nn/engines/x86/kernels/onnx/matmul_kernel.cc:45-52   (matmul_ndarray_fp32)
 *     Softmax  src/ppl/nn/engines/x86/kernels/onnx/softmax_kernel.cc:41-51  (softmax_ndarray_fp32)
 *     threads  src/ppl/nn/engines/x86/threading.cc:24-26                    (OpenMP, one pool)
 * Those kernels live in ppl.kernel.cpu, which is not in the reference tree, so they cannot be built
 * here; this file restates the graph with the same structure:
 *     xgb_dequant    int8 codes x fp16 group scales -> dense fp32 K and V, one [kvlen, head_dim]
 *                    matrix per (sequence, kv head) (what the graph's inputs would be)
 *     xgb_attention  for every (sequence, query head): GEMV q.K^T, scale, softmax with max
 *                    subtraction, GEMV p.V; ONE OpenMP loop over all (sequence, head) pairs.
 * Compile with -O3 -march=native -fopenmp: every inner loop is a contiguous fp32 loop over head_dim
 * or kvlen that the compiler vectorises; the exponential is a polynomial (below) so that it
 * vectorises too, as the exponentials of SIMD softmax kernels do.
 * Only decode sequences (one query token each) are handled: that is the benchmark's workload.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* binary16 -> binary32 (normal, subnormal, zero, inf, nan) */
static inline float xgb_half_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t em = h & 0x7fffu;
    uint32_t bits;
    if (em >= 0x7c00u) {
        bits = sign | 0x7f800000u | ((em & 0x3ffu) << 13);
    } else if (em >= 0x0400u) {
        bits = sign | ((em << 13) + 0x38000000u);
    } else { /* subnormal or zero: em * 2^-24, exact in fp32 */
        float f = (float)em * 5.9604644775390625e-8f;
        memcpy(&bits, &f, 4);
        bits |= sign;
    }
    float out;
    memcpy(&out, &bits, 4);
    return out;
}

/* binary32 -> binary16, round to nearest even (finite inputs of moderate size only: attention outputs) */
static inline uint16_t xgb_float_to_half(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    x &= 0x7fffffffu;
    if (x >= 0x477ff000u) {
        return (uint16_t)(sign | (x > 0x7f800000u ? 0x7e00u : 0x7c00u));
    }
    if (x < 0x38800000u) { /* result is subnormal or zero: scale into the integer grid of 2^-24 */
        float a;
        memcpy(&a, &x, 4);
        const float r = rintf(a * 16777216.0f);
        return (uint16_t)(sign | (uint16_t)r);
    }
    const uint32_t rounded = x + 0xfffu + ((x >> 13) & 1u);
    return (uint16_t)(sign | ((rounded - 0x38000000u) >> 13));
}

/* e^x for x <= 0 (softmax arguments after max subtraction): n = rint(x log2 e), r = x - n ln 2 in two
 * pieces, degree-6 polynomial for e^r on [-ln2/2, ln2/2], scaled by 2^n through the exponent field.
 * Relative error below 2e-7; branch-free, so loops over it vectorise. */
static inline float xgb_expf(float x) {
    x = x < -87.0f ? -87.0f : x;
    const float n = rintf(x * 1.44269504088896341f);
    float r = x - n * 0.693359375f;
    r = r - n * -2.12194440e-4f;
    float p = 1.9875691500e-4f;
    p = p * r + 1.3981999507e-3f;
    p = p * r + 8.3334519073e-3f;
    p = p * r + 4.1665795894e-2f;
    p = p * r + 1.6666665459e-1f;
    p = p * r + 5.0000001201e-1f;
    p = p * r * r + r + 1.0f;
    int32_t bits;
    memcpy(&bits, &p, 4);
    bits += (int32_t)n << 23;
    memcpy(&p, &bits, 4);
    return p;
}

/* Element offset of channel 0 of (row, k|v, head) in a cache tensor whose innermost extent is `inner`
 * (head_dim for codes, head_dim/8 for scales); layouts as in
 * src/ppl/nn/engines/llm_cuda/kernels/opmx/dynamic_batching/multi_head_cache_attention_kernel.cc:141-155. */
static inline int64_t xgb_cache_off(int layout, int64_t max_tokens, int64_t num_layer, int64_t layer, int64_t H,
                                    int64_t row, int kv, int64_t head, int64_t inner) {
    if (layout == 0) { /* (MaxT, L, 2, H, inner) */
        return (((row * num_layer + layer) * 2 + kv) * H + head) * inner;
    }
    /* layout 3: (L, 2, H, MaxT, inner) */
    return (((layer * 2 + kv) * H + head) * max_tokens + row) * inner;
}

/* Dequantise the cached rows [0, kvlen_b) of sequences [0, batch) (contiguous cache mode: row =
 * cachestarts[b] + position).  k_out / v_out receive, sequence after sequence and head after head, one dense
 * fp32 matrix [kvlen_b, head_dim] per (sequence, kv head); mat_starts[b] is the first ROW of sequence b's
 * matrices in units of rows, i.e. the prefix sum of kvlen_b * num_kv_heads (batch + 1 entries). */
int xgb_dequant(int32_t num_kv_heads, int32_t head_dim, int32_t num_layer, int32_t layer_idx, int32_t cache_layout,
                int64_t max_tokens, int64_t batch, const int64_t* kvlens, const int64_t* cachestarts,
                const int64_t* mat_starts, const int8_t* cache, const uint16_t* scale, float* k_out, float* v_out) {
    const int64_t Dh = head_dim, H = num_kv_heads, Gs = Dh / 8;
    if ((cache_layout != 0 && cache_layout != 3) || Dh % 8 != 0) {
        return 1;
    }
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int64_t b = 0; b < batch; ++b) {
        for (int64_t h = 0; h < H; ++h) {
            const int64_t n = kvlens[b];
            for (int kv = 0; kv < 2; ++kv) {
                float* dst = (kv ? v_out : k_out) + (mat_starts[b] + h * n) * Dh;
                for (int64_t j = 0; j < n; ++j) {
                    const int64_t row = cachestarts[b] + j;
                    const int8_t* c = cache + xgb_cache_off(cache_layout, max_tokens, num_layer, layer_idx, H, row, kv, h, Dh);
                    const uint16_t* s = scale + xgb_cache_off(cache_layout, max_tokens, num_layer, layer_idx, H, row, kv, h, Gs);
                    float* o = dst + j * Dh;
                    for (int64_t g = 0; g < Gs; ++g) {
                        const float sf = xgb_half_to_float(s[g]);
                        for (int e = 0; e < 8; ++e) {
                            o[g * 8 + e] = (float)c[g * 8 + e] * sf;
                        }
                    }
                }
            }
        }
    }
    return 0;
}

/* Decode attention over the dequantised cache: query [batch, num_heads, head_dim] fp16 (one token per
 * sequence), K/V as written by xgb_dequant, out [batch, num_heads, head_dim] fp16.  `scores` is scratch of
 * num_threads * max_kvlen floats.  One OpenMP loop over all (sequence, query head) pairs. */
int xgb_attention(int32_t num_heads, int32_t num_kv_heads, int32_t head_dim, int64_t batch, const int64_t* kvlens,
                  const int64_t* mat_starts, const uint16_t* query, const float* k_mat, const float* v_mat,
                  float* scores, int64_t max_kvlen, uint16_t* out) {
    const int64_t Dh = head_dim, Hq = num_heads, Hkv = num_kv_heads;
    if (Hkv <= 0 || Hq % Hkv != 0 || Dh > 256) {
        return 1;
    }
    const int64_t group = Hq / Hkv;
    const float inv_sqrt = 1.0f / sqrtf((float)Dh);
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t w = 0; w < batch * Hq; ++w) {
        const int64_t b = w / Hq, h = w % Hq;
        const int64_t n = kvlens[b];
        const int64_t kvh = h / group;
#ifdef _OPENMP
        float* s = scores + (int64_t)omp_get_thread_num() * max_kvlen;
#else
        float* s = scores;
#endif
        float q[256], acc[256];
        const uint16_t* q16 = query + (b * Hq + h) * Dh;
        for (int64_t e = 0; e < Dh; ++e) {
            q[e] = xgb_half_to_float(q16[e]);
        }
        const float* K = k_mat + (mat_starts[b] + kvh * n) * Dh;
        const float* V = v_mat + (mat_starts[b] + kvh * n) * Dh;
        /* MatMul(Q, K^T) and Mul: a GEMV, one dot product per cached token */
        float mx = -INFINITY;
        for (int64_t j = 0; j < n; ++j) {
            const float* kr = K + j * Dh;
            float d = 0.0f;
#pragma omp simd reduction(+ : d)
            for (int64_t e = 0; e < Dh; ++e) {
                d += q[e] * kr[e];
            }
            d *= inv_sqrt;
            s[j] = d;
            mx = d > mx ? d : mx;
        }
        /* Softmax(axis=-1) */
        float denom = 0.0f;
#pragma omp simd reduction(+ : denom)
        for (int64_t j = 0; j < n; ++j) {
            const float p = xgb_expf(s[j] - mx);
            s[j] = p;
            denom += p;
        }
        const float inv = 1.0f / denom;
        /* MatMul(P, V): a GEMV, one axpy per cached token */
        for (int64_t e = 0; e < Dh; ++e) {
            acc[e] = 0.0f;
        }
        for (int64_t j = 0; j < n; ++j) {
            const float p = s[j] * inv;
            const float* vr = V + j * Dh;
#pragma omp simd
            for (int64_t e = 0; e < Dh; ++e) {
                acc[e] += p * vr[e];
            }
        }
        uint16_t* o = out + (b * Hq + h) * Dh;
        for (int64_t e = 0; e < Dh; ++e) {
            o[e] = xgb_float_to_half(acc[e]);
        }
    }
    return 0;
}

int xgb_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Launchers such as torch.distributed.run export OMP_NUM_THREADS=1 to their children; the benchmark sets
 * the count it wants explicitly. */
void xgb_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) {
        omp_set_num_threads(n);
    }
#else
    (void)n;
#endif
}
