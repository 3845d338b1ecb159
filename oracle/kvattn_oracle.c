/*
 * CPU oracle for the INT8-KV cache attention path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is a plain-C restatement of what ppl.nn's llm_cuda engine asks of its two
 * operators
 *   opmx.dynamic_batching.KeyValueCache
 *       (src/ppl/nn/engines/llm_cuda/kernels/opmx/dynamic_batching/key_value_cache_kernel.cc:23-114)
 *   opmx.dynamic_batching.MultiHeadCacheAttention
 *       (src/ppl/nn/engines/llm_cuda/kernels/opmx/dynamic_batching/multi_head_cache_attention_kernel.cc:24-231)
 * It is linked by the tests, by the smoke check and by the CPU-baseline leg of the benchmark,
 * always as the checker (or as the timed CPU stand-in), never by the CUDA product path.
 *
 * PARITY UNPINNED.  The arithmetic of those operators lives in a third-party module that the
 * reference fetches at configure time -- ppl.llm.kernel.cuda, git
 * https://github.com/OpenPPL/ppl.llm.kernel.cuda.git at "master" (no commit pinned;
 * cmake/deps.cmake:290-304) -- and that module is not part of the reference tree.  The
 * reference tree holds no test, golden vector or fixture for this path either.  What is
 * restated here is therefore (1) the tensor contract, read off the call site
 * (multi_head_cache_attention_kernel.cc:170-212: argument order, strides, batch and
 * decoding_batches), (2) the cache geometry (cache_layout 0 and 3, same file :141-155, paged
 * mode :161-168), (3) the ragged index semantics of the reference's own driver
 * (tools/benchmark_llama/generation_state.cc:60-192), and (4) the published description of the
 * quantisation: symmetric INT8, one fp16 scale per group of 8 channels, scale = absmax / 127.
 *
 * Quantisation formula fixed by this oracle (all choices in one place, see orc_quant_group):
 *     a   = max_i |float(x_i)|                      over the 8 halves of the group
 *     s16 = fp16_round_nearest_even(a / 127.0f)     (fp32 divide, then one rounding to fp16)
 *     s   = float(s16)
 *     c_i = s == 0 ? 0 : clamp(rint(float(x_i) / s), -127, 127)     (rint = half-to-even)
 *     dequant(c, s16) = float(c) * float(s16)
 *
 * Attention: fp32 throughout over the dequantised cache; scores scaled by 1/sqrt(head_dim);
 * softmax with max subtraction; query head h reads kv head h / (num_heads/num_kv_heads);
 * causal mask kv_pos <= start_pos + q_idx; the output is rounded to fp16 once.  The first
 * decoding_batches sequences are decode sequences, the rest prefill.  Prefill sequences attend
 * to the fp16 current_key/current_value of this call (no history) unless enable_cache_prefill
 * is set, in which case they read the INT8 cache including the start_pos tokens of history.
 * The append happens before attention, so decode reads this step's token back quantised.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

typedef struct {
    int32_t num_heads;
    int32_t num_kv_heads;
    int32_t head_dim;
    int32_t is_causal;
    int32_t num_layer;
    int32_t layer_idx;
    int32_t quant_group; /* must be 8 */
    int32_t cache_mode; /* 0 contiguous rows per sequence, 1 paged */
    int32_t cache_layout; /* 0: (MaxT,L,2,H,Dh)   3: (L,2,H,MaxT,Dh) */
    int32_t page_size;
    int32_t enable_cache_prefill;
    int32_t reserved;
    int64_t batch;
    int64_t decoding_batches;
    int64_t max_tokens; /* MaxT: rows of the cache */
    int64_t cachestart_stride_b; /* paged: entries of cachestarts per sequence */
} orc_desc;

/* ---------------------------------------------------------------- fp16 <-> fp32 ------ */

float orc_half_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: normalise */
            int e = -1;
            do {
                ++e;
                man <<= 1;
            } while ((man & 0x400u) == 0);
            man &= 0x3ffu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* round-to-nearest-even, IEEE binary32 -> binary16 */
uint16_t orc_float_to_half(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    x &= 0x7fffffffu;
    if (x >= 0x7f800000u) { /* inf / nan */
        return (uint16_t)(sign | 0x7c00u | ((x > 0x7f800000u) ? 0x200u : 0u));
    }
    if (x >= 0x477ff000u) { /* >= 65520 rounds to inf */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (x < 0x38800000u) { /* below the smallest normal half (2^-14): subnormal or zero */
        if (x < 0x33000000u) { /* < 2^-25 rounds to zero (2^-25 itself ties to even = 0) */
            return sign;
        }
        const int e = (int)(x >> 23); /* biased fp32 exponent, 102..112 */
        uint32_t man = (x & 0x7fffffu) | 0x800000u; /* 24-bit significand */
        const int shift = 126 - e; /* 14..24: drop so that the unit is 2^-24 */
        const uint32_t q = man >> shift;
        const uint32_t rem = man & ((1u << shift) - 1u);
        const uint32_t halfway = 1u << (shift - 1);
        uint32_t r = q;
        if (rem > halfway || (rem == halfway && (q & 1u))) {
            ++r;
        }
        return (uint16_t)(sign | r); /* r == 0x400 is the smallest normal: still right */
    }
    /* normal */
    uint32_t e = (x >> 23) - 127 + 15;
    uint32_t man = x & 0x7fffffu;
    uint32_t r = (e << 10) | (man >> 13);
    const uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1u))) {
        ++r; /* carries into the exponent correctly */
    }
    return (uint16_t)(sign | r);
}

/* ---------------------------------------------------------------- quantisation -------- */

/* One group of 8 channels: 8 halves in, 8 codes + 1 fp16 scale out. */
void orc_quant_group(const uint16_t* x, int8_t* codes, uint16_t* scale16) {
    float v[8];
    float a = 0.0f;
    for (int i = 0; i < 8; ++i) {
        v[i] = orc_half_to_float(x[i]);
        const float m = fabsf(v[i]);
        if (m > a) {
            a = m; /* NaN never compares greater: a NaN lane is ignored by the max */
        }
    }
    const uint16_t s16 = orc_float_to_half(a / 127.0f);
    const float s = orc_half_to_float(s16);
    *scale16 = s16;
    for (int i = 0; i < 8; ++i) {
        float q = 0.0f;
        if (s != 0.0f) {
            q = rintf(v[i] / s);
            if (!(q >= -127.0f)) { /* also catches NaN */
                q = -127.0f;
            }
            if (q > 127.0f) {
                q = 127.0f;
            }
        }
        codes[i] = (int8_t)q;
    }
}

static inline int64_t cache_row(const orc_desc* d, const int64_t* cachestarts, int64_t b, int64_t pos) {
    if (d->cache_mode == 0) {
        return cachestarts[b] + pos;
    }
    return cachestarts[b * d->cachestart_stride_b + pos / d->page_size] + pos % d->page_size;
}

/* element offset of channel 0 of (row, kv, head) for a tensor with `dh` elements per head */
static inline int64_t cache_off(const orc_desc* d, int64_t row, int kv, int head, int64_t dh) {
    const int64_t L = d->num_layer, H = d->num_kv_heads, l = d->layer_idx;
    if (d->cache_layout == 0) {
        return (((row * L + l) * 2 + kv) * H + head) * dh;
    }
    return ((((l * 2 + kv) * H) + head) * d->max_tokens + row) * dh;
}

/* KeyValueCache, write side: quantise current_key/current_value and append them at row
 * cachestarts[b] + start_pos[b] + i for token i of sequence b. */
int orc_kv_append(const orc_desc* d, const uint16_t* cur_k, const uint16_t* cur_v, const int64_t* seqstarts,
                  const int64_t* cachestarts, const int64_t* start_pos, int8_t* cache, uint16_t* scale) {
    if (d->quant_group != 8 || (d->head_dim % 8) != 0) {
        return 1;
    }
    const int64_t Dh = d->head_dim, H = d->num_kv_heads, Gs = Dh / 8;
    for (int64_t b = 0; b < d->batch; ++b) {
        for (int64_t tok = seqstarts[b]; tok < seqstarts[b + 1]; ++tok) {
            const int64_t row = cache_row(d, cachestarts, b, start_pos[b] + (tok - seqstarts[b]));
            for (int kv = 0; kv < 2; ++kv) {
                const uint16_t* src = (kv == 0 ? cur_k : cur_v) + tok * H * Dh;
                for (int h = 0; h < H; ++h) {
                    int8_t* c = cache + cache_off(d, row, kv, h, Dh);
                    uint16_t* s = scale + cache_off(d, row, kv, h, Gs);
                    for (int64_t g = 0; g < Gs; ++g) {
                        orc_quant_group(src + h * Dh + g * 8, c + g * 8, s + g);
                    }
                }
            }
        }
    }
    return 0;
}

/* KeyValueCache, read side: key/value outputs = dequantised history, [kvstarts[B], H, Dh] fp16
 * (shape: src/ppl/nn/oputils/opmx/reshape_dynamic_batching_key_value_cache.cc:26-41). */
int orc_kv_gather_dequant(const orc_desc* d, const int64_t* kvstarts, const int64_t* cachestarts,
                          const int8_t* cache, const uint16_t* scale, uint16_t* key_out, uint16_t* value_out) {
    const int64_t Dh = d->head_dim, H = d->num_kv_heads, Gs = Dh / 8;
    for (int64_t b = 0; b < d->batch; ++b) {
        const int64_t kvlen = kvstarts[b + 1] - kvstarts[b];
        for (int64_t j = 0; j < kvlen; ++j) {
            const int64_t row = cache_row(d, cachestarts, b, j);
            for (int kv = 0; kv < 2; ++kv) {
                uint16_t* dst = (kv == 0 ? key_out : value_out) + (kvstarts[b] + j) * H * Dh;
                for (int h = 0; h < H; ++h) {
                    const int8_t* c = cache + cache_off(d, row, kv, h, Dh);
                    const uint16_t* s = scale + cache_off(d, row, kv, h, Gs);
                    for (int64_t e = 0; e < Dh; ++e) {
                        dst[h * Dh + e] = orc_float_to_half((float)c[e] * orc_half_to_float(s[e / 8]));
                    }
                }
            }
        }
    }
    return 0;
}

/* ---------------------------------------------------------------- attention ----------- */

/* The optional attn_mask input of both attention operators.  The reference only forwards its shape and
 * pointer to the external kernel library (multi_head_cache_attention_kernel.cc:105-110,179-180;
 * multi_head_attention_kernel.cc:96-103,114-115), so the convention is fixed here, after the operator
 * description of the OPMX dynamic-batching attention ops: an ADDITIVE fp16 mask of shape [T, C] or
 * [num_heads, T, C], T = seqstarts[batch] query tokens, C >= kvstarts[batch]; the element for query token i and
 * kv position j of sequence b is [.., seqstarts[b] + i, kvstarts[b] + j]; it is added to the scaled score
 * before the softmax, on top of the causal mask when is_causal is set.  A row whose visible positions are all
 * masked with -inf yields zeros.  data == NULL: no mask. */
typedef struct {
    const uint16_t* data;
    int64_t heads; /* 1: one mask for all heads */
    int64_t rows;
    int64_t cols;
} orc_mask;

static const uint16_t* mask_row_ptr(const orc_mask* m, int64_t head, int64_t tok, int64_t col0) {
    if (!m || !m->data) {
        return NULL;
    }
    const int64_t hh = m->heads > 1 ? head : 0;
    return m->data + (hh * m->rows + tok) * m->cols + col0;
}

/* One (sequence, query token, query head): scores over kv positions [0, n_kv), softmax, PV.
 * K/V rows come from `fetch` = 0: INT8 cache, 1: fp16 current tensors. */
static void attend_one(const orc_desc* d, const float* q, int64_t n_kv, int fetch, int64_t b, int kvh,
                       const int64_t* cachestarts, const int8_t* cache, const uint16_t* scale,
                       const uint16_t* cur_k, const uint16_t* cur_v, int64_t cur_base, const uint16_t* mask_row,
                       float* scores, float* krow, uint16_t* out) {
    const int64_t Dh = d->head_dim, H = d->num_kv_heads, Gs = Dh / 8;
    const float inv_sqrt = 1.0f / sqrtf((float)Dh);
    float mx = -INFINITY;
    for (int64_t j = 0; j < n_kv; ++j) {
        if (fetch == 0) {
            const int64_t row = cache_row(d, cachestarts, b, j);
            const int8_t* c = cache + cache_off(d, row, 0, kvh, Dh);
            const uint16_t* s = scale + cache_off(d, row, 0, kvh, Gs);
            for (int64_t g = 0; g < Gs; ++g) {
                const float sf = orc_half_to_float(s[g]);
                for (int e = 0; e < 8; ++e) {
                    krow[g * 8 + e] = (float)c[g * 8 + e] * sf;
                }
            }
        } else {
            const uint16_t* k = cur_k + ((cur_base + j) * H + kvh) * Dh;
            for (int64_t e = 0; e < Dh; ++e) {
                krow[e] = orc_half_to_float(k[e]);
            }
        }
        float acc = 0.0f;
        for (int64_t e = 0; e < Dh; ++e) {
            acc += q[e] * krow[e];
        }
        scores[j] = acc * inv_sqrt;
        if (mask_row) { /* additive mask, applied to the scaled score */
            scores[j] += orc_half_to_float(mask_row[j]);
        }
        if (scores[j] > mx) {
            mx = scores[j];
        }
    }
    if (!(mx > -INFINITY)) { /* every visible position is masked with -inf: the row attends to nothing */
        for (int64_t e = 0; e < Dh; ++e) {
            out[e] = 0;
        }
        return;
    }
    float denom = 0.0f;
    for (int64_t j = 0; j < n_kv; ++j) {
        scores[j] = expf(scores[j] - mx);
        denom += scores[j];
    }
    for (int64_t e = 0; e < Dh; ++e) {
        krow[e] = 0.0f; /* reuse as the output accumulator */
    }
    for (int64_t j = 0; j < n_kv; ++j) {
        const float p = scores[j];
        if (fetch == 0) {
            const int64_t row = cache_row(d, cachestarts, b, j);
            const int8_t* c = cache + cache_off(d, row, 1, kvh, Dh);
            const uint16_t* s = scale + cache_off(d, row, 1, kvh, Gs);
            for (int64_t g = 0; g < Gs; ++g) {
                const float sf = orc_half_to_float(s[g]);
                for (int e = 0; e < 8; ++e) {
                    krow[g * 8 + e] += p * ((float)c[g * 8 + e] * sf);
                }
            }
        } else {
            const uint16_t* v = cur_v + ((cur_base + j) * H + kvh) * Dh;
            for (int64_t e = 0; e < Dh; ++e) {
                krow[e] += p * orc_half_to_float(v[e]);
            }
        }
    }
    for (int64_t e = 0; e < Dh; ++e) {
        out[e] = orc_float_to_half(krow[e] / denom);
    }
}

/* MultiHeadCacheAttention, read side only: attention over a cache that already holds this
 * step's tokens.  seq_lo/seq_hi restrict the work to sequences [seq_lo, seq_hi) so that the
 * benchmark can time a bounded sample.  Parallel over (sequence, query token, head). */
int orc_attention_masked(const orc_desc* d, const uint16_t* query, const uint16_t* cur_k, const uint16_t* cur_v,
                         const int64_t* seqstarts, const int64_t* kvstarts, const int64_t* cachestarts,
                         const int64_t* start_pos, const int8_t* cache, const uint16_t* scale, uint16_t* out,
                         int64_t seq_lo, int64_t seq_hi, const orc_mask* mask) {
    const int64_t Dh = d->head_dim, Hq = d->num_heads, Hkv = d->num_kv_heads;
    if (Hkv <= 0 || Hq % Hkv != 0 || d->quant_group != 8) {
        return 1;
    }
    const int group = (int)(Hq / Hkv);
    int64_t max_kv = 0;
    for (int64_t b = seq_lo; b < seq_hi; ++b) {
        const int64_t n = start_pos[b] + (seqstarts[b + 1] - seqstarts[b]);
        if (n > max_kv) {
            max_kv = n;
        }
    }
    int failed = 0;
#pragma omp parallel
    {
        float* scores = (float*)malloc(sizeof(float) * (size_t)(max_kv > 0 ? max_kv : 1));
        float* krow = (float*)malloc(sizeof(float) * (size_t)Dh);
        float* qf = (float*)malloc(sizeof(float) * (size_t)Dh);
        if (!scores || !krow || !qf) {
#pragma omp atomic write
            failed = 1;
        } else {
            for (int64_t b = seq_lo; b < seq_hi; ++b) {
                const int64_t seqlen = seqstarts[b + 1] - seqstarts[b];
                const int is_decode = b < d->decoding_batches;
                const int from_cache = is_decode || d->enable_cache_prefill;
                const int64_t hist = from_cache ? start_pos[b] : 0;
                const int64_t work = seqlen * Hq;
#pragma omp for schedule(dynamic, 1) nowait
                for (int64_t w = 0; w < work; ++w) {
                    const int64_t i = w / Hq;
                    const int h = (int)(w % Hq);
                    const int64_t tok = seqstarts[b] + i;
                    const uint16_t* q16 = query + (tok * Hq + h) * Dh;
                    for (int64_t e = 0; e < Dh; ++e) {
                        qf[e] = orc_half_to_float(q16[e]);
                    }
                    const int64_t n_kv = d->is_causal ? hist + i + 1 : hist + seqlen;
                    /* kv position 0 of what this row reads: position 0 of the sequence, or its first new token */
                    const uint16_t* mrow = (mask && mask->data)
                        ? mask_row_ptr(mask, h, tok, kvstarts[b] + (from_cache ? 0 : start_pos[b])) : NULL;
                    attend_one(d, qf, n_kv, from_cache ? 0 : 1, b, h / group, cachestarts, cache, scale, cur_k,
                               cur_v, seqstarts[b], mrow, scores, krow, out + (tok * Hq + h) * Dh);
                }
            }
        }
        free(scores);
        free(krow);
        free(qf);
    }
    return failed;
}

int orc_attention(const orc_desc* d, const uint16_t* query, const uint16_t* cur_k, const uint16_t* cur_v,
                  const int64_t* seqstarts, const int64_t* cachestarts, const int64_t* start_pos,
                  const int8_t* cache, const uint16_t* scale, uint16_t* out, int64_t seq_lo, int64_t seq_hi) {
    return orc_attention_masked(d, query, cur_k, cur_v, seqstarts, NULL, cachestarts, start_pos, cache, scale, out,
                                seq_lo, seq_hi, NULL);
}

/* The whole MultiHeadCacheAttention op: append this step's K/V, then attend. */
int orc_mhca(const orc_desc* d, const uint16_t* query, const uint16_t* cur_k, const uint16_t* cur_v,
             const int64_t* seqstarts, const int64_t* cachestarts, const int64_t* start_pos, int8_t* cache,
             uint16_t* scale, uint16_t* out) {
    int rc = orc_kv_append(d, cur_k, cur_v, seqstarts, cachestarts, start_pos, cache, scale);
    if (rc != 0) {
        return rc;
    }
    return orc_attention(d, query, cur_k, cur_v, seqstarts, cachestarts, start_pos, cache, scale, out, 0,
                         d->batch);
}

/* The same with the optional attn_mask input (see orc_mask). */
int orc_mhca_masked(const orc_desc* d, const uint16_t* query, const uint16_t* cur_k, const uint16_t* cur_v,
                    const int64_t* seqstarts, const int64_t* kvstarts, const int64_t* cachestarts,
                    const int64_t* start_pos, int8_t* cache, uint16_t* scale, uint16_t* out, const orc_mask* mask) {
    int rc = orc_kv_append(d, cur_k, cur_v, seqstarts, cachestarts, start_pos, cache, scale);
    if (rc != 0) {
        return rc;
    }
    return orc_attention_masked(d, query, cur_k, cur_v, seqstarts, kvstarts, cachestarts, start_pos, cache, scale,
                                out, 0, d->batch, mask);
}

/* MultiHeadAttention without a cache (contract: src/ppl/nn/engines/llm_cuda/kernels/opmx/dynamic_batching/
 * multi_head_attention_kernel.cc:24-128; the arithmetic is not in the reference tree).  Sequence b owns query
 * rows [seqstarts[b], seqstarts[b+1]) and key/value rows [kvstarts[b], kvstarts[b+1]) of tensors shaped
 * [rows, heads, head_dim].  With is_causal, query row i sees kv positions <= (kvlen - seqlen) + i (the mask
 * is aligned to the end of the kv range; a choice of this repository); a row that sees nothing gives zeros.
 * Only num_heads, num_kv_heads, head_dim, is_causal and batch of the descriptor are read. */
int orc_mha_masked(const orc_desc* d, const uint16_t* query, const uint16_t* key, const uint16_t* value,
                   const int64_t* seqstarts, const int64_t* kvstarts, uint16_t* out, const orc_mask* mask) {
    const int64_t Dh = d->head_dim, Hq = d->num_heads, Hkv = d->num_kv_heads;
    if (Hkv <= 0 || Hq % Hkv != 0) {
        return 1;
    }
    const int group = (int)(Hq / Hkv);
    int64_t max_kv = 0;
    for (int64_t b = 0; b < d->batch; ++b) {
        const int64_t n = kvstarts[b + 1] - kvstarts[b];
        if (n > max_kv) {
            max_kv = n;
        }
    }
    int failed = 0;
#pragma omp parallel
    {
        float* scores = (float*)malloc(sizeof(float) * (size_t)(max_kv > 0 ? max_kv : 1));
        float* krow = (float*)malloc(sizeof(float) * (size_t)Dh);
        float* qf = (float*)malloc(sizeof(float) * (size_t)Dh);
        if (!scores || !krow || !qf) {
#pragma omp atomic write
            failed = 1;
        } else {
            for (int64_t b = 0; b < d->batch; ++b) {
                const int64_t seqlen = seqstarts[b + 1] - seqstarts[b];
                const int64_t kvlen = kvstarts[b + 1] - kvstarts[b];
                const int64_t work = seqlen * Hq;
#pragma omp for schedule(dynamic, 1) nowait
                for (int64_t w = 0; w < work; ++w) {
                    const int64_t i = w / Hq;
                    const int h = (int)(w % Hq);
                    const int64_t tok = seqstarts[b] + i;
                    uint16_t* o = out + (tok * Hq + h) * Dh;
                    int64_t n_kv = d->is_causal ? (kvlen - seqlen) + i + 1 : kvlen;
                    n_kv = n_kv > kvlen ? kvlen : n_kv;
                    if (n_kv <= 0) {
                        for (int64_t e = 0; e < Dh; ++e) {
                            o[e] = 0;
                        }
                        continue;
                    }
                    const uint16_t* q16 = query + (tok * Hq + h) * Dh;
                    for (int64_t e = 0; e < Dh; ++e) {
                        qf[e] = orc_half_to_float(q16[e]);
                    }
                    attend_one(d, qf, n_kv, 1, b, h / group, NULL, NULL, NULL, key, value, kvstarts[b],
                               mask_row_ptr(mask, h, tok, kvstarts[b]), scores, krow, o);
                }
            }
        }
        free(scores);
        free(krow);
        free(qf);
    }
    return failed;
}

int orc_mha(const orc_desc* d, const uint16_t* query, const uint16_t* key, const uint16_t* value,
            const int64_t* seqstarts, const int64_t* kvstarts, uint16_t* out) {
    return orc_mha_masked(d, query, key, value, seqstarts, kvstarts, out, NULL);
}

/* RotaryPositionEmbedding for ragged batches (contract: src/ppl/nn/engines/llm_cuda/kernels/opmx/
 * dynamic_batching/rotary_position_embedding_kernel.cc:24-132, attributes params/opmx/
 * rotary_position_embedding_param.h; the arithmetic is not in the reference tree, so the convention below
 * is this repository's): channel pairs (2j, 2j+1), j < rotary_dim/2, of every head are rotated by
 * pos_eff * inv_freq[j], inv_freq[j] = (float)pow(theta_eff, -2j/rotary_dim) in double; pos = start_pos[b] + i;
 * scaling_type 0: pos_eff = pos; 1 (linear): pos_eff = (float)pos / scaling_factor; 2 (dynamic): with
 * L = start_pos[b] + seqlen[b] > max_position_embeddings,
 * theta_eff = theta * pow(scaling_factor * L / max_pos - (scaling_factor - 1), rotary_dim / (rotary_dim - 2)).
 * float throughout after that: angle = pos_eff * inv_freq[j]; products and sums rounded one by one (no fma). */
static void rope_rows(const uint16_t* in, uint16_t* out, int64_t heads, int64_t Dh, int64_t half_rot, float pos_eff,
                      const float* inv_freq, int rotate) {
    for (int64_t h = 0; h < heads; ++h) {
        const uint16_t* x = in + h * Dh;
        uint16_t* y = out + h * Dh;
        for (int64_t e = 0; e < Dh; ++e) {
            y[e] = x[e];
        }
        if (!rotate) {
            continue;
        }
        for (int64_t j = 0; j < half_rot; ++j) {
            const volatile float angle = pos_eff * inv_freq[j];
            const float sn = sinf(angle), cs = cosf(angle);
            const float x0 = orc_half_to_float(x[2 * j]), x1 = orc_half_to_float(x[2 * j + 1]);
            const volatile float p0 = x0 * cs, p1 = x1 * sn, p2 = x0 * sn, p3 = x1 * cs;
            y[2 * j] = orc_float_to_half(p0 - p1);
            y[2 * j + 1] = orc_float_to_half(p2 + p3);
        }
    }
}

int orc_rope(int64_t num_heads, int64_t num_kv_heads, int64_t head_dim, int64_t rotary_dim, int bypass_key,
             int scaling_type, int64_t max_position_embeddings, float theta, float scaling_factor, int64_t batch,
             const uint16_t* query, const uint16_t* key, const int64_t* seqstarts, const int64_t* start_pos,
             uint16_t* rotated_query, uint16_t* rotated_key) {
    const int64_t rot = rotary_dim == 0 ? head_dim : rotary_dim;
    if (rot < 2 || rot > head_dim || (rot & 1) || scaling_type < 0 || scaling_type > 2) {
        return 1;
    }
    const int64_t half_rot = rot / 2;
    float* inv_freq = (float*)malloc(sizeof(float) * (size_t)half_rot);
    if (!inv_freq) {
        return 1;
    }
    for (int64_t b = 0; b < batch; ++b) {
        const int64_t seqlen = seqstarts[b + 1] - seqstarts[b];
        double theta_eff = (double)theta;
        if (scaling_type == 2) {
            const double len = (double)(start_pos[b] + seqlen);
            if (len > (double)max_position_embeddings) {
                theta_eff = (double)theta * pow((double)scaling_factor * len / (double)max_position_embeddings -
                                                    ((double)scaling_factor - 1.0),
                                                (double)rot / ((double)rot - 2.0));
            }
        }
        for (int64_t j = 0; j < half_rot; ++j) {
            inv_freq[j] = (float)pow(theta_eff, -2.0 * (double)j / (double)rot);
        }
        for (int64_t i = 0; i < seqlen; ++i) {
            const int64_t tok = seqstarts[b] + i;
            float pos_eff = (float)(start_pos[b] + i);
            if (scaling_type == 1) {
                pos_eff = pos_eff / scaling_factor;
            }
            rope_rows(query + tok * num_heads * head_dim, rotated_query + tok * num_heads * head_dim, num_heads, head_dim,
                      half_rot, pos_eff, inv_freq, 1);
            rope_rows(key + tok * num_kv_heads * head_dim, rotated_key + tok * num_kv_heads * head_dim, num_kv_heads,
                      head_dim, half_rot, pos_eff, inv_freq, !bypass_key);
        }
    }
    free(inv_freq);
    return 0;
}

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
