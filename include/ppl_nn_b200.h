/*
 * ppl_nn_b200.h -- C ABI of the B200 (sm_100a) kernels behind ppl.nn's llm_cuda operators
 *   opmx.dynamic_batching.KeyValueCache            and
 *   opmx.dynamic_batching.MultiHeadCacheAttention.
 *
 * In ppl.nn these operators call into an external kernel library through C++ entry points
 * (namespace ppl::kernel::llm::cuda::pmx).  The functions below are what a binding for this path
 * would bind instead: plain pointers and sizes, `int` status codes, no C++ or torch types.  All
 * device pointers belong to the caller; every function only enqueues work on `stream` (a
 * cudaStream_t passed as void*) and returns without synchronising, unless stated otherwise.
 * Citations are paths inside the ppl.nn source tree.
 *
 * Tensor contract (src/ppl/nn/engines/llm_cuda/kernels/opmx/dynamic_batching/
 * multi_head_cache_attention_kernel.cc:27-41; index tensors are int64 on the device):
 *   query          [T, num_heads, head_dim]        fp16
 *   current_key    [T, num_kv_heads, head_dim]     fp16
 *   current_value  [T, num_kv_heads, head_dim]     fp16
 *   seqstarts      [batch+1]   prefix sum of the query lengths
 *   kvstarts       [batch+1]   prefix sum of start_pos + query length
 *   cachestarts    [batch]     first cache row of each sequence
 *                  ([batch, cachestart_stride_b] page start rows when cache_mode == 1)
 *   start_pos      [batch]     tokens already cached
 *   cache          int8,  cache_layout 0: (MaxT, L, 2, Hkv, Dh)       3: (L, 2, Hkv, MaxT, Dh)
 *   scale          fp16,  same with Dh/quant_group in place of Dh
 *   attn_output    [T, num_heads, head_dim]        fp16, 32-byte aligned (PPLB200_INVALID_VALUE otherwise)
 * All tensors are dense (no padding between rows); query, current_key, current_value, cache and scale
 * must be 16-byte aligned, which every device allocation is.
 * The first `decoding_batches` sequences are decode sequences (one query token each); the rest
 * are prefill sequences.
 */
#ifndef PPL_NN_B200_H_
#define PPL_NN_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes.  ppl.nn reports ppl::common::RetCode; its numeric values are defined in the
 * ppl.common module, so the host layer maps these by name (RC_SUCCESS, RC_UNSUPPORTED, ...). */
enum {
    PPLB200_SUCCESS = 0,
    PPLB200_INVALID_VALUE = 1,       /* RC_INVALID_VALUE                                          */
    PPLB200_UNSUPPORTED = 2,         /* RC_UNSUPPORTED                                            */
    PPLB200_OUT_OF_MEMORY = 3,       /* RC_OUT_OF_MEMORY: workspace too small                     */
    PPLB200_DEVICE_RUNTIME_ERROR = 4,/* RC_DEVICE_RUNTIME_ERROR: a CUDA call or launch failed     */
    PPLB200_NOT_FOUND = 5,           /* RC_NOT_FOUND: a required pointer is null                  */
    PPLB200_NO_DEVICE_CODE = 6       /* the library was built without sm_100a device code        */
};

/* Phases of MultiHeadCacheAttention, for pplb200_attn_params.phase_mask (0 means all). */
enum {
    PPLB200_PHASE_APPEND = 1,  /* quantise + append current_key/current_value                     */
    PPLB200_PHASE_DECODE = 2,  /* split-k attention of the first decoding_batches sequences       */
    PPLB200_PHASE_PREFILL = 4  /* causal attention of the remaining sequences                     */
};

/*
 * Operator attributes + engine knobs + launch geometry, i.e. everything that
 * dynamic_batching_multi_head_cache_attention::heuristic_prepare() receives as scalars
 * (multi_head_cache_attention_kernel.cc:170-212), plus the attributes of KeyValueCacheParam
 * (src/ppl/nn/params/opmx/key_value_cache_param.h:10-18) that the append needs.
 */
typedef struct pplb200_attn_params {
    /* MultiHeadCacheAttentionParam (src/ppl/nn/params/opmx/multi_head_cache_attention_param.h:10-22) */
    int32_t num_heads;
    int32_t num_kv_heads;
    int32_t head_dim;           /* 64 or 128                                                      */
    int32_t is_causal;
    int32_t num_layer;
    int32_t layer_idx;
    int32_t quant_bit;          /* must be 8                                                      */
    int32_t quant_group;        /* must be 8                                                      */
    int32_t cache_mode;         /* 0: one contiguous row range per sequence, 1: paged             */
    int32_t cache_layout;       /* 0 or 3                                                         */
    int32_t page_size;          /* paged mode only; a multiple of 16                              */
    /* EngineConfig knobs (src/ppl/nn/engines/llm_cuda/engine_config.h:30-35) */
    int32_t enable_cache_prefill;  /* prefill reads the INT8 cache including start_pos history    */
    int32_t split_k_mode;          /* specify_decoding_attn_split_k: 0 off, 1 heuristic, 2 always */
    int32_t phase_mask;            /* 0 = all phases; else an OR of PPLB200_PHASE_*               */
    /* host scalars of the call (multi_head_cache_attention_kernel.cc:114-134) */
    int64_t batch;              /* start_pos.dim(0)                                               */
    int64_t decoding_batches;
    int64_t max_seqlen;
    int64_t max_kvlen;
    int64_t total_tokens;       /* T = query.dim(0)                                               */
    int64_t max_tokens;         /* MaxT: cache rows (cache.dim(0) for layout 0, dim(3) for 3)     */
    /* cache strides in elements of `cache` (same file :141-155); the scale tensor uses the same
     * strides divided by quant_group */
    int64_t cache_stride_s;
    int64_t cache_stride_l;
    int64_t cache_stride_h;
    int64_t cache_stride_kv;
    int64_t cachestart_stride_b; /* cachestarts.dim(1) when cache_mode == 1, else 0 (:161-168)    */
} pplb200_attn_params;

/* Fills the four cache strides from (cache_layout, num_layer, num_kv_heads, head_dim, max_tokens)
 * exactly as multi_head_cache_attention_kernel.cc:141-155 does.  Host only. */
int pplb200_fill_cache_strides(pplb200_attn_params* p);

/*
 * KeyValueCache, write side.  Replaces the quantise-and-append that the reference performs
 * inside dynamic_batching_multi_head_cache_attention::forward (call site
 * multi_head_cache_attention_kernel.cc:230; operator contract
 * kernels/opmx/dynamic_batching/key_value_cache_kernel.cc:26-35).
 * Token i of sequence b goes to cache row cachestarts[b] + start_pos[b] + i.
 * Codes: int8 in [-127,127]; scale: fp16(absmax/127) per group of 8 channels.
 */
int pplb200_kv_append_i8g8(const pplb200_attn_params* p, const void* current_key, const void* current_value,
                           const int64_t* seqstarts, const int64_t* cachestarts, const int64_t* start_pos,
                           void* cache, void* scale, void* stream);

/*
 * KeyValueCache, read side: the operator's `key` and `value` outputs, i.e. the dequantised
 * history of every sequence packed as [total_kv, num_kv_heads, head_dim] fp16 with
 * total_kv = kvstarts[batch]
 * (src/ppl/nn/oputils/opmx/reshape_dynamic_batching_key_value_cache.cc:26-41;
 *  src/ppl/nn/engines/llm_cuda/ops/opmx/dynamic_batching/key_value_cache_op.cc:37-56).
 */
int pplb200_kv_gather_dequant(const pplb200_attn_params* p, const int64_t* kvstarts, const int64_t* cachestarts,
                              const void* cache, const void* scale, int64_t total_kv, void* key_out,
                              void* value_out, void* stream);

/*
 * Scratch bytes that pplb200_mhca_forward needs for these params.  Replaces
 * heuristic_prepare()'s cfg.workspace_size (multi_head_cache_attention_kernel.cc:170-218).
 * Host only; depends on batch, decoding_batches, max_seqlen, max_kvlen, head counts and knobs.
 */
int pplb200_mhca_workspace_size(const pplb200_attn_params* p, uint64_t* bytes);

/*
 * MultiHeadCacheAttention.  Replaces heuristic_prepare() + forward()
 * (multi_head_cache_attention_kernel.cc:170-230): append (unless masked out), split-k decode
 * over the INT8 cache for sequences [0, decoding_batches), causal prefill for the rest.
 * `workspace` is caller-allocated device memory of at least pplb200_mhca_workspace_size() bytes,
 * 256-byte aligned; its contents need not be initialised and are undefined afterwards.
 * Calls that share a workspace must not overlap on the device.
 */
int pplb200_mhca_forward(const pplb200_attn_params* p, const void* query, const void* current_key,
                         const void* current_value, const int64_t* seqstarts, const int64_t* kvstarts,
                         const int64_t* cachestarts, const int64_t* start_pos, void* cache, void* scale,
                         void* workspace, uint64_t workspace_bytes, void* attn_output, void* stream);

/*
 * The optional attn_mask input of both attention operators.  The reference hands its shape and pointer
 * to the external kernel (multi_head_cache_attention_kernel.cc:105-110,179-180;
 * multi_head_attention_kernel.cc:96-103,114-115) and treats a tensor of zero elements as absent; the meaning
 * of the values is fixed by this library as follows.  The mask is ADDITIVE, fp16, dense, of shape
 * [T, C] (one mask for all heads) or [num_heads, T, C]; T = seqstarts[batch] query tokens, C >= kvstarts[batch]
 * and C % 8 == 0.  The element for query token i and kv position j of sequence b is
 * [.., seqstarts[b] + i, kvstarts[b] + j]; it is added to the scaled score q.k / sqrt(head_dim) before the
 * softmax, in addition to the causal mask when is_causal is set.  -inf removes a position; a query row whose
 * visible positions are all removed yields zeros; +inf and NaN entries count as -inf.  Entries the tensor
 * is too narrow to hold read as 0 and set PPLB200_DEV_MASK_OUT_OF_RANGE in the device status word.
 * data == NULL (or a NULL pplb200_attn_mask pointer): no mask.
 */
typedef struct pplb200_attn_mask {
    const void* data; /* device pointer, fp16 */
    int32_t ndim;     /* 2 or 3 */
    int32_t reserved;
    int64_t dims[3];  /* the first `ndim` entries are used */
} pplb200_attn_mask;

/* Host-only shape check of a mask against the operator's head count and query rows: PPLB200_SUCCESS (also
 * for an absent mask) or PPLB200_INVALID_VALUE.  The forward calls run the same check. */
int pplb200_attn_mask_check(const pplb200_attn_mask* attn_mask, int32_t num_heads, int64_t total_tokens);

/* pplb200_mhca_forward with the attn_mask input (multi_head_cache_attention_kernel.cc:39, input 12). */
int pplb200_mhca_forward_masked(const pplb200_attn_params* p, const void* query, const void* current_key,
                                const void* current_value, const int64_t* seqstarts, const int64_t* kvstarts,
                                const int64_t* cachestarts, const int64_t* start_pos, void* cache, void* scale,
                                const pplb200_attn_mask* attn_mask, void* workspace, uint64_t workspace_bytes,
                                void* attn_output, void* stream);

/*
 * MultiHeadCacheAttention without a caller workspace.  This entry point has no counterpart in the
 * reference: ppl.nn always borrows the scratch from its engine's tmp-buffer pool
 * (multi_head_cache_attention_kernel.cc:218-228).  It is for callers that cannot allocate device
 * memory at all -- an operator invoked outside an engine's device context has no pool to borrow
 * from, and a server that gave every free byte to the KV cache, or that must not call cudaMalloc
 * behind its own allocator's back, has nowhere to get a buffer.  Same arguments and results as
 * pplb200_mhca_forward, minus `workspace`: the scratch is a fixed 32 MiB array inside the library's
 * device image (pplb200_static_scratch_bytes(); every GPU that loads the library carries it until
 * the process exits).  The call allocates and frees nothing.
 *   - Calls whose pplb200_mhca_workspace_size() exceeds that capacity return PPLB200_OUT_OF_MEMORY
 *     and enqueue nothing.
 *   - The first call on each device looks up the array's device address (with that device
 *     current); make that first call before starting any stream capture.
 *   - All calls on a device share the one array, which keeps whatever the previous call left in
 *     it; the kernels re-initialise what they rely on, but two calls that overlap on the GPU
 *     (different streams) race on it.  The status word is read with pplb200_static_scratch_status.
 */
int pplb200_mhca_forward_noalloc(const pplb200_attn_params* p, const void* query, const void* current_key,
                                 const void* current_value, const int64_t* seqstarts, const int64_t* kvstarts,
                                 const int64_t* cachestarts, const int64_t* start_pos, void* cache, void* scale,
                                 void* attn_output, void* stream);

/* Capacity in bytes of the built-in scratch used by pplb200_mhca_forward_noalloc. */
uint64_t pplb200_static_scratch_bytes(void);

/* pplb200_mhca_device_status for the built-in scratch of the current device: the status word the last
 * pplb200_mhca_forward_noalloc call on this device left behind.  Synchronises `stream`.  The library does
 * not follow a cudaDeviceReset: the looked-up address is kept for the life of the process. */
int pplb200_static_scratch_status(void* stream, uint32_t* status);

/*
 * MultiHeadAttention without a cache (opmx.dynamic_batching.MultiHeadAttention).  Replaces
 * ppl::kernel::llm::cuda::pmx::dynamic_batching_multi_head_attention as called from
 * src/ppl/nn/engines/llm_cuda/kernels/opmx/dynamic_batching/multi_head_attention_kernel.cc:96-121
 * (attributes: src/ppl/nn/params/opmx/multi_head_attention_param.h).
 *   query [total_tokens, num_heads, head_dim], key/value [total_kv_tokens, num_kv_heads, head_dim], fp16;
 *   sequence b owns query rows [seqstarts[b], seqstarts[b+1]) and kv rows [kvstarts[b], kvstarts[b+1]).
 *   is_causal: query row i of a sequence sees kv positions <= (kvlen - seqlen) + i, i.e. the mask is
 *   aligned to the end of the kv range; a row that sees nothing yields zeros.  Scores are scaled by
 *   1/sqrt(head_dim).  `decoding_batches` is accepted for symmetry with the cached operator and not used.
 * is_alibi of the reference operator is not supported (the reference refuses it as well,
 * multi_head_attention_kernel.cc:72-75); the attn_mask input goes through pplb200_mha_forward_masked.
 * `workspace`: at least pplb200_mha_workspace_size() bytes of device memory
 * (it only holds the device status word, readable with pplb200_mhca_device_status).
 */
typedef struct pplb200_mha_params {
    int32_t num_heads;
    int32_t num_kv_heads;
    int32_t head_dim; /* 64 or 128 */
    int32_t is_causal;
    int64_t batch;
    int64_t decoding_batches;
    int64_t max_seqlen;
    int64_t max_kvlen;
    int64_t total_tokens;    /* = seqstarts[batch] */
    int64_t total_kv_tokens; /* = kvstarts[batch] */
} pplb200_mha_params;

int pplb200_mha_workspace_size(const pplb200_mha_params* p, uint64_t* bytes);

int pplb200_mha_forward(const pplb200_mha_params* p, const void* query, const void* key, const void* value,
                        const int64_t* seqstarts, const int64_t* kvstarts, void* workspace, uint64_t workspace_bytes,
                        void* attn_output, void* stream);

/* pplb200_mha_forward with the attn_mask input (multi_head_attention_kernel.cc:30, input 3); see
 * pplb200_attn_mask for the convention. */
int pplb200_mha_forward_masked(const pplb200_mha_params* p, const void* query, const void* key, const void* value,
                               const int64_t* seqstarts, const int64_t* kvstarts, const pplb200_attn_mask* attn_mask,
                               void* workspace, uint64_t workspace_bytes, void* attn_output, void* stream);

/*
 * RotaryPositionEmbedding for ragged batches (opmx.dynamic_batching.RotaryPositionEmbedding).  Replaces
 * ppl::kernel::llm::cuda::pmx::dynamic_batching_rotary_position_embedding as called from
 * src/ppl/nn/engines/llm_cuda/kernels/opmx/dynamic_batching/rotary_position_embedding_kernel.cc:107-129
 * (attributes: src/ppl/nn/params/opmx/rotary_position_embedding_param.h).
 *   query [total_tokens, num_heads, head_dim], key [total_tokens, num_kv_heads, head_dim], fp16;
 *   the token at index i of sequence b has position start_pos[b] + i.
 *   Channel pairs (2j, 2j+1), j < rotary_dim/2 (rotary_dim 0 = head_dim), are rotated by
 *   pos_eff * theta_eff^(-2j/rotary_dim); the other channels pass through.  scaling_type 0 none,
 *   1 linear (pos / scaling_factor), 2 dynamic (theta grows once start_pos + seqlen exceeds
 *   max_position_embeddings).  bypass_key != 0: the key passes through unrotated.
 *   rotated_query / rotated_key may alias query / key (the reference hands the input buffers over when it can).
 * `workspace`: pplb200_rope_workspace_size() bytes of device memory (the inverse-frequency table).
 */
typedef struct pplb200_rope_params {
    int32_t num_heads;
    int32_t num_kv_heads;
    int32_t head_dim;   /* 64 or 128 */
    int32_t rotary_dim; /* even, <= head_dim; 0 = head_dim */
    int32_t bypass_key;
    int32_t scaling_type; /* 0 none, 1 linear, 2 dynamic */
    int32_t max_position_embeddings;
    int32_t reserved;
    float theta;
    float scaling_factor;
    int64_t batch;
    int64_t max_seqlen;
    int64_t total_tokens;
} pplb200_rope_params;

int pplb200_rope_workspace_size(const pplb200_rope_params* p, uint64_t* bytes);

int pplb200_rope_forward(const pplb200_rope_params* p, const void* query, const void* key, const int64_t* seqstarts,
                         const int64_t* start_pos, void* workspace, uint64_t workspace_bytes, void* rotated_query,
                         void* rotated_key, void* stream);

/*
 * The rotary embedding and the KeyValueCache write side in one call (one kernel for the small batches of
 * decode steps; rotation and append kernels back to back for batches of 1024 tokens and more when
 * `rotated_key` is given, which is faster there): rotates the query into
 * `rotated_query`, rotates the key, rounds it to fp16 (written to `rotated_key` unless that is null),
 * quantises it and `value` and appends both to the cache.  The cache rows are bit-identical to
 * pplb200_rope_forward followed by pplb200_kv_append_i8g8; a following pplb200_mhca_forward is called with
 * phase_mask = PPLB200_PHASE_DECODE | PPLB200_PHASE_PREFILL.  No counterpart in the reference, whose
 * graph runs the two operators separately; `rotated_key` may only be null when the step has no prefill
 * sequence reading it.  `attn` supplies the cache geometry (layer, layout, strides, paging).
 */
int pplb200_rope_kv_append_i8g8(const pplb200_rope_params* p, const pplb200_attn_params* attn, const void* query,
                                const void* key, const void* value, const int64_t* seqstarts,
                                const int64_t* cachestarts, const int64_t* start_pos, void* workspace,
                                uint64_t workspace_bytes, void* rotated_query, void* rotated_key, void* cache,
                                void* scale, void* stream);

/*
 * Reads the device-side status word that the kernels of the last pplb200_mhca_forward on this
 * workspace left behind (0 = clean; non-zero = a bounded wait gave up, see PPLB200_DEV_*).
 * Synchronises `stream`.  Has no counterpart in the reference; it exists because every wait
 * in these kernels is bounded and reports instead of hanging.
 */
int pplb200_mhca_device_status(const void* workspace, void* stream, uint32_t* status);

enum {
    PPLB200_DEV_OK = 0,
    PPLB200_DEV_TMA_WAIT_TIMEOUT = 1,  /* a wait for a bulk-tensor copy ran out of iterations    */
    PPLB200_DEV_MMA_WAIT_TIMEOUT = 2,  /* a wait for a tensor-core commit ran out of iterations   */
    PPLB200_DEV_LENGTH_CLAMPED = 4,    /* a sequence exceeded max_kvlen / max_seqlen and was cut   */
    PPLB200_DEV_ROW_OUT_OF_RANGE = 8,  /* cachestarts/start_pos named a row outside [0, max_tokens):
                                          that row was neither read nor written                     */
    PPLB200_DEV_MASK_OUT_OF_RANGE = 16 /* attn_mask has fewer columns than kvstarts needs: the missing
                                          entries were read as 0                                    */
};

/* Name of a status code ("RC_SUCCESS", ...).  Never null. */
const char* pplb200_status_str(int status);

/* 1 if the library contains sm_100a device code and a CUDA device is present, else 0. */
int pplb200_device_ready(void);

/* Number of kernels launched by this library since load (all entry points).  For benchmarks. */
uint64_t pplb200_launch_count(void);

/*
 * Measurement aid, in the spirit of the reference's PPLNN_ENABLE_KERNEL_PROFILING event pairs
 * (src/ppl/nn/engines/llm_cuda/kernel.cc:93-160), but per CUDA kernel instead of per operator:
 * while enabled, each launch of the kernel families below is bracketed by a pair of CUDA events
 * recorded on the launching stream.  pplb200_profile_read() synchronises those events, returns
 * the summed device time and the launch count of one family since the last read, and clears them.
 * Off by default; not thread-safe against concurrent launches.
 */
enum {
    PPLB200_KERNEL_APPEND = 0,   /* kv_append_i8g8_kernel   */
    PPLB200_KERNEL_DECODE = 1,   /* decode_splitk_kernel    */
    PPLB200_KERNEL_PREFILL = 2,  /* prefill_tcgen05_kernel  */
    PPLB200_KERNEL_FAMILIES = 3
};
int pplb200_profile_enable(int enable);
int pplb200_profile_read(int kernel_family, double* total_ms, uint64_t* launches);

#ifdef __cplusplus
}
#endif
#endif /* PPL_NN_B200_H_ */
