// Operator and kernel classes of the two ops; see b200_ops.h.
#include "b200_ops.h"

#include "ppl_nn_b200.h"

using namespace ppl::common;

namespace ppl { namespace nn { namespace llm { namespace cuda { namespace opmx {

namespace {

RetCode FromStatus(int s) {
    switch (s) {
        case PPLB200_SUCCESS: return RC_SUCCESS;
        case PPLB200_INVALID_VALUE: return RC_INVALID_VALUE;
        case PPLB200_OUT_OF_MEMORY: return RC_OUT_OF_MEMORY;
        case PPLB200_NOT_FOUND: return RC_NOT_FOUND;
        case PPLB200_DEVICE_RUNTIME_ERROR: return RC_DEVICE_RUNTIME_ERROR;
        default: return RC_UNSUPPORTED;  // PPLB200_UNSUPPORTED, PPLB200_NO_DEVICE_CODE
    }
}

// Input/output slot lookup.  A slot beyond the node's arity or an empty slot yields null; a missing
// REQUIRED tensor is RC_NOT_FOUND with the engine's message (src/ppl/nn/engines/llm_cuda/macros.h:84-89).
struct Slots {
    explicit Slots(KernelExecContext* c) : ctx(c) {}
    TensorImpl* In(uint32_t idx) const { return idx < ctx->GetInputCount() ? ctx->GetInput<TensorImpl>(idx) : nullptr; }
    TensorImpl* Out(uint32_t idx) const { return idx < ctx->GetOutputCount() ? ctx->GetOutput<TensorImpl>(idx) : nullptr; }
    bool Need(TensorImpl* t, const char* kind, const char* name) {
        if (!t) {
            LOG(ERROR) << kind << " \"" << name << "\" is required.";
            rc = RC_NOT_FOUND;
            return false;
        }
        return true;
    }
    KernelExecContext* ctx;
    RetCode rc = RC_SUCCESS;
};

// host scalars arrive as tensors that normally live on the host device
RetCode ReadScalar(const TensorImpl* t, int64_t* v, const char* name) {
    if (t->CopyToHost(v) != RC_SUCCESS) {
        LOG(ERROR) << name << "->CopyToHost() failed";
        return RC_DEVICE_MEMORY_ERROR;
    }
    return RC_SUCCESS;
}

// Every tensor whose pointer is handed to the GPU kernels must live on the engine's GPU; a host tensor
// here would make the kernels read a host address.
RetCode RequireOnDevice(const TensorImpl* t, const Device* dev) {
    if (t->GetDevice() != dev || !t->GetBufferPtr()) {
        LOG(ERROR) << "tensor[" << t->GetName() << "] must have a buffer on the engine's GPU";
        return RC_INVALID_VALUE;
    }
    return RC_SUCCESS;
}

// The optional attn_mask input: shape and pointer are handed down as the reference hands them down
// (multi_head_cache_attention_kernel.cc:105-110,179-180); a tensor without elements counts as absent.
// Fills `m` (data stays null without a mask); the tensor must be fp16 and live on the device.
RetCode MaskFromTensor(TensorImpl* attn_mask, const Device* dev, int32_t num_heads, int64_t tokens,
                       pplb200_attn_mask* m) {
    memset(m, 0, sizeof(*m));
    if (!attn_mask || attn_mask->GetShape()->CalcElementsExcludingPadding() == 0) {
        return RC_SUCCESS;
    }
    const TensorShape* shape = attn_mask->GetShape();
    if (shape->GetDataType() != DATATYPE_FLOAT16) {
        LOG(ERROR) << "attn_mask must be fp16";
        return RC_UNSUPPORTED;
    }
    if (shape->GetDimCount() != 2 && shape->GetDimCount() != 3) {
        LOG(ERROR) << "attn_mask must be a 2d or 3d tensor";
        return RC_INVALID_VALUE;
    }
    const RetCode rc = RequireOnDevice(attn_mask, dev);
    if (rc != RC_SUCCESS) {
        return rc;
    }
    m->data = attn_mask->GetBufferPtr();
    m->ndim = static_cast<int32_t>(shape->GetDimCount());
    for (uint32_t i = 0; i < shape->GetDimCount(); ++i) {
        m->dims[i] = shape->GetDim(i);
    }
    return FromStatus(pplb200_attn_mask_check(m, num_heads, tokens));
}


// The kernels index [tokens, heads, head_dim] tensors with the attribute values, so a tensor of another
// shape would be read out of bounds; the reference leaves this to its kernel library.
RetCode RequireTokenTensor(const TensorImpl* t, int64_t tokens, int64_t heads, int64_t head_dim) {
    const TensorShape& s = *t->GetShape();
    if (s.GetDimCount() != 3 || (tokens >= 0 && s.GetDim(0) != tokens) || s.GetDim(1) != heads || s.GetDim(2) != head_dim) {
        LOG(ERROR) << "tensor[" << t->GetName() << "] must be [tokens, " << heads << ", " << head_dim << "]";
        return RC_INVALID_VALUE;
    }
    return RC_SUCCESS;
}

RetCode RequireIndexTensor(const TensorImpl* t, int64_t min_rows) {
    const TensorShape& s = *t->GetShape();
    if (s.GetDataType() != DATATYPE_INT64 || s.GetDimCount() < 1 || s.GetDim(0) < min_rows) {
        LOG(ERROR) << "tensor[" << t->GetName() << "] must be int64 with at least " << min_rows << " rows";
        return RC_INVALID_VALUE;
    }
    return RC_SUCCESS;
}

RetCode ReallocOn(TensorImpl* t, Device* dev) {
    t->SetDevice(dev);
    const RetCode rc = t->ReallocBuffer();
    if (rc != RC_SUCCESS) {
        LOG(ERROR) << "ReallocBuffer for tensor[" << t->GetName() << "] failed: " << GetRetCodeStr(rc);
    }
    return rc;
}

}  // namespace

// =================================================================================================
// MultiHeadCacheAttention
// =================================================================================================
RetCode DynamicBatchingMultiHeadCacheAttentionOp::DoInit(const OptKernelOptions& options) {
    const RetCode rc = GenericLoadParam<ppl::nn::opmx::MultiHeadCacheAttentionParam>(options, &param_);
    if (rc != RC_SUCCESS) {
        LOG(ERROR) << "GenericLoadParam failed: " << GetRetCodeStr(rc);
        return rc;
    }
    infer_type_and_format_func_ = GenericInferTypeAndFormat;
    infer_dims_func_ = GenericInferDims;  // attn_output has query's shape
    return RC_SUCCESS;
}

KernelImpl* DynamicBatchingMultiHeadCacheAttentionOp::CreateKernelImpl() const {
    return CreateKernelImplWithParam<DynamicBatchingMultiHeadCacheAttentionKernel>(param_.get());
}

RetCode DynamicBatchingMultiHeadCacheAttentionKernel::DoExecute(KernelExecContext* ctx) {
    // inputs by index: 0 query, 1 current_key, 2 current_value, 3 seqstarts, 4 kvstarts, 5 cachestarts,
    // 6 start_pos, 7 decoding_batches, 8 max_seqlen, 9 max_kvlen, 10 cache, 11 scale (optional),
    // 12 attn_mask (optional); output 0 attn_output
    static const char* const kNames[11] = {"query",       "current_key", "current_value",    "seqstarts",  "kvstarts",
                                           "cachestarts", "start_pos",   "decoding_batches", "max_seqlen", "max_kvlen",
                                           "cache"};
    Slots s(ctx);
    TensorImpl* in[13];
    for (uint32_t i = 0; i < 13; ++i) {
        in[i] = s.In(i);
        if (i < 11 && !s.Need(in[i], "Input", kNames[i])) {
            return s.rc;
        }
    }
    TensorImpl* attn_output = s.Out(0);
    if (!s.Need(attn_output, "Output", "attn_output")) {
        return s.rc;
    }
    TensorImpl *query = in[0], *current_key = in[1], *current_value = in[2], *seqstarts = in[3], *kvstarts = in[4],
               *cachestarts = in[5], *start_pos = in[6], *cache = in[10], *scale = in[11], *attn_mask = in[12];

    RetCode rc = Reshape(ctx);
    if (rc != RC_SUCCESS) {
        LOG(ERROR) << "Reshape kernel[" << GetName() << "] failed: " << GetRetCodeStr(rc);
        return rc;
    }

    // The reference rejects only when BOTH differ from 8; nothing else is implemented here, so either
    // one differing is rejected.
    if (param_->quant_bit != 8 || param_->quant_group != 8) {
        LOG(ERROR) << "currently only support quant_bit == quant_group == 8";
        return RC_UNSUPPORTED;
    }
    if (param_->is_alibi) {
        LOG(ERROR) << "currently only support is_alibi == false";
        return RC_UNSUPPORTED;
    }
    if (!scale || scale->GetShape()->CalcElementsExcludingPadding() == 0) {
        LOG(ERROR) << "currently only support quantized cache but scale not found";
        return RC_UNSUPPORTED;
    }
    pplb200_attn_mask mask;
    if ((rc = MaskFromTensor(attn_mask, GetCudaDevice(), param_->num_heads,
                             query->GetShape()->GetDimCount() > 0 ? query->GetShape()->GetDim(0) : 0, &mask)) !=
        RC_SUCCESS) {
        return rc;
    }
    if (query->GetShape()->GetDataType() != DATATYPE_FLOAT16) {
        LOG(ERROR) << "currently only support fp16";
        return RC_UNSUPPORTED;
    }

    {
        const int64_t tokens = query->GetShape()->GetDimCount() > 0 ? query->GetShape()->GetDim(0) : 0;
        const int64_t batch = start_pos->GetShape()->GetDimCount() > 0 ? start_pos->GetShape()->GetDim(0) : 0;
        if ((rc = RequireTokenTensor(query, -1, param_->num_heads, param_->head_dim)) != RC_SUCCESS ||
            (rc = RequireTokenTensor(current_key, tokens, param_->num_kv_heads, param_->head_dim)) != RC_SUCCESS ||
            (rc = RequireTokenTensor(current_value, tokens, param_->num_kv_heads, param_->head_dim)) != RC_SUCCESS ||
            (rc = RequireIndexTensor(start_pos, 0)) != RC_SUCCESS ||
            (rc = RequireIndexTensor(seqstarts, batch + 1)) != RC_SUCCESS ||
            (rc = RequireIndexTensor(kvstarts, batch + 1)) != RC_SUCCESS ||
            (rc = RequireIndexTensor(cachestarts, batch)) != RC_SUCCESS) {
            return rc;
        }
        if (cache->GetShape()->GetDimCount() != 5 || scale->GetShape()->GetDimCount() != 5) {
            LOG(ERROR) << "cache and scale must be 5-d tensors";
            return RC_INVALID_VALUE;
        }
    }
    for (TensorImpl* t : {query, current_key, current_value, seqstarts, kvstarts, cachestarts, start_pos, cache, scale}) {
        if ((rc = RequireOnDevice(t, GetCudaDevice())) != RC_SUCCESS) {
            return rc;
        }
    }
    if ((rc = ReallocOn(attn_output, GetCudaDevice())) != RC_SUCCESS) {
        return rc;
    }

    int64_t decoding_batches = 0, max_seqlen = 0, max_kvlen = 0;
    if ((rc = ReadScalar(in[7], &decoding_batches, "decoding_batches")) != RC_SUCCESS) return rc;
    if ((rc = ReadScalar(in[8], &max_seqlen, "max_seqlen")) != RC_SUCCESS) return rc;
    if ((rc = ReadScalar(in[9], &max_kvlen, "max_kvlen")) != RC_SUCCESS) return rc;

    pplb200_attn_params p;
    memset(&p, 0, sizeof(p));
    p.num_heads = param_->num_heads;
    p.num_kv_heads = param_->num_kv_heads;
    p.head_dim = param_->head_dim;
    p.is_causal = param_->is_causal ? 1 : 0;
    p.num_layer = param_->num_layer;
    p.layer_idx = param_->layer_idx;
    p.quant_bit = param_->quant_bit;
    p.quant_group = param_->quant_group;
    p.cache_mode = param_->cache_mode;
    p.cache_layout = param_->cache_layout;
    p.page_size = param_->page_size;
    p.enable_cache_prefill = GetEngineConfig().enable_cache_prefill ? 1 : 0;
    p.split_k_mode = GetEngineConfig().specify_decoding_attn_split_k;
    p.batch = start_pos->GetShape()->GetDim(0);  // the batch comes from start_pos, not seqstarts
    p.decoding_batches = decoding_batches;
    p.max_seqlen = max_seqlen;
    p.max_kvlen = max_kvlen;
    p.total_tokens = query->GetShape()->GetDim(0);
    if (param_->cache_layout == 0) {
        p.max_tokens = cache->GetShape()->GetDim(0);  // (MaxT, L, 2, H, Dh)
    } else if (param_->cache_layout == 3) {
        p.max_tokens = cache->GetShape()->GetDim(3);  // (L, 2, H, MaxT, Dh)
    } else {
        LOG(ERROR) << "currently only support cache_layout == 0 or cache_layout == 3";
        return RC_UNSUPPORTED;
    }
    if ((rc = FromStatus(pplb200_fill_cache_strides(&p))) != RC_SUCCESS) {
        return rc;
    }
    if (param_->cache_mode == 1) {
        if (cachestarts->GetShape()->GetDimCount() != 2) {
            LOG(ERROR) << "cachestarts must be a 2d tensor in cache_mode 1";
            return RC_INVALID_VALUE;
        }
        p.cachestart_stride_b = cachestarts->GetShape()->GetDim(1);
    }

    uint64_t workspace_bytes = 0;
    if ((rc = FromStatus(pplb200_mhca_workspace_size(&p, &workspace_bytes))) != RC_SUCCESS) {
        return rc;
    }
    BufferDesc tmp;
    rc = GetCudaDevice()->AllocTmpBuffer(workspace_bytes, &tmp);
    if (rc != RC_SUCCESS) {
        LOG(ERROR) << "alloc tmp buffer size[" << workspace_bytes << "] for kernel[" << GetName()
                   << "] failed: " << GetRetCodeStr(rc);
        return rc;
    }
    Destructor tmp_guard([this, &tmp]() { GetCudaDevice()->FreeTmpBuffer(&tmp); });

    return FromStatus(pplb200_mhca_forward_masked(
        &p, query->GetBufferPtr(), current_key->GetBufferPtr(), current_value->GetBufferPtr(),
        seqstarts->GetBufferPtr<int64_t>(), kvstarts->GetBufferPtr<int64_t>(), cachestarts->GetBufferPtr<int64_t>(),
        start_pos->GetBufferPtr<int64_t>(), cache->GetBufferPtr(), scale->GetBufferPtr(), &mask, tmp.addr,
        workspace_bytes, attn_output->GetBufferPtr(), GetStream()));
}

// =================================================================================================
// MultiHeadAttention (no cache)
// =================================================================================================
RetCode DynamicBatchingMultiHeadAttentionOp::DoInit(const OptKernelOptions& options) {
    const RetCode rc = GenericLoadParam<ppl::nn::opmx::MultiHeadAttentionParam>(options, &param_);
    if (rc != RC_SUCCESS) {
        LOG(ERROR) << "GenericLoadParam failed: " << GetRetCodeStr(rc);
        return rc;
    }
    infer_type_and_format_func_ = GenericInferTypeAndFormat;
    infer_dims_func_ = GenericInferDims;  // attn_output has query's shape
    return RC_SUCCESS;
}

KernelImpl* DynamicBatchingMultiHeadAttentionOp::CreateKernelImpl() const {
    return CreateKernelImplWithParam<DynamicBatchingMultiHeadAttentionKernel>(param_.get());
}

RetCode DynamicBatchingMultiHeadAttentionKernel::DoExecute(KernelExecContext* ctx) {
    // inputs by index: 0 query, 1 key, 2 value, 3 seqstarts, 4 kvstarts, 5 decoding_batches, 6 max_seqlen,
    // 7 max_kvlen, 8 attn_mask (optional); output 0 attn_output
    // (src/ppl/nn/engines/llm_cuda/kernels/opmx/dynamic_batching/multi_head_attention_kernel.cc:27-37)
    static const char* const kNames[8] = {"query",    "key",        "value",     "seqstarts", "kvstarts", "decoding_batches",
                                          "max_seqlen", "max_kvlen"};
    Slots s(ctx);
    TensorImpl* in[9];
    for (uint32_t i = 0; i < 9; ++i) {
        in[i] = s.In(i);
        if (i < 8 && !s.Need(in[i], "Input", kNames[i])) {
            return s.rc;
        }
    }
    TensorImpl* attn_output = s.Out(0);
    if (!s.Need(attn_output, "Output", "attn_output")) {
        return s.rc;
    }
    TensorImpl *query = in[0], *key = in[1], *value = in[2], *seqstarts = in[3], *kvstarts = in[4], *attn_mask = in[8];

    RetCode rc = Reshape(ctx);
    if (rc != RC_SUCCESS) {
        LOG(ERROR) << "Reshape kernel[" << GetName() << "] failed: " << GetRetCodeStr(rc);
        return rc;
    }
    if (param_->is_alibi) {
        LOG(ERROR) << "currently only support is_alibi == false";
        return RC_UNSUPPORTED;
    }
    pplb200_attn_mask mask;
    if ((rc = MaskFromTensor(attn_mask, GetCudaDevice(), param_->num_heads,
                             query->GetShape()->GetDimCount() > 0 ? query->GetShape()->GetDim(0) : 0, &mask)) !=
        RC_SUCCESS) {
        return rc;
    }
    if (query->GetShape()->GetDataType() != DATATYPE_FLOAT16) {
        LOG(ERROR) << "currently only support fp16";
        return RC_UNSUPPORTED;
    }
    {
        const int64_t kv_tokens = key->GetShape()->GetDimCount() > 0 ? key->GetShape()->GetDim(0) : 0;
        if ((rc = RequireTokenTensor(query, -1, param_->num_heads, param_->head_dim)) != RC_SUCCESS ||
            (rc = RequireTokenTensor(key, -1, param_->num_kv_heads, param_->head_dim)) != RC_SUCCESS ||
            (rc = RequireTokenTensor(value, kv_tokens, param_->num_kv_heads, param_->head_dim)) != RC_SUCCESS ||
            (rc = RequireIndexTensor(seqstarts, 1)) != RC_SUCCESS ||
            (rc = RequireIndexTensor(kvstarts, seqstarts->GetShape()->GetDim(0))) != RC_SUCCESS) {
            return rc;
        }
    }
    for (TensorImpl* t : {query, key, value, seqstarts, kvstarts}) {
        if ((rc = RequireOnDevice(t, GetCudaDevice())) != RC_SUCCESS) {
            return rc;
        }
    }
    if ((rc = ReallocOn(attn_output, GetCudaDevice())) != RC_SUCCESS) {
        return rc;
    }

    int64_t decoding_batches = 0, max_seqlen = 0, max_kvlen = 0;
    if ((rc = ReadScalar(in[5], &decoding_batches, "decoding_batches")) != RC_SUCCESS) return rc;
    if ((rc = ReadScalar(in[6], &max_seqlen, "max_seqlen")) != RC_SUCCESS) return rc;
    if ((rc = ReadScalar(in[7], &max_kvlen, "max_kvlen")) != RC_SUCCESS) return rc;

    pplb200_mha_params p;
    memset(&p, 0, sizeof(p));
    p.num_heads = param_->num_heads;
    p.num_kv_heads = param_->num_kv_heads;
    p.head_dim = param_->head_dim;
    p.is_causal = param_->is_causal ? 1 : 0;
    p.batch = seqstarts->GetShape()->GetDim(0) - 1;  // here the batch does come from seqstarts
    p.decoding_batches = decoding_batches;
    p.max_seqlen = max_seqlen;
    p.max_kvlen = max_kvlen;
    p.total_tokens = query->GetShape()->GetDim(0);
    p.total_kv_tokens = key->GetShape()->GetDim(0);

    uint64_t workspace_bytes = 0;
    if ((rc = FromStatus(pplb200_mha_workspace_size(&p, &workspace_bytes))) != RC_SUCCESS) {
        return rc;
    }
    BufferDesc tmp;
    rc = GetCudaDevice()->AllocTmpBuffer(workspace_bytes, &tmp);
    if (rc != RC_SUCCESS) {
        LOG(ERROR) << "alloc tmp buffer size[" << workspace_bytes << "] for kernel[" << GetName()
                   << "] failed: " << GetRetCodeStr(rc);
        return rc;
    }
    Destructor tmp_guard([this, &tmp]() { GetCudaDevice()->FreeTmpBuffer(&tmp); });

    return FromStatus(pplb200_mha_forward_masked(&p, query->GetBufferPtr(), key->GetBufferPtr(), value->GetBufferPtr(),
                                                 seqstarts->GetBufferPtr<int64_t>(), kvstarts->GetBufferPtr<int64_t>(),
                                                 &mask, tmp.addr, workspace_bytes, attn_output->GetBufferPtr(),
                                                 GetStream()));
}

// =================================================================================================
// RotaryPositionEmbedding
// =================================================================================================
RetCode DynamicBatchingRotaryPositionEmbeddingOp::DoInit(const OptKernelOptions& options) {
    const RetCode rc = GenericLoadParam<ppl::nn::opmx::RotaryPositionEmbeddingParam>(options, &param_);
    if (rc != RC_SUCCESS) {
        LOG(ERROR) << "GenericLoadParam failed: " << GetRetCodeStr(rc);
        return rc;
    }
    infer_type_and_format_func_ = GenericInferTypeAndFormat;
    // rotated_query takes query's dims, rotated_key takes key's
    // (src/ppl/nn/oputils/opmx/reshape_rotary_position_embedding.cc:26-35)
    infer_dims_func_ = [](InputOutputInfo* info) -> RetCode {
        for (uint32_t i = 0; i < 2 && i < info->GetOutputCount(); ++i) {
            auto in = info->GetInput<TensorImpl>(i);
            auto out = info->GetOutput<TensorImpl>(i);
            if (in && out) {
                out->GetShape()->Reshape(in->GetShape()->GetDims(), in->GetShape()->GetDimCount());
            }
        }
        return RC_SUCCESS;
    };
    return RC_SUCCESS;
}

KernelImpl* DynamicBatchingRotaryPositionEmbeddingOp::CreateKernelImpl() const {
    return CreateKernelImplWithParam<DynamicBatchingRotaryPositionEmbeddingKernel>(param_.get());
}

RetCode DynamicBatchingRotaryPositionEmbeddingKernel::DoExecute(KernelExecContext* ctx) {
    // inputs by index: 0 query, 1 key, 2 seqstarts, 3 start_pos, 4 max_seqlen; outputs 0 rotated_query,
    // 1 rotated_key (src/ppl/nn/engines/llm_cuda/kernels/opmx/dynamic_batching/rotary_position_embedding_kernel.cc:27-34)
    static const char* const kNames[5] = {"query", "key", "seqstarts", "start_pos", "max_seqlen"};
    Slots s(ctx);
    TensorImpl* in[5];
    for (uint32_t i = 0; i < 5; ++i) {
        in[i] = s.In(i);
        if (!s.Need(in[i], "Input", kNames[i])) {
            return s.rc;
        }
    }
    TensorImpl* rotated_query = s.Out(0);
    TensorImpl* rotated_key = s.Out(1);
    if (!s.Need(rotated_query, "Output", "rotated_query") || !s.Need(rotated_key, "Output", "rotated_key")) {
        return s.rc;
    }
    TensorImpl *query = in[0], *key = in[1], *seqstarts = in[2], *start_pos = in[3];

    RetCode rc = Reshape(ctx);
    if (rc != RC_SUCCESS) {
        LOG(ERROR) << "Reshape kernel[" << GetName() << "] failed: " << GetRetCodeStr(rc);
        return rc;
    }
    if (query->GetShape()->GetDataType() != DATATYPE_FLOAT16) {
        LOG(ERROR) << "currently only support fp16";
        return RC_UNSUPPORTED;
    }
    {
        const TensorShape& qs = *query->GetShape();
        const TensorShape& ks = *key->GetShape();
        if (qs.GetDimCount() != 3 || ks.GetDimCount() != 3 || ks.GetDim(0) != qs.GetDim(0) || ks.GetDim(2) != qs.GetDim(2)) {
            LOG(ERROR) << "query and key must be [tokens, heads, head_dim] with the same tokens and head_dim";
            return RC_INVALID_VALUE;
        }
        if ((rc = RequireIndexTensor(start_pos, 0)) != RC_SUCCESS ||
            (rc = RequireIndexTensor(seqstarts, start_pos->GetShape()->GetDim(0) + 1)) != RC_SUCCESS) {
            return rc;
        }
    }
    for (TensorImpl* t : {query, key, seqstarts, start_pos}) {
        if ((rc = RequireOnDevice(t, GetCudaDevice())) != RC_SUCCESS) {
            return rc;
        }
    }
    // The input buffers are handed over to the outputs when this kernel is their last consumer, as the
    // reference does (:55-75); the kernels rotate in place then (the C ABI allows the aliasing).
    const bool can_trans_query = ctx->IsLastConsumerOfInput(0) && query->GetType() == TENSORTYPE_NORMAL;
    const bool can_trans_key = ctx->IsLastConsumerOfInput(1) && key->GetType() == TENSORTYPE_NORMAL;
    void* query_data = query->GetBufferPtr();
    void* key_data = key->GetBufferPtr();
    if (can_trans_query) {
        rotated_query->TransferBufferFrom(query);
    } else if ((rc = ReallocOn(rotated_query, GetCudaDevice())) != RC_SUCCESS) {
        return rc;
    }
    if (can_trans_key) {
        rotated_key->TransferBufferFrom(key);
    } else if ((rc = ReallocOn(rotated_key, GetCudaDevice())) != RC_SUCCESS) {
        return rc;
    }

    int64_t max_seqlen = 0;
    if ((rc = ReadScalar(in[4], &max_seqlen, "max_seqlen")) != RC_SUCCESS) return rc;

    pplb200_rope_params p;
    memset(&p, 0, sizeof(p));
    p.num_heads = static_cast<int32_t>(query->GetShape()->GetDim(1));
    p.num_kv_heads = static_cast<int32_t>(key->GetShape()->GetDim(1));
    p.head_dim = static_cast<int32_t>(query->GetShape()->GetDim(2));
    p.rotary_dim = param_->rotary_dim;
    p.bypass_key = param_->bypass_key;
    // The reference's mapping of the scaling type tests with != where == is meant (:94-103), which sends
    // every type to its neighbour; the attribute's own meaning is used here.
    p.scaling_type = param_->scaling_type;
    p.max_position_embeddings = param_->max_position_embeddings;
    p.theta = param_->theta;
    p.scaling_factor = param_->scaling_factor;
    p.batch = start_pos->GetShape()->GetDim(0);
    p.max_seqlen = max_seqlen;
    p.total_tokens = query->GetShape()->GetDim(0);

    uint64_t workspace_bytes = 0;
    if ((rc = FromStatus(pplb200_rope_workspace_size(&p, &workspace_bytes))) != RC_SUCCESS) {
        return rc;
    }
    BufferDesc tmp;
    rc = GetCudaDevice()->AllocTmpBuffer(workspace_bytes, &tmp);
    if (rc != RC_SUCCESS) {
        LOG(ERROR) << "alloc tmp buffer size[" << workspace_bytes << "] for kernel[" << GetName()
                   << "] failed: " << GetRetCodeStr(rc);
        return rc;
    }
    Destructor tmp_guard([this, &tmp]() { GetCudaDevice()->FreeTmpBuffer(&tmp); });
    return FromStatus(pplb200_rope_forward(&p, query_data, key_data, seqstarts->GetBufferPtr<int64_t>(),
                                           start_pos->GetBufferPtr<int64_t>(), tmp.addr, workspace_bytes,
                                           rotated_query->GetBufferPtr(), rotated_key->GetBufferPtr(), GetStream()));
}

// =================================================================================================
// KeyValueCache
// =================================================================================================
RetCode DynamicBatchingKeyValueCacheOp::DoInit(const OptKernelOptions& options) {
    const RetCode rc = GenericLoadParam<ppl::nn::opmx::KeyValueCacheParam>(options, &param_);
    if (rc != RC_SUCCESS) {
        LOG(ERROR) << "GenericLoadParam failed: " << GetRetCodeStr(rc);
        return rc;
    }
    infer_type_and_format_func_ = GenericInferTypeAndFormat;
    // key/value = current_key's dims with dim 0 replaced by the total kv length kvstarts[-1], read from
    // wherever kvstarts lives; without a buffer the outputs get length 0 and the caller is told
    infer_dims_func_ = [](InputOutputInfo* info) -> RetCode {
        const TensorImpl* current_key = info->GetInput<TensorImpl>(0);
        const TensorImpl* kvstarts = info->GetInput<TensorImpl>(3);
        const TensorShape& ks = *current_key->GetShape();
        std::vector<int64_t> dims(ks.GetDims(), ks.GetDims() + ks.GetDimCount());
        int64_t kv_length = 0;
        RetCode status = RC_SUCCESS;
        if (!kvstarts->GetBufferPtr()) {
            status = RC_NOT_FOUND;
        } else {
            const int64_t* last = kvstarts->GetBufferPtr<int64_t>() + kvstarts->GetShape()->GetDim(0) - 1;
            status = kvstarts->GetDevice()->CopyToHost(&kv_length, BufferDesc(const_cast<int64_t*>(last)), sizeof(int64_t));
            if (status != RC_SUCCESS) {
                LOG(ERROR) << "kvstarts->GetDevice()->CopyToHost() failed: " << GetRetCodeStr(status);
                return status;
            }
        }
        if (!dims.empty()) {
            dims[0] = kv_length;
        }
        info->GetOutput<TensorImpl>(0)->GetShape()->Reshape(dims);
        info->GetOutput<TensorImpl>(1)->GetShape()->Reshape(dims);
        return status;
    };
    return RC_SUCCESS;
}

KernelImpl* DynamicBatchingKeyValueCacheOp::CreateKernelImpl() const {
    return CreateKernelImplWithParam<DynamicBatchingKeyValueCacheKernel>(param_.get());
}

RetCode DynamicBatchingKeyValueCacheKernel::DoExecute(KernelExecContext* ctx) {
    // inputs: 0 current_key, 1 current_value, 2 seqstarts, 3 kvstarts, 4 cachestarts, 5 start_pos,
    // 6 max_seqlen, 7 max_kvlen, 8 cache, 9 scale (optional); outputs: 0 key, 1 value
    static const char* const kNames[9] = {"current_key", "current_value", "seqstarts",  "kvstarts", "cachestarts",
                                          "start_pos",   "max_seqlen",    "max_kvlen", "cache"};
    Slots s(ctx);
    TensorImpl* in[10];
    for (uint32_t i = 0; i < 10; ++i) {
        in[i] = s.In(i);
        if (i < 9 && !s.Need(in[i], "Input", kNames[i])) {
            return s.rc;
        }
    }
    TensorImpl *key = s.Out(0), *value = s.Out(1);
    if (!s.Need(key, "Output", "key") || !s.Need(value, "Output", "value")) {
        return s.rc;
    }
    TensorImpl *current_key = in[0], *current_value = in[1], *seqstarts = in[2], *kvstarts = in[3],
               *cachestarts = in[4], *start_pos = in[5], *cache = in[8], *scale = in[9];

    RetCode rc = Reshape(ctx);
    if (rc != RC_SUCCESS) {
        LOG(ERROR) << "Reshape kernel[" << GetName() << "] failed: " << GetRetCodeStr(rc);
        return rc;
    }
    if (!scale) {
        LOG(ERROR) << "currently only support quantized cache but scale not found";
        return RC_UNSUPPORTED;
    }
    if (param_->quant_bit != 8 || param_->quant_group != 8) {
        LOG(ERROR) << "currently only support quant_bit == quant_group == 8";
        return RC_UNSUPPORTED;
    }
    if (param_->cache_layout != 0 && param_->cache_layout != 3) {  // the reference's contract names layout 0 only
        LOG(ERROR) << "currently only support cache_layout == 0 or cache_layout == 3";
        return RC_UNSUPPORTED;
    }
    if (param_->cache_mode != 0 && param_->cache_mode != 1) {
        LOG(ERROR) << "currently only support cache_mode == 0 or cache_mode == 1";
        return RC_UNSUPPORTED;
    }
    if (param_->num_repeat != 1) {
        LOG(ERROR) << "currently only support num_repeat == 1";
        return RC_UNSUPPORTED;
    }
    {
        const TensorShape& cs = *current_key->GetShape();
        if (cs.GetDimCount() != 3) {
            LOG(ERROR) << "current_key must be [tokens, num_kv_heads, head_dim]";
            return RC_INVALID_VALUE;
        }
        const int64_t batch = start_pos->GetShape()->GetDimCount() > 0 ? start_pos->GetShape()->GetDim(0) : 0;
        if ((rc = RequireTokenTensor(current_value, cs.GetDim(0), cs.GetDim(1), cs.GetDim(2))) != RC_SUCCESS ||
            (rc = RequireIndexTensor(start_pos, 0)) != RC_SUCCESS ||
            (rc = RequireIndexTensor(seqstarts, batch + 1)) != RC_SUCCESS ||
            (rc = RequireIndexTensor(kvstarts, batch + 1)) != RC_SUCCESS ||
            (rc = RequireIndexTensor(cachestarts, batch)) != RC_SUCCESS) {
            return rc;
        }
        if (cache->GetShape()->GetDimCount() != 5 || scale->GetShape()->GetDimCount() != 5) {
            LOG(ERROR) << "cache and scale must be 5-d tensors";
            return RC_INVALID_VALUE;
        }
    }
    for (TensorImpl* t : {current_key, current_value, seqstarts, kvstarts, cachestarts, start_pos, cache, scale}) {
        if ((rc = RequireOnDevice(t, GetCudaDevice())) != RC_SUCCESS) {
            return rc;
        }
    }
    if ((rc = ReallocOn(key, GetCudaDevice())) != RC_SUCCESS) return rc;
    if ((rc = ReallocOn(value, GetCudaDevice())) != RC_SUCCESS) return rc;
    const TensorShape& ks = *current_key->GetShape();
    if (ks.GetDataType() != DATATYPE_FLOAT16) {
        LOG(ERROR) << "currently only support fp16";
        return RC_UNSUPPORTED;
    }

    pplb200_attn_params p;
    memset(&p, 0, sizeof(p));
    p.num_heads = p.num_kv_heads = static_cast<int32_t>(ks.GetDim(1));
    p.head_dim = static_cast<int32_t>(ks.GetDim(2));
    p.is_causal = 1;
    p.num_layer = param_->num_layer;
    p.layer_idx = param_->layer_idx;
    p.quant_bit = param_->quant_bit;
    p.quant_group = param_->quant_group;
    p.cache_mode = param_->cache_mode;
    p.cache_layout = param_->cache_layout;
    p.page_size = param_->page_size;
    p.batch = start_pos->GetShape()->GetDim(0);
    p.total_tokens = ks.GetDim(0);
    p.max_tokens = cache->GetShape()->GetDim(param_->cache_layout == 0 ? 0 : 3);
    if ((rc = FromStatus(pplb200_fill_cache_strides(&p))) != RC_SUCCESS) {
        return rc;
    }
    if (param_->cache_mode == 1) {
        if (cachestarts->GetShape()->GetDimCount() != 2) {
            LOG(ERROR) << "cachestarts must be a 2d tensor in cache_mode 1";
            return RC_INVALID_VALUE;
        }
        p.cachestart_stride_b = cachestarts->GetShape()->GetDim(1);
    }
    rc = FromStatus(pplb200_kv_append_i8g8(&p, current_key->GetBufferPtr(), current_value->GetBufferPtr(),
                                           seqstarts->GetBufferPtr<int64_t>(), cachestarts->GetBufferPtr<int64_t>(),
                                           start_pos->GetBufferPtr<int64_t>(), cache->GetBufferPtr(),
                                           scale->GetBufferPtr(), GetStream()));
    if (rc != RC_SUCCESS) {
        return rc;
    }
    const int64_t total_kv = key->GetShape()->GetDim(0);
    return FromStatus(pplb200_kv_gather_dequant(&p, kvstarts->GetBufferPtr<int64_t>(),
                                                cachestarts->GetBufferPtr<int64_t>(), cache->GetBufferPtr(),
                                                scale->GetBufferPtr(), total_kv, key->GetBufferPtr(),
                                                value->GetBufferPtr(), GetStream()));
}

}  // namespace opmx

// =================================================================================================
// registration
// =================================================================================================
template <typename T>
static LlmCudaOptKernel* CreateOp(const ir::Node* node) {
    return new T(node);
}

void RegisterB200OpImpls() {
    auto mgr = OptKernelCreatorManager::GetInstance();
    const char* domain = "opmx.dynamic_batching";
    mgr->Remove(domain, "MultiHeadCacheAttention");
    mgr->Register(domain, "MultiHeadCacheAttention", utils::VersionRange(1, 1),
                  CreateOp<opmx::DynamicBatchingMultiHeadCacheAttentionOp>);
    mgr->Remove(domain, "KeyValueCache");
    mgr->Register(domain, "KeyValueCache", utils::VersionRange(1, 1), CreateOp<opmx::DynamicBatchingKeyValueCacheOp>);
    mgr->Remove(domain, "RotaryPositionEmbedding");
    mgr->Register(domain, "RotaryPositionEmbedding", utils::VersionRange(1, 1),
                  CreateOp<opmx::DynamicBatchingRotaryPositionEmbeddingOp>);
    mgr->Remove(domain, "MultiHeadAttention");
    mgr->Register(domain, "MultiHeadAttention", utils::VersionRange(1, 1),
                  CreateOp<opmx::DynamicBatchingMultiHeadAttentionOp>);
}

}}}}  // namespace ppl::nn::llm::cuda
