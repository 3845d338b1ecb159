// Devices, kernel/operator bases, attribute parsers and the operator registry of the host layer.
#include "llm_cuda.h"

#include <string.h>

#include <stdlib.h>

using namespace ppl::common;

namespace ppl { namespace nn {

namespace opmx {

static bool Lookup(const AttrMap& attrs, const char* key, int64_t* v) {
    auto it = attrs.find(key);
    if (it == attrs.end()) {
        return false;
    }
    *v = it->second;
    return true;
}

template <typename T>
static RetCode Required(const AttrMap& attrs, const char* key, T* dst) {
    int64_t v = 0;
    if (!Lookup(attrs, key, &v)) {
        LOG(ERROR) << "attribute \"" << key << "\" is required.";
        return RC_NOT_FOUND;
    }
    *dst = static_cast<T>(v);
    return RC_SUCCESS;
}

template <typename T>
static void Optional(const AttrMap& attrs, const char* key, T* dst, T dflt) {
    int64_t v = 0;
    *dst = Lookup(attrs, key, &v) ? static_cast<T>(v) : dflt;
}

RetCode ParseKeyValueCacheParam(const AttrMap& attrs, KeyValueCacheParam* p) {
    RetCode rc;
    if ((rc = Required(attrs, "num_layer", &p->num_layer)) != RC_SUCCESS) return rc;
    if ((rc = Required(attrs, "layer_idx", &p->layer_idx)) != RC_SUCCESS) return rc;
    Optional(attrs, "quant_bit", &p->quant_bit, 0);
    Optional(attrs, "quant_group", &p->quant_group, 8);
    Optional(attrs, "num_repeat", &p->num_repeat, 1);
    Optional(attrs, "cache_mode", &p->cache_mode, 0);
    Optional(attrs, "cache_layout", &p->cache_layout, 0);
    Optional(attrs, "page_size", &p->page_size, 128);
    return RC_SUCCESS;
}

RetCode ParseMultiHeadCacheAttentionParam(const AttrMap& attrs, MultiHeadCacheAttentionParam* p) {
    RetCode rc;
    if ((rc = Required(attrs, "num_heads", &p->num_heads)) != RC_SUCCESS) return rc;
    if ((rc = Required(attrs, "head_dim", &p->head_dim)) != RC_SUCCESS) return rc;
    if ((rc = Required(attrs, "num_layer", &p->num_layer)) != RC_SUCCESS) return rc;
    if ((rc = Required(attrs, "layer_idx", &p->layer_idx)) != RC_SUCCESS) return rc;
    Optional(attrs, "num_kv_heads", &p->num_kv_heads, p->num_heads);
    Optional(attrs, "is_causal", &p->is_causal, true);
    Optional(attrs, "is_alibi", &p->is_alibi, false);
    Optional(attrs, "quant_bit", &p->quant_bit, 0);
    Optional(attrs, "quant_group", &p->quant_group, 8);
    Optional(attrs, "cache_mode", &p->cache_mode, 0);
    Optional(attrs, "cache_layout", &p->cache_layout, 0);
    Optional(attrs, "page_size", &p->page_size, 128);
    return RC_SUCCESS;
}

RetCode ParseMultiHeadAttentionParam(const AttrMap& attrs, MultiHeadAttentionParam* p) {
    RetCode rc;
    if ((rc = Required(attrs, "num_heads", &p->num_heads)) != RC_SUCCESS) return rc;
    if ((rc = Required(attrs, "head_dim", &p->head_dim)) != RC_SUCCESS) return rc;
    Optional(attrs, "num_kv_heads", &p->num_kv_heads, p->num_heads);
    Optional(attrs, "is_causal", &p->is_causal, true);
    Optional(attrs, "is_alibi", &p->is_alibi, false);
    return RC_SUCCESS;
}

static float FloatFromBits(int64_t v) {
    const uint32_t u = static_cast<uint32_t>(v);
    float f;
    memcpy(&f, &u, sizeof(f));
    return f;
}

RetCode ParseRotaryPositionEmbeddingParam(const AttrMap& attrs, RotaryPositionEmbeddingParam* p) {
    int64_t v = 0;
    if (!Lookup(attrs, "theta", &v)) {  // parse_rotary_position_embedding_param.cc:13-16
        LOG(ERROR) << "attribute \"theta\" is required.";
        return RC_NOT_FOUND;
    }
    p->theta = FloatFromBits(v);
    Optional(attrs, "bypass_key", &p->bypass_key, 0);
    Optional(attrs, "rotary_dim", &p->rotary_dim, 0);
    p->scaling_factor = Lookup(attrs, "scaling_factor", &v) ? FloatFromBits(v) : 1.0f;
    Optional(attrs, "max_position_embeddings", &p->max_position_embeddings, 2048);
    Optional(attrs, "scaling_type", &p->scaling_type, 0);
    if (p->scaling_type < 0 || p->scaling_type > 2) {
        LOG(ERROR) << "unsupported scaling_type: " << p->scaling_type;
        return RC_UNSUPPORTED;
    }
    return RC_SUCCESS;
}

}  // namespace opmx

namespace llm { namespace cuda {

// ---- host device ---------------------------------------------------------------------------------
RetCode LlmHostDevice::Realloc(uint64_t bytes, BufferDesc* buffer) {
    buffer->addr = malloc(bytes ? bytes : 1);
    return buffer->addr ? RC_SUCCESS : RC_OUT_OF_MEMORY;
}
void LlmHostDevice::Free(BufferDesc* buffer) {
    free(buffer->addr);
    buffer->addr = nullptr;
}
RetCode LlmHostDevice::CopyToHost(void* dst, const BufferDesc& src, uint64_t bytes) const {
    memcpy(dst, src.addr, bytes);
    return RC_SUCCESS;
}
RetCode LlmHostDevice::CopyFromHost(BufferDesc* dst, const void* src, uint64_t bytes) const {
    memcpy(dst->addr, src, bytes);
    return RC_SUCCESS;
}

// ---- cuda device ---------------------------------------------------------------------------------
LlmCudaDevice::~LlmCudaDevice() {
    if (pool_) {
        cudaFree(pool_);
    }
}
RetCode LlmCudaDevice::Realloc(uint64_t bytes, BufferDesc* buffer) {
    void* p = nullptr;
    if (cudaMalloc(&p, bytes ? bytes : 1) != cudaSuccess) {
        (void)cudaGetLastError();
        return RC_OUT_OF_MEMORY;
    }
    buffer->addr = p;
    return RC_SUCCESS;
}
void LlmCudaDevice::Free(BufferDesc* buffer) {
    if (buffer->addr) {
        cudaFree(buffer->addr);
        buffer->addr = nullptr;
    }
}
// A device-to-host copy of a tensor that lives on the GPU synchronises the stream, as the reference's
// does (src/ppl/nn/engines/llm_cuda/llm_cuda_device.cc:187-200).
RetCode LlmCudaDevice::CopyToHost(void* dst, const BufferDesc& src, uint64_t bytes) const {
    if (cudaMemcpyAsync(dst, src.addr, bytes, cudaMemcpyDeviceToHost, stream_) != cudaSuccess ||
        cudaStreamSynchronize(stream_) != cudaSuccess) {
        (void)cudaGetLastError();
        return RC_DEVICE_MEMORY_ERROR;
    }
    return RC_SUCCESS;
}
RetCode LlmCudaDevice::CopyFromHost(BufferDesc* dst, const void* src, uint64_t bytes) const {
    if (cudaMemcpyAsync(dst->addr, src, bytes, cudaMemcpyHostToDevice, stream_) != cudaSuccess) {
        (void)cudaGetLastError();
        return RC_DEVICE_MEMORY_ERROR;
    }
    return RC_SUCCESS;
}
RetCode LlmCudaDevice::AllocTmpBuffer(uint64_t bytes, BufferDesc* buffer) {
    if (pool_in_use_) {
        return RC_INVALID_VALUE;  // one operator at a time per device, like the sequential scheduler
    }
    if (bytes > pool_bytes_) {
        // grow: earlier work on the stream may still use the old block, so drain the stream first
        if (pool_) {
            cudaStreamSynchronize(stream_);
            cudaFree(pool_);
            pool_ = nullptr;
            pool_bytes_ = 0;
        }
        const uint64_t want = (bytes + (1u << 20) - 1) & ~uint64_t((1u << 20) - 1);
        if (cudaMalloc(&pool_, want) != cudaSuccess) {
            (void)cudaGetLastError();
            pool_ = nullptr;
            return RC_OUT_OF_MEMORY;
        }
        pool_bytes_ = want;
    }
    buffer->addr = pool_;
    pool_in_use_ = true;
    return RC_SUCCESS;
}
void LlmCudaDevice::FreeTmpBuffer(BufferDesc* buffer) {
    buffer->addr = nullptr;
    pool_in_use_ = false;
}
RetCode LlmCudaDevice::Synchronize() const {
    if (cudaStreamSynchronize(stream_) != cudaSuccess) {
        (void)cudaGetLastError();
        return RC_DEVICE_RUNTIME_ERROR;
    }
    return RC_SUCCESS;
}

// ---- kernel / operator bases -----------------------------------------------------------------------
RetCode LlmCudaKernel::Execute(KernelExecContext* ctx) {
    const RetCode rc = DoExecute(ctx);
    if (rc != RC_SUCCESS) {
        return rc;
    }
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        LOG(ERROR) << "kernel[" << GetName() << "] left a CUDA error: " << cudaGetErrorString(e);
        return RC_DEVICE_RUNTIME_ERROR;
    }
    return RC_SUCCESS;
}

RetCode LlmCudaOptKernel::GenericInferDims(InputOutputInfo* info) {
    const TensorShape& in0 = *info->GetInput<TensorImpl>(0)->GetShape();
    for (uint32_t i = 0; i < info->GetOutputCount(); ++i) {
        TensorShape* out = info->GetOutput<TensorImpl>(i)->GetShape();
        if (in0.IsScalar()) {
            out->ReshapeAsScalar();
        } else {
            out->Reshape(in0.GetDims(), in0.GetDimCount());
        }
    }
    return RC_SUCCESS;
}

RetCode LlmCudaOptKernel::GenericInferTypeAndFormat(InputOutputInfo* info) {
    const TensorShape& in0 = *info->GetInput<TensorImpl>(0)->GetShape();
    for (uint32_t i = 0; i < info->GetOutputCount(); ++i) {
        TensorShape* out = info->GetOutput<TensorImpl>(i)->GetShape();
        out->SetDataType(in0.GetDataType());
        out->SetDataFormat(in0.GetDataFormat());
    }
    return RC_SUCCESS;
}

// ---- registry ----------------------------------------------------------------------------------------
OptKernelCreatorManager* OptKernelCreatorManager::GetInstance() {
    static OptKernelCreatorManager mgr;
    return &mgr;
}

RetCode OptKernelCreatorManager::Register(const std::string& domain, const std::string& type,
                                          const utils::VersionRange& ver, OptKernelCreator creator) {
    if (ver.last < ver.first || !creator) {
        return RC_INVALID_VALUE;
    }
    std::lock_guard<std::mutex> lock(mu_);
    Versions& versions = info_[domain][type];
    auto pos = versions.begin();
    for (; pos != versions.end(); ++pos) {  // kept sorted by first version; ranges never overlap
        const utils::VersionRange& cur = pos->first;
        if (ver.last < cur.first) {
            break;
        }
        if (ver.first <= cur.last) {
            return RC_EXISTS;
        }
    }
    versions.insert(pos, std::make_pair(ver, creator));
    return RC_SUCCESS;
}

OptKernelCreator OptKernelCreatorManager::Find(const std::string& domain, const std::string& type,
                                               uint64_t version) const {
    std::lock_guard<std::mutex> lock(mu_);
    auto d = info_.find(domain);
    if (d == info_.end()) {
        return nullptr;
    }
    auto t = d->second.find(type);
    if (t == d->second.end()) {
        return nullptr;
    }
    for (const auto& entry : t->second) {
        if (entry.first.first <= version && version <= entry.first.last) {
            return entry.second;
        }
    }
    return nullptr;
}

void OptKernelCreatorManager::Remove(const std::string& domain, const std::string& type) {
    std::lock_guard<std::mutex> lock(mu_);
    auto d = info_.find(domain);
    if (d == info_.end()) {
        return;
    }
    d->second.erase(type);
    if (d->second.empty()) {
        info_.erase(d);
    }
}

uint64_t OptKernelCreatorManager::GetSize() const {
    std::lock_guard<std::mutex> lock(mu_);
    return info_.size();
}

}}  // namespace llm::cuda

}}  // namespace ppl::nn
