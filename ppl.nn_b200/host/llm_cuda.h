// The part of ppl.nn's llm_cuda engine that an operator plugs into, restated for this path:
//   EngineConfig                  src/ppl/nn/engines/llm_cuda/engine_config.h:25-36
//   LlmCudaDevice / LlmHostDevice src/ppl/nn/engines/llm_cuda/llm_cuda_device.h:97-156, llm_host_device.h
//   LlmCudaKernel                 src/ppl/nn/engines/llm_cuda/kernel.h:36-105, kernel.cc:156-196
//   LlmCudaOptKernel              src/ppl/nn/engines/llm_cuda/opt_kernel.h:41-139
//   OptKernelCreatorManager       src/ppl/nn/engines/llm_cuda/opt_kernel_creator_manager.h:27-29,
//                                 src/ppl/nn/utils/op_info_manager.h:30-110
// and the two parameter structs with their ONNX attribute parsers
//   src/ppl/nn/params/opmx/{key_value_cache,multi_head_cache_attention,multi_head_attention}_param.h
//   src/ppl/nn/models/onnx/parsers/opmx/parse_{key_value_cache,multi_head_cache_attention,multi_head_attention}_param.cc
#pragma once

#include <cuda_runtime.h>

#include <list>
#include <mutex>
#include <utility>

#include "compat.h"

namespace ppl { namespace nn {

// ---------------------------------------------------------------------------------------------
// operator parameters
// ---------------------------------------------------------------------------------------------
namespace opmx {

struct KeyValueCacheParam final : public ir::TypedAttr<KeyValueCacheParam> {
    int32_t num_layer = 0;
    int32_t layer_idx = 0;
    int32_t quant_bit = 0;
    int32_t quant_group = 8;
    int32_t num_repeat = 1;
    int32_t cache_mode = 0;
    int32_t cache_layout = 0;
    int32_t page_size = 128;
};

struct MultiHeadCacheAttentionParam final : public ir::TypedAttr<MultiHeadCacheAttentionParam> {
    int32_t num_heads = 0;
    int32_t num_kv_heads = 0;
    int32_t head_dim = 0;
    bool is_causal = true;
    bool is_alibi = false;
    int32_t num_layer = 0;
    int32_t layer_idx = 0;
    int32_t quant_bit = 0;
    int32_t quant_group = 8;
    int32_t cache_mode = 0;
    int32_t cache_layout = 0;
    int32_t page_size = 128;
};

// src/ppl/nn/params/opmx/multi_head_attention_param.h; parser
// src/ppl/nn/models/onnx/parsers/opmx/parse_multi_head_attention_param.cc
struct MultiHeadAttentionParam final : public ir::TypedAttr<MultiHeadAttentionParam> {
    int32_t num_heads = 0;
    int32_t num_kv_heads = 0;
    int32_t head_dim = 0;
    bool is_causal = true;
    bool is_alibi = false;
};

// src/ppl/nn/params/opmx/rotary_position_embedding_param.h; parser
// src/ppl/nn/models/onnx/parsers/opmx/parse_rotary_position_embedding_param.cc
struct RotaryPositionEmbeddingParam final : public ir::TypedAttr<RotaryPositionEmbeddingParam> {
    enum { SCALING_TYPE_NONE = 0, SCALING_TYPE_LINEAR = 1, SCALING_TYPE_DYNAMIC = 2 };
    int32_t bypass_key = 0;
    int32_t rotary_dim = 0;
    float theta = 10000.0f;
    int32_t max_position_embeddings = 2048;
    int32_t scaling_type = SCALING_TYPE_NONE;
    float scaling_factor = 1.0f;
};

// Attributes of a node as name -> integer.  A float attribute (theta, scaling_factor) travels as the bit
// pattern of the float in the low 32 bits; the string attribute scaling_type as 0 "", 1 "linear", 2 "dynamic".
using AttrMap = std::map<std::string, int64_t>;

// Same required attributes and defaults as the ONNX parsers: a missing required attribute is
// RC_NOT_FOUND, everything else falls back to its default.
ppl::common::RetCode ParseKeyValueCacheParam(const AttrMap& attrs, KeyValueCacheParam* param);
ppl::common::RetCode ParseMultiHeadCacheAttentionParam(const AttrMap& attrs, MultiHeadCacheAttentionParam* param);
ppl::common::RetCode ParseMultiHeadAttentionParam(const AttrMap& attrs, MultiHeadAttentionParam* param);
ppl::common::RetCode ParseRotaryPositionEmbeddingParam(const AttrMap& attrs, RotaryPositionEmbeddingParam* param);

}  // namespace opmx

namespace llm { namespace cuda {

struct EngineConfig final {
    bool enable_cache_prefill = false;
    // one algorithm per regime here: the next three and specify_decoding_attn_tpb are accepted and ignored
    bool enable_decoding_sharemem_mhca = true;
    bool enable_decoding_infinity_mhca = true;
    bool enable_decoding_infinity_gqca = true;
    int32_t specify_decoding_attn_split_k = 1;
    int32_t specify_decoding_attn_tpb = 0;
};

// ---------------------------------------------------------------------------------------------
// devices
// ---------------------------------------------------------------------------------------------
class LlmHostDevice final : public Device {
public:
    const char* GetTypeStr() const override { return "cpu"; }
    ppl::common::RetCode Realloc(uint64_t bytes, BufferDesc* buffer) override;
    void Free(BufferDesc* buffer) override;
    ppl::common::RetCode CopyToHost(void* dst, const BufferDesc& src, uint64_t bytes) const override;
    ppl::common::RetCode CopyFromHost(BufferDesc* dst, const void* src, uint64_t bytes) const override;
};

// One stream, one GPU.  Output tensors come from cudaMalloc; the per-call scratch comes from a
// grow-only pool (the reference offers PLAIN/COMPACT/BEST_FIT policies; this is the simplest one that
// never allocates in steady state).
class LlmCudaDevice final : public Device {
public:
    LlmCudaDevice(int device_id, cudaStream_t stream) : device_id_(device_id), stream_(stream) {}
    ~LlmCudaDevice() override;
    const char* GetTypeStr() const override { return "cuda"; }
    int GetDeviceId() const { return device_id_; }
    cudaStream_t GetStream() const { return stream_; }
    ppl::common::RetCode Realloc(uint64_t bytes, BufferDesc* buffer) override;
    void Free(BufferDesc* buffer) override;
    ppl::common::RetCode CopyToHost(void* dst, const BufferDesc& src, uint64_t bytes) const override;
    ppl::common::RetCode CopyFromHost(BufferDesc* dst, const void* src, uint64_t bytes) const override;
    ppl::common::RetCode AllocTmpBuffer(uint64_t bytes, BufferDesc* buffer);
    void FreeTmpBuffer(BufferDesc* buffer);
    ppl::common::RetCode Synchronize() const;
    uint64_t GetTmpPoolBytes() const { return pool_bytes_; }

private:
    int device_id_;
    cudaStream_t stream_;
    void* pool_ = nullptr;
    uint64_t pool_bytes_ = 0;
    bool pool_in_use_ = false;
};

struct LlmCudaEngineContext final {
    LlmCudaDevice* cuda_device = nullptr;
    LlmHostDevice* host_device = nullptr;
    EngineConfig config;
};

// ---------------------------------------------------------------------------------------------
// kernel and operator bases
// ---------------------------------------------------------------------------------------------
class LlmCudaKernel : public KernelImpl {
public:
    explicit LlmCudaKernel(const ir::Node* node) : KernelImpl(node) {}
    ppl::common::RetCode Init() { return ppl::common::RC_SUCCESS; }
    void SetReshapeFunc(const std::function<ppl::common::RetCode(InputOutputInfo*)>& f) { reshape_func_ = f; }
    ppl::common::RetCode Reshape(InputOutputInfo* info) const override final { return reshape_func_(info); }
    // DoExecute, then cudaGetLastError -> RC_DEVICE_RUNTIME_ERROR, like the engine does after every kernel
    ppl::common::RetCode Execute(KernelExecContext* ctx) override final;

    LlmCudaDevice* GetCudaDevice() const { return Context()->cuda_device; }
    LlmHostDevice* GetHostDevice() const { return Context()->host_device; }
    const EngineConfig& GetEngineConfig() const { return Context()->config; }
    cudaStream_t GetStream() const { return GetCudaDevice()->GetStream(); }
    int GetDeviceId() const { return GetCudaDevice()->GetDeviceId(); }

protected:
    virtual ppl::common::RetCode DoExecute(KernelExecContext*) = 0;

private:
    LlmCudaEngineContext* Context() const { return static_cast<LlmCudaEngineContext*>(GetEngineContext()); }
    std::function<ppl::common::RetCode(InputOutputInfo*)> reshape_func_;
};

struct OptKernelOptions final {
    ir::Graph* graph = nullptr;
    LlmCudaDevice* device = nullptr;
    const EngineConfig* engine_config = nullptr;
};

class LlmCudaOptKernel {
public:
    explicit LlmCudaOptKernel(const ir::Node* node) : node_(node) {}
    virtual ~LlmCudaOptKernel() {}
    const ir::Node* GetNode() const { return node_; }
    ppl::common::RetCode Init(const OptKernelOptions& options) { return DoInit(options); }
    virtual KernelImpl* CreateKernelImpl() const = 0;

protected:
    virtual ppl::common::RetCode DoInit(const OptKernelOptions&) = 0;

    // the typed attribute object that the model front-end stored under this node's id
    template <typename T>
    ppl::common::RetCode GenericLoadParam(const OptKernelOptions& options, std::shared_ptr<T>* param) const {
        const auto& attrs = options.graph->data->attrs;
        auto it = attrs.find(node_->GetId());
        if (it == attrs.end()) {
            return ppl::common::RC_NOT_FOUND;
        }
        *param = std::static_pointer_cast<T>(it->second);
        return ppl::common::RC_SUCCESS;
    }

    template <typename KernelType, typename ParamType>
    KernelType* CreateKernelImplWithParam(const ParamType param) const {
        auto kernel = new KernelType(node_);
        const auto rc = kernel->Init();
        if (rc != ppl::common::RC_SUCCESS) {
            LOG(ERROR) << "init kernel for [" << node_->GetName() << "] failed: " << ppl::common::GetRetCodeStr(rc);
            delete kernel;
            return nullptr;
        }
        kernel->SetParam(param);
        kernel->SetReshapeFunc([this](InputOutputInfo* info) -> ppl::common::RetCode {
            const auto r = infer_type_and_format_func_(info);
            return r != ppl::common::RC_SUCCESS ? r : infer_dims_func_(info);
        });
        return kernel;
    }

    // every output takes the first input's dims / type and format
    static ppl::common::RetCode GenericInferDims(InputOutputInfo* info);
    static ppl::common::RetCode GenericInferTypeAndFormat(InputOutputInfo* info);

    std::function<ppl::common::RetCode(InputOutputInfo*)> infer_dims_func_;
    std::function<ppl::common::RetCode(InputOutputInfo*)> infer_type_and_format_func_;

private:
    const ir::Node* node_;
};

// ---------------------------------------------------------------------------------------------
// registry: (domain, type, version range) -> creator
// ---------------------------------------------------------------------------------------------
namespace utils {
struct VersionRange final {
    VersionRange(uint64_t f = 0, uint64_t l = 0) : first(f), last(l) {}
    uint64_t first, last;
};
}  // namespace utils

typedef LlmCudaOptKernel* (*OptKernelCreator)(const ir::Node*);

class OptKernelCreatorManager final {
public:
    static OptKernelCreatorManager* GetInstance();
    // RC_EXISTS when [first, last] overlaps a registered range of the same (domain, type)
    ppl::common::RetCode Register(const std::string& domain, const std::string& type, const utils::VersionRange& ver,
                                  OptKernelCreator creator);
    OptKernelCreator Find(const std::string& domain, const std::string& type, uint64_t version) const;
    void Remove(const std::string& domain, const std::string& type);
    uint64_t GetSize() const;

private:
    typedef std::list<std::pair<utils::VersionRange, OptKernelCreator>> Versions;
    mutable std::mutex mu_;
    std::map<std::string, std::map<std::string, Versions>> info_;
};

// Registers this library's operators under the names the engine serves
// (src/ppl/nn/engines/llm_cuda/register_ops.cc), replacing whatever is registered for them.
void RegisterB200OpImpls();

}}  // namespace llm::cuda

}}  // namespace ppl::nn
