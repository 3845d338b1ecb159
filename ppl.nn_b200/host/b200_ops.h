// The two operators of this path as llm_cuda engine operators (Op = graph-build-time object that
// loads attributes and infers shapes; Kernel = run-time object that validates inputs and calls the
// C ABI of include/ppl_nn_b200.h).  Class names match the reference's:
//   DynamicBatchingMultiHeadCacheAttentionOp / ...Kernel
//       src/ppl/nn/engines/llm_cuda/{ops,kernels}/opmx/dynamic_batching/multi_head_cache_attention_*
//   DynamicBatchingKeyValueCacheOp / ...Kernel
//       src/ppl/nn/engines/llm_cuda/{ops,kernels}/opmx/dynamic_batching/key_value_cache_*
//   DynamicBatchingMultiHeadAttentionOp / ...Kernel (attention over the call's own key/value, no cache)
//       src/ppl/nn/engines/llm_cuda/{ops,kernels}/opmx/dynamic_batching/multi_head_attention_*
#pragma once

#include "llm_cuda.h"

namespace ppl { namespace nn { namespace llm { namespace cuda { namespace opmx {

class DynamicBatchingMultiHeadCacheAttentionKernel final : public LlmCudaKernel {
public:
    explicit DynamicBatchingMultiHeadCacheAttentionKernel(const ir::Node* node) : LlmCudaKernel(node) {}
    void SetParam(const ppl::nn::opmx::MultiHeadCacheAttentionParam* p) { param_ = p; }

private:
    ppl::common::RetCode DoExecute(KernelExecContext*) override;
    const ppl::nn::opmx::MultiHeadCacheAttentionParam* param_ = nullptr;
};

class DynamicBatchingMultiHeadCacheAttentionOp final : public LlmCudaOptKernel {
public:
    explicit DynamicBatchingMultiHeadCacheAttentionOp(const ir::Node* node) : LlmCudaOptKernel(node) {}
    KernelImpl* CreateKernelImpl() const override;

private:
    ppl::common::RetCode DoInit(const OptKernelOptions&) override;
    std::shared_ptr<ppl::nn::opmx::MultiHeadCacheAttentionParam> param_;
};

class DynamicBatchingKeyValueCacheKernel final : public LlmCudaKernel {
public:
    explicit DynamicBatchingKeyValueCacheKernel(const ir::Node* node) : LlmCudaKernel(node) {}
    void SetParam(const ppl::nn::opmx::KeyValueCacheParam* p) { param_ = p; }

private:
    ppl::common::RetCode DoExecute(KernelExecContext*) override;
    const ppl::nn::opmx::KeyValueCacheParam* param_ = nullptr;
};

class DynamicBatchingKeyValueCacheOp final : public LlmCudaOptKernel {
public:
    explicit DynamicBatchingKeyValueCacheOp(const ir::Node* node) : LlmCudaOptKernel(node) {}
    KernelImpl* CreateKernelImpl() const override;

private:
    ppl::common::RetCode DoInit(const OptKernelOptions&) override;
    std::shared_ptr<ppl::nn::opmx::KeyValueCacheParam> param_;
};

class DynamicBatchingMultiHeadAttentionKernel final : public LlmCudaKernel {
public:
    explicit DynamicBatchingMultiHeadAttentionKernel(const ir::Node* node) : LlmCudaKernel(node) {}
    void SetParam(const ppl::nn::opmx::MultiHeadAttentionParam* p) { param_ = p; }

private:
    ppl::common::RetCode DoExecute(KernelExecContext*) override;
    const ppl::nn::opmx::MultiHeadAttentionParam* param_ = nullptr;
};

class DynamicBatchingMultiHeadAttentionOp final : public LlmCudaOptKernel {
public:
    explicit DynamicBatchingMultiHeadAttentionOp(const ir::Node* node) : LlmCudaOptKernel(node) {}
    KernelImpl* CreateKernelImpl() const override;

private:
    ppl::common::RetCode DoInit(const OptKernelOptions&) override;
    std::shared_ptr<ppl::nn::opmx::MultiHeadAttentionParam> param_;
};

// DynamicBatchingRotaryPositionEmbeddingOp / ...Kernel
//     src/ppl/nn/engines/llm_cuda/{ops,kernels}/opmx/dynamic_batching/rotary_position_embedding_*
class DynamicBatchingRotaryPositionEmbeddingKernel final : public LlmCudaKernel {
public:
    explicit DynamicBatchingRotaryPositionEmbeddingKernel(const ir::Node* node) : LlmCudaKernel(node) {}
    void SetParam(const ppl::nn::opmx::RotaryPositionEmbeddingParam* p) { param_ = p; }

private:
    ppl::common::RetCode DoExecute(KernelExecContext*) override;
    const ppl::nn::opmx::RotaryPositionEmbeddingParam* param_ = nullptr;
};

class DynamicBatchingRotaryPositionEmbeddingOp final : public LlmCudaOptKernel {
public:
    explicit DynamicBatchingRotaryPositionEmbeddingOp(const ir::Node* node) : LlmCudaOptKernel(node) {}
    KernelImpl* CreateKernelImpl() const override;

private:
    ppl::common::RetCode DoInit(const OptKernelOptions&) override;
    std::shared_ptr<ppl::nn::opmx::RotaryPositionEmbeddingParam> param_;
};

}}}}}  // namespace ppl::nn::llm::cuda::opmx
