// extern "C" harness over the host layer; see include/ppl_nn_b200_host.h.
#include "ppl_nn_b200_host.h"

#include "b200_ops.h"

using namespace ppl::common;
using namespace ppl::nn;
using namespace ppl::nn::llm::cuda;

namespace {

struct Engine {
    LlmCudaDevice* cuda = nullptr;
    LlmHostDevice host;
    LlmCudaEngineContext ctx;
    ~Engine() { delete cuda; }
};

struct Op {
    Engine* engine = nullptr;
    std::unique_ptr<ir::Node> node;
    ir::Graph graph;
    std::unique_ptr<LlmCudaOptKernel> opt;
    std::unique_ptr<KernelImpl> kernel;
    std::vector<std::unique_ptr<TensorImpl>> inputs, outputs;
    uint32_t last_consumer_mask = 0;  // bit i: this op is the last consumer of its input i
};

datatype_t ToDataType(int32_t dt) {
    switch (dt) {
        case PPLB200_DT_FLOAT16: return DATATYPE_FLOAT16;
        case PPLB200_DT_FLOAT32: return DATATYPE_FLOAT32;
        case PPLB200_DT_INT8: return DATATYPE_INT8;
        case PPLB200_DT_INT32: return DATATYPE_INT32;
        case PPLB200_DT_INT64: return DATATYPE_INT64;
        default: return DATATYPE_UNKNOWN;
    }
}
int32_t FromDataType(datatype_t dt) {
    switch (dt) {
        case DATATYPE_FLOAT16: return PPLB200_DT_FLOAT16;
        case DATATYPE_FLOAT32: return PPLB200_DT_FLOAT32;
        case DATATYPE_INT8: return PPLB200_DT_INT8;
        case DATATYPE_INT32: return PPLB200_DT_INT32;
        case DATATYPE_INT64: return PPLB200_DT_INT64;
        default: return 0;
    }
}

LlmCudaOptKernel* DummyCreator(const ir::Node*) {
    return nullptr;
}

}  // namespace

extern "C" {

void* pplb200_host_engine_create(int device_id, void* stream) {
    Engine* e = new Engine;
    e->cuda = new LlmCudaDevice(device_id, static_cast<cudaStream_t>(stream));
    e->ctx.cuda_device = e->cuda;
    e->ctx.host_device = &e->host;
    return e;
}

void pplb200_host_engine_destroy(void* engine) {
    delete static_cast<Engine*>(engine);
}

int pplb200_host_engine_configure(void* engine, const char* key, int64_t value) {
    if (!engine || !key) {
        return RC_INVALID_VALUE;
    }
    EngineConfig& c = static_cast<Engine*>(engine)->ctx.config;
    const std::string k(key);
    if (k == "cache_prefill") {
        c.enable_cache_prefill = value != 0;
    } else if (k == "decoding_attn_split_k") {
        if (value < 0 || value > 2) {
            return RC_INVALID_VALUE;
        }
        c.specify_decoding_attn_split_k = static_cast<int32_t>(value);
    } else if (k == "decoding_attn_tpb") {
        if (value != 0 && value != 256 && value != 512) {
            return RC_INVALID_VALUE;
        }
        c.specify_decoding_attn_tpb = static_cast<int32_t>(value);
    } else if (k == "decoding_shm_mha") {
        c.enable_decoding_sharemem_mhca = value != 0;
    } else if (k == "decoding_inf_mha") {
        c.enable_decoding_infinity_mhca = value != 0;
    } else if (k == "decoding_inf_gqa") {
        c.enable_decoding_infinity_gqca = value != 0;
    } else {
        return RC_INVALID_VALUE;
    }
    return RC_SUCCESS;
}

uint64_t pplb200_host_engine_tmp_pool_bytes(void* engine) {
    return engine ? static_cast<Engine*>(engine)->cuda->GetTmpPoolBytes() : 0;
}

void pplb200_host_register_ops(void) {
    RegisterB200OpImpls();
}

int pplb200_host_registry_has(const char* domain, const char* type, uint64_t version) {
    return OptKernelCreatorManager::GetInstance()->Find(domain, type, version) != nullptr;
}

void pplb200_host_registry_remove(const char* domain, const char* type) {
    OptKernelCreatorManager::GetInstance()->Remove(domain, type);
}

int pplb200_host_registry_register_again(const char* domain, const char* type, uint64_t first, uint64_t last) {
    return OptKernelCreatorManager::GetInstance()->Register(domain, type, utils::VersionRange(first, last), DummyCreator);
}

void* pplb200_host_op_create(void* engine, const char* domain, const char* type, uint64_t version,
                             const char* const* attr_names, const int64_t* attr_values, int num_attrs, int* rc_out) {
    int dummy;
    int& rc = rc_out ? *rc_out : dummy;
    rc = RC_SUCCESS;
    if (!engine || !domain || !type) {
        rc = RC_INVALID_VALUE;
        return nullptr;
    }
    auto creator = OptKernelCreatorManager::GetInstance()->Find(domain, type, version);
    if (!creator) {
        LOG(ERROR) << "op[" << domain << ":" << type << ":" << version << "] is not registered";
        rc = RC_NOT_FOUND;
        return nullptr;
    }
    std::unique_ptr<Op> op(new Op);
    op->engine = static_cast<Engine*>(engine);
    ir::NodeType nt;
    nt.domain = domain;
    nt.name = type;
    nt.version = version;
    op->node.reset(new ir::Node(1, std::string(type) + "_0", nt));
    // what the model front-end does: parse the node's attributes into the typed param object
    ppl::nn::opmx::AttrMap attrs;
    for (int i = 0; i < num_attrs; ++i) {
        attrs[attr_names[i]] = attr_values[i];
    }
    const std::string t(type);
    if (t == "MultiHeadCacheAttention") {
        auto p = std::make_shared<ppl::nn::opmx::MultiHeadCacheAttentionParam>();
        rc = ppl::nn::opmx::ParseMultiHeadCacheAttentionParam(attrs, p.get());
        op->graph.data->attrs[op->node->GetId()] = p;
    } else if (t == "KeyValueCache") {
        auto p = std::make_shared<ppl::nn::opmx::KeyValueCacheParam>();
        rc = ppl::nn::opmx::ParseKeyValueCacheParam(attrs, p.get());
        op->graph.data->attrs[op->node->GetId()] = p;
    } else if (t == "RotaryPositionEmbedding") {
        auto p = std::make_shared<ppl::nn::opmx::RotaryPositionEmbeddingParam>();
        rc = ppl::nn::opmx::ParseRotaryPositionEmbeddingParam(attrs, p.get());
        op->graph.data->attrs[op->node->GetId()] = p;
    } else if (t == "MultiHeadAttention") {
        auto p = std::make_shared<ppl::nn::opmx::MultiHeadAttentionParam>();
        rc = ppl::nn::opmx::ParseMultiHeadAttentionParam(attrs, p.get());
        op->graph.data->attrs[op->node->GetId()] = p;
    }
    if (rc != RC_SUCCESS) {
        return nullptr;
    }
    op->opt.reset(creator(op->node.get()));
    if (!op->opt) {
        rc = RC_OTHER_ERROR;
        return nullptr;
    }
    OptKernelOptions options;
    options.graph = &op->graph;
    options.device = op->engine->cuda;
    options.engine_config = &op->engine->ctx.config;
    rc = op->opt->Init(options);
    if (rc != RC_SUCCESS) {
        return nullptr;
    }
    op->kernel.reset(op->opt->CreateKernelImpl());
    if (!op->kernel) {
        rc = RC_OTHER_ERROR;
        return nullptr;
    }
    op->kernel->SetEngineContext(&op->engine->ctx);
    return op.release();
}

void pplb200_host_op_destroy(void* op) {
    delete static_cast<Op*>(op);
}

int pplb200_host_op_run(void* opv, const pplb200_host_tensor* inputs, int num_inputs, pplb200_host_tensor* outputs,
                        int num_outputs) {
    if (!opv || num_inputs < 0 || num_outputs < 0 || (num_inputs && !inputs) || (num_outputs && !outputs)) {
        return RC_INVALID_VALUE;
    }
    Op* op = static_cast<Op*>(opv);
    Engine* e = op->engine;
    auto bind = [e](std::vector<std::unique_ptr<TensorImpl>>& slots, const pplb200_host_tensor* ts, int n,
                    const char* prefix, std::vector<TensorImpl*>* raw) {
        slots.resize(n);
        raw->assign(n, nullptr);
        for (int i = 0; i < n; ++i) {
            if (ts[i].absent) {
                slots[i].reset();
                continue;
            }
            if (!slots[i]) {
                slots[i].reset(new TensorImpl(std::string(prefix) + std::to_string(i)));
            }
            TensorImpl* t = slots[i].get();
            t->GetShape()->SetDataType(ToDataType(ts[i].dtype));
            t->GetShape()->SetDataFormat(DATAFORMAT_NDARRAY);
            if (ts[i].ndim == 0) {
                t->GetShape()->ReshapeAsScalar();
            } else {
                t->GetShape()->Reshape(ts[i].dims, static_cast<uint32_t>(ts[i].ndim));
            }
            t->SetDevice(ts[i].on_host ? static_cast<Device*>(&e->host) : static_cast<Device*>(e->cuda));
            if (ts[i].data) {
                t->SetBufferPtr(ts[i].data);  // borrowed
            } else if (!t->IsBufferOwner()) {
                t->SetBufferPtr(nullptr);
            }
            (*raw)[i] = t;
        }
    };
    std::vector<TensorImpl*> in_raw, out_raw;
    bind(op->inputs, inputs, num_inputs, "input", &in_raw);
    bind(op->outputs, outputs, num_outputs, "output", &out_raw);
    KernelExecContext ctx;
    ctx.SetInputs(in_raw);
    ctx.SetOutputs(out_raw);
    ctx.SetLastConsumerMask(op->last_consumer_mask);
    const RetCode rc = op->kernel->Execute(&ctx);
    for (int i = 0; i < num_outputs; ++i) {
        if (!out_raw[i]) {
            continue;
        }
        const TensorShape& s = *out_raw[i]->GetShape();
        outputs[i].dtype = FromDataType(s.GetDataType());
        outputs[i].ndim = static_cast<int32_t>(s.GetDimCount() > 6 ? 6 : s.GetDimCount());
        for (int d = 0; d < outputs[i].ndim; ++d) {
            outputs[i].dims[d] = s.GetDim(d);
        }
        outputs[i].data = out_raw[i]->GetBufferPtr();
        outputs[i].on_host = 0;
    }
    return rc;
}

void pplb200_host_op_set_last_consumer(void* op, uint32_t input_mask) {
    if (op) {
        static_cast<Op*>(op)->last_consumer_mask = input_mask;
    }
}

int pplb200_host_engine_synchronize(void* engine) {
    return engine ? static_cast<Engine*>(engine)->cuda->Synchronize() : RC_INVALID_VALUE;
}

const char* pplb200_host_retcode_str(int rc) {
    return GetRetCodeStr(static_cast<RetCode>(rc));
}

}  // extern "C"
