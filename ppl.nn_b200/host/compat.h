// Stand-ins for the few ppl.nn / ppl.common types that the two operators of this path touch, so that
// the operator and kernel classes in this directory can be written against the llm_cuda engine's
// plug-in interface and built without a ppl.nn checkout.  Each type carries only the members this
// path uses; names and meanings follow ppl.nn (citations are paths in its tree):
//   RetCode / GetRetCodeStr        ppl.common (external); only the codes the llm_cuda engine returns on this path
//   TensorShape                    include/ppl/nn/common/tensor_shape.h:21-25 (alias of ppl::common's)
//   BufferDesc                     include/ppl/nn/common/buffer_desc.h:25-36
//   Device                         include/ppl/nn/common/device.h:30-137
//   TensorImpl                     src/ppl/nn/runtime/tensor_impl.h:36-155
//   InputOutputInfo / KernelExecContext   src/ppl/nn/common/input_output_info.h:47-76,
//                                         src/ppl/nn/runtime/kernel_exec_context.h:28-48
//   ir::Node, ir::Attr             src/ppl/nn/ir/node.h, src/ppl/nn/ir/attr.h
//   KernelImpl                     src/ppl/nn/runtime/kernel_impl.h:65-71
// Inside a ppl.nn build this header is not used at all: b200_ops.* and llm_cuda.* then include the real
// headers these stand-ins are named after (see INTEGRATION.md for the file-by-file mapping).
#pragma once

#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <functional>
#include <map>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

namespace ppl { namespace common {

// The numeric values of ppl.common's RetCode are not part of the reference tree; these are this
// library's own stable values and are only ever compared by name.
enum RetCode : int {
    RC_SUCCESS = 0,
    RC_INVALID_VALUE = 1,
    RC_UNSUPPORTED = 2,
    RC_OUT_OF_MEMORY = 3,
    RC_DEVICE_RUNTIME_ERROR = 4,
    RC_NOT_FOUND = 5,
    RC_EXISTS = 6,
    RC_DEVICE_MEMORY_ERROR = 7,
    RC_OTHER_ERROR = 8,
    RC_INTERNAL_ERROR = 9
};

inline const char* GetRetCodeStr(RetCode rc) {
    switch (rc) {
        case RC_SUCCESS: return "RC_SUCCESS";
        case RC_INVALID_VALUE: return "RC_INVALID_VALUE";
        case RC_UNSUPPORTED: return "RC_UNSUPPORTED";
        case RC_OUT_OF_MEMORY: return "RC_OUT_OF_MEMORY";
        case RC_DEVICE_RUNTIME_ERROR: return "RC_DEVICE_RUNTIME_ERROR";
        case RC_NOT_FOUND: return "RC_NOT_FOUND";
        case RC_EXISTS: return "RC_EXISTS";
        case RC_DEVICE_MEMORY_ERROR: return "RC_DEVICE_MEMORY_ERROR";
        case RC_INTERNAL_ERROR: return "RC_INTERNAL_ERROR";
        default: return "RC_OTHER_ERROR";
    }
}

enum datatype_t : int {
    DATATYPE_UNKNOWN = 0,
    DATATYPE_FLOAT16 = 1,
    DATATYPE_FLOAT32 = 2,
    DATATYPE_INT8 = 3,
    DATATYPE_INT32 = 4,
    DATATYPE_INT64 = 5,
    DATATYPE_BOOL = 6
};

inline uint32_t GetSizeOfDataType(datatype_t t) {
    switch (t) {
        case DATATYPE_FLOAT16: return 2;
        case DATATYPE_FLOAT32: return 4;
        case DATATYPE_INT8: return 1;
        case DATATYPE_INT32: return 4;
        case DATATYPE_INT64: return 8;
        case DATATYPE_BOOL: return 1;
        default: return 0;
    }
}

enum dataformat_t : int { DATAFORMAT_UNKNOWN = 0, DATAFORMAT_NDARRAY = 1 };

class TensorShape final {
public:
    uint32_t GetDimCount() const { return static_cast<uint32_t>(dims_.size()); }
    int64_t GetDim(uint32_t i) const { return dims_[i]; }
    const int64_t* GetDims() const { return dims_.data(); }
    bool IsScalar() const { return is_scalar_; }
    void ReshapeAsScalar() {
        dims_.clear();
        is_scalar_ = true;
    }
    void Reshape(const int64_t* dims, uint32_t count) {
        dims_.assign(dims, dims + count);
        is_scalar_ = false;
    }
    void Reshape(const std::vector<int64_t>& dims) { Reshape(dims.data(), static_cast<uint32_t>(dims.size())); }
    datatype_t GetDataType() const { return type_; }
    void SetDataType(datatype_t t) { type_ = t; }
    dataformat_t GetDataFormat() const { return format_; }
    void SetDataFormat(dataformat_t f) { format_ = f; }
    uint64_t CalcElementsExcludingPadding() const {
        if (is_scalar_) {
            return 1;
        }
        if (dims_.empty()) {
            return 0;
        }
        uint64_t n = 1;
        for (auto d : dims_) {
            n *= static_cast<uint64_t>(d < 0 ? 0 : d);
        }
        return n;
    }
    uint64_t CalcElementsIncludingPadding() const { return CalcElementsExcludingPadding(); }
    uint64_t CalcBytesIncludingPadding() const { return CalcElementsExcludingPadding() * GetSizeOfDataType(type_); }

private:
    std::vector<int64_t> dims_;
    bool is_scalar_ = false;
    datatype_t type_ = DATATYPE_UNKNOWN;
    dataformat_t format_ = DATAFORMAT_NDARRAY;
};

// Runs a callable when it leaves scope (ppl::common::Destructor).
class Destructor final {
public:
    explicit Destructor(std::function<void()> f) : f_(std::move(f)) {}
    ~Destructor() {
        if (f_) {
            f_();
        }
    }
    Destructor(const Destructor&) = delete;
    Destructor& operator=(const Destructor&) = delete;

private:
    std::function<void()> f_;
};

// LOG(LEVEL) << ... : one line to stderr when the statement ends.
class LogLine final {
public:
    LogLine(const char* level, const char* file, int line) { os_ << "[" << level << "][" << file << ":" << line << "] "; }
    ~LogLine() {
        os_ << "\n";
        fputs(os_.str().c_str(), stderr);
    }
    std::ostream& stream() { return os_; }

private:
    std::ostringstream os_;
};

}}  // namespace ppl::common

#ifndef LOG
#define LOG(LEVEL) ::ppl::common::LogLine(#LEVEL, __FILE__, __LINE__).stream()
#endif

namespace ppl { namespace nn {

using TensorShape = ppl::common::TensorShape;

struct BufferDesc final {
    BufferDesc(void* a = nullptr) : addr(a), desc(0) {}
    void* addr;
    uint64_t desc;
};

class Device {
public:
    virtual ~Device() {}
    virtual const char* GetTypeStr() const = 0;
    virtual ppl::common::RetCode Realloc(uint64_t bytes, BufferDesc* buffer) = 0;
    virtual void Free(BufferDesc* buffer) = 0;
    virtual ppl::common::RetCode CopyToHost(void* dst, const BufferDesc& src, uint64_t bytes) const = 0;
    virtual ppl::common::RetCode CopyFromHost(BufferDesc* dst, const void* src, uint64_t bytes) const = 0;
};

// include/ppl/nn/common/types.h: tensors the runtime may recycle are "normal"; inputs, outputs and constants
// of the whole graph are reserved.  The harness only makes normal ones.
enum tensortype_t : int { TENSORTYPE_NORMAL = 0, TENSORTYPE_RESERVED = 1 };

// A tensor of the runtime: shape + a buffer on some device.  The buffer is either owned (allocated by
// ReallocBuffer through the device) or borrowed (SetBufferPtr: user-owned memory such as the KV cache,
// tools/benchmark_llama/text_generator.cc:223-224).
class TensorImpl final {
public:
    explicit TensorImpl(const std::string& name) : name_(name) {}
    ~TensorImpl() { FreeBuffer(); }
    TensorImpl(const TensorImpl&) = delete;
    TensorImpl& operator=(const TensorImpl&) = delete;

    const char* GetName() const { return name_.c_str(); }
    TensorShape* GetShape() { return &shape_; }
    const TensorShape* GetShape() const { return &shape_; }
    Device* GetDevice() const { return device_; }
    void SetDevice(Device* d) { device_ = d; }

    template <typename T = void>
    T* GetBufferPtr() const {
        return static_cast<T*>(buffer_.addr);
    }
    void SetBufferPtr(void* p) {
        FreeBuffer();
        buffer_.addr = p;
        owner_ = false;
    }
    bool IsBufferOwner() const { return owner_; }
    tensortype_t GetType() const { return TENSORTYPE_NORMAL; }

    // Takes over `another`'s buffer together with its ownership; this tensor's old buffer is freed (or let
    // go, if borrowed) and `another` is left without one (src/ppl/nn/runtime/tensor_impl.h:83-93).
    void TransferBufferFrom(TensorImpl* another) {
        FreeBuffer();
        buffer_ = another->buffer_;
        capacity_ = another->capacity_;
        owner_ = another->owner_;
        device_ = another->device_;
        another->DetachBuffer();
    }
    BufferDesc DetachBuffer() {
        const BufferDesc b = buffer_;
        buffer_.addr = nullptr;
        capacity_ = 0;
        owner_ = false;
        return b;
    }

    // No-op when the tensor borrows a buffer that is already set (src/ppl/nn/runtime/tensor_impl.cc:25-32).
    ppl::common::RetCode ReallocBuffer() {
        if (!owner_ && buffer_.addr) {
            return ppl::common::RC_SUCCESS;
        }
        if (!device_) {
            return ppl::common::RC_INVALID_VALUE;
        }
        const uint64_t bytes = shape_.CalcBytesIncludingPadding();
        if (owner_ && buffer_.addr && bytes <= capacity_) {
            return ppl::common::RC_SUCCESS;
        }
        FreeBuffer();
        if (bytes == 0) {
            owner_ = true;
            return ppl::common::RC_SUCCESS;
        }
        auto rc = device_->Realloc(bytes, &buffer_);
        if (rc == ppl::common::RC_SUCCESS) {
            owner_ = true;
            capacity_ = bytes;
        }
        return rc;
    }
    void FreeBuffer() {
        if (owner_ && buffer_.addr && device_) {
            device_->Free(&buffer_);
        }
        buffer_.addr = nullptr;
        capacity_ = 0;
        owner_ = false;
    }
    ppl::common::RetCode CopyToHost(void* dst) const {
        if (!device_ || !buffer_.addr) {
            return ppl::common::RC_INVALID_VALUE;
        }
        return device_->CopyToHost(dst, buffer_, shape_.CalcBytesIncludingPadding());
    }

private:
    std::string name_;
    TensorShape shape_;
    Device* device_ = nullptr;
    BufferDesc buffer_;
    uint64_t capacity_ = 0;
    bool owner_ = false;
};

// The inputs and outputs a kernel sees.  Optional inputs that the graph leaves out are null entries.
class InputOutputInfo {
public:
    virtual ~InputOutputInfo() {}
    uint32_t GetInputCount() const { return static_cast<uint32_t>(inputs_.size()); }
    uint32_t GetOutputCount() const { return static_cast<uint32_t>(outputs_.size()); }
    template <typename T>
    T* GetInput(uint32_t i) const {
        return static_cast<T*>(inputs_[i]);
    }
    template <typename T>
    T* GetOutput(uint32_t i) const {
        return static_cast<T*>(outputs_[i]);
    }
    void SetInputs(const std::vector<TensorImpl*>& v) { inputs_ = v; }
    void SetOutputs(const std::vector<TensorImpl*>& v) { outputs_ = v; }

private:
    std::vector<TensorImpl*> inputs_, outputs_;
};

class KernelExecContext final : public InputOutputInfo {
public:
    bool IsProfilingEnabled() const { return false; }
    // Whether this kernel is the last one to read input `idx` (src/ppl/nn/runtime/kernel_exec_context.h:37-43
    // derives it from the graph's edge-to-last-consumer list; the harness states it as a bit mask).
    bool IsLastConsumerOfInput(uint32_t idx) const { return idx < 32 && ((last_consumer_mask_ >> idx) & 1u) != 0; }
    void SetLastConsumerMask(uint32_t mask) { last_consumer_mask_ = mask; }

private:
    uint32_t last_consumer_mask_ = 0;
};

namespace ir {

struct NodeType final {
    std::string domain, name;
    uint64_t version = 0;
};

class Node final {
public:
    Node(uint32_t id, const std::string& name, const NodeType& type) : id_(id), name_(name), type_(type) {}
    uint32_t GetId() const { return id_; }
    const std::string& GetName() const { return name_; }
    const NodeType& GetType() const { return type_; }

private:
    uint32_t id_;
    std::string name_;
    NodeType type_;
};

class Attr {
public:
    virtual ~Attr() {}
};

template <typename T>
class TypedAttr : public Attr {};

// graph->data->attrs: node id -> parsed attribute object (src/ppl/nn/engines/llm_cuda/opt_kernel.h:49-61)
struct GraphData final {
    std::map<uint32_t, std::shared_ptr<Attr>> attrs;
};
struct Graph final {
    std::shared_ptr<GraphData> data = std::make_shared<GraphData>();
};

}  // namespace ir

class KernelImpl {
public:
    explicit KernelImpl(const ir::Node* node) : node_(node) {}
    virtual ~KernelImpl() {}
    const ir::Node* GetNode() const { return node_; }
    const std::string& GetName() const { return node_->GetName(); }
    void SetEngineContext(void* ctx) { engine_context_ = ctx; }
    void* GetEngineContext() const { return engine_context_; }
    virtual ppl::common::RetCode Reshape(InputOutputInfo*) const = 0;
    virtual ppl::common::RetCode Execute(KernelExecContext*) = 0;

private:
    const ir::Node* node_;
    void* engine_context_ = nullptr;
};

}}  // namespace ppl::nn
