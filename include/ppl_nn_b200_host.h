/*
 * ppl_nn_b200_host.h -- C harness over the C++ host layer (ppl.nn_b200/host/): creates the two
 * operators through the llm_cuda-style registry, exactly as ppl.nn's graph builder would
 * (OptKernelCreatorManager::Find -> creator -> Init -> CreateKernelImpl;
 *  src/ppl/nn/engines/llm_cuda/opt_graph.cc:31-80, src/ppl/nn/runtime/runtime_impl.cc:57-79), and
 * executes their kernels on caller-provided tensors.  It exists so that tests and the benchmark
 * can drive the reference-facing operator interface from Python; ppl.nn itself would link the
 * C++ classes directly.  Return values are ppl::common::RetCode values of this library
 * (pplb200_host_retcode_str gives their names).
 */
#ifndef PPL_NN_B200_HOST_H_
#define PPL_NN_B200_HOST_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { PPLB200_DT_FLOAT16 = 1, PPLB200_DT_FLOAT32 = 2, PPLB200_DT_INT8 = 3, PPLB200_DT_INT32 = 4, PPLB200_DT_INT64 = 5 };

typedef struct pplb200_host_tensor {
    void* data;        /* buffer; null = the slot is present but has no buffer yet                       */
    int32_t dtype;     /* PPLB200_DT_*                                                                  */
    int32_t ndim;      /* 0 = scalar                                                                    */
    int64_t dims[6];
    int32_t on_host;   /* 1: `data` is host memory (host device), 0: device memory of the engine's GPU  */
    int32_t absent;    /* 1: optional input left out of the graph                                       */
} pplb200_host_tensor;

/* Engine context: one GPU, one stream (cudaStream_t as void*), one tmp-buffer pool. */
void* pplb200_host_engine_create(int device_id, void* stream);
void pplb200_host_engine_destroy(void* engine);
/* Engine knobs by the names of ENGINE_CONF_* (include/ppl/nn/engines/llm_cuda/options.h:139-148,111-137):
 * "cache_prefill", "decoding_attn_split_k", "decoding_attn_tpb", "decoding_shm_mha", "decoding_inf_mha",
 * "decoding_inf_gqa".  Unknown key: RC_INVALID_VALUE. */
int pplb200_host_engine_configure(void* engine, const char* key, int64_t value);
uint64_t pplb200_host_engine_tmp_pool_bytes(void* engine);

/* Registry. */
void pplb200_host_register_ops(void);                                            /* RegisterB200OpImpls()            */
int pplb200_host_registry_has(const char* domain, const char* type, uint64_t version);
void pplb200_host_registry_remove(const char* domain, const char* type);
int pplb200_host_registry_register_again(const char* domain, const char* type, uint64_t first, uint64_t last);

/* Creates node + attribute object + Op (Init) + Kernel.  attr_names/attr_values: the node's attributes
 * as integers; a float attribute (theta, scaling_factor) is passed as the bit pattern of the float in the
 * low 32 bits, the string attribute scaling_type as 0 (""), 1 ("linear") or 2 ("dynamic").  On failure returns null and stores the RetCode in *rc. */
void* pplb200_host_op_create(void* engine, const char* domain, const char* type, uint64_t version,
                             const char* const* attr_names, const int64_t* attr_values, int num_attrs, int* rc);
void pplb200_host_op_destroy(void* op);

/* Executes the kernel.  Outputs: on return dims/ndim/dtype hold the inferred shape; if `data` was
 * null the kernel allocated the buffer on the engine's GPU and `data` points to it (owned by the op,
 * valid until the next run or destroy). */
int pplb200_host_op_run(void* op, const pplb200_host_tensor* inputs, int num_inputs, pplb200_host_tensor* outputs,
                        int num_outputs);
/* States which inputs (bit i = input i) the op is the LAST consumer of, what the runtime's
 * KernelExecContext::IsLastConsumerOfInput() answers from the graph; default 0.  A kernel may then hand such an
 * input's buffer over to an output instead of allocating one (the rotary embedding does, like the reference):
 * after the run the output's `data` is the input's pointer. */
void pplb200_host_op_set_last_consumer(void* op, uint32_t input_mask);
int pplb200_host_engine_synchronize(void* engine);

const char* pplb200_host_retcode_str(int rc);

#ifdef __cplusplus
}
#endif
#endif
