// Host-side declarations shared by the translation units of the library: one launcher per kernel
// family, the launch counter and the post-launch error check.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ppl_nn_b200.h"

namespace pplb200 {

struct CacheGeom;
struct MaskDev;

constexpr int kMaxDevices = 64;  // devices per process that per-device launch state is kept for

// cudaGetLastError() after a launch -> PPLB200_SUCCESS / PPLB200_DEVICE_RUNTIME_ERROR (logged to
// stderr with the kernel name), and bumps the launch counter.  Mirrors what ppl.nn does after every
// kernel (src/ppl/nn/engines/llm_cuda/kernel.cc:179-185).
int check_launch(const char* kernel_name);

// Event bracketing of one kernel launch for pplb200_profile_*: a no-op unless profiling is on.
// Usage: { KernelTimer t(PPLB200_KERNEL_DECODE, stream); kernel<<<...>>>(...); }
class KernelTimer {
public:
    KernelTimer(int family, cudaStream_t stream);
    ~KernelTimer();

private:
    cudaStream_t stream_;
    cudaEvent_t stop_;
};

// Launch with programmatic stream serialisation: the grid may be scheduled while its predecessor in the
// stream drains, and runs its prologue there; every kernel launched this way executes
// grid_dependency_wait() (common.cuh) before it touches anything a predecessor wrote, which waits for the
// predecessor's completion and memory flush.  Saves the launch gap between the short kernels of a step.
#ifndef PPLB200_PDL
#define PPLB200_PDL 1
#endif
template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = PPLB200_PDL;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Properties of the current device, cached per device id.
struct DeviceInfo {
    int device_id;
    int sm_count;
    int cc_major;
    int cc_minor;
    int max_smem_optin;
};
int current_device_info(DeviceInfo* info);

// Appends the tokens of sequences [first_seq, batch) (all of them with first_seq 0).  `status` (nullable)
// receives kDevRowOutOfRange when an index tensor names a row outside the cache; such rows are skipped.
int launch_kv_append(const pplb200_attn_params& p, const CacheGeom& geom, const void* cur_k, const void* cur_v,
                     const int64_t* seqstarts, const int64_t* cachestarts, const int64_t* start_pos, void* cache,
                     void* scale, int64_t first_seq, uint32_t* status, int sm_count, cudaStream_t stream);

int launch_kv_gather_dequant(const pplb200_attn_params& p, const CacheGeom& geom, const int64_t* kvstarts,
                             const int64_t* cachestarts, const void* cache, const void* scale, int64_t total_kv,
                             void* key_out, void* value_out, int sm_count, cudaStream_t stream);

// ---- decode (split-k over the INT8 cache) ------------------------------------------------------
// Host-side plan: pure function of the params and the SM count, used both for the workspace size
// and for the launch, so the two always agree.
struct DecodePlan {
    int32_t octets;            // ceil(group / 8): query-head octets per kv head
    int64_t num_vheads;        // num_kv_heads * octets: segments per sequence
    int32_t head_lanes;        // 4, 2 or 1 head classes: warps of a CTA that stream adjacent heads of the same rows
    int64_t class_heads;       // num_vheads / head_lanes
    int64_t grid;              // persistent CTAs (4 warps each)
    int64_t workers;           // resident warps per head class
    int64_t max_ranges;        // upper bound of the ranges (per class) the planning kernel may create
    int64_t partial_slots;     // fp32 partial records in the workspace (2 per range and class)
    // workspace layout (byte offsets)
    uint64_t off_header, off_tile_prefix, off_part_ml, off_part_o, bytes;
};
int make_decode_plan(const pplb200_attn_params& p, int sm_count, DecodePlan* plan);

// `append_key` / `append_value` non-null: the decode kernel also quantises and appends the new token of
// every decode sequence (query row seqstarts[b+1]-1, position start_pos[b]+seqlen-1) and attends to it;
// null: the cache already holds that token.
int launch_decode(const pplb200_attn_params& p, const CacheGeom& geom, const DecodePlan& plan, const void* query,
                  const void* append_key, const void* append_value, const int64_t* seqstarts,
                  const int64_t* cachestarts, const int64_t* start_pos, void* cache, void* scale, const MaskDev& mask,
                  void* workspace, void* attn_output, cudaStream_t stream);

// ---- prefill (causal, tcgen05) -------------------------------------------------------------------
struct PrefillPlan {
    int64_t prefill_batches;
    int64_t q_tiles_per_seq;   // ceil(max_seqlen / 128)
    int64_t kv_rows_bound;     // rows of the dequantised fp16 K/V staging buffer (cache prefill only)
    uint64_t off_kv_stage, off_stage_starts, bytes;  // relative to the prefill region of the workspace
};
int make_prefill_plan(const pplb200_attn_params& p, PrefillPlan* plan);

int launch_prefill(const pplb200_attn_params& p, const CacheGeom& geom, const PrefillPlan& plan, const void* query,
                   const void* cur_k, const void* cur_v, const int64_t* seqstarts, const int64_t* cachestarts,
                   const int64_t* start_pos, const void* cache, const void* scale, const MaskDev& mask,
                   void* workspace_region, uint32_t* status_word, void* attn_output, cudaStream_t stream);

// The un-cached attention operator through the prefill kernel (K/V from their own tensors).
int launch_mha(int num_heads, int num_kv_heads, int head_dim, int is_causal, int64_t batch, int64_t max_seqlen,
               int64_t max_kvlen, int64_t total_q, int64_t total_kv, const void* query, const void* key,
               const void* value, const int64_t* seqstarts, const int64_t* kvstarts, const MaskDev& mask,
               uint32_t* status_word, void* attn_output, cudaStream_t stream);

// Rotary position embedding, alone (append == nullptr) or fused with the cache append.
uint64_t rope_workspace_bytes(const pplb200_rope_params& p);
int launch_rope(const pplb200_rope_params& p, const pplb200_attn_params* append, const CacheGeom* geom,
                const void* query, const void* key, const void* value, const int64_t* seqstarts,
                const int64_t* start_pos, const int64_t* cachestarts, void* workspace, void* rotated_query,
                void* rotated_key, void* cache, void* scale, int sm_count, cudaStream_t stream);

}  // namespace pplb200
