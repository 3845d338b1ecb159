// placeholder while the tcgen05 prefill kernel is being written
#include "common.cuh"
#include "launch.h"

namespace pplb200 {

int make_prefill_plan(const pplb200_attn_params& p, PrefillPlan* plan) {
    plan->prefill_batches = p.batch - p.decoding_batches;
    plan->q_tiles_per_seq = (p.max_seqlen + 127) / 128;
    plan->kv_rows_bound = 0;
    plan->off_kv_stage = 0;
    plan->off_stage_starts = 0;
    plan->bytes = 0;
    return PPLB200_SUCCESS;
}

int launch_prefill(const pplb200_attn_params&, const CacheGeom&, const PrefillPlan&, const void*, const void*,
                   const void*, const int64_t*, const int64_t*, const int64_t*, const void*, const void*, void*,
                   uint32_t*, void*, cudaStream_t) {
    return PPLB200_UNSUPPORTED;
}

}  // namespace pplb200
