// extern "C" layer: argument validation, workspace layout and kernel sequencing for the two operators.
// Nothing here allocates device memory or synchronises, except pplb200_mhca_device_status (waits for the
// stream) and pplb200_profile_read (waits for the recorded events).
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>

#include <atomic>
#include <initializer_list>
#include <mutex>
#include <utility>
#include <vector>

#include "common.cuh"
#include "launch.h"

namespace pplb200 {

static std::atomic<uint64_t> g_launches{0};

int check_launch(const char* kernel_name) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        fprintf(stderr, "[ppl_nn_b200] launch of %s failed: %s\n", kernel_name, cudaGetErrorString(e));
        return PPLB200_DEVICE_RUNTIME_ERROR;
    }
    return PPLB200_SUCCESS;
}

// ---- optional per-kernel event timing ------------------------------------------------------------
struct ProfileState {
    std::mutex mu;
    std::atomic<bool> enabled{false};
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> pending[PPLB200_KERNEL_FAMILIES];
};
static ProfileState& profile_state() {
    static ProfileState s;
    return s;
}

KernelTimer::KernelTimer(int family, cudaStream_t stream) : stream_(stream), stop_(nullptr) {
    ProfileState& ps = profile_state();
    if (!ps.enabled.load(std::memory_order_relaxed)) {
        return;
    }
    cudaEvent_t start = nullptr;
    if (cudaEventCreate(&start) != cudaSuccess) {
        (void)cudaGetLastError();
        return;
    }
    if (cudaEventCreate(&stop_) != cudaSuccess) {
        (void)cudaGetLastError();
        cudaEventDestroy(start);
        stop_ = nullptr;
        return;
    }
    cudaEventRecord(start, stream_);
    std::lock_guard<std::mutex> lock(ps.mu);
    ps.pending[family].emplace_back(start, stop_);
}

KernelTimer::~KernelTimer() {
    if (stop_) {
        cudaEventRecord(stop_, stream_);
    }
}

int current_device_info(DeviceInfo* info) {
    constexpr int kMaxDevices = 64;
    static DeviceInfo cache[kMaxDevices];
    static bool known[kMaxDevices] = {};
    static std::mutex mu;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        (void)cudaGetLastError();
        return PPLB200_DEVICE_RUNTIME_ERROR;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (!known[dev]) {
        DeviceInfo d;
        d.device_id = dev;
        if (cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&d.cc_minor, cudaDevAttrComputeCapabilityMinor, dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) {
            (void)cudaGetLastError();
            return PPLB200_DEVICE_RUNTIME_ERROR;
        }
        cache[dev] = d;
        known[dev] = true;
    }
    *info = cache[dev];
    return PPLB200_SUCCESS;
}

static int fail(int code, const char* what) {
    fprintf(stderr, "[ppl_nn_b200] %s: %s\n", pplb200_status_str(code), what);
    return code;
}

// Attribute and geometry checks shared by all entry points.  The reference rejects
// quant_bit/quant_group only when BOTH differ from 8 (multi_head_cache_attention_kernel.cc:90-93);
// here either one differing is rejected, because no other format is implemented.
static int validate(const pplb200_attn_params* p) {
    if (!p) {
        return fail(PPLB200_NOT_FOUND, "params is null");
    }
    if (p->quant_bit != 8 || p->quant_group != 8) {
        return fail(PPLB200_UNSUPPORTED, "only quant_bit == quant_group == 8 is supported");
    }
    if (p->head_dim != 64 && p->head_dim != 128) {
        return fail(PPLB200_UNSUPPORTED, "head_dim must be 64 or 128");
    }
    if (p->num_heads <= 0 || p->num_kv_heads <= 0 || p->num_heads % p->num_kv_heads != 0) {
        return fail(PPLB200_INVALID_VALUE, "num_heads must be a positive multiple of num_kv_heads");
    }
    if (p->cache_layout != 0 && p->cache_layout != 3) {
        return fail(PPLB200_UNSUPPORTED, "only cache_layout 0 and 3 are supported");
    }
    if (p->cache_mode != 0 && p->cache_mode != 1) {
        return fail(PPLB200_UNSUPPORTED, "only cache_mode 0 and 1 are supported");
    }
    if (p->cache_mode == 1 && (p->page_size <= 0 || p->page_size % 16 != 0 || p->cachestart_stride_b <= 0)) {
        return fail(PPLB200_INVALID_VALUE, "paged cache needs page_size % 16 == 0 and 2-d cachestarts");
    }
    if (p->cache_mode == 1 && p->max_kvlen > p->cachestart_stride_b * static_cast<int64_t>(p->page_size)) {
        return fail(PPLB200_INVALID_VALUE, "max_kvlen exceeds what a page-table row (cachestarts.dim(1) pages) can hold");
    }
    if (p->num_layer <= 0 || p->layer_idx < 0 || p->layer_idx >= p->num_layer) {
        return fail(PPLB200_INVALID_VALUE, "layer_idx out of range");
    }
    if (p->batch < 0 || p->decoding_batches < 0 || p->decoding_batches > p->batch || p->total_tokens < 0 ||
        p->batch > 0x7fffffff || p->total_tokens > 0x7fffffff || p->max_seqlen < 0 || p->max_kvlen < 0) {
        return fail(PPLB200_INVALID_VALUE, "batch / decoding_batches / total_tokens / max lengths out of range");
    }
    if (p->max_tokens <= 0 || p->max_tokens > 0x7fffffff) {
        return fail(PPLB200_INVALID_VALUE, "max_tokens (cache rows) out of range");
    }
    const int64_t s[4] = {p->cache_stride_s, p->cache_stride_l, p->cache_stride_h, p->cache_stride_kv};
    for (int i = 0; i < 4; ++i) {
        if (s[i] <= 0 || s[i] % 64 != 0) {
            return fail(PPLB200_INVALID_VALUE, "cache strides must be positive multiples of 64 elements");
        }
    }
    if (p->split_k_mode < 0 || p->split_k_mode > 2) {
        return fail(PPLB200_INVALID_VALUE, "split_k_mode must be 0, 1 or 2");
    }
    return PPLB200_SUCCESS;
}

// The kernels use 16-byte vector accesses and TMA on the payload tensors and 8-byte loads on the index
// tensors; a misaligned pointer would fault on the device, so it is refused here.
static bool misaligned(std::initializer_list<const void*> payload, std::initializer_list<const void*> index) {
    for (const void* q : payload) {
        if (reinterpret_cast<uintptr_t>(q) & 15u) {
            return true;
        }
    }
    for (const void* q : index) {
        if (reinterpret_cast<uintptr_t>(q) & 7u) {
            return true;
        }
    }
    return false;
}

static CacheGeom make_geom(const pplb200_attn_params& p) {
    CacheGeom g;
    g.stride_s = p.cache_stride_s;
    g.stride_l = p.cache_stride_l;
    g.stride_h = p.cache_stride_h;
    g.stride_kv = p.cache_stride_kv;
    g.layer_idx = p.layer_idx;
    g.cachestart_stride_b = p.cachestart_stride_b;
    g.cache_mode = p.cache_mode;
    g.page_size = p.page_size > 0 ? p.page_size : 1;
    return g;
}

// The library only carries sm_100a code; on any other device it must fail loudly, never fall back.
static int require_device(DeviceInfo* di) {
    const int rc = current_device_info(di);
    if (rc != PPLB200_SUCCESS) {
        return fail(PPLB200_NO_DEVICE_CODE, "no usable CUDA device");
    }
    if (di->cc_major != 10) {
        return fail(PPLB200_NO_DEVICE_CODE, "this library holds sm_100a code only; the current device is not sm_100");
    }
    return PPLB200_SUCCESS;
}

struct WorkspaceLayout {
    DecodePlan decode;
    PrefillPlan prefill;
    uint64_t off_prefill;
    uint64_t bytes;
};

static int make_layout(const pplb200_attn_params& p, int sm_count, WorkspaceLayout* w) {
    int rc = make_decode_plan(p, sm_count, &w->decode);
    if (rc != PPLB200_SUCCESS) {
        return rc;
    }
    rc = make_prefill_plan(p, &w->prefill);
    if (rc != PPLB200_SUCCESS) {
        return rc;
    }
    w->off_prefill = w->decode.bytes;
    w->bytes = w->decode.bytes + w->prefill.bytes;
    return PPLB200_SUCCESS;
}

}  // namespace pplb200

using namespace pplb200;

extern "C" {

int pplb200_fill_cache_strides(pplb200_attn_params* p) {
    if (!p) {
        return PPLB200_NOT_FOUND;
    }
    const int64_t L = p->num_layer, H = p->num_kv_heads, D = p->head_dim, M = p->max_tokens;
    if (p->cache_layout == 0) {  // (MaxT, L, 2, H, Dh)
        p->cache_stride_s = L * 2 * H * D;
        p->cache_stride_l = 2 * H * D;
        p->cache_stride_h = D;
        p->cache_stride_kv = H * D;
    } else if (p->cache_layout == 3) {  // (L, 2, H, MaxT, Dh)
        p->cache_stride_s = D;
        p->cache_stride_l = 2 * H * M * D;
        p->cache_stride_h = M * D;
        p->cache_stride_kv = H * M * D;
    } else {
        return fail(PPLB200_UNSUPPORTED, "only cache_layout 0 and 3 are supported");
    }
    return PPLB200_SUCCESS;
}

int pplb200_kv_append_i8g8(const pplb200_attn_params* p, const void* current_key, const void* current_value,
                           const int64_t* seqstarts, const int64_t* cachestarts, const int64_t* start_pos,
                           void* cache, void* scale, void* stream) {
    int rc = validate(p);
    if (rc != PPLB200_SUCCESS) {
        return rc;
    }
    if (!scale) {
        return fail(PPLB200_UNSUPPORTED, "only a quantised cache is supported but scale is null");
    }
    if (p->batch == 0 || p->total_tokens == 0) {
        return PPLB200_SUCCESS;  // nothing to append, whatever the pointers are
    }
    if (!current_key || !current_value || !seqstarts || !cachestarts || !start_pos || !cache) {
        return fail(PPLB200_NOT_FOUND, "a required tensor pointer is null");
    }
    if (misaligned({current_key, current_value, cache, scale}, {seqstarts, cachestarts, start_pos})) {
        return fail(PPLB200_INVALID_VALUE, "tensor pointers must be 16-byte aligned (index tensors 8-byte)");
    }
    DeviceInfo di;
    rc = require_device(&di);
    if (rc != PPLB200_SUCCESS) {
        return rc;
    }
    return launch_kv_append(*p, make_geom(*p), current_key, current_value, seqstarts, cachestarts, start_pos, cache,
                            scale, 0, nullptr, di.sm_count, static_cast<cudaStream_t>(stream));
}

int pplb200_kv_gather_dequant(const pplb200_attn_params* p, const int64_t* kvstarts, const int64_t* cachestarts,
                              const void* cache, const void* scale, int64_t total_kv, void* key_out,
                              void* value_out, void* stream) {
    int rc = validate(p);
    if (rc != PPLB200_SUCCESS) {
        return rc;
    }
    if (!scale) {
        return fail(PPLB200_UNSUPPORTED, "only a quantised cache is supported but scale is null");
    }
    if (!kvstarts || !cachestarts || !cache || (total_kv > 0 && (!key_out || !value_out))) {
        return fail(PPLB200_NOT_FOUND, "a required tensor pointer is null");
    }
    if (total_kv < 0) {
        return fail(PPLB200_INVALID_VALUE, "total_kv is negative");
    }
    if (misaligned({cache, scale, key_out, value_out}, {kvstarts, cachestarts})) {
        return fail(PPLB200_INVALID_VALUE, "tensor pointers must be 16-byte aligned (index tensors 8-byte)");
    }
    DeviceInfo di;
    rc = require_device(&di);
    if (rc != PPLB200_SUCCESS) {
        return rc;
    }
    return launch_kv_gather_dequant(*p, make_geom(*p), kvstarts, cachestarts, cache, scale, total_kv, key_out,
                                    value_out, di.sm_count, static_cast<cudaStream_t>(stream));
}

// The SM count enters the split heuristic.  Without a device (host-only callers sizing buffers
// ahead of time) the B200 count is assumed; with a device its own count is used, and the forward
// call uses the same rule, so the two agree on the machine that runs the kernels.
static int planning_sm_count() {
    DeviceInfo di;
    if (current_device_info(&di) == PPLB200_SUCCESS && di.sm_count > 0) {
        return di.sm_count;
    }
    return 148;
}

int pplb200_mhca_workspace_size(const pplb200_attn_params* p, uint64_t* bytes) {
    int rc = validate(p);
    if (rc != PPLB200_SUCCESS) {
        return rc;
    }
    if (!bytes) {
        return fail(PPLB200_NOT_FOUND, "bytes is null");
    }
    WorkspaceLayout w;
    rc = make_layout(*p, planning_sm_count(), &w);
    if (rc != PPLB200_SUCCESS) {
        return rc;
    }
    *bytes = w.bytes;
    return PPLB200_SUCCESS;
}

// Shape checks of the optional attn_mask input; fills `m` (data == nullptr when there is no mask).
static int make_mask(const pplb200_attn_mask* in, int num_heads, int64_t total_tokens, const int64_t* kvstarts,
                     MaskDev* m) {
    m->data = nullptr;
    m->kvstarts = kvstarts;
    m->cols = 0;
    m->head_stride = 0;
    if (!in || !in->data) {
        return PPLB200_SUCCESS;
    }
    if (in->ndim != 2 && in->ndim != 3) {
        return fail(PPLB200_INVALID_VALUE, "attn_mask must have 2 or 3 dimensions");
    }
    const int64_t heads = in->ndim == 3 ? in->dims[0] : 1;
    const int64_t rows = in->dims[in->ndim - 2], cols = in->dims[in->ndim - 1];
    if ((in->ndim == 3 && heads != num_heads) || rows < total_tokens || cols <= 0 || cols % 8 != 0) {
        return fail(PPLB200_INVALID_VALUE,
                    "attn_mask must be [T, C] or [num_heads, T, C] with T >= query rows and C a multiple of 8");
    }
    if (reinterpret_cast<uintptr_t>(in->data) & 1u) {
        return fail(PPLB200_INVALID_VALUE, "attn_mask must be 2-byte aligned");
    }
    m->data = static_cast<const __half*>(in->data);
    m->cols = cols;
    m->head_stride = in->ndim == 3 ? rows * cols : 0;
    return PPLB200_SUCCESS;
}

int pplb200_attn_mask_check(const pplb200_attn_mask* attn_mask, int32_t num_heads, int64_t total_tokens) {
    MaskDev m;
    return make_mask(attn_mask, num_heads, total_tokens, nullptr, &m);
}

int pplb200_mhca_forward(const pplb200_attn_params* p, const void* query, const void* current_key,
                         const void* current_value, const int64_t* seqstarts, const int64_t* kvstarts,
                         const int64_t* cachestarts, const int64_t* start_pos, void* cache, void* scale,
                         void* workspace, uint64_t workspace_bytes, void* attn_output, void* stream_v) {
    return pplb200_mhca_forward_masked(p, query, current_key, current_value, seqstarts, kvstarts, cachestarts,
                                       start_pos, cache, scale, nullptr, workspace, workspace_bytes, attn_output,
                                       stream_v);
}

int pplb200_mhca_forward_masked(const pplb200_attn_params* p, const void* query, const void* current_key,
                                const void* current_value, const int64_t* seqstarts, const int64_t* kvstarts,
                                const int64_t* cachestarts, const int64_t* start_pos, void* cache, void* scale,
                                const pplb200_attn_mask* attn_mask, void* workspace, uint64_t workspace_bytes,
                                void* attn_output, void* stream_v) {
    int rc = validate(p);
    if (rc != PPLB200_SUCCESS) {
        return rc;
    }
    if (!scale) {
        return fail(PPLB200_UNSUPPORTED, "only a quantised cache is supported but scale is null");
    }
    // an empty batch is a no-op whatever the pointers are (empty tensors have none)
    if (p->batch == 0 || p->total_tokens == 0) {
        return PPLB200_SUCCESS;
    }
    if (!query || !current_key || !current_value || !seqstarts || !kvstarts || !cachestarts || !start_pos || !cache ||
        !attn_output) {
        return fail(PPLB200_NOT_FOUND, "a required tensor pointer is null");
    }
    if (misaligned({query, current_key, current_value, cache, scale, attn_output},
                   {seqstarts, kvstarts, cachestarts, start_pos})) {
        return fail(PPLB200_INVALID_VALUE, "tensor pointers must be 16-byte aligned (index tensors 8-byte)");
    }
    MaskDev amask;
    rc = make_mask(attn_mask, p->num_heads, p->total_tokens, kvstarts, &amask);
    if (rc != PPLB200_SUCCESS) {
        return rc;
    }
    DeviceInfo di;
    rc = require_device(&di);
    if (rc != PPLB200_SUCCESS) {
        return rc;
    }
    WorkspaceLayout w;
    rc = make_layout(*p, di.sm_count, &w);
    if (rc != PPLB200_SUCCESS) {
        return rc;
    }
    if (!workspace) {
        return fail(PPLB200_NOT_FOUND, "workspace is null");
    }
    if (workspace_bytes < w.bytes) {
        return fail(PPLB200_OUT_OF_MEMORY, "workspace is smaller than pplb200_mhca_workspace_size()");
    }
    if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) {
        return fail(PPLB200_INVALID_VALUE, "workspace must be 256-byte aligned");
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const CacheGeom geom = make_geom(*p);
    const int mask = p->phase_mask ? p->phase_mask : (PPLB200_PHASE_APPEND | PPLB200_PHASE_DECODE | PPLB200_PHASE_PREFILL);
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    uint32_t* status = reinterpret_cast<uint32_t*>(ws + w.decode.off_header);  // first word of the header

    // Order of the launches.  The planning kernel of the decode part (or a memset) clears the status word
    // first, so that every later kernel of the call can report through it.  The decode kernel appends the new
    // tokens of the decode sequences itself; the append kernel only sees the remaining sequences, and runs
    // behind the decode part, which does not depend on it.
    const bool do_append = (mask & PPLB200_PHASE_APPEND) != 0;
    const bool do_decode = (mask & PPLB200_PHASE_DECODE) != 0 && p->decoding_batches > 0;
    const bool do_prefill = (mask & PPLB200_PHASE_PREFILL) != 0 && p->decoding_batches < p->batch;
    // PPLB200_FUSE_APPEND=0 (measurement only): the append kernel handles every token ahead of the decode part
    const char* fuse_env = getenv("PPLB200_FUSE_APPEND");
    const bool fuse = do_append && do_decode && !(fuse_env && fuse_env[0] == '0');
    if (do_append && do_decode && !fuse) {
        rc = launch_kv_append(*p, geom, current_key, current_value, seqstarts, cachestarts, start_pos, cache, scale, 0,
                              nullptr, di.sm_count, stream);
        if (rc != PPLB200_SUCCESS) {
            return rc;
        }
    }
    if (do_decode) {
        rc = launch_decode(*p, geom, w.decode, query, fuse ? current_key : nullptr, fuse ? current_value : nullptr,
                           seqstarts, cachestarts, start_pos, cache, scale, amask, workspace, attn_output, stream);
        if (rc != PPLB200_SUCCESS) {
            return rc;
        }
    } else if (cudaMemsetAsync(status, 0, 4, stream) != cudaSuccess) {
        (void)cudaGetLastError();
        return fail(PPLB200_DEVICE_RUNTIME_ERROR, "cudaMemsetAsync(status) failed");
    }
    if (do_append && (fuse || !do_decode)) {
        rc = launch_kv_append(*p, geom, current_key, current_value, seqstarts, cachestarts, start_pos, cache, scale,
                              fuse ? p->decoding_batches : 0, status, di.sm_count, stream);
        if (rc != PPLB200_SUCCESS) {
            return rc;
        }
    }
    if (do_prefill) {
        rc = launch_prefill(*p, geom, w.prefill, query, current_key, current_value, seqstarts, cachestarts, start_pos,
                            cache, scale, amask, ws + w.off_prefill, status, attn_output, stream);
        if (rc != PPLB200_SUCCESS) {
            return rc;
        }
    }
    return PPLB200_SUCCESS;
}

int pplb200_mha_workspace_size(const pplb200_mha_params* p, uint64_t* bytes) {
    if (!p || !bytes) {
        return fail(PPLB200_NOT_FOUND, "null argument");
    }
    *bytes = 256;  // the device status word
    return PPLB200_SUCCESS;
}

int pplb200_mha_forward(const pplb200_mha_params* p, const void* query, const void* key, const void* value,
                        const int64_t* seqstarts, const int64_t* kvstarts, void* workspace, uint64_t workspace_bytes,
                        void* attn_output, void* stream_v) {
    return pplb200_mha_forward_masked(p, query, key, value, seqstarts, kvstarts, nullptr, workspace, workspace_bytes,
                                      attn_output, stream_v);
}

int pplb200_mha_forward_masked(const pplb200_mha_params* p, const void* query, const void* key, const void* value,
                               const int64_t* seqstarts, const int64_t* kvstarts, const pplb200_attn_mask* attn_mask,
                               void* workspace, uint64_t workspace_bytes, void* attn_output, void* stream_v) {
    if (!p) {
        return fail(PPLB200_NOT_FOUND, "params is null");
    }
    if (p->head_dim != 64 && p->head_dim != 128) {
        return fail(PPLB200_UNSUPPORTED, "head_dim must be 64 or 128");
    }
    if (p->num_heads <= 0 || p->num_kv_heads <= 0 || p->num_heads % p->num_kv_heads != 0) {
        return fail(PPLB200_INVALID_VALUE, "num_heads must be a positive multiple of num_kv_heads");
    }
    if (p->batch < 0 || p->max_seqlen < 0 || p->max_kvlen < 0 || p->total_tokens < 0 || p->total_kv_tokens < 0 ||
        p->decoding_batches < 0 || p->decoding_batches > p->batch) {
        return fail(PPLB200_INVALID_VALUE, "negative size or decoding_batches > batch");
    }
    if (p->total_tokens > 0x7fffffff || p->total_kv_tokens > 0x7fffffff) {
        return fail(PPLB200_UNSUPPORTED, "more than 2^31 rows");
    }
    // an empty batch is a no-op whatever the pointers are (empty tensors have none)
    if (p->batch == 0 || p->total_tokens == 0) {
        return PPLB200_SUCCESS;
    }
    if (!query || !key || !value || !seqstarts || !kvstarts || !attn_output) {
        return fail(PPLB200_NOT_FOUND, "a required tensor pointer is null");
    }
    if (misaligned({query, key, value, attn_output}, {seqstarts, kvstarts})) {
        return fail(PPLB200_INVALID_VALUE, "tensor pointers must be 16-byte aligned (index tensors 8-byte)");
    }
    MaskDev amask;
    int rc = make_mask(attn_mask, p->num_heads, p->total_tokens, kvstarts, &amask);
    if (rc != PPLB200_SUCCESS) {
        return rc;
    }
    DeviceInfo di;
    rc = require_device(&di);
    if (rc != PPLB200_SUCCESS) {
        return rc;
    }
    if (!workspace) {
        return fail(PPLB200_NOT_FOUND, "workspace is null");
    }
    if (workspace_bytes < 256) {
        return fail(PPLB200_OUT_OF_MEMORY, "workspace is smaller than pplb200_mha_workspace_size()");
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    uint32_t* status = static_cast<uint32_t*>(workspace);
    if (cudaMemsetAsync(status, 0, 4, stream) != cudaSuccess) {
        (void)cudaGetLastError();
        return fail(PPLB200_DEVICE_RUNTIME_ERROR, "cudaMemsetAsync(status) failed");
    }
    return launch_mha(p->num_heads, p->num_kv_heads, p->head_dim, p->is_causal, p->batch, p->max_seqlen, p->max_kvlen,
                      p->total_tokens, p->total_kv_tokens, query, key, value, seqstarts, kvstarts, amask, status,
                      attn_output, stream);
}

static int validate_rope(const pplb200_rope_params* p) {
    if (!p) {
        return fail(PPLB200_NOT_FOUND, "params is null");
    }
    if (p->head_dim != 64 && p->head_dim != 128) {
        return fail(PPLB200_UNSUPPORTED, "head_dim must be 64 or 128");
    }
    const int rot = p->rotary_dim == 0 ? p->head_dim : p->rotary_dim;
    if (rot < 2 || rot > p->head_dim || (rot & 1)) {
        return fail(PPLB200_INVALID_VALUE, "rotary_dim must be even and within head_dim");
    }
    if (p->num_heads <= 0 || p->num_kv_heads <= 0) {
        return fail(PPLB200_INVALID_VALUE, "head counts must be positive");
    }
    if (p->scaling_type < 0 || p->scaling_type > 2) {
        return fail(PPLB200_INVALID_VALUE, "invalid scaling type");
    }
    if (!(p->theta > 0.0f) || (p->scaling_type != 0 && !(p->scaling_factor > 0.0f))) {
        return fail(PPLB200_INVALID_VALUE, "theta and scaling_factor must be positive");
    }
    if (p->scaling_type == 2 && (p->max_position_embeddings <= 0 || rot <= 2)) {
        return fail(PPLB200_INVALID_VALUE, "dynamic scaling needs max_position_embeddings > 0 and rotary_dim > 2");
    }
    if (p->batch < 0 || p->total_tokens < 0 || p->batch > 0x7fffffff || p->total_tokens > 0x7fffffff) {
        return fail(PPLB200_INVALID_VALUE, "batch / total_tokens out of range");
    }
    return PPLB200_SUCCESS;
}

int pplb200_rope_workspace_size(const pplb200_rope_params* p, uint64_t* bytes) {
    const int rc = validate_rope(p);
    if (rc != PPLB200_SUCCESS) {
        return rc;
    }
    if (!bytes) {
        return fail(PPLB200_NOT_FOUND, "null argument");
    }
    *bytes = rope_workspace_bytes(*p);
    return PPLB200_SUCCESS;
}

int pplb200_rope_forward(const pplb200_rope_params* p, const void* query, const void* key, const int64_t* seqstarts,
                         const int64_t* start_pos, void* workspace, uint64_t workspace_bytes, void* rotated_query,
                         void* rotated_key, void* stream) {
    int rc = validate_rope(p);
    if (rc != PPLB200_SUCCESS) {
        return rc;
    }
    // an empty batch is a no-op whatever the pointers are (empty tensors have none)
    if (p->batch == 0 || p->total_tokens == 0) {
        return PPLB200_SUCCESS;
    }
    if (!query || !key || !seqstarts || !start_pos || !rotated_query || !rotated_key) {
        return fail(PPLB200_NOT_FOUND, "a required tensor pointer is null");
    }
    if (misaligned({query, key, rotated_query, rotated_key}, {seqstarts, start_pos})) {
        return fail(PPLB200_INVALID_VALUE, "tensor pointers must be 16-byte aligned (index tensors 8-byte)");
    }
    DeviceInfo di;
    rc = require_device(&di);
    if (rc != PPLB200_SUCCESS) {
        return rc;
    }
    if (!workspace) {
        return fail(PPLB200_NOT_FOUND, "workspace is null");
    }
    if (workspace_bytes < rope_workspace_bytes(*p)) {
        return fail(PPLB200_OUT_OF_MEMORY, "workspace is smaller than pplb200_rope_workspace_size()");
    }
    return launch_rope(*p, nullptr, nullptr, query, key, nullptr, seqstarts, start_pos, nullptr, workspace,
                       rotated_query, rotated_key, nullptr, nullptr, di.sm_count, static_cast<cudaStream_t>(stream));
}

int pplb200_rope_kv_append_i8g8(const pplb200_rope_params* p, const pplb200_attn_params* attn, const void* query,
                                const void* key, const void* value, const int64_t* seqstarts,
                                const int64_t* cachestarts, const int64_t* start_pos, void* workspace,
                                uint64_t workspace_bytes, void* rotated_query, void* rotated_key, void* cache,
                                void* scale, void* stream) {
    int rc = validate_rope(p);
    if (rc != PPLB200_SUCCESS) {
        return rc;
    }
    rc = validate(attn);
    if (rc != PPLB200_SUCCESS) {
        return rc;
    }
    if (attn->num_heads != p->num_heads || attn->num_kv_heads != p->num_kv_heads || attn->head_dim != p->head_dim ||
        attn->batch != p->batch || attn->total_tokens != p->total_tokens) {
        return fail(PPLB200_INVALID_VALUE, "the two parameter blocks disagree on heads, head_dim, batch or tokens");
    }
    // an empty batch is a no-op whatever the pointers are (empty tensors have none)
    if (p->batch == 0 || p->total_tokens == 0) {
        return PPLB200_SUCCESS;
    }
    if (!query || !key || !value || !seqstarts || !cachestarts || !start_pos || !rotated_query || !cache || !scale) {
        return fail(PPLB200_NOT_FOUND, "a required tensor pointer is null");
    }
    if (misaligned({query, key, value, rotated_query, rotated_key, cache, scale}, {seqstarts, cachestarts, start_pos})) {
        return fail(PPLB200_INVALID_VALUE, "tensor pointers must be 16-byte aligned (index tensors 8-byte)");
    }
    DeviceInfo di;
    rc = require_device(&di);
    if (rc != PPLB200_SUCCESS) {
        return rc;
    }
    if (!workspace) {
        return fail(PPLB200_NOT_FOUND, "workspace is null");
    }
    if (workspace_bytes < rope_workspace_bytes(*p)) {
        return fail(PPLB200_OUT_OF_MEMORY, "workspace is smaller than pplb200_rope_workspace_size()");
    }
    const CacheGeom geom = make_geom(*attn);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // One kernel pays off while the step is bound by launches (decode steps).  On big batches the rotation
    // is memory-bound and the quantiser issue-bound, and two kernels, each at its own limit, are faster
    // (measured: 333 vs 480 us for 65 536 tokens); the cache rows are the same either way.
    if (rotated_key && p->total_tokens >= 1024) {
        rc = launch_rope(*p, nullptr, nullptr, query, key, nullptr, seqstarts, start_pos, nullptr, workspace,
                         rotated_query, rotated_key, nullptr, nullptr, di.sm_count, st);
        if (rc != PPLB200_SUCCESS) {
            return rc;
        }
        return launch_kv_append(*attn, geom, rotated_key, value, seqstarts, cachestarts, start_pos, cache, scale, 0,
                                nullptr, di.sm_count, st);
    }
    return launch_rope(*p, attn, &geom, query, key, value, seqstarts, start_pos, cachestarts, workspace, rotated_query,
                       rotated_key, cache, scale, di.sm_count, st);
}

int pplb200_mhca_device_status(const void* workspace, void* stream, uint32_t* status) {
    if (!workspace || !status) {
        return PPLB200_NOT_FOUND;
    }
    if (cudaStreamSynchronize(static_cast<cudaStream_t>(stream)) != cudaSuccess) {
        (void)cudaGetLastError();
        return PPLB200_DEVICE_RUNTIME_ERROR;
    }
    if (cudaMemcpy(status, workspace, 4, cudaMemcpyDeviceToHost) != cudaSuccess) {
        (void)cudaGetLastError();
        return PPLB200_DEVICE_RUNTIME_ERROR;
    }
    return PPLB200_SUCCESS;
}

const char* pplb200_status_str(int status) {
    switch (status) {
        case PPLB200_SUCCESS: return "RC_SUCCESS";
        case PPLB200_INVALID_VALUE: return "RC_INVALID_VALUE";
        case PPLB200_UNSUPPORTED: return "RC_UNSUPPORTED";
        case PPLB200_OUT_OF_MEMORY: return "RC_OUT_OF_MEMORY";
        case PPLB200_DEVICE_RUNTIME_ERROR: return "RC_DEVICE_RUNTIME_ERROR";
        case PPLB200_NOT_FOUND: return "RC_NOT_FOUND";
        case PPLB200_NO_DEVICE_CODE: return "RC_NO_DEVICE_CODE";
        default: return "RC_OTHER_ERROR";
    }
}

int pplb200_device_ready(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) {
        (void)cudaGetLastError();
        return 0;
    }
    DeviceInfo di;
    if (current_device_info(&di) != PPLB200_SUCCESS) {
        return 0;
    }
    return di.cc_major == 10 ? 1 : 0;
}

uint64_t pplb200_launch_count(void) {
    return g_launches.load(std::memory_order_relaxed);
}

int pplb200_profile_enable(int enable) {
    ProfileState& ps = profile_state();
    ps.enabled.store(enable != 0, std::memory_order_relaxed);
    return PPLB200_SUCCESS;
}

int pplb200_profile_read(int kernel_family, double* total_ms, uint64_t* launches) {
    if (kernel_family < 0 || kernel_family >= PPLB200_KERNEL_FAMILIES || !total_ms || !launches) {
        return PPLB200_INVALID_VALUE;
    }
    ProfileState& ps = profile_state();
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> taken;
    {
        std::lock_guard<std::mutex> lock(ps.mu);
        taken.swap(ps.pending[kernel_family]);
    }
    double sum = 0.0;
    int rc = PPLB200_SUCCESS;
    for (auto& pr : taken) {
        float ms = 0.0f;
        if (cudaEventSynchronize(pr.second) != cudaSuccess || cudaEventElapsedTime(&ms, pr.first, pr.second) != cudaSuccess) {
            (void)cudaGetLastError();
            rc = PPLB200_DEVICE_RUNTIME_ERROR;
        }
        sum += ms;
        cudaEventDestroy(pr.first);
        cudaEventDestroy(pr.second);
    }
    *total_ms = sum;
    *launches = taken.size();
    return rc;
}

}  // extern "C"
