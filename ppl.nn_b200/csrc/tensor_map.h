// Host-side construction of the TMA tensor maps over the caller's cache and scale tensors.
#pragma once

#include <cuda.h>
#include <stdint.h>

#include "../../include/ppl_nn_b200.h"

namespace pplb200 {

// Encodes a tiled tensor map through the driver entry point (resolved once at run time, so the
// library does not link against libcuda).  `rank` <= 5; dims/box in elements, strides in bytes for
// dimensions 1..rank-1.  Returns PPLB200_SUCCESS or PPLB200_DEVICE_RUNTIME_ERROR (logged).
int encode_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, uint32_t rank, const void* base,
                      const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                      CUtensorMapSwizzle swizzle);

// Position (1..4) of each logical cache dimension in the tensor maps below.  Dimension 0 is always
// the channel; the other four are ordered by increasing stride, which depends on cache_layout.
struct CacheMapOrder {
    int32_t pos_row, pos_head, pos_kv, pos_layer;
};

// Five-dimensional map over `cache` (uint8 view, innermost extent head_dim) whose outer dimensions
// are (row, kv head, k|v, layer) with the strides of the params, sorted by stride.  The box is one
// head's rows of `tile_tokens` consecutive cache rows.  Code rows of 128 bytes use the 128-byte swizzle
// so that the kernels' 16-byte shared-memory reads are bank-conflict free.
int make_cache_tensor_map(const pplb200_attn_params& p, const void* cache, int tile_tokens, CUtensorMap* codes,
                          CacheMapOrder* order);

}  // namespace pplb200
