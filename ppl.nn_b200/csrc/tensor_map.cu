#include "tensor_map.h"

#include <cuda_runtime.h>
#include <cudaTypedefs.h>
#include <stdio.h>

#include <mutex>

#ifndef PPLB200_L2_PROMO
#define PPLB200_L2_PROMO CU_TENSOR_MAP_L2_PROMOTION_L2_256B
#endif

namespace pplb200 {

namespace {

PFN_cuTensorMapEncodeTiled_v12000 resolve_encode() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    static std::once_flag once;
    std::call_once(once, []() {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &sym, 12000, cudaEnableDefault, &qres);
        if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(sym);
        } else {
            fprintf(stderr, "[ppl_nn_b200] cannot resolve cuTensorMapEncodeTiled: %s\n", cudaGetErrorString(e));
        }
    });
    return fn;
}

}  // namespace

int encode_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, uint32_t rank, const void* base,
                      const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                      CUtensorMapSwizzle swizzle) {
    auto fn = resolve_encode();
    if (!fn) {
        return PPLB200_DEVICE_RUNTIME_ERROR;
    }
    cuuint64_t gdims[5];
    cuuint64_t gstrides[4];
    cuuint32_t gbox[5];
    cuuint32_t estr[5];
    for (uint32_t i = 0; i < rank; ++i) {
        gdims[i] = dims[i];
        gbox[i] = box[i];
        estr[i] = 1;
        if (i + 1 < rank) {
            gstrides[i] = strides_bytes[i];
        }
    }
    CUresult r = fn(map, dtype, rank, const_cast<void*>(base), gdims, gstrides, gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle, PPLB200_L2_PROMO, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        fprintf(stderr, "[ppl_nn_b200] cuTensorMapEncodeTiled failed: CUresult %d (rank %u, dims", static_cast<int>(r), rank);
        for (uint32_t i = 0; i < rank; ++i) {
            fprintf(stderr, " %llu", static_cast<unsigned long long>(dims[i]));
        }
        fprintf(stderr, ")\n");
        return PPLB200_DEVICE_RUNTIME_ERROR;
    }
    return PPLB200_SUCCESS;
}

int make_cache_tensor_map(const pplb200_attn_params& p, const void* cache, int tile_tokens, CUtensorMap* codes,
                          CacheMapOrder* order) {
    // logical outer dimensions: 0 row, 1 kv head, 2 k|v, 3 layer
    const uint64_t extent[4] = {static_cast<uint64_t>(p.max_tokens), static_cast<uint64_t>(p.num_kv_heads), 2,
                                static_cast<uint64_t>(p.num_layer)};
    const uint64_t stride[4] = {static_cast<uint64_t>(p.cache_stride_s), static_cast<uint64_t>(p.cache_stride_h),
                                static_cast<uint64_t>(p.cache_stride_kv), static_cast<uint64_t>(p.cache_stride_l)};
    int idx[4] = {0, 1, 2, 3};
    // Insertion sort by stride; among equal strides the row dimension goes last, so that a one-layer
    // token-major cache (row and layer strides tie) gets the same order as a multi-layer one.
    auto before = [&](int x, int y) {
        return stride[x] < stride[y] || (stride[x] == stride[y] && y == 0 && x != 0);
    };
    for (int i = 1; i < 4; ++i) {
        for (int j = i; j > 0 && before(idx[j], idx[j - 1]); --j) {
            const int tmp = idx[j];
            idx[j] = idx[j - 1];
            idx[j - 1] = tmp;
        }
    }
    int pos[4];
    for (int i = 0; i < 4; ++i) {
        pos[idx[i]] = i + 1;
    }
    order->pos_row = pos[0];
    order->pos_head = pos[1];
    order->pos_kv = pos[2];
    order->pos_layer = pos[3];

    const uint64_t dh = static_cast<uint64_t>(p.head_dim);
    uint64_t dims_c[5], str_c[4];
    uint32_t box_c[5];
    dims_c[0] = dh;
    box_c[0] = static_cast<uint32_t>(dh);
    for (int i = 0; i < 4; ++i) {
        const int d = idx[i];
        dims_c[i + 1] = extent[d];
        str_c[i] = stride[d];  // int8: elements == bytes
        box_c[i + 1] = (d == 0) ? static_cast<uint32_t>(tile_tokens) : 1u;
    }
    return encode_tensor_map(codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, 5, cache, dims_c, str_c, box_c,
                             p.head_dim == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE);
}

}  // namespace pplb200
