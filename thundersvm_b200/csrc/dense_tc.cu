// Tensor maps for the tcgen05 kernel-row engine (dense_tc2.cu) and the engine's entry point used by km.cu.
#include "tc_common.cuh"

namespace tsvm {

typedef CUresult (*encode_fn_t)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static encode_fn_t get_encode() {
    static encode_fn_t fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (encode_fn_t) p;
    }
    return fn;
}

// rows x row_len matrix of 32-bit words (or FP16 halves) with row stride ld elements; box = one 128-byte
// swizzle row (32 words / 64 halves) x box_rows rows.
tsvm_status make_map(CUtensorMap *map, const void *ptr, int rows, int row_len, long long ld, int box_rows, bool f16) {
    encode_fn_t enc = get_encode();
    if (!enc) { set_error("cuTensorMapEncodeTiled is not available from the driver"); return TSVM_ERR_CUDA; }
    const size_t esz = f16 ? 2 : 4;
    cuuint64_t dims[2] = {(cuuint64_t) row_len, (cuuint64_t) rows};
    cuuint64_t strides[1] = {(cuuint64_t) ld * esz};
    cuuint32_t box[2] = {(cuuint32_t) (128 / esz), (cuuint32_t) box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void *) ptr, dims,
                     strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed with code %d", (int) r); return TSVM_ERR_CUDA; }
    return TSVM_OK;
}

// Whi/Wlo (m x plane_ld) and sd_rows are staged in the handle's scratch by the caller.
tsvm_status launch_dense_tc2(tsvm_km *km, int m, float *out, long long ld_out, cudaStream_t st);   // dense_tc2.cu

tsvm_status launch_dense_tc(tsvm_km *km, int m, float *out, long long ld_out, cudaStream_t st) {
    return launch_dense_tc2(km, m, out, ld_out, st);
}

}  // namespace tsvm
