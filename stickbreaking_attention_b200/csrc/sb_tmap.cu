// Host side of TMA: encodes tiled tensor maps through the driver entry point (no link-time dependency on libcuda).
#include <mutex>

#include "sb_sm100.cuh"

namespace sb {

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
std::once_flag g_once;

void resolve() {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
        g_encode = (EncodeTiledFn)fn;
}
}  // namespace

int encode_tile_map(CUtensorMap* map, const void* ptr, int elem_kind, int64_t D, int64_t T, int64_t H, int64_t B,
                    int64_t stride_t, int64_t stride_h, int64_t stride_b, int box_rows) {
    std::call_once(g_once, resolve);
    if (!g_encode) return -1;
    if (H < 1) H = 1;
    if (B < 1) B = 1;
    // a dimension of extent 1 never moves the address: give it a stride the encoder accepts
    if (H == 1) stride_h = stride_t * T;
    if (B == 1) stride_b = (stride_h > stride_t ? stride_h * H : stride_t * T);
    const cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)T, (cuuint64_t)H, (cuuint64_t)B};
    const cuuint64_t strides[3] = {(cuuint64_t)stride_t * 2, (cuuint64_t)stride_h * 2, (cuuint64_t)stride_b * 2};
    const cuuint32_t box[4] = {64u, (cuuint32_t)box_rows, 1u, 1u};
    const cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
    const CUtensorMapDataType dt = elem_kind == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    const CUresult r = g_encode(map, dt, 4, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)r;
}

}  // namespace sb
