// Host side of the TMA helpers: tensor-map encoding through the driver entry point that the
// CUDA runtime hands out (the library does not link libcuda).
#include "tma.cuh"
#include <mutex>

flare_encode_tiled_fn flare_get_encode_tiled() {
    static flare_encode_tiled_fn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<flare_encode_tiled_fn>(p);
    });
    return fn;
}

int flare_make_tensor_map(CUtensorMap* out, CUtensorMapDataType dt, int rank, void* base, const uint64_t* dims,
                          const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swz) {
    flare_encode_tiled_fn enc = flare_get_encode_tiled();
    if (!enc) return -1;
    cuuint64_t gdim[5], gstr[4];
    cuuint32_t bx[5], es[5];
    for (int i = 0; i < rank; i++) { gdim[i] = dims[i]; bx[i] = box[i]; es[i] = 1; }
    for (int i = 0; i + 1 < rank; i++) gstr[i] = strides_bytes[i];
    CUresult r = enc(out, dt, (cuuint32_t)rank, base, gdim, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return (int)r;
}
