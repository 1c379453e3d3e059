// Per-process runtime: one stream (blocking, so that it orders itself against
// work the caller queued on the legacy default stream, as the reference's
// calc_stream does), the device error word that
// kernels raise instead of trapping, and the TMA tensor-map encoder (fetched
// from the driver at run time so the library links against cudart only).
// Plays the role of the reference's global stream/handle set-up
// (src/utils.cu:13-23) without cuBLAS.
#include "common.cuh"

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        CUDA_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres));
        if (sym == nullptr || qres != cudaDriverEntryPointSuccess) {
            throw std::runtime_error("cpmcu_b200: driver does not export cuTensorMapEncodeTiled");
        }
        fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

}  // namespace

Runtime& runtime() {
    static Runtime rt;
    static bool ready = false;
    if (!ready) {
        int count = 0;
        cudaError_t e = cudaGetDeviceCount(&count);
        if (e != cudaSuccess || count == 0) {
            throw std::runtime_error("cpmcu_b200: no CUDA device visible; this library has no CPU path");
        }
        CUDA_CHECK(cudaGetDevice(&rt.device));
        cudaDeviceProp prop;
        CUDA_CHECK(cudaGetDeviceProperties(&prop, rt.device));
        if (prop.major != 10) {
            throw std::runtime_error("cpmcu_b200: kernels are built for sm_100a only (found sm_" +
                                     std::to_string(prop.major * 10 + prop.minor) + ")");
        }
        rt.num_sms = prop.multiProcessorCount;
        rt.pdl = (getenv("CPMCU_NO_PDL") == nullptr);
        CUDA_CHECK(cudaStreamCreate(&rt.stream));
        CUDA_CHECK(cudaMalloc(&rt.d_error, sizeof(int)));
        CUDA_CHECK(cudaMemset(rt.d_error, 0, sizeof(int)));
        CUDA_CHECK(cudaMalloc(&rt.d_accept_ticket, sizeof(unsigned)));
        CUDA_CHECK(cudaMemset(rt.d_accept_ticket, 0, sizeof(unsigned)));
        ready = true;
    }
    return rt;
}

int read_and_clear_error() {
    Runtime& rt = runtime();
    int h = 0;
    CUDA_CHECK(cudaMemcpyAsync(&h, rt.d_error, sizeof(int), cudaMemcpyDeviceToHost, rt.stream));
    CUDA_CHECK(cudaStreamSynchronize(rt.stream));
    if (h != 0) {
        CUDA_CHECK(cudaMemsetAsync(rt.d_error, 0, sizeof(int), rt.stream));
        CUDA_CHECK(cudaStreamSynchronize(rt.stream));
    }
    return h;
}

CUtensorMap make_tmap_2d(const void* base, uint64_t inner, uint64_t outer, uint64_t outer_stride_bytes,
                         uint32_t box_inner, uint32_t box_outer) {
    CPM_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, "tensor map base must be 16-byte aligned");
    CPM_REQUIRE(outer_stride_bytes % 16 == 0, "tensor map stride must be a multiple of 16 bytes");
    CPM_REQUIRE(box_inner * 2 == 128 && box_outer >= 1 && box_outer <= 256, "tensor map box out of range");
    CUtensorMap tm;
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {outer_stride_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode_fn()(&tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                             estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) throw std::runtime_error("cpmcu_b200: cuTensorMapEncodeTiled (2-D) failed: " + std::to_string(r));
    return tm;
}

CUtensorMap make_tmap_3d(const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_bytes,
                         uint64_t stride2_bytes, uint32_t b0, uint32_t b1, uint32_t b2) {
    CPM_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, "tensor map base must be 16-byte aligned");
    CPM_REQUIRE(stride1_bytes % 16 == 0 && stride2_bytes % 16 == 0, "tensor map strides must be multiples of 16 bytes");
    CPM_REQUIRE(b0 * 2 == 128 && b1 >= 1 && b1 <= 256 && b2 >= 1 && b2 <= 256, "tensor map box out of range");
    CUtensorMap tm;
    cuuint64_t dims[3] = {d0, d1, d2};
    cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
    cuuint32_t box[3] = {b0, b1, b2};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = encode_fn()(&tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box,
                             estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) throw std::runtime_error("cpmcu_b200: cuTensorMapEncodeTiled (3-D) failed: " + std::to_string(r));
    return tm;
}

ProfileScope::ProfileScope(int kind_, cudaStream_t s_) : s(s_), kind(kind_), on(false) {
    Runtime& rt = runtime();
    if (!rt.profile) return;
    on = true;
    cudaEvent_t e0;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    cudaEventRecord(e0, s);
    rt.prof[kind].push_back(std::make_pair(e0, e1));
}

ProfileScope::~ProfileScope() {
    if (on) cudaEventRecord(e1, s);
}

CUtensorMap make_tmap_2d_u8(const void* base, uint64_t inner_bytes, uint64_t outer, uint64_t outer_stride_bytes,
                            uint32_t box_inner_bytes, uint32_t box_outer) {
    CPM_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, "tensor map base must be 16-byte aligned");
    CPM_REQUIRE(outer_stride_bytes % 16 == 0 && box_inner_bytes % 16 == 0, "tensor map stride/box must be multiples of 16 bytes");
    CPM_REQUIRE(box_inner_bytes <= 256 && box_outer >= 1 && box_outer <= 256, "tensor map box out of range");
    CUtensorMap tm;
    cuuint64_t dims[2] = {inner_bytes, outer};
    cuuint64_t strides[1] = {outer_stride_bytes};
    cuuint32_t box[2] = {box_inner_bytes, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode_fn()(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) throw std::runtime_error("cpmcu_b200: cuTensorMapEncodeTiled (u8) failed: " + std::to_string(r));
    return tm;
}
