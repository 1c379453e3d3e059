// TEST INFRASTRUCTURE, not product code: one C entry point around the reference project's own W4A16
// GEMM (src/qgemm/gptq_marlin/gptq_marlin.cu, compiled where it lies together with this file into
// oracle/_ref/libcpmcu_ref_marlin.so by oracle/build_ref.py; it needs the PyTorch headers the
// reference's own build uses).  Arguments as W4A16GPTQMarlinLinear::prefill passes them
// (src/model/w4a16_gptq_marlin/w4a16_gptq_marlin_linear.cuh:100-142): symmetric int4 with bias 8,
// group size 128, no act-order, fp32 reduce.
#include <cstdint>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include "qgemm/gptq_marlin/marlin.cuh"
#include "qgemm/gptq_marlin/gptq_marlin.cuh"
#include "qgemm/gptq_marlin/core/scalar_type.hpp"

extern "C" {

// x: [M][K] bf16, qweight: int32 [K/16][N*16/8] (Marlin tiles), scales: [K/128][N] bf16 (Marlin column
// order), y: [M][N] bf16.  Scratch (lock words, fp32 reduce buffer) is allocated and zeroed per call.
// Returns the CUDA error code, or -1 for an exception from the reference's argument checks.
int refk_marlin_gemm(const void* x, const int32_t* qweight, const void* scales, void* y, int M, int N, int K) {
    using T = __nv_bfloat16;
    const vllm::ScalarType wtype(static_cast<uint8_t>(0), static_cast<uint8_t>(4), false, static_cast<int32_t>(8),
                                 false);
    const int num_groups = K / 128;
    const size_t ws_bytes = size_t(N / 64) * 16 * sizeof(int32_t);
    const size_t ct_bytes = size_t(marlin::determine_reduce_max_m(M, marlin::max_par)) * N * sizeof(float);
    int32_t* workspace = nullptr;
    float* c_tmp = nullptr;
    T* a_tmp = nullptr;
    if (cudaMalloc(&workspace, ws_bytes) != cudaSuccess) return int(cudaGetLastError());
    if (cudaMalloc(&c_tmp, ct_bytes) != cudaSuccess) return int(cudaGetLastError());
    if (cudaMalloc(&a_tmp, size_t(M) * K * sizeof(T)) != cudaSuccess) return int(cudaGetLastError());
    cudaMemset(workspace, 0, ws_bytes);
    cudaMemset(c_tmp, 0, ct_bytes);
    int rc = 0;
    try {
        gptq_marlin_gemm<T>((T*)x, (int32_t*)qweight, (T*)scales, nullptr, nullptr, nullptr, workspace, wtype, M, N, K,
                            true, false, true, (T*)y, num_groups, 128, 2 * N, false, nullptr, a_tmp, c_tmp);
    } catch (const std::exception&) {
        rc = -1;
    }
    cudaError_t e = cudaDeviceSynchronize();
    if (rc == 0 && e == cudaSuccess) e = cudaGetLastError();
    if (rc == 0) rc = int(e);
    cudaFree(workspace);
    cudaFree(c_tmp);
    cudaFree(a_tmp);
    return rc;
}

// Times `iters` back-to-back calls of the reference's Marlin GEMM with CUDA events, cycling through `copies`
// weight buffers (HBM, not L2).  Any bit pattern is a valid int4 weight; scales are 0x3c3c (about 0.0115).
int refk_bench_marlin(int M, int N, int K, int copies, int iters, float* avg_us) {
    using T = __nv_bfloat16;
    const vllm::ScalarType wtype(static_cast<uint8_t>(0), static_cast<uint8_t>(4), false, static_cast<int32_t>(8),
                                 false);
    const size_t wq_bytes = size_t(N) * K / 2, sc_bytes = size_t(K / 128) * N * 2;
    const size_t ws_bytes = size_t(N / 64) * 16 * sizeof(int32_t);
    const size_t ct_bytes = size_t(marlin::determine_reduce_max_m(M, marlin::max_par)) * N * sizeof(float);
    char *wq = nullptr, *sc = nullptr;
    T *x = nullptr, *y = nullptr, *a_tmp = nullptr;
    int32_t* workspace = nullptr;
    float* c_tmp = nullptr;
    if (cudaMalloc(&wq, wq_bytes * copies) != cudaSuccess || cudaMalloc(&sc, sc_bytes * copies) != cudaSuccess ||
        cudaMalloc(&x, size_t(M) * K * 2) != cudaSuccess || cudaMalloc(&y, size_t(M) * N * 2) != cudaSuccess ||
        cudaMalloc(&a_tmp, size_t(M) * K * 2) != cudaSuccess || cudaMalloc(&workspace, ws_bytes) != cudaSuccess ||
        cudaMalloc(&c_tmp, ct_bytes) != cudaSuccess)
        return int(cudaGetLastError());
    cudaMemset(wq, 0x5a, wq_bytes * copies);
    cudaMemset(sc, 0x3c, sc_bytes * copies);
    cudaMemset(x, 0x3c, size_t(M) * K * 2);
    cudaMemset(workspace, 0, ws_bytes);
    cudaMemset(c_tmp, 0, ct_bytes);
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    int rc = 0;
    try {
        for (int i = -3; i < iters; ++i) {
            if (i == 0) cudaEventRecord(e0, nullptr);
            const int c = (i + 3) % copies;
            gptq_marlin_gemm<T>(x, (int32_t*)(wq + wq_bytes * c), (T*)(sc + sc_bytes * c), nullptr, nullptr, nullptr,
                                workspace, wtype, M, N, K, true, false, true, y, K / 128, 128, 2 * N, false, nullptr,
                                a_tmp, c_tmp);
        }
        cudaEventRecord(e1, nullptr);
    } catch (const std::exception&) {
        rc = -1;
    }
    cudaError_t e = cudaDeviceSynchronize();
    if (rc == 0 && e == cudaSuccess) e = cudaGetLastError();
    if (rc == 0) rc = int(e);
    if (rc == 0) {
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        *avg_us = ms * 1000.f / iters;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaFree(wq); cudaFree(sc); cudaFree(x); cudaFree(y); cudaFree(a_tmp); cudaFree(workspace); cudaFree(c_tmp);
    return rc;
}

}  // extern "C"
