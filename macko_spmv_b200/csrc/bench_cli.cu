// Command-line benchmark with the interface of the reference's `c_benchmarking/benchmark`
// (c_benchmarking/utils.cuh:63-101 for the ten positional arguments, c_benchmarking/benchmark.cu:128-233
// for the protocol and the output), so that its result lines drop into the same tables:
//
//   macko_bench <bits_per_value> <rows> <cols> <warmup> <timing> <flush> <debug> <kernel_id> <seed> <density>
//
// kernel_id 7 is the MACKO SpMV (here: macko_spmv_fp16 of this library), 8 the int8 MACKO SpMV (bits_per_value 8:
// macko_spmv_int8), 1 and 2 are cuBLAS GemmEx with fp16 and fp32 accumulation on the dense matrix, 3 is cuSPARSE
// SpMM on a CSR copy (CUSPARSE_SPMM_CSR_ALG1, fp16 values, fp32 compute: c_benchmarking/benchmark.cu:76-90,
// utils.cuh:405-462), 0 is the fp32 cuBLAS GEMV every result is checked against. The protocol is the
// reference's: one checked run, warm-up, 100 launches timed on the host for the launch cost, then `timing`
// launches timed one by one with CUDA events, each after an optional flush of L2 (a memset of twice its size).
// The data follows the reference's generator call for call (c_benchmarking/utils.cuh:464-519 after
// srand(seed), benchmark.cu:138): every matrix entry drawn as (rand() % 101 - 50) / 100 (bits 16) or
// rand() % 101 - 50 (bits 8) until non-zero, the vector likewise, then exactly int(density * rows * cols)
// entries kept by sequential selection sampling with rand(); so a run sees the matrix the reference CLI sees
// for the same arguments on the same C library. It is compressed on the GPU through the C ABI, and the last line is
//   Final results:\t<bits>\t<rows>\t<cols>\t<kernel_id>\t<density>\t<mean us>\t<dense Gflops>\t<sparse Gflops>
#include <cublas_v2.h>
#include <cusparse.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <string>
#include <vector>

#include "macko_b200.h"

namespace {

#define CUDA_OK(expr)                                                                                      \
    do {                                                                                                   \
        cudaError_t e_ = (expr);                                                                           \
        if (e_ != cudaSuccess) {                                                                           \
            std::cerr << "CUDA error " << cudaGetErrorString(e_) << " at " << __FILE__ << ":" << __LINE__ << std::endl; \
            std::exit(2);                                                                                  \
        }                                                                                                  \
    } while (0)

#define CUBLAS_OK(expr)                                                                                    \
    do {                                                                                                   \
        cublasStatus_t s_ = (expr);                                                                        \
        if (s_ != CUBLAS_STATUS_SUCCESS) {                                                                 \
            std::cerr << "cuBLAS error " << (int)s_ << " at " << __FILE__ << ":" << __LINE__ << std::endl;  \
            std::exit(2);                                                                                  \
        }                                                                                                  \
    } while (0)

#define CUSPARSE_OK(expr)                                                                                  \
    do {                                                                                                   \
        cusparseStatus_t s_ = (expr);                                                                      \
        if (s_ != CUSPARSE_STATUS_SUCCESS) {                                                               \
            std::cerr << "cuSPARSE error " << (int)s_ << " at " << __FILE__ << ":" << __LINE__ << std::endl; \
            std::exit(2);                                                                                  \
        }                                                                                                  \
    } while (0)

#define MACKO_CALL(expr)                                                                                   \
    do {                                                                                                   \
        int st_ = (expr);                                                                                  \
        if (st_ != MACKO_OK) {                                                                             \
            std::cerr << "macko error " << macko_status_string(st_) << ": " << macko_last_error() << std::endl; \
            std::exit(2);                                                                                  \
        }                                                                                                  \
    } while (0)

struct Args {
    int bits = 16, rows = 0, cols = 0, warmup = 10, timing = 10, flush = 0, debug = 0, kernel_id = 7, seed = 0;
    float density = 1.f;
};

// One draw of the reference generator: uniform over {-50, ..., 50} \ {0} by rejection (utils.cuh:464-489)
int draw_nonzero()
{
    int k;
    do {
        k = rand() % 101 - 50;
    } while (k == 0);
    return k;
}

struct Data {
    Args a;
    size_t n = 0;
    std::vector<float> m32, v32;
    float *m32_d = nullptr, *v32_d = nullptr, *y32_d = nullptr;
    __half *m16_d = nullptr, *v16_d = nullptr, *y16_d = nullptr;
    void *values_d = nullptr, *deltas_d = nullptr;
    int32_t *ri_d = nullptr;
    int64_t padded = 0;
    bool last_output_is_half = true;
    // cuSPARSE CSR copy of the dense fp16 matrix (kernel id 3), built on first use
    cusparseHandle_t sp = nullptr;
    cusparseSpMatDescr_t sp_a = nullptr;
    cusparseDnMatDescr_t dn_a = nullptr, dn_b = nullptr, dn_c = nullptr;
    void *sp_buffer = nullptr;
    const float sp_alpha = 1.f, sp_beta = 0.f;

    explicit Data(const Args &args) : a(args)
    {
        n = (size_t)a.rows * a.cols;
        srand((unsigned)a.seed);
        m32.resize(n);
        v32.resize(a.cols);
        // bits 8: integer values, as the int8 matrix needs them
        for (size_t i = 0; i < n; ++i) m32[i] = a.bits == 16 ? float(draw_nonzero()) / 100 : float(draw_nonzero());
        for (int i = 0; i < a.cols; ++i) v32[i] = float(draw_nonzero()) / 100;
        // exactly int(density * n) non-zeros survive: entry i stays with probability (still to keep) / (still to see)
        int ones_to_sample = int(a.density * float((int)n));
        int zeros_to_sample = (int)n - ones_to_sample;
        for (size_t i = 0; i < n; ++i) {
            const bool is_one = (rand() % (ones_to_sample + zeros_to_sample)) < ones_to_sample;
            if (!is_one) {
                m32[i] = 0.f;
                --zeros_to_sample;
            } else {
                --ones_to_sample;
            }
        }
        std::vector<__half> m16(n), v16(a.cols);
        for (size_t i = 0; i < n; ++i) m16[i] = __float2half(m32[i]);
        for (int i = 0; i < a.cols; ++i) v16[i] = __float2half(v32[i]);
        // the fp32 copies hold the fp16-rounded values, so that the check compares like with like
        for (size_t i = 0; i < n; ++i) m32[i] = __half2float(m16[i]);
        for (int i = 0; i < a.cols; ++i) v32[i] = __half2float(v16[i]);

        CUDA_OK(cudaMalloc(&m32_d, std::max<size_t>(n, 1) * sizeof(float)));
        CUDA_OK(cudaMalloc(&v32_d, std::max(a.cols, 1) * sizeof(float)));
        CUDA_OK(cudaMalloc(&y32_d, std::max(a.rows, 1) * sizeof(float)));
        CUDA_OK(cudaMalloc(&m16_d, std::max<size_t>(n, 8) * sizeof(__half)));
        CUDA_OK(cudaMalloc(&v16_d, std::max(a.cols, 8) * sizeof(__half)));
        CUDA_OK(cudaMalloc(&y16_d, std::max(a.rows, 1) * sizeof(__half)));
        CUDA_OK(cudaMemcpy(m32_d, m32.data(), n * sizeof(float), cudaMemcpyHostToDevice));
        CUDA_OK(cudaMemcpy(v32_d, v32.data(), a.cols * sizeof(float), cudaMemcpyHostToDevice));
        CUDA_OK(cudaMemcpy(m16_d, m16.data(), n * sizeof(__half), cudaMemcpyHostToDevice));
        CUDA_OK(cudaMemcpy(v16_d, v16.data(), a.cols * sizeof(__half), cudaMemcpyHostToDevice));

        // MACKO buffers from the GPU compressor
        CUDA_OK(cudaMalloc(&ri_d, ((size_t)a.rows + 1) * sizeof(int32_t)));
        if (a.bits == 8) {
            std::vector<int8_t> m8(n);
            for (size_t i = 0; i < n; ++i) m8[i] = (int8_t)m32[i];
            int8_t *m8_d = nullptr;
            CUDA_OK(cudaMalloc(&m8_d, std::max<size_t>(n, 8)));
            CUDA_OK(cudaMemcpy(m8_d, m8.data(), n, cudaMemcpyHostToDevice));
            MACKO_CALL(macko_compress_count_int8(m8_d, a.rows, a.cols, ri_d, nullptr));
            int32_t stored8 = 0;
            CUDA_OK(cudaMemcpy(&stored8, ri_d + a.rows, sizeof(int32_t), cudaMemcpyDeviceToHost));
            padded = ((int64_t)stored8 + 7) / 8 * 8;
            void *ws8 = nullptr;
            CUDA_OK(cudaMalloc(&values_d, std::max<int64_t>(padded, 16)));
            CUDA_OK(cudaMalloc(&deltas_d, std::max<int64_t>(padded / 2, 4)));
            CUDA_OK(cudaMalloc(&ws8, std::max<int64_t>(macko_compress_workspace_bytes(padded), 8)));
            MACKO_CALL(macko_compress_emit_int8(m8_d, a.rows, a.cols, ri_d, padded, values_d, deltas_d, ws8,
                                                macko_compress_workspace_bytes(padded), nullptr));
            CUDA_OK(cudaDeviceSynchronize());
            CUDA_OK(cudaFree(ws8));
            CUDA_OK(cudaFree(m8_d));
            return;
        }
        MACKO_CALL(macko_compress_count(m16_d, a.rows, a.cols, ri_d, nullptr));
        int32_t stored = 0;
        CUDA_OK(cudaMemcpy(&stored, ri_d + a.rows, sizeof(int32_t), cudaMemcpyDeviceToHost));
        padded = ((int64_t)stored + 7) / 8 * 8;
        void *ws = nullptr;
        CUDA_OK(cudaMalloc(&values_d, std::max<int64_t>(padded, 8) * 2));
        CUDA_OK(cudaMalloc(&deltas_d, std::max<int64_t>(padded / 2, 4)));
        CUDA_OK(cudaMalloc(&ws, std::max<int64_t>(macko_compress_workspace_bytes(padded), 8)));
        MACKO_CALL(macko_compress_emit(m16_d, a.rows, a.cols, ri_d, padded, values_d, deltas_d, ws,
                                       macko_compress_workspace_bytes(padded), nullptr));
        CUDA_OK(cudaDeviceSynchronize());
        CUDA_OK(cudaFree(ws));
    }

    // CSR copy of the dense fp16 matrix through cuSPARSE's own dense-to-sparse conversion, and the SpMM buffer
    void setup_cusparse()
    {
        if (sp) return;
        int *row_ptr = nullptr, *col_ind = nullptr;
        __half *csr_val = nullptr;
        CUDA_OK(cudaMalloc(&row_ptr, sizeof(int) * ((size_t)a.rows + 1)));
        CUSPARSE_OK(cusparseCreate(&sp));
        CUSPARSE_OK(cusparseCreateDnMat(&dn_a, a.rows, a.cols, a.cols, m16_d, CUDA_R_16F, CUSPARSE_ORDER_ROW));
        CUSPARSE_OK(cusparseCreateDnMat(&dn_b, a.cols, 1, a.cols, v16_d, CUDA_R_16F, CUSPARSE_ORDER_COL));
        CUSPARSE_OK(cusparseCreateDnMat(&dn_c, a.rows, 1, a.rows, y16_d, CUDA_R_16F, CUSPARSE_ORDER_COL));
        CUSPARSE_OK(cusparseCreateCsr(&sp_a, a.rows, a.cols, 0, row_ptr, nullptr, nullptr, CUSPARSE_INDEX_32I, CUSPARSE_INDEX_32I,
                                      CUSPARSE_INDEX_BASE_ZERO, CUDA_R_16F));
        size_t bytes = 0;
        void *tmp = nullptr;
        CUSPARSE_OK(cusparseDenseToSparse_bufferSize(sp, dn_a, sp_a, CUSPARSE_DENSETOSPARSE_ALG_DEFAULT, &bytes));
        CUDA_OK(cudaMalloc(&tmp, std::max<size_t>(bytes, 8)));
        CUSPARSE_OK(cusparseDenseToSparse_analysis(sp, dn_a, sp_a, CUSPARSE_DENSETOSPARSE_ALG_DEFAULT, tmp));
        int64_t r = 0, c = 0, nnz = 0;
        CUSPARSE_OK(cusparseSpMatGetSize(sp_a, &r, &c, &nnz));
        CUDA_OK(cudaMalloc(&col_ind, std::max<int64_t>(nnz, 1) * sizeof(int)));
        CUDA_OK(cudaMalloc(&csr_val, std::max<int64_t>(nnz, 1) * sizeof(__half)));
        CUSPARSE_OK(cusparseCsrSetPointers(sp_a, row_ptr, col_ind, csr_val));
        CUSPARSE_OK(cusparseDenseToSparse_convert(sp, dn_a, sp_a, CUSPARSE_DENSETOSPARSE_ALG_DEFAULT, tmp));
        CUDA_OK(cudaFree(tmp));
        CUSPARSE_OK(cusparseSpMM_bufferSize(sp, CUSPARSE_OPERATION_NON_TRANSPOSE, CUSPARSE_OPERATION_NON_TRANSPOSE, &sp_alpha, sp_a,
                                            dn_b, &sp_beta, dn_c, CUDA_R_32F, CUSPARSE_SPMM_CSR_ALG1, &bytes));
        CUDA_OK(cudaMalloc(&sp_buffer, std::max<size_t>(bytes, 8)));
    }

    double dense_gflops(double us) const { return 2.0 * a.rows * a.cols / (us * 1e3); }
    double sparse_gflops(double us) const { return 2.0 * a.rows * a.cols * a.density / (us * 1e3); }
    double dense_bandwidth(double us) const { return 2.0 * ((double)n + a.rows + a.cols) / (us * 1e3); }
    double compressed_bandwidth(double us) const
    {
        return ((a.bits == 8 ? 1.5 : 2.5) * padded + 4.0 * (a.rows + 1) + 2.0 * a.cols + 2.0 * a.rows) / (us * 1e3);
    }
    double effective_density() const { return ((a.bits == 8 ? 1.5 : 2.5) * padded + 4.0 * a.cols) / ((a.bits == 8 ? 1.0 : 2.0) * (double)n); }
};

void run(int kernel_id, Data &d, cudaStream_t stream, cublasHandle_t handle)
{
    const Args &a = d.a;
    d.last_output_is_half = true;
    switch (kernel_id) {
        case 0: {   // fp32 cuBLAS GEMV: the reference result
            const float alpha = 1.f, beta = 0.f;
            CUBLAS_OK(cublasSgemv(handle, CUBLAS_OP_T, a.cols, a.rows, &alpha, d.m32_d, a.cols, d.v32_d, 1, &beta, d.y32_d, 1));
            d.last_output_is_half = false;
            break;
        }
        case 1: {   // cuBLAS, fp16 accumulation
            const __half alpha = __float2half(1.f), beta = __float2half(0.f);
            CUBLAS_OK(cublasGemmEx(handle, CUBLAS_OP_T, CUBLAS_OP_N, a.rows, 1, a.cols, &alpha, d.m16_d, CUDA_R_16F, a.cols,
                                   d.v16_d, CUDA_R_16F, a.cols, &beta, d.y16_d, CUDA_R_16F, a.rows, CUBLAS_COMPUTE_16F,
                                   CUBLAS_GEMM_DEFAULT));
            break;
        }
        case 2: {   // cuBLAS, fp32 accumulation
            const float alpha = 1.f, beta = 0.f;
            CUBLAS_OK(cublasGemmEx(handle, CUBLAS_OP_T, CUBLAS_OP_N, a.rows, 1, a.cols, &alpha, d.m16_d, CUDA_R_16F, a.cols,
                                   d.v16_d, CUDA_R_16F, a.cols, &beta, d.y16_d, CUDA_R_16F, a.rows, CUBLAS_COMPUTE_32F,
                                   CUBLAS_GEMM_DEFAULT));
            break;
        }
        case 3:     // cuSPARSE SpMM on the CSR copy
            d.setup_cusparse();
            CUSPARSE_OK(cusparseSetStream(d.sp, stream));
            CUSPARSE_OK(cusparseSpMM(d.sp, CUSPARSE_OPERATION_NON_TRANSPOSE, CUSPARSE_OPERATION_NON_TRANSPOSE, &d.sp_alpha, d.sp_a,
                                     d.dn_b, &d.sp_beta, d.dn_c, CUDA_R_32F, CUSPARSE_SPMM_CSR_ALG1, d.sp_buffer));
            break;
        case 7:     // MACKO SpMV
            if (a.bits != 16) { std::cerr << "NO KERNEL (kernel id 7 takes 16 bits per value)" << std::endl; std::exit(1); }
            MACKO_CALL(macko_spmv_fp16(d.values_d, d.deltas_d, d.ri_d, a.rows, a.cols, d.padded, d.v16_d, d.y16_d, 1.f, 0.f, stream));
            break;
        case 8:     // MACKO SpMV, int8 values
            if (a.bits != 8) { std::cerr << "NO KERNEL (kernel id 8 takes 8 bits per value)" << std::endl; std::exit(1); }
            MACKO_CALL(macko_spmv_int8(d.values_d, d.deltas_d, d.ri_d, a.rows, a.cols, d.padded, d.v16_d, d.y16_d, 1.f, 0.f, 0u, stream));
            break;
        default:
            std::cerr << "NO KERNEL (this library has kernel ids 0, 1, 2, 3, 7 and 8)" << std::endl;
            std::exit(1);
    }
}

}  // namespace

int main(int argc, char **argv)
{
    Args a;
    if (argc != 11) {
        std::cerr << "Wrong usage." << std::endl;
        std::cerr << "<bits_per_value> <rows> <cols> <warmup> <timing> <flush> <debug> <kernel_id> <seed> <density>" << std::endl;
        return 1;
    }
    try {
        a.bits = std::stoi(argv[1]);
        a.rows = std::stoi(argv[2]);
        a.cols = std::stoi(argv[3]);
        a.warmup = std::stoi(argv[4]);
        a.timing = std::stoi(argv[5]);
        a.flush = std::stoi(argv[6]);
        a.debug = std::stoi(argv[7]);
        a.kernel_id = std::stoi(argv[8]);
        a.seed = std::stoi(argv[9]);
        a.density = std::stof(argv[10]);
    } catch (const std::exception &e) {
        std::cerr << "Error: Invalid arguments: " << e.what() << std::endl;
        return 1;
    }
    if (a.bits != 16 && a.bits != 8) {
        std::cerr << "Only 16 and 8 bits per value are built in this library." << std::endl;
        return 1;
    }
    if ((int64_t)a.rows * a.cols >= (1LL << 31)) {
        std::cerr << "Error: Invalid arguments: rows * cols must stay below 2^31" << std::endl;
        return 1;
    }
    if (a.rows <= 0 || a.cols <= 0 || a.timing <= 0 || a.warmup < 0 || a.density < 0.f || a.density > 1.f) {
        std::cerr << "Error: Invalid arguments: sizes and repetitions must be positive, density in [0, 1]" << std::endl;
        return 1;
    }
    std::cout << "Kernel id: " << a.kernel_id << std::endl;
    std::cout << "M_rows, M_cols, density: " << a.rows << " " << a.cols << " " << a.density << std::endl;
    std::cout << "Warmup reps / timing reps: " << a.warmup << "/" << a.timing << std::endl;
    std::cout << "Seed: " << a.seed << std::endl;
    std::cout << "Flush: " << a.flush << std::endl << std::endl;

    int device = 0;
    CUDA_OK(cudaSetDevice(device));
    int l2_bytes = 0;
    CUDA_OK(cudaDeviceGetAttribute(&l2_bytes, cudaDevAttrL2CacheSize, device));
    const size_t flush_bytes = (size_t)l2_bytes * 2;
    void *flush_d = nullptr;
    CUDA_OK(cudaMalloc(&flush_d, std::max<size_t>(flush_bytes, 1)));
    std::cout << "Cache size: " << l2_bytes << std::endl;

    cublasHandle_t handle;
    CUBLAS_OK(cublasCreate(&handle));
    cudaStream_t stream;
    CUDA_OK(cudaStreamCreate(&stream));
    CUBLAS_OK(cublasSetStream(handle, stream));
    cudaEvent_t start, stop;
    CUDA_OK(cudaEventCreate(&start));
    CUDA_OK(cudaEventCreate(&stop));

    Data data(a);

    // one checked run against the fp32 GEMV
    run(a.kernel_id, data, stream, handle);
    CUDA_OK(cudaStreamSynchronize(stream));
    const bool out_half = data.last_output_is_half;
    std::vector<float> got(a.rows), ref(a.rows);
    if (out_half) {
        std::vector<__half> tmp(a.rows);
        CUDA_OK(cudaMemcpy(tmp.data(), data.y16_d, a.rows * sizeof(__half), cudaMemcpyDeviceToHost));
        for (int i = 0; i < a.rows; ++i) got[i] = __half2float(tmp[i]);
    } else {
        CUDA_OK(cudaMemcpy(got.data(), data.y32_d, a.rows * sizeof(float), cudaMemcpyDeviceToHost));
    }
    run(0, data, stream, handle);
    CUDA_OK(cudaStreamSynchronize(stream));
    CUDA_OK(cudaMemcpy(ref.data(), data.y32_d, a.rows * sizeof(float), cudaMemcpyDeviceToHost));
    float maxdiff = 0.f;
    for (int i = 0; i < a.rows; ++i) maxdiff = std::max(maxdiff, std::abs(got[i] - ref[i]));
    if (a.debug)
        for (int i = 0; i < std::min(a.rows, 16); ++i) std::cout << "y[" << i << "] " << got[i] << " ref " << ref[i] << std::endl;
    std::cout << "Max diff: " << maxdiff << std::endl;
    if (maxdiff > 0.1f) std::cout << "@@@@@@ LOOKS BIG @@@@@@@@" << std::endl;
    std::cout << std::endl;

    for (int i = 0; i < a.warmup; ++i) run(a.kernel_id, data, stream, handle);
    CUDA_OK(cudaStreamSynchronize(stream));

    // host-side cost of a launch
    const int launch_reps = 100;
    double launch_us = 0.0;
    for (int i = 0; i < launch_reps; ++i) {
        const auto t0 = std::chrono::high_resolution_clock::now();
        run(a.kernel_id, data, stream, handle);
        const auto t1 = std::chrono::high_resolution_clock::now();
        launch_us += std::chrono::duration<double, std::micro>(t1 - t0).count();
    }
    launch_us /= launch_reps;
    CUDA_OK(cudaStreamSynchronize(stream));

    std::vector<float> times_us;
    times_us.reserve(a.timing);
    float ms = 0.f;
    for (int i = 0; i < a.timing; ++i) {
        if (a.flush) {
            CUDA_OK(cudaMemset(flush_d, 0, flush_bytes));
            CUDA_OK(cudaDeviceSynchronize());
        }
        CUDA_OK(cudaEventRecord(start, stream));
        run(a.kernel_id, data, stream, handle);
        CUDA_OK(cudaEventRecord(stop, stream));
        CUDA_OK(cudaEventSynchronize(stop));
        CUDA_OK(cudaGetLastError());
        CUDA_OK(cudaEventElapsedTime(&ms, start, stop));
        times_us.push_back(ms * 1000.f);
    }
    const float t_min = *std::min_element(times_us.begin(), times_us.end());
    const float t_max = *std::max_element(times_us.begin(), times_us.end());
    double t_mean = 0.0;
    for (float t : times_us) t_mean += t;
    t_mean /= times_us.size();

    std::cout << "Kernel id: " << a.kernel_id << std::endl;
    std::cout << "Bits per value: " << a.bits << std::endl;
    std::cout << "Last time (us): " << ms * 1000.f << std::endl;
    std::cout << "Max  time (us): " << t_max << std::endl;
    std::cout << "Min  time (us): " << t_min << std::endl;
    std::cout << "Mean time (us): " << t_mean << std::endl;
    std::cout << "Mean kernel launch time (us): " << launch_us << std::endl;
    std::cout << "Dense Bandwidth best (Gbps): " << data.dense_bandwidth(t_min) << std::endl;
    std::cout << "Dense Bandwidth mean (Gbps): " << data.dense_bandwidth(t_mean) << std::endl;
    std::cout << "Compressed Bandwidth best (Gbps): " << data.compressed_bandwidth(t_min) << std::endl;
    std::cout << "Compressed Bandwidth mean (Gbps): " << data.compressed_bandwidth(t_mean) << std::endl;
    std::cout << "Dense flops best (Gflops): " << data.dense_gflops(t_min) << std::endl;
    std::cout << "Dense flops mean (Gflops): " << data.dense_gflops(t_mean) << std::endl;
    std::cout << "Sparse flops best (Gflops): " << data.sparse_gflops(t_min) << std::endl;
    std::cout << "Sparse flops mean (Gflops): " << data.sparse_gflops(t_mean) << std::endl;
    std::cout << "Effective density: " << data.effective_density() << " " << a.density << std::endl;
    std::cout << std::endl;
    std::cout << "Final results:\t" << a.bits << "\t" << a.rows << "\t" << a.cols << "\t" << a.kernel_id << "\t" << a.density
              << "\t" << (int)t_mean << "\t" << (int)data.dense_gflops(t_mean) << "\t" << (int)data.sparse_gflops(t_mean) << std::endl;
    return 0;
}
