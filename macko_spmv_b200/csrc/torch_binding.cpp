// PyTorch operator boundary of the sm_100a MACKO library.
//
// Registers `macko_spmv::multiply` with the schema of the reference
// (src/macko_spmv/__init__.py:56-63) and a CUDA implementation that forwards to the C ABI
// (macko_spmv_fp16) instead of a JIT-compiled kernel; mirrors the argument checks of
// `macko_spmv_launcher` (src/macko_spmv/cuda/kernels_torch_launchers.cuh:3-48) and of
// `cpu_compress` (src/macko_spmv/cuda/cpu_compressor_torch_launcher.cuh:6-39).
// Everything is allocated through the caching allocator and enqueued on the current stream,
// so the op can be captured in CUDA graphs.
#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <tuple>

#include "macko_b200.h"

namespace {

void check_status(int status, const char *what)
{
    TORCH_CHECK(status == MACKO_OK, what, ": ", macko_status_string(status), " (", macko_last_error(), ")");
}

void check_compressed(const at::Tensor &values, const at::Tensor &deltas, const at::Tensor &ri,
                      int64_t rows, int64_t cols)
{
    TORCH_CHECK(values.dtype() == at::kHalf, "M must be torch.half");
    TORCH_CHECK(deltas.dtype() == at::kByte, "M_deltas must be torch.uint8");
    TORCH_CHECK(ri.dtype() == at::kInt, "M_row_indices must be torch.int32");
    TORCH_CHECK(values.is_cuda() && deltas.is_cuda() && ri.is_cuda(), "compressed buffers must be CUDA tensors");
    TORCH_CHECK(values.device() == deltas.device() && values.device() == ri.device(),
                "compressed buffers must live on one device");
    TORCH_CHECK(values.is_contiguous() && deltas.is_contiguous() && ri.is_contiguous(),
                "compressed buffers must be contiguous");
    TORCH_CHECK(rows >= 0 && cols >= 0, "negative matrix shape");
    TORCH_CHECK(ri.numel() == rows + 1, "M_row_indices must have M_rows + 1 entries");
    TORCH_CHECK(values.numel() % 8 == 0 && deltas.numel() * 2 == values.numel(),
                "values / deltas sizes are not a MACKO pair");
}

// y[..., rows] for V[..., cols]; one SpMV per leading index.
at::Tensor multiply_cuda(const at::Tensor &values, const at::Tensor &deltas, const at::Tensor &ri,
                         int64_t rows, int64_t cols, const at::Tensor &V)
{
    check_compressed(values, deltas, ri, rows, cols);
    TORCH_CHECK(V.dtype() == at::kHalf, "V must be torch.half");
    TORCH_CHECK(V.is_cuda() && V.device() == values.device(), "V must be on the device of M");
    TORCH_CHECK(V.is_contiguous(), "V must be contiguous");
    TORCH_CHECK(V.dim() == 1 && V.size(0) == cols, "V must have shape [M_cols]");

    const c10::cuda::CUDAGuard guard(values.device());
    at::Tensor y = at::empty({rows}, values.options());
    cudaStream_t stream = c10::cuda::getCurrentCUDAStream();
    check_status(macko_spmv_fp16(values.data_ptr(), deltas.data_ptr(), ri.data_ptr<int32_t>(), rows, cols,
                                 values.numel(), V.data_ptr(), y.data_ptr(), 1.0f, 0.0f, stream),
                 "macko_spmv_fp16");
    return y;
}

// In-place y = alpha * M x + beta * y (the `reuse_value_from_c` epilogue of kernels.cuh:113-122).
void multiply_out_cuda(const at::Tensor &values, const at::Tensor &deltas, const at::Tensor &ri,
                       int64_t rows, int64_t cols, const at::Tensor &V, at::Tensor y, double alpha, double beta)
{
    check_compressed(values, deltas, ri, rows, cols);
    TORCH_CHECK(V.dtype() == at::kHalf && y.dtype() == at::kHalf, "V and y must be torch.half");
    TORCH_CHECK(V.is_cuda() && V.device() == values.device() && y.device() == values.device(),
                "V and y must be on the device of M");
    TORCH_CHECK(V.is_contiguous() && y.is_contiguous(), "V and y must be contiguous");
    TORCH_CHECK(V.dim() == 1 && V.size(0) == cols && y.dim() == 1 && y.size(0) == rows, "bad vector shapes");
    const c10::cuda::CUDAGuard guard(values.device());
    cudaStream_t stream = c10::cuda::getCurrentCUDAStream();
    check_status(macko_spmv_fp16(values.data_ptr(), deltas.data_ptr(), ri.data_ptr<int32_t>(), rows, cols,
                                 values.numel(), V.data_ptr(), y.data_ptr(), (float)alpha, (float)beta, stream),
                 "macko_spmv_fp16");
}

// Y[batch, rows] for V[batch, cols]: up to 8 vectors per pass over the compressed matrix.
at::Tensor multiply_batched_cuda(const at::Tensor &values, const at::Tensor &deltas, const at::Tensor &ri,
                                 int64_t rows, int64_t cols, const at::Tensor &V)
{
    check_compressed(values, deltas, ri, rows, cols);
    TORCH_CHECK(V.dtype() == at::kHalf, "V must be torch.half");
    TORCH_CHECK(V.is_cuda() && V.device() == values.device(), "V must be on the device of M");
    TORCH_CHECK(V.is_contiguous(), "V must be contiguous");
    TORCH_CHECK(V.dim() == 2 && V.size(1) == cols, "V must have shape [batch, M_cols]");
    const c10::cuda::CUDAGuard guard(values.device());
    at::Tensor y = at::empty({V.size(0), rows}, values.options());
    cudaStream_t stream = c10::cuda::getCurrentCUDAStream();
    check_status(macko_spmm_fp16(values.data_ptr(), deltas.data_ptr(), ri.data_ptr<int32_t>(), rows, cols,
                                 values.numel(), V.data_ptr(), y.data_ptr(), V.size(0), 1.0f, 0.0f, stream),
                 "macko_spmm_fp16");
    return y;
}

at::Tensor decompress_cuda(const at::Tensor &values, const at::Tensor &deltas, const at::Tensor &ri,
                           int64_t rows, int64_t cols)
{
    check_compressed(values, deltas, ri, rows, cols);
    const c10::cuda::CUDAGuard guard(values.device());
    at::Tensor dense = at::empty({rows, cols}, values.options());
    cudaStream_t stream = c10::cuda::getCurrentCUDAStream();
    check_status(macko_decompress_fp16(values.data_ptr(), deltas.data_ptr(), ri.data_ptr<int32_t>(), rows, cols,
                                       values.numel(), dense.data_ptr(), stream),
                 "macko_decompress_fp16");
    return dense;
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> compress_cuda(const at::Tensor &M)
{
    TORCH_CHECK(M.is_cuda(), "M must be a CUDA tensor");
    TORCH_CHECK(M.dtype() == at::kHalf, "M must be torch.half");
    TORCH_CHECK(M.dim() == 2, "M must be a matrix");
    TORCH_CHECK(M.is_contiguous(), "M must be contiguous");
    const int64_t rows = M.size(0), cols = M.size(1);

    const c10::cuda::CUDAGuard guard(M.device());
    cudaStream_t stream = c10::cuda::getCurrentCUDAStream();
    at::Tensor ri = at::empty({rows + 1}, M.options().dtype(at::kInt));
    check_status(macko_compress_count(M.data_ptr(), rows, cols, ri.data_ptr<int32_t>(), stream),
                 "macko_compress_count");
    const int64_t n = ri[rows].item<int32_t>();  // the one device->host read that sizes the outputs
    const int64_t padded = (n + 7) / 8 * 8;
    at::Tensor values = at::empty({padded}, M.options());
    at::Tensor deltas = at::empty({padded / 2}, M.options().dtype(at::kByte));
    const int64_t ws_bytes = macko_compress_workspace_bytes(padded);
    at::Tensor ws = at::empty({ws_bytes}, M.options().dtype(at::kByte));
    check_status(macko_compress_emit(M.data_ptr(), rows, cols, ri.data_ptr<int32_t>(), padded,
                                     values.data_ptr(), deltas.data_ptr(), ws.data_ptr(), ws_bytes, stream),
                 "macko_compress_emit");
    return std::make_tuple(values, deltas, ri);
}

}  // namespace

TORCH_LIBRARY(macko_spmv, m)
{
    m.def("multiply(Tensor M_values, Tensor M_deltas, Tensor M_row_indices, int M_rows, int M_cols, Tensor V) -> Tensor");
    m.def("multiply_out(Tensor M_values, Tensor M_deltas, Tensor M_row_indices, int M_rows, int M_cols, Tensor V, "
          "Tensor(a!) y, float alpha, float beta) -> ()");
    m.def("compress_dense(Tensor M) -> (Tensor, Tensor, Tensor)");
    m.def("multiply_batched(Tensor M_values, Tensor M_deltas, Tensor M_row_indices, int M_rows, int M_cols, Tensor V) -> Tensor");
    m.def("decompress(Tensor M_values, Tensor M_deltas, Tensor M_row_indices, int M_rows, int M_cols) -> Tensor");
}

TORCH_LIBRARY_IMPL(macko_spmv, CUDA, m)
{
    m.impl("multiply", &multiply_cuda);
    m.impl("multiply_out", &multiply_out_cuda);
    m.impl("compress_dense", &compress_cuda);
    m.impl("multiply_batched", &multiply_batched_cuda);
    m.impl("decompress", &decompress_cuda);
}
