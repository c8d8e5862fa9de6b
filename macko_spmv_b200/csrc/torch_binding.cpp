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
    // fp16 is the reference's type; bfloat16 runs the same layout through the bf16 kernel, int8 the reference's
    // int8 variant of the format (values one byte each, vectors fp16)
    TORCH_CHECK(values.dtype() == at::kHalf || values.dtype() == at::kBFloat16 || values.dtype() == at::kChar,
                "M must be torch.half");
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

// y[rows] for V[cols]. `flags`: MACKO_SPMV_MATRIX_IMMUTABLE or 0.
at::Tensor multiply_flags(const at::Tensor &values, const at::Tensor &deltas, const at::Tensor &ri,
                          int64_t rows, int64_t cols, const at::Tensor &V, uint32_t flags)
{
    check_compressed(values, deltas, ri, rows, cols);
    const bool int8 = values.dtype() == at::kChar;
    TORCH_CHECK(V.dtype() == (int8 ? at::ScalarType::Half : values.scalar_type()), "V must be torch.half");
    TORCH_CHECK(V.is_cuda() && V.device() == values.device(), "V must be on the device of M");
    TORCH_CHECK(V.is_contiguous(), "V must be contiguous");
    TORCH_CHECK(V.dim() == 1 && V.size(0) == cols, "V must have shape [M_cols]");

    const c10::cuda::CUDAGuard guard(values.device());
    at::Tensor y = at::empty({rows}, V.options());
    cudaStream_t stream = c10::cuda::getCurrentCUDAStream();
    if (int8)
        check_status(macko_spmv_int8(values.data_ptr(), deltas.data_ptr(), ri.data_ptr<int32_t>(), rows, cols,
                                     values.numel(), V.data_ptr(), y.data_ptr(), 1.0f, 0.0f, flags, stream),
                     "macko_spmv_int8");
    else if (values.dtype() == at::kBFloat16)
        check_status(macko_spmv_bf16(values.data_ptr(), deltas.data_ptr(), ri.data_ptr<int32_t>(), rows, cols,
                                     values.numel(), V.data_ptr(), y.data_ptr(), 1.0f, 0.0f, flags, stream),
                     "macko_spmv_bf16");
    else
        check_status(macko_spmv_fp16_ex(values.data_ptr(), deltas.data_ptr(), ri.data_ptr<int32_t>(), rows, cols,
                                        values.numel(), V.data_ptr(), y.data_ptr(), 1.0f, 0.0f, flags, stream),
                     "macko_spmv_fp16");
    return y;
}

at::Tensor multiply_cuda(const at::Tensor &values, const at::Tensor &deltas, const at::Tensor &ri,
                         int64_t rows, int64_t cols, const at::Tensor &V)
{
    return multiply_flags(values, deltas, ri, rows, cols, V, 0u);
}

// The same product for a matrix the caller has declared immutable (weights): the kernel may fetch matrix
// data before the previous kernel of the stream has finished.
at::Tensor multiply_frozen_cuda(const at::Tensor &values, const at::Tensor &deltas, const at::Tensor &ri,
                                int64_t rows, int64_t cols, const at::Tensor &V)
{
    return multiply_flags(values, deltas, ri, rows, cols, V, MACKO_SPMV_MATRIX_IMMUTABLE);
}

// Plan of a compressed matrix: (plan buffer on the device, int64[8] on the host =
// plan_bytes, rows, padded_count, virtual_rows, segment_elements, longest_row, split_rows, recommended).
std::tuple<at::Tensor, at::Tensor> plan_build_cuda(const at::Tensor &deltas, const at::Tensor &ri, int64_t rows,
                                                   int64_t cols, int64_t padded, int64_t segment_elements)
{
    TORCH_CHECK(deltas.is_cuda() && ri.is_cuda() && deltas.device() == ri.device(), "compressed buffers must be CUDA tensors");
    TORCH_CHECK(deltas.dtype() == at::kByte && ri.dtype() == at::kInt, "M_deltas must be uint8 and M_row_indices int32");
    TORCH_CHECK(deltas.is_contiguous() && ri.is_contiguous(), "compressed buffers must be contiguous");
    TORCH_CHECK(ri.numel() == rows + 1 && deltas.numel() * 2 == padded, "sizes are not those of a MACKO matrix");
    const int64_t bytes = macko_spmv_plan_bytes(rows, cols, padded, (int32_t)segment_elements);
    TORCH_CHECK(bytes >= 0, "macko_spmv_plan_bytes: ", macko_last_error());
    const c10::cuda::CUDAGuard guard(deltas.device());
    at::Tensor plan = at::empty({bytes}, deltas.options());
    macko_spmv_plan_info info;
    cudaStream_t stream = c10::cuda::getCurrentCUDAStream();
    check_status(macko_spmv_plan(deltas.data_ptr(), ri.data_ptr<int32_t>(), rows, cols, padded, (int32_t)segment_elements,
                                 plan.data_ptr(), bytes, &info, stream),
                 "macko_spmv_plan");
    at::Tensor meta = at::empty({8}, at::TensorOptions().dtype(at::kLong).device(at::kCPU));
    int64_t *m = meta.data_ptr<int64_t>();
    m[0] = info.plan_bytes; m[1] = info.rows; m[2] = info.padded_count; m[3] = info.virtual_rows;
    m[4] = info.segment_elements; m[5] = info.longest_row; m[6] = info.split_rows; m[7] = info.recommended;
    return std::make_tuple(plan, meta);
}

at::Tensor multiply_planned_cuda(const at::Tensor &values, const at::Tensor &deltas, const at::Tensor &ri,
                                 int64_t rows, int64_t cols, const at::Tensor &plan, int64_t virtual_rows,
                                 int64_t segment_elements, int64_t split_rows, const at::Tensor &V, bool frozen)
{
    check_compressed(values, deltas, ri, rows, cols);
    TORCH_CHECK(values.dtype() == at::kHalf && V.dtype() == at::kHalf, "the planned product is built for torch.half");
    TORCH_CHECK(V.is_cuda() && V.device() == values.device() && plan.is_cuda() && plan.device() == values.device(),
                "V and the plan must be on the device of M");
    TORCH_CHECK(V.is_contiguous() && plan.is_contiguous(), "V and the plan must be contiguous");
    TORCH_CHECK(V.dim() == 1 && V.size(0) == cols, "V must have shape [M_cols]");
    macko_spmv_plan_info info = {};
    info.plan_bytes = macko_spmv_plan_bytes(rows, cols, values.numel(), (int32_t)segment_elements);
    TORCH_CHECK(info.plan_bytes >= 0 && plan.numel() * plan.element_size() >= info.plan_bytes, "plan buffer too small for this matrix");
    info.rows = rows;
    info.padded_count = values.numel();
    info.virtual_rows = (int32_t)virtual_rows;
    info.segment_elements = (int32_t)segment_elements;
    info.split_rows = (int32_t)split_rows;
    const c10::cuda::CUDAGuard guard(values.device());
    at::Tensor y = at::empty({rows}, values.options());
    cudaStream_t stream = c10::cuda::getCurrentCUDAStream();
    check_status(macko_spmv_fp16_planned(values.data_ptr(), deltas.data_ptr(), ri.data_ptr<int32_t>(), rows, cols,
                                         values.numel(), plan.data_ptr(), &info, V.data_ptr(), y.data_ptr(), 1.0f, 0.0f,
                                         frozen ? MACKO_SPMV_MATRIX_IMMUTABLE : 0u, stream),
                 "macko_spmv_fp16_planned");
    return y;
}

// In-place y = alpha * M x + beta * y (the `reuse_value_from_c` epilogue of kernels.cuh:113-122).
void multiply_out_cuda(const at::Tensor &values, const at::Tensor &deltas, const at::Tensor &ri,
                       int64_t rows, int64_t cols, const at::Tensor &V, at::Tensor y, double alpha, double beta)
{
    check_compressed(values, deltas, ri, rows, cols);
    const bool int8 = values.dtype() == at::kChar;
    TORCH_CHECK(V.dtype() == (int8 ? at::ScalarType::Half : values.scalar_type()) && y.dtype() == V.dtype(), "V and y must be torch.half");
    TORCH_CHECK(V.is_cuda() && V.device() == values.device() && y.device() == values.device(),
                "V and y must be on the device of M");
    TORCH_CHECK(V.is_contiguous() && y.is_contiguous(), "V and y must be contiguous");
    TORCH_CHECK(V.dim() == 1 && V.size(0) == cols && y.dim() == 1 && y.size(0) == rows, "bad vector shapes");
    const c10::cuda::CUDAGuard guard(values.device());
    cudaStream_t stream = c10::cuda::getCurrentCUDAStream();
    if (int8)
        check_status(macko_spmv_int8(values.data_ptr(), deltas.data_ptr(), ri.data_ptr<int32_t>(), rows, cols,
                                     values.numel(), V.data_ptr(), y.data_ptr(), (float)alpha, (float)beta, 0u, stream),
                     "macko_spmv_int8");
    else if (values.dtype() == at::kBFloat16)
        check_status(macko_spmv_bf16(values.data_ptr(), deltas.data_ptr(), ri.data_ptr<int32_t>(), rows, cols,
                                     values.numel(), V.data_ptr(), y.data_ptr(), (float)alpha, (float)beta, 0u, stream),
                     "macko_spmv_bf16");
    else
        check_status(macko_spmv_fp16(values.data_ptr(), deltas.data_ptr(), ri.data_ptr<int32_t>(), rows, cols,
                                     values.numel(), V.data_ptr(), y.data_ptr(), (float)alpha, (float)beta, stream),
                     "macko_spmv_fp16");
}

// multiply_out with flag bits (MACKO_SPMV_MATRIX_IMMUTABLE): the product into a caller-owned y.
void multiply_ex_cuda(const at::Tensor &values, const at::Tensor &deltas, const at::Tensor &ri,
                      int64_t rows, int64_t cols, const at::Tensor &V, at::Tensor y, double alpha, double beta, int64_t flags)
{
    check_compressed(values, deltas, ri, rows, cols);
    const bool int8 = values.dtype() == at::kChar;
    TORCH_CHECK(V.dtype() == (int8 ? at::ScalarType::Half : values.scalar_type()) && y.dtype() == V.dtype(), "V and y must be torch.half");
    TORCH_CHECK(V.is_cuda() && V.device() == values.device() && y.device() == values.device(),
                "V and y must be on the device of M");
    TORCH_CHECK(V.is_contiguous() && y.is_contiguous(), "V and y must be contiguous");
    TORCH_CHECK(V.dim() == 1 && V.size(0) == cols && y.dim() == 1 && y.size(0) == rows, "bad vector shapes");
    const c10::cuda::CUDAGuard guard(values.device());
    cudaStream_t stream = c10::cuda::getCurrentCUDAStream();
    if (int8)
        check_status(macko_spmv_int8(values.data_ptr(), deltas.data_ptr(), ri.data_ptr<int32_t>(), rows, cols,
                                     values.numel(), V.data_ptr(), y.data_ptr(), (float)alpha, (float)beta, (uint32_t)flags, stream),
                     "macko_spmv_int8");
    else if (values.dtype() == at::kBFloat16)
        check_status(macko_spmv_bf16(values.data_ptr(), deltas.data_ptr(), ri.data_ptr<int32_t>(), rows, cols,
                                     values.numel(), V.data_ptr(), y.data_ptr(), (float)alpha, (float)beta, (uint32_t)flags, stream),
                     "macko_spmv_bf16");
    else
        check_status(macko_spmv_fp16_ex(values.data_ptr(), deltas.data_ptr(), ri.data_ptr<int32_t>(), rows, cols,
                                        values.numel(), V.data_ptr(), y.data_ptr(), (float)alpha, (float)beta, (uint32_t)flags, stream),
                     "macko_spmv_fp16_ex");
}

// Y[batch, rows] for V[batch, cols]: up to 8 vectors per pass over the compressed matrix.
at::Tensor multiply_batched_cuda(const at::Tensor &values, const at::Tensor &deltas, const at::Tensor &ri,
                                 int64_t rows, int64_t cols, const at::Tensor &V)
{
    check_compressed(values, deltas, ri, rows, cols);
    TORCH_CHECK(values.dtype() == at::kHalf && V.dtype() == at::kHalf, "M and V must be torch.half");
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
    TORCH_CHECK(values.dtype() != at::kChar, "decompress is built for 16-bit values");
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
    TORCH_CHECK(M.dtype() == at::kHalf || M.dtype() == at::kBFloat16 || M.dtype() == at::kChar, "M must be torch.half");
    TORCH_CHECK(M.dim() == 2, "M must be a matrix");
    TORCH_CHECK(M.is_contiguous(), "M must be contiguous");
    const int64_t rows = M.size(0), cols = M.size(1);

    const c10::cuda::CUDAGuard guard(M.device());
    cudaStream_t stream = c10::cuda::getCurrentCUDAStream();
    at::Tensor ri = at::empty({rows + 1}, M.options().dtype(at::kInt));
    const bool int8 = M.dtype() == at::kChar;
    if (int8)
        check_status(macko_compress_count_int8(M.data_ptr(), rows, cols, ri.data_ptr<int32_t>(), stream),
                     "macko_compress_count_int8");
    else
        check_status(macko_compress_count(M.data_ptr(), rows, cols, ri.data_ptr<int32_t>(), stream),
                     "macko_compress_count");
    const int64_t n = ri[rows].item<int32_t>();  // the one device->host read that sizes the outputs
    const int64_t padded = (n + 7) / 8 * 8;
    at::Tensor values = at::empty({padded}, M.options());
    at::Tensor deltas = at::empty({padded / 2}, M.options().dtype(at::kByte));
    const int64_t ws_bytes = macko_compress_workspace_bytes(padded);
    at::Tensor ws = at::empty({ws_bytes}, M.options().dtype(at::kByte));
    if (int8)
        check_status(macko_compress_emit_int8(M.data_ptr(), rows, cols, ri.data_ptr<int32_t>(), padded,
                                              values.data_ptr(), deltas.data_ptr(), ws.data_ptr(), ws_bytes, stream),
                     "macko_compress_emit_int8");
    else if (M.dtype() == at::kBFloat16)
        check_status(macko_compress_emit_bf16(M.data_ptr(), rows, cols, ri.data_ptr<int32_t>(), padded,
                                              values.data_ptr(), deltas.data_ptr(), ws.data_ptr(), ws_bytes, stream),
                     "macko_compress_emit_bf16");
    else
        check_status(macko_compress_emit(M.data_ptr(), rows, cols, ri.data_ptr<int32_t>(), padded,
                                         values.data_ptr(), deltas.data_ptr(), ws.data_ptr(), ws_bytes, stream),
                     "macko_compress_emit");
    return std::make_tuple(values, deltas, ri);
}

// ---- decode helpers (macko_decode_*): the steps between the products of a batch-1 decode step ------------

void check_half_vec(const at::Tensor &t, const char *name)
{
    TORCH_CHECK(t.is_cuda() && t.dtype() == at::kHalf && t.is_contiguous(), name, " must be a contiguous CUDA fp16 tensor");
}

at::Tensor add_rmsnorm_impl(at::Tensor x, const at::Tensor &pending, const at::Tensor &weight, double eps,
                            int64_t flags_address, int64_t world, int64_t spin_limit);

// x[n] += rows of pending[k, n] (k may be 0); returns rmsnorm(x) * weight
at::Tensor add_rmsnorm_cuda(at::Tensor x, const at::Tensor &pending, const at::Tensor &weight, double eps)
{
    return add_rmsnorm_impl(x, pending, weight, eps, 0, 0, 0);
}

// The same with the bounded wait for the other ranks' slices of `pending` inside the kernel; `flags_address` is the
// device address of this rank's flag words (sharded.PeerGather keeps it).
at::Tensor add_rmsnorm_peer_cuda(at::Tensor x, const at::Tensor &pending, const at::Tensor &weight, double eps,
                                 int64_t flags_address, int64_t world, int64_t spin_limit)
{
    TORCH_CHECK(flags_address != 0 && world >= 1, "add_rmsnorm_peer needs the flag words of the exchange");
    return add_rmsnorm_impl(x, pending, weight, eps, flags_address, world, spin_limit);
}

at::Tensor add_rmsnorm_impl(at::Tensor x, const at::Tensor &pending, const at::Tensor &weight, double eps,
                            int64_t flags_address, int64_t world, int64_t spin_limit)
{
    check_half_vec(x, "x");
    check_half_vec(weight, "weight");
    check_half_vec(pending, "pending");
    TORCH_CHECK(x.dim() == 1 && weight.dim() == 1 && weight.size(0) == x.size(0), "x and weight must be vectors of one length");
    TORCH_CHECK(pending.dim() == 2 && (pending.size(0) == 0 || pending.size(1) == x.size(0)), "pending must be [k, n]");
    TORCH_CHECK(pending.device() == x.device() && weight.device() == x.device(), "tensors on different devices");
    const c10::cuda::CUDAGuard guard(x.device());
    at::Tensor out = at::empty_like(x);
    const int k = (int)pending.size(0);
    if (flags_address != 0)
        check_status(macko_decode_add_rmsnorm_peer(x.data_ptr(), k ? pending.data_ptr() : nullptr, k, x.size(0), weight.data_ptr(),
                                                   out.data_ptr(), x.size(0), (float)eps,
                                                   reinterpret_cast<uint32_t *>(static_cast<uintptr_t>(flags_address)), (int)world,
                                                   (uint32_t)spin_limit, c10::cuda::getCurrentCUDAStream()),
                     "macko_decode_add_rmsnorm_peer");
    else
        check_status(macko_decode_add_rmsnorm(x.data_ptr(), k ? pending.data_ptr() : nullptr, k, x.size(0), weight.data_ptr(),
                                              out.data_ptr(), x.size(0), (float)eps, c10::cuda::getCurrentCUDAStream()),
                     "macko_decode_add_rmsnorm");
    return out;
}

at::Tensor rope_attention_cuda(const at::Tensor &qkv, const at::Tensor &cos_table, const at::Tensor &sin_table,
                               const at::Tensor &position, at::Tensor k_cache, at::Tensor v_cache)
{
    check_half_vec(qkv, "qkv");
    check_half_vec(cos_table, "cos_table");
    check_half_vec(sin_table, "sin_table");
    check_half_vec(k_cache, "k_cache");
    check_half_vec(v_cache, "v_cache");
    TORCH_CHECK(position.is_cuda() && position.dtype() == at::kLong && position.numel() == 1, "position must be one int64 on the device");
    TORCH_CHECK(k_cache.dim() >= 3 && k_cache.sizes() == v_cache.sizes(), "caches must be [..., heads, max_len, head_dim]");
    const int64_t hd = k_cache.size(-1), max_len = k_cache.size(-2), heads = k_cache.numel() / (hd * max_len);
    TORCH_CHECK(qkv.numel() == 3 * heads * hd, "qkv must hold q, k and v of ", heads, " heads");
    TORCH_CHECK(cos_table.dim() == 2 && cos_table.size(1) == hd && cos_table.size(0) >= max_len && sin_table.sizes() == cos_table.sizes(),
                "cos/sin tables must be [>= max_len, head_dim]");
    const c10::cuda::CUDAGuard guard(qkv.device());
    at::Tensor out = at::empty({heads * hd}, qkv.options());
    check_status(macko_decode_rope_attention(qkv.data_ptr(), cos_table.data_ptr(), sin_table.data_ptr(),
                                             position.data_ptr<int64_t>(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
                                             (int)heads, (int)hd, (int)max_len, c10::cuda::getCurrentCUDAStream()),
                 "macko_decode_rope_attention");
    return out;
}

at::Tensor silu_mul_cuda(const at::Tensor &gate_up)
{
    check_half_vec(gate_up, "gate_up");
    TORCH_CHECK(gate_up.dim() == 1 && gate_up.size(0) % 2 == 0, "gate_up must be a vector of 2n elements");
    const c10::cuda::CUDAGuard guard(gate_up.device());
    const int64_t n = gate_up.size(0) / 2;
    at::Tensor out = at::empty({n}, gate_up.options());
    if (n > 0)
        check_status(macko_decode_silu_mul(gate_up.data_ptr(), out.data_ptr(), n, c10::cuda::getCurrentCUDAStream()),
                     "macko_decode_silu_mul");
    return out;
}

at::Tensor argmax_cuda(const at::Tensor &values)
{
    check_half_vec(values, "values");
    TORCH_CHECK(values.dim() == 1 && values.size(0) > 0, "values must be a non-empty vector");
    const c10::cuda::CUDAGuard guard(values.device());
    at::Tensor out = at::empty({1}, values.options().dtype(at::kLong));
    check_status(macko_decode_argmax(values.data_ptr(), values.size(0), out.data_ptr<int64_t>(), c10::cuda::getCurrentCUDAStream()),
                 "macko_decode_argmax");
    return out;
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
    m.def("multiply_ex(Tensor M_values, Tensor M_deltas, Tensor M_row_indices, int M_rows, int M_cols, Tensor V, "
          "Tensor(a!) y, float alpha, float beta, int flags) -> ()");
    m.def("multiply_frozen(Tensor M_values, Tensor M_deltas, Tensor M_row_indices, int M_rows, int M_cols, Tensor V) -> Tensor");
    m.def("plan_build(Tensor M_deltas, Tensor M_row_indices, int M_rows, int M_cols, int padded_count, int segment_elements) -> (Tensor, Tensor)");
    m.def("multiply_planned(Tensor M_values, Tensor M_deltas, Tensor M_row_indices, int M_rows, int M_cols, Tensor plan, "
          "int virtual_rows, int segment_elements, int split_rows, Tensor V, bool frozen) -> Tensor");
    m.def("add_rmsnorm(Tensor(a!) x, Tensor pending, Tensor weight, float eps) -> Tensor");
    m.def("add_rmsnorm_peer(Tensor(a!) x, Tensor pending, Tensor weight, float eps, int flags_address, int world, "
          "int spin_limit) -> Tensor");
    m.def("rope_attention(Tensor qkv, Tensor cos_table, Tensor sin_table, Tensor position, Tensor(a!) k_cache, "
          "Tensor(b!) v_cache) -> Tensor");
    m.def("silu_mul(Tensor gate_up) -> Tensor");
    m.def("argmax(Tensor values) -> Tensor");
}

TORCH_LIBRARY_IMPL(macko_spmv, CUDA, m)
{
    m.impl("multiply", &multiply_cuda);
    m.impl("multiply_out", &multiply_out_cuda);
    m.impl("compress_dense", &compress_cuda);
    m.impl("multiply_batched", &multiply_batched_cuda);
    m.impl("decompress", &decompress_cuda);
    m.impl("multiply_ex", &multiply_ex_cuda);
    m.impl("multiply_frozen", &multiply_frozen_cuda);
    m.impl("plan_build", &plan_build_cuda);
    m.impl("multiply_planned", &multiply_planned_cuda);
    m.impl("add_rmsnorm", &add_rmsnorm_cuda);
    m.impl("add_rmsnorm_peer", &add_rmsnorm_peer_cuda);
    m.impl("rope_attention", &rope_attention_cuda);
    m.impl("silu_mul", &silu_mul_cuda);
    m.impl("argmax", &argmax_cuda);
}
