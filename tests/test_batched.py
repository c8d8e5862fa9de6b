"""GPU tests of the two callers' helpers next to the single-vector product: the multi-vector product
(`multiply_batched` / `macko_spmm_fp16`) and the GPU decompressor (`decompress` / `macko_decompress_fp16`).

Every vector of a batched product must meet the bounds of the single-vector product against the oracle
    |y - y_ref| <= 1e-3 * sum_k |val_k * x[col_k]|  per row,  ||y - y_ref||_2 <= 5e-3 * ||y_ref||_2
and the decompressor must reproduce the oracle's dense matrix bit for bit."""
import numpy as np
import pytest
import torch

import oracle
import macko_spmv_b200 as macko_spmv
from macko_spmv_b200 import cabi, workloads
from macko_spmv_b200.linear import MackoLinear

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _u16(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def _comp_np(comp):
    return (_u16(comp[0]), comp[1].cpu().numpy(), comp[2].cpu().numpy(), comp[3], comp[4])


def _check_vector(y, comp_np, x_np, what):
    y64, _, l1 = oracle.spmv(comp_np, x_np)
    got = y.float().cpu().numpy().astype(np.float64)
    err = np.abs(got - y64)
    assert not (err > 1e-3 * l1 + 1e-12).any(), f"{what}: worst {float((err / (l1 + 1e-30)).max()):.3e} of L1"
    nrm = np.linalg.norm(y64)
    if nrm > 0:
        assert np.linalg.norm(got - y64) <= 5e-3 * nrm, what


@pytest.mark.parametrize("shape", [(512, 4096, 0.5), (4096, 1024, 0.1), (333, 515, 0.3), (20000, 256, 0.5), (64, 11008, 0.9)])
def test_batched_product_every_batch_size(shape):
    rows, cols, d = shape
    M = workloads.bernoulli_matrix(rows, cols, d, seed=rows + cols, device=DEV)
    comp = macko_spmv.compress(M)
    cnp = _comp_np(comp)
    g = torch.Generator(device=DEV).manual_seed(7)
    for batch in (1, 2, 3, 4, 5, 7, 8, 9, 16, 17):
        V = torch.randn(batch, cols, generator=g, device=DEV).half()
        Y = macko_spmv.multiply_batched(comp, V)
        assert Y.shape == (batch, rows) and Y.dtype == torch.float16
        for b in (0, batch // 2, batch - 1):
            _check_vector(Y[b], cnp, _u16(V[b]), f"{shape} batch {batch} vector {b}")
        # and against the single-vector product of the same library
        single = torch.stack([macko_spmv.multiply(comp, V[b].contiguous()) for b in range(batch)])
        assert torch.allclose(Y.float(), single.float(), rtol=2e-3, atol=2e-3 * float(single.float().abs().max()))
        if 8 < batch <= macko_spmv.DENSE_BATCH_THRESHOLD:
            # 9..16 vectors: the API picks two passes of the kernel or the dense copy by density; the kernel itself
            Yk = torch.ops.macko_spmv.multiply_batched.default(*comp[:5], V)
            assert torch.allclose(Yk.float(), single.float(), rtol=2e-3, atol=2e-3 * float(single.float().abs().max()))


def test_batched_product_edge_cases():
    lib = cabi.load()
    stream = torch.cuda.current_stream().cuda_stream
    # empty rows, rows that start in the middle of an 8-element unit, one very long row, empty matrix
    M = torch.zeros(70, 3000, dtype=torch.float16, device=DEV)
    M[3, ::7] = 1.5
    M[4, 5] = -2.0
    M[9] = 0.25
    M[69, 2999] = 3.0
    comp = macko_spmv.compress(M)
    V = workloads.dense_vector(3 * 3000, 5, DEV).view(3, 3000).contiguous()
    Y = macko_spmv.multiply_batched(comp, V)
    ref = V.float() @ M.float().t()
    assert torch.allclose(Y.float(), ref, rtol=2e-3, atol=2e-2)
    # alpha / beta through the C ABI
    Y2 = torch.ones(3, 70, dtype=torch.float16, device=DEV)
    cabi.check(lib, lib.macko_spmm_fp16(comp[0].data_ptr(), comp[1].data_ptr(), comp[2].data_ptr(), 70, 3000,
                                        comp[0].numel(), V.data_ptr(), Y2.data_ptr(), 3, 2.0, -1.0, stream))
    assert torch.allclose(Y2.float(), 2.0 * ref - 1.0, rtol=2e-3, atol=4e-2)
    # zero vectors, zero rows
    assert macko_spmv.multiply_batched(comp, V[:0].contiguous()).shape == (0, 70)
    empty = macko_spmv.compress(torch.zeros(0, 64, dtype=torch.float16, device=DEV))
    assert macko_spmv.multiply_batched(empty, V[:, :64].contiguous()).shape == (3, 0)
    assert lib.macko_spmm_fp16(comp[0].data_ptr(), comp[1].data_ptr(), comp[2].data_ptr(), 70, 3000,
                               comp[0].numel(), V.data_ptr(), Y2.data_ptr(), -1, 1.0, 0.0, stream) == cabi.ERR_INVALID_ARGUMENT
    with pytest.raises(RuntimeError):
        macko_spmv.multiply_batched(comp, V[:, :100].contiguous())


def test_batched_product_wide_matrix_uses_fewer_vectors_per_pass():
    # 8 interleaved copies of a 20000-column x do not fit shared memory: the library drops to 4 per pass
    rows, cols = 300, 20000
    M = workloads.bernoulli_matrix(rows, cols, 0.2, seed=3, device=DEV)
    comp = macko_spmv.compress(M)
    V = workloads.dense_vector(8 * cols, 11, DEV).view(8, cols).contiguous()
    Y = macko_spmv.multiply_batched(comp, V)
    cnp = _comp_np(comp)
    for b in (0, 5, 7):
        _check_vector(Y[b], cnp, _u16(V[b]), f"wide vector {b}")


def test_large_batch_goes_through_dense_copy():
    rows, cols = 1024, 2048
    M = workloads.magnitude_pruned_matrix(rows, cols, 0.5, seed=21, device=DEV)
    comp = macko_spmv.compress(M)
    V = workloads.dense_vector(64 * cols, 12, DEV).view(64, cols).contiguous()
    assert V.shape[0] > macko_spmv.DENSE_BATCH_THRESHOLD
    Y = macko_spmv.multiply_batched(comp, V)
    ref = V.float() @ M.float().t()
    assert float((Y.float() - ref).norm() / ref.norm()) < 5e-3


@pytest.mark.parametrize("shape", [(257, 1000, 0.3), (64, 4096, 0.02), (1000, 33, 0.5), (5, 40000, 0.001), (300, 4099, 0.9), (40, 11008, 0.5),
                                   (3, 130000, 0.01)])
def test_decompress_bit_exact_against_oracle(shape):
    # rows of up to about 116 000 columns are assembled whole in shared memory by one CTA (several passes of 2048
    # stored elements for the dense 4099-column case); wider rows take the warp-per-row kernel with a window
    rows, cols, d = shape
    M = workloads.bernoulli_matrix(rows, cols, d, seed=rows * 3 + cols, device=DEV)
    M[0] = 0                                  # an empty row
    M[1, : min(cols, 40)] = -0.0               # negative zeros: dropped or stored as pads; both decode to +0
    M[2, cols - 1] = float("nan")
    comp = macko_spmv.compress(M)
    dense = macko_spmv.decompress(comp)
    exp = oracle.decompress(_comp_np(comp))
    assert np.array_equal(_u16(dense), exp)
    # round trip: equal to the source except that dropped negative zeros come back positive and NaNs are canonical
    src = _u16(M)
    back = _u16(dense)
    differ = src != back
    is_nan = (src & 0x7fff) > 0x7c00
    assert np.all((src[differ] == 0x8000) | is_nan[differ])
    assert np.all(back[is_nan] == 0x7fff)


def test_decompress_full_size_round_trip():
    M = workloads.magnitude_pruned_matrix(11008, 4096, 0.5, seed=2012, device=DEV)
    comp = macko_spmv.compress(M)
    dense = macko_spmv.decompress(comp)
    assert torch.equal(dense, M)                       # as numbers: the -0.0 the pruning left behind come back as +0
    assert not bool((dense.view(torch.int16) == -32768).any())
    again = macko_spmv.compress(dense)
    assert torch.equal(again[0], comp[0]) and torch.equal(again[1], comp[1]) and torch.equal(again[2], comp[2])


def test_linear_layer_routes_batches():
    W = workloads.magnitude_pruned_matrix(768, 1024, 0.4, seed=31, device=DEV)
    layer = MackoLinear(macko_spmv.compress(W), bias=torch.full((768,), 0.5, dtype=torch.float16, device=DEV))
    g = torch.Generator(device=DEV).manual_seed(1)
    for lead in ((), (1,), (3,), (2, 4), (40,)):
        x = torch.randn(*lead, 1024, generator=g, device=DEV).half()
        y = layer(x)
        ref = x.float() @ W.float().t() + 0.5
        assert y.shape == (*lead, 768)
        assert float((y.float() - ref).norm() / ref.norm()) < 5e-3
