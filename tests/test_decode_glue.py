"""The three kernels that run between the products of a decode step (residual add + RMSNorm, rotary embedding +
KV-cache append + attention, SwiGLU gate) against the same steps in plain PyTorch fp32, and the decode loop that
uses them against the one built from PyTorch operators."""
import math

import pytest
import torch

import macko_spmv_b200  # noqa: F401  (registers torch.ops.macko_spmv)

pytestmark = pytest.mark.gpu
ops = torch.ops.macko_spmv


def _gen(seed):
    return torch.Generator(device="cuda").manual_seed(seed)


@pytest.mark.parametrize("n,k", [(4096, 0), (4096, 1), (4096, 4), (256, 2), (250, 1), (11008, 3), (8, 1)])
def test_add_rmsnorm(n, k):
    g = _gen(n + k)
    x = torch.randn(n, device="cuda", generator=g).half()
    pending = (0.5 * torch.randn(k, n, device="cuda", generator=g)).half()
    w = (1.0 + 0.1 * torch.randn(n, device="cuda", generator=g)).half()
    x_ref = x.float()
    for p in range(k):
        x_ref = x_ref + pending[p].float()
    x_ref = x_ref.half()                     # the residual stream is fp16: one rounding after the fp32 sum
    xf = x_ref.float()
    out_ref = xf * torch.rsqrt(xf.pow(2).mean() + 1e-5) * w.float()
    x_run = x.clone()
    out = ops.add_rmsnorm(x_run, pending, w, 1e-5)
    assert torch.equal(x_run, x_ref)
    assert out.dtype == torch.float16 and out.shape == (n,)
    # fp32 arithmetic, one rounding: within one fp16 unit in the last place of the reference
    assert torch.allclose(out.float(), out_ref, rtol=2e-3, atol=1e-4)


@pytest.mark.parametrize("n", [11008, 5504, 688, 37, 8])
def test_silu_mul(n):
    gu = torch.randn(2 * n, device="cuda", generator=_gen(n)).mul(3).half()
    ref = torch.nn.functional.silu(gu[:n].float()) * gu[n:].float()
    out = ops.silu_mul(gu)
    assert out.shape == (n,)
    assert torch.allclose(out.float(), ref, rtol=2e-3, atol=1e-4)


def _rope_ref(t, cos, sin):
    half = t.shape[-1] // 2
    rot = torch.cat((-t[..., half:], t[..., :half]), dim=-1)
    return t * cos + rot * sin


@pytest.mark.parametrize("heads,head_dim,max_len", [(32, 128, 80), (4, 64, 48), (2, 256, 20), (8, 128, 300), (40, 128, 40), (160, 64, 24)])
def test_rope_attention(heads, head_dim, max_len):
    g = _gen(heads * head_dim)
    half = head_dim // 2
    inv = 1.0 / (10000.0 ** (torch.arange(half, device="cuda", dtype=torch.float32) / half))
    ang = torch.arange(max_len, device="cuda", dtype=torch.float32)[:, None] * inv[None, :]
    ang = torch.cat((ang, ang), dim=-1)
    cos_t, sin_t = ang.cos().half(), ang.sin().half()
    k_cache = torch.zeros(1, heads, max_len, head_dim, dtype=torch.float16, device="cuda")
    v_cache = torch.zeros_like(k_cache)
    k_ref = torch.zeros(heads, max_len, head_dim, device="cuda")
    v_ref = torch.zeros_like(k_ref)
    steps = list(range(min(max_len, 19))) + ([max_len - 1] if max_len > 19 else [])
    for pos in steps:
        if pos == max_len - 1 and max_len > 19:
            # fill the rows in between, in both caches, so that the last position attends over a long, full cache
            fill = torch.randn(heads, max_len, head_dim, device="cuda", generator=g).half()
            k_cache[0, :, 19:pos] = fill[:, 19:pos]
            v_cache[0, :, 19:pos] = fill.flip(1)[:, 19:pos]
            k_ref[:, 19:pos] = fill[:, 19:pos].float()
            v_ref[:, 19:pos] = fill.flip(1)[:, 19:pos].float()
        qkv = torch.randn(3, heads, head_dim, device="cuda", generator=g).half()
        position = torch.tensor([pos], device="cuda")
        out = ops.rope_attention(qkv, cos_t, sin_t, position, k_cache, v_cache)
        q = _rope_ref(qkv[0].float(), cos_t[pos].float(), sin_t[pos].float()).half().float()
        k = _rope_ref(qkv[1].float(), cos_t[pos].float(), sin_t[pos].float()).half().float()
        k_ref[:, pos] = k
        v_ref[:, pos] = qkv[2].float()
        assert torch.equal(v_cache[0, :, pos], qkv[2])
        assert torch.allclose(k_cache[0, :, pos].float(), k, rtol=1e-3, atol=1e-3)
        scores = torch.einsum("hd,htd->ht", q, k_ref[:, : pos + 1]) / math.sqrt(head_dim)
        ref = torch.einsum("ht,htd->hd", torch.softmax(scores, dim=-1), v_ref[:, : pos + 1])
        assert out.shape == (heads * head_dim,)
        err = (out.float().view(heads, head_dim) - ref).abs().max().item()
        assert err < 4e-3 * max(1.0, ref.abs().max().item()), (pos, err)


def test_rope_attention_clamps_a_position_outside_the_cache():
    heads, head_dim, max_len = 2, 64, 8
    cos_t = torch.ones(max_len, head_dim, dtype=torch.float16, device="cuda")
    sin_t = torch.zeros_like(cos_t)
    k_cache = torch.zeros(heads, max_len, head_dim, dtype=torch.float16, device="cuda")
    v_cache = torch.zeros_like(k_cache)
    guard = torch.full((4096,), 7.0, dtype=torch.float16, device="cuda")   # a neighbouring allocation must stay untouched
    qkv = torch.randn(3, heads, head_dim, device="cuda", generator=_gen(3)).half()
    out = ops.rope_attention(qkv, cos_t, sin_t, torch.tensor([1000], device="cuda"), k_cache, v_cache)
    torch.cuda.synchronize()
    assert torch.equal(v_cache[:, max_len - 1], qkv[2]) and bool((guard == 7.0).all())
    assert torch.isfinite(out.float()).all()


def test_fused_decode_step_matches_the_pytorch_step():
    from macko_spmv_b200 import llama_decode

    cfg = dict(hidden=256, heads=4, ffn=512, vocab=1000, layers=3, eps=1e-5, rope_theta=10000.0)
    with torch.no_grad():
        for density in (0.5, 1.0):
            a = llama_decode.LlamaDecoder(density, cfg=cfg, max_len=32, seed=21, fused_glue=True)
            b = llama_decode.LlamaDecoder(density, cfg=cfg, max_len=32, seed=21, fused_glue=False)
            for i, tok in enumerate([3, 999, 17, 0, 512, 44, 8, 250, 77, 1]):
                token, pos = torch.tensor([tok], device="cuda"), torch.tensor([i], device="cuda")
                la, lb = a.logits(token, pos).float(), b.logits(token, pos).float()
                assert float((la - lb).norm() / lb.norm()) < 1e-2, (density, i)
            for blk_a, blk_b in zip(a.blocks, b.blocks):
                ka, kb = blk_a.k_cache[:, :, :10].float(), blk_b.k_cache[:, :, :10].float()
                assert float((ka - kb).norm() / kb.norm()) < 1e-2


@pytest.mark.parametrize("n", [32000, 1000, 37, 8, 1])
def test_argmax(n):
    v = torch.randn(n, device="cuda", generator=_gen(n)).half()
    assert int(ops.argmax(v)) == int(torch.argmax(v.float()))
    v[n // 2] = 100.0
    v[n - 1] = 100.0                          # equal maxima: the lowest index wins
    assert int(ops.argmax(v)) == n // 2
    v[0] = float("nan")                       # NaN never wins
    assert int(ops.argmax(v)) == (n // 2 if n > 1 else 0)
    v.fill_(float("-inf"))
    assert int(ops.argmax(v)) == 0


def test_add_rmsnorm_peer_wait_is_bounded_and_says_who_was_missing():
    """The kernel that adds up the partial rows of a column-sharded layer waits for the other ranks itself: with
    an arrival counter that never comes the wait runs out after `spin_limit` polls, records the rank, and the
    kernel still produces its result; with all counters there nothing is recorded."""
    n, world = 256, 2
    g = _gen(9)
    x0 = torch.randn(n, device="cuda", generator=g).half()
    pending = torch.randn(world, n, device="cuda", generator=g).half()
    w = torch.ones(n, dtype=torch.float16, device="cuda")
    xr = x0.clone()
    ref = ops.add_rmsnorm(xr, pending, w, 1e-5)
    flags = torch.zeros(world + 3 + 13, dtype=torch.int32, device="cuda")
    flags[world] = 1          # this rank has issued one exchange
    flags[0] = 1              # rank 0 (itself) has delivered it, rank 1 has not
    xa = x0.clone()
    out = ops.add_rmsnorm_peer(xa, pending, w, 1e-5, flags.data_ptr(), world, 1000)
    torch.cuda.synchronize()
    assert int(flags[world + 2]) == 2
    assert torch.equal(out, ref) and torch.equal(xa, xr)
    flags[world + 2] = 0
    flags[1] = 1
    xb = x0.clone()
    out = ops.add_rmsnorm_peer(xb, pending, w, 1e-5, flags.data_ptr(), world, 1000)
    torch.cuda.synchronize()
    assert int(flags[world + 2]) == 0 and torch.equal(out, ref)
