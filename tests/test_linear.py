"""MackoLinear and the compressed-checkpoint key layout (CPU part: key handling; GPU part: numerics)."""
import numpy as np
import pytest
import torch
from torch import nn

import oracle
from macko_spmv_b200 import linear, workloads


def _oracle_comp(W):
    v, d, ri, r, c = oracle.compress(W.numpy().view(np.uint16))
    return (torch.from_numpy(v.view(np.float16).copy()), torch.from_numpy(d.copy()), torch.from_numpy(ri.copy()), r, c)


def test_checkpoint_key_layout_and_module_swap_cpu():
    W = workloads.bernoulli_matrix(6, 40, 0.3, seed=3)
    comp = _oracle_comp(W)   # the test builds the buffers with the oracle: no GPU needed for key handling
    sd = {"model.layers.0.mlp.up_proj.c_0": comp[0], "model.layers.0.mlp.up_proj.c_1": comp[1],
          "model.layers.0.mlp.up_proj.c_2": comp[2], "model.layers.0.mlp.up_proj.c_3": comp[3],
          "model.layers.0.mlp.up_proj.c_4": comp[4], "model.norm.weight": torch.ones(40)}
    assert linear.compressed_prefixes(sd) == ["model.layers.0.mlp.up_proj"]

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.mlp = nn.Module()
            self.mlp.up_proj = nn.Linear(40, 6, bias=False)

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.model = nn.Module()
            self.model.layers = nn.ModuleList([Block()])

    net = linear.replace_linears(Net(), sd, device="cpu")
    layer = net.model.layers[0].mlp.up_proj
    assert isinstance(layer, linear.MackoLinear)
    assert layer.in_features == 40 and layer.out_features == 6
    assert torch.equal(layer.c_0.view(torch.int16), comp[0].view(torch.int16))
    assert set(k for k in layer.state_dict()) == {"c_0", "c_1", "c_2"}
    with pytest.raises(RuntimeError):
        layer(torch.zeros(3, 41, dtype=torch.float16))


@pytest.mark.gpu
def test_macko_linear_forward_and_checkpoint_roundtrip(tmp_path):
    torch.manual_seed(0)
    lin = nn.Linear(512, 300, bias=True).half().cuda()
    with torch.no_grad():
        lin.weight.mul_((torch.rand_like(lin.weight) < 0.4).half())
    layer = linear.MackoLinear.from_linear(lin)
    x = torch.randn(2, 3, 512, device="cuda").half()
    ref = torch.nn.functional.linear(x.float(), lin.weight.float(), lin.bias.float())
    got = layer(x)
    assert got.shape == (2, 3, 300)
    assert torch.allclose(got.float(), ref, rtol=2e-3, atol=2e-3)
    assert torch.allclose(layer(x[0, 0]).float(), ref[0, 0], rtol=2e-3, atol=2e-3)
    # checkpoint: compress a state dict with the reference's key selection, save, load, rebuild
    sd = {"model.layers.0.self_attn.q_proj.weight": lin.weight.detach().cpu(),
          "model.layers.0.self_attn.q_proj.bias": lin.bias.detach().cpu(),
          "model.embed_tokens.weight": torch.randn(10, 512).half()}
    csd = linear.compress_state_dict(sd)
    assert "model.layers.0.self_attn.q_proj.weight" not in csd and "model.embed_tokens.weight" in csd
    assert csd["model.layers.0.self_attn.q_proj.c_3"] == 300 and csd["model.layers.0.self_attn.q_proj.c_4"] == 512
    path = tmp_path / "compressed.pt"
    torch.save(csd, path)
    back = torch.load(path)
    rebuilt = linear.MackoLinear.from_state_dict_entry(back, "model.layers.0.self_attn.q_proj", device="cuda")
    assert torch.equal(rebuilt(x), got)
    exp = oracle.compress(lin.weight.detach().cpu().numpy().view(np.uint16))
    assert np.array_equal(back["model.layers.0.self_attn.q_proj.c_1"].numpy(), exp[1])


@pytest.mark.gpu
def test_llama_decode_step_matches_dense_twin():
    """A small Llama-architecture decoder on MACKO layers against the same decoder on dense layers
    holding the decompressed weights; CUDA-graph decode must reproduce eager decode token for token."""
    from macko_spmv_b200 import llama_decode

    cfg = dict(hidden=256, heads=4, ffn=512, vocab=1000, layers=2, eps=1e-5, rope_theta=10000.0)
    model = llama_decode.LlamaDecoder(0.5, cfg=cfg, max_len=48, seed=11)
    twin = llama_decode.LlamaDecoder(0.5, cfg=cfg, max_len=48, seed=11)

    def densify(layer):
        comp = tuple(t.cpu().numpy() if torch.is_tensor(t) else t for t in layer.compressed)
        dense = oracle.decompress((comp[0].view(np.uint16), comp[1], comp[2], comp[3], comp[4]))
        lin = nn.Linear(layer.in_features, layer.out_features, bias=False, device="cuda", dtype=torch.float16)
        with torch.no_grad():
            lin.weight.copy_(torch.from_numpy(dense.view(np.float16).copy()))
        return lin

    for blk in twin.blocks:
        for name in ("qkv_proj", "o_proj", "gate_up_proj", "down_proj"):
            setattr(blk, name, densify(getattr(blk, name)))
    twin.lm_head = densify(twin.lm_head)

    prompt = torch.randint(0, 1000, (16,), device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
    with torch.no_grad():
        for i in range(4):  # same hidden state through both stacks, one token at a time
            tok, pos = prompt[i : i + 1], torch.tensor([i], device="cuda")
            x = model.embed.index_select(0, tok)[0]
            cos, sin = model.cos_table[i], model.sin_table[i]
            mask = torch.where(model.positions <= pos, model.zero, model.neg_inf).view(1, 1, 1, -1)
            xa, xb = x, x
            for ba, bb in zip(model.blocks, twin.blocks):
                xa, xb = ba(xa, pos, cos, sin, mask), bb(xb, pos, cos, sin, mask)
            la, lb = model.lm_head(model.norm(xa)).float(), twin.lm_head(twin.norm(xb)).float()
            assert float((la - lb).norm() / lb.norm()) < 2e-2
    fresh = llama_decode.LlamaDecoder(0.5, cfg=cfg, max_len=48, seed=11)
    eager, _, _ = llama_decode.generate(fresh, prompt, 12, use_graph=False)
    fresh2 = llama_decode.LlamaDecoder(0.5, cfg=cfg, max_len=48, seed=11)
    graphed, _, _ = llama_decode.generate(fresh2, prompt, 12, use_graph=True)
    assert torch.equal(eager, graphed)


@pytest.mark.gpu
def test_batched_prefill_matches_token_by_token():
    """The prompt run in one pass (linear layers take the [tokens, hidden] batch: multi-vector kernel for the
    short prompt, dense-copy GEMM for the long one) must leave the same KV cache and produce the same logits
    as feeding the tokens one at a time through the decode step."""
    from macko_spmv_b200 import llama_decode

    cfg = dict(hidden=256, heads=4, ffn=512, vocab=1000, layers=2, eps=1e-5, rope_theta=10000.0)
    for T in (6, 40):
        a = llama_decode.LlamaDecoder(0.5, cfg=cfg, max_len=64, seed=5)
        b = llama_decode.LlamaDecoder(0.5, cfg=cfg, max_len=64, seed=5)
        prompt = torch.randint(0, 1000, (T,), device="cuda", generator=torch.Generator(device="cuda").manual_seed(2))
        with torch.no_grad():
            for i in range(T):
                last = a.logits(prompt[i : i + 1], torch.tensor([i], device="cuda"))
            b.prefill(prompt)
            nxt = torch.tensor([7], device="cuda")
            pos = torch.tensor([T], device="cuda")
            la, lb = a.logits(nxt, pos), b.logits(nxt, pos)      # both continue from their own cache
        for blk_a, blk_b in zip(a.blocks, b.blocks):
            ka, kb = blk_a.k_cache[:, :, :T].float(), blk_b.k_cache[:, :, :T].float()
            assert float((ka - kb).norm() / ka.norm()) < 1e-2
        assert float((la.float() - lb.float()).norm() / la.float().norm()) < 2e-2
        assert last.shape == (1000,)
