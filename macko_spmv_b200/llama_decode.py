"""Batch-1 decode of a Llama-2-architecture transformer whose linear layers run through `multiply`.

The reference measures end-to-end tokens/s by swapping the attention/MLP projections of a pruned
Llama-2-7B for MACKO layers and decoding under CUDA graphs (python_scripts/util_run_pruned_llm.py).
No checkpoint is available offline, so this module builds the same architecture (RMSNorm, rotary
embeddings, multi-head attention with a static KV cache, SwiGLU MLP) with seeded random weights
N(0, 0.02), prunes every linear layer per row by magnitude to the requested density, compresses it on
the GPU, and decodes greedily with one captured CUDA graph per token. Prompt tokens go through the
same single-token step. It is a caller of the hot path, used to report tokens/s; it is not a model zoo.

    python -m macko_spmv_b200.llama_decode --density 0.5 --layers 32
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m macko_spmv_b200.llama_decode --density 0.5

Tensor parallel (one process per GPU): the attention heads are split over the ranks. A rank holds the rows
of the q/k/v projection that belong to its heads and the matching rows of gate/up (plain local products, no
exchange: their input is the replicated hidden state), its heads' slice of the KV cache, and the columns of
the o and down projections that its slice of the attention output / MLP activation feeds
(`ColumnShardedMackoLinear`: partial products of all ranks are exchanged by the SpMV kernel itself and added).
A token therefore costs two fused product+exchange kernels per block plus one for the row-sharded LM head
(`RowShardedMackoLinear`), and no collective call; norms and rotary embedding are replicated.

The decode step runs the code between the products as three kernels of this package per block
(`torch.ops.macko_spmv.add_rmsnorm`, `rope_attention`, `silu_mul`: residual add + RMSNorm, rotary embedding +
KV-cache append + attention, SwiGLU gate), eight launches per block in all, for MACKO and dense layers alike;
`LlamaDecoder(..., fused_glue=False)` and `Block.forward` keep the same step in plain PyTorch operators.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch
from torch import nn

from . import compress, workloads
from .linear import ColumnShardedMackoLinear, MackoLinear, RowShardedMackoLinear

LLAMA2_7B = dict(hidden=4096, heads=32, ffn=11008, vocab=32000, layers=32, eps=1e-5, rope_theta=10000.0)


def _local_rows(w: torch.Tensor, parts: int, rank: int, world: int) -> torch.Tensor:
    """Rows of `w` = `parts` matrices stacked (q/k/v or gate/up): this rank's block of each part, stacked again."""
    n = w.shape[0] // parts
    if n % world:
        raise ValueError(f"{n} output features do not split over {world} ranks")
    b = n // world
    return torch.cat([w[p * n + rank * b: p * n + (rank + 1) * b] for p in range(parts)], dim=0).contiguous()


def _tp_linear(out_features: int, in_features: int, density: float, seed: int, device, peer, split: str, parts: int = 1):
    """One rank's share of a pruned linear layer under tensor parallelism. The full matrix is generated and
    pruned per row exactly as on one GPU, then cut: split="rows" keeps this rank's output features (of each of
    the `parts` stacked matrices) as a local MackoLinear; split="cols" keeps its input features as a
    ColumnShardedMackoLinear whose partial products are exchanged and added."""
    if density >= 1.0:
        raise ValueError("the tensor-parallel path runs MACKO layers only (density < 1)")
    w = workloads.magnitude_pruned_matrix(out_features, in_features, density, seed, device=device)
    if split == "rows":
        return MackoLinear(compress(_local_rows(w, parts, peer.rank, peer.world))).freeze()
    if in_features % peer.world:
        raise ValueError(f"{in_features} input features do not split over {peer.world} ranks")
    b = in_features // peer.world
    return ColumnShardedMackoLinear(w[:, peer.rank * b:(peer.rank + 1) * b], peer)


def _pruned_linear(out_features: int, in_features: int, density: float, seed: int, device, peer=None, slot=None) -> nn.Module:
    """A MackoLinear (density < 1) or a dense nn.Linear (density >= 1, the cuBLAS baseline); with `peer`
    (a `sharded.PeerGather`) this rank's row block as a RowShardedMackoLinear."""
    w = workloads.magnitude_pruned_matrix(out_features, in_features, min(density, 1.0), seed, device=device)
    if peer is not None:
        if density >= 1.0:
            raise ValueError("the tensor-parallel path runs MACKO layers only (density < 1)")
        from .sharded import row_block

        lo, hi = row_block(out_features, peer.rank, peer.world)
        return RowShardedMackoLinear(w[lo:hi], lo, out_features, peer, slot=slot, copy_result=False)   # consumed at once
    if density >= 1.0:
        lin = nn.Linear(in_features, out_features, bias=False, device=device, dtype=torch.float16)
        with torch.no_grad():
            lin.weight.copy_(w)
        return lin
    return MackoLinear(compress(w)).freeze()   # weights are final: see MackoLinear.freeze


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float, device):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=torch.float16, device=device), requires_grad=False)
        self.eps = eps
        self.dim = dim

    def forward(self, x):
        return torch.nn.functional.rms_norm(x, (self.dim,), self.weight, self.eps)


class Block(nn.Module):
    """One transformer block. q/k/v and gate/up are stored as one matrix each (rows concatenated), so a
    token costs four SpMVs per block; the glue around them is kept to a handful of kernels."""

    def __init__(self, cfg, density, seed, device, max_len, peer=None):
        super().__init__()
        h, f = cfg["hidden"], cfg["ffn"]
        world = peer.world if peer is not None else 1
        if cfg["heads"] % world or f % world:
            raise ValueError(f"{cfg['heads']} heads / {f} MLP features do not split over {world} ranks")
        self.head_dim = h // cfg["heads"]
        self.heads = cfg["heads"] // world          # heads held by this rank
        self.hidden, self.ffn = h, f // world       # ffn: this rank's share of the MLP width
        if peer is None:
            self.qkv_proj = _pruned_linear(3 * h, h, density, seed + 0, device)
            self.o_proj = _pruned_linear(h, h, density, seed + 3, device)
            self.gate_up_proj = _pruned_linear(2 * f, h, density, seed + 4, device)
            self.down_proj = _pruned_linear(h, f, density, seed + 6, device)
        else:
            self.qkv_proj = _tp_linear(3 * h, h, density, seed + 0, device, peer, "rows", parts=3)
            self.o_proj = _tp_linear(h, h, density, seed + 3, device, peer, "cols")
            self.gate_up_proj = _tp_linear(2 * f, h, density, seed + 4, device, peer, "rows", parts=2)
            self.down_proj = _tp_linear(h, f, density, seed + 6, device, peer, "cols")
        self.input_norm = RMSNorm(h, cfg["eps"], device)
        self.post_norm = RMSNorm(h, cfg["eps"], device)
        self.register_buffer("k_cache", torch.zeros(1, self.heads, max_len, self.head_dim, dtype=torch.float16, device=device))
        self.register_buffer("v_cache", torch.zeros(1, self.heads, max_len, self.head_dim, dtype=torch.float16, device=device))

    def forward(self, x, pos, cos, sin, mask):
        # x [hidden]; pos int64[1] on the device (graph-friendly); cos/sin [head_dim] fp16; mask [1,1,1,max_len]
        qkv = self.qkv_proj(self.input_norm(x)).view(3, self.heads, self.head_dim)
        qk = _rope(qkv[:2], cos, sin)                       # q and k rotated together
        self.k_cache.index_copy_(2, pos, qk[1].view(1, self.heads, 1, self.head_dim))
        self.v_cache.index_copy_(2, pos, qkv[2].view(1, self.heads, 1, self.head_dim))
        attn = torch.nn.functional.scaled_dot_product_attention(
            qk[0].view(1, self.heads, 1, self.head_dim), self.k_cache, self.v_cache, attn_mask=mask)
        x = x + self.o_proj(attn.reshape(-1))
        gu = self.gate_up_proj(self.post_norm(x))
        return x + self.down_proj(torch.nn.functional.silu(gu[: self.ffn]) * gu[self.ffn :])


    def step_fused(self, x, pending, pos, cos_table, sin_table):
        """The same block as `forward` with three kernels of this package between the four products. `x` [hidden]
        is the residual stream, updated in place; `pending` [k, hidden] holds output vectors that have not been
        added to it yet (the previous block's down projection: one vector, or one partial vector per rank), as
        the pair that `_pending_output` returns. Returns this block's own pending output."""
        ops = torch.ops.macko_spmv
        qkv = self.qkv_proj(_add_norm(x, pending, self.input_norm))
        attn = ops.rope_attention(qkv, cos_table, sin_table, pos, self.k_cache, self.v_cache)
        gu = self.gate_up_proj(_add_norm(x, _pending_output(self.o_proj, attn), self.post_norm))
        return _pending_output(self.down_proj, ops.silu_mul(gu))

    def prefill(self, x, cos, sin):
        """All prompt positions at once: x [T, hidden], cos/sin [T, head_dim]. Fills cache rows 0..T-1."""
        T = x.shape[0]
        qkv = self.qkv_proj(self.input_norm(x)).view(T, 3, self.heads, self.head_dim)
        qk = _rope(qkv[:, :2], cos[:, None, None, :], sin[:, None, None, :])          # [T, 2, heads, head_dim]
        q = qk[:, 0].transpose(0, 1).unsqueeze(0)                                      # [1, heads, T, head_dim]
        k = qk[:, 1].transpose(0, 1).unsqueeze(0)
        v = qkv[:, 2].transpose(0, 1).unsqueeze(0)
        self.k_cache[:, :, :T] = k
        self.v_cache[:, :, :T] = v
        attn = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.o_proj(attn[0].transpose(0, 1).reshape(T, self.hidden))
        gu = self.gate_up_proj(self.post_norm(x))
        return x + self.down_proj(torch.nn.functional.silu(gu[:, : self.ffn]) * gu[:, self.ffn :])


def _pending_output(layer, x):
    """The output of a projection as rows still to be added to the residual stream, with the exchange they wait
    for: ([1, out], None), or ([N, out], peer) for the partial vectors of a column-sharded layer, which stay in
    the exchange buffer; the product kernel has only published this rank's row, and the kernel that adds the rows
    up waits for the other ranks itself."""
    if isinstance(layer, ColumnShardedMackoLinear):
        return layer.partials(x, defer_wait=True), layer.peer
    return layer(x).view(1, -1), None


def _add_norm(x, pending, norm):
    """x += the pending rows; returns rmsnorm(x) * weight (one kernel; with an exchange pending, its wait too)."""
    rows, peer = pending
    if peer is None:
        return torch.ops.macko_spmv.add_rmsnorm(x, rows, norm.weight, norm.eps)
    return torch.ops.macko_spmv.add_rmsnorm_peer(x, rows, norm.weight, norm.eps, peer.flags_address, peer.world, peer.spin_limit)


def _rope(t, cos, sin):
    # rotate-half convention: (t1, t2) -> (t1*cos - t2*sin, t2*cos + t1*sin), cos/sin repeated over both halves
    half = t.shape[-1] // 2
    rot = torch.cat((-t[..., half:], t[..., :half]), dim=-1)
    return t * cos + rot * sin


class LlamaDecoder(nn.Module):
    def __init__(self, density: float, cfg=None, layers=None, device="cuda", max_len=384, seed=4000,
                 prune_lm_head=True, peer=None, fused_glue=True):
        super().__init__()
        self.fused_glue = fused_glue
        cfg = dict(LLAMA2_7B if cfg is None else cfg)
        if layers is not None:
            cfg["layers"] = layers
        self.cfg, self.max_len, self.device = cfg, max_len, device
        h = cfg["hidden"]
        g = torch.Generator(device=device).manual_seed(seed)
        self.embed = (0.02 * torch.randn(cfg["vocab"], h, generator=g, device=device)).to(torch.float16)
        self.blocks = nn.ModuleList([Block(cfg, density, seed + 100 * (i + 1), device, max_len, peer) for i in range(cfg["layers"])])
        self.norm = RMSNorm(h, cfg["eps"], device)
        # A decode step is two exchanges per block plus this one: an odd number. Replayed as one captured graph,
        # its last exchange would be followed by its first in the same slot; the LM head takes the spare slot.
        self.lm_head = _pruned_linear(cfg["vocab"], h, density if prune_lm_head else 1.0, seed + 7, device,
                                      peer if prune_lm_head else None, slot=2)
        half = (h // cfg["heads"]) // 2
        inv = 1.0 / (cfg["rope_theta"] ** (torch.arange(half, device=device, dtype=torch.float32) / half))
        ang = torch.arange(max_len, device=device, dtype=torch.float32)[:, None] * inv[None, :]
        ang = torch.cat((ang, ang), dim=-1)
        self.cos_table, self.sin_table = ang.cos().to(torch.float16), ang.sin().to(torch.float16)
        self.neg_inf = torch.tensor(float("-inf"), dtype=torch.float16, device=device)
        self.zero = torch.zeros((), dtype=torch.float16, device=device)
        self.positions = torch.arange(max_len, device=device)

    def step(self, token, pos):
        """token int64[1], pos int64[1] (device tensors) -> next token int64[1] (greedy)."""
        if self.fused_glue:
            return torch.ops.macko_spmv.argmax(self.logits(token, pos))
        return torch.argmax(self.logits(token, pos).float(), dim=-1, keepdim=True)

    def prefill(self, tokens):
        """Runs the whole prompt (int64 [T]) in one pass (the linear layers see a [T, hidden] batch and route
        it through the multi-vector product or the dense-copy GEMM); returns the greedy next token [1]."""
        T = tokens.numel()
        x = self.embed.index_select(0, tokens)
        cos, sin = self.cos_table[:T], self.sin_table[:T]
        for blk in self.blocks:
            x = blk.prefill(x, cos, sin)
        logits = self.lm_head(self.norm(x[T - 1]))
        return torch.argmax(logits.float(), dim=-1, keepdim=True)

    def logits(self, token, pos):
        """fp16 logits [vocab] of the token at position `pos`; updates the KV cache."""
        x = self.embed.index_select(0, token)[0]
        if self.fused_glue:
            pending = (x.new_empty((0, x.shape[0])), None)
            for blk in self.blocks:
                pending = blk.step_fused(x, pending, pos, self.cos_table, self.sin_table)
            return self.lm_head(_add_norm(x, pending, self.norm))
        cos = self.cos_table.index_select(0, pos)[0]
        sin = self.sin_table.index_select(0, pos)[0]
        mask = torch.where(self.positions <= pos, self.zero, self.neg_inf).view(1, 1, 1, -1)
        for blk in self.blocks:
            x = blk(x, pos, cos, sin, mask)
        return self.lm_head(self.norm(x))


@torch.no_grad()
def generate(model: LlamaDecoder, prompt: torch.Tensor, new_tokens: int, use_graph: bool = True,
             batched_prefill: bool = False):
    """Feeds the prompt (token by token through the decode step, or in one batched pass), then generates
    greedily. Returns (tokens, seconds for the generated part, seconds for the prompt part)."""
    dev = model.device
    token = torch.zeros(1, dtype=torch.int64, device=dev)
    pos = torch.zeros(1, dtype=torch.int64, device=dev)
    out_token = torch.zeros(1, dtype=torch.int64, device=dev)
    graph = None
    if use_graph:
        token.copy_(prompt[:1])
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                out_token.copy_(model.step(token, pos))
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out_token.copy_(model.step(token, pos))

    def run_step():
        if graph is not None:
            graph.replay()
        else:
            out_token.copy_(model.step(token, pos))

    if batched_prefill:
        model.prefill(prompt)   # untimed first pass, like the warm-up runs of the decode step: allocator growth, GEMM set-up
    tokens = []
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    if batched_prefill:
        out_token.copy_(model.prefill(prompt))
    else:
        for i in range(prompt.numel()):
            token.copy_(prompt[i : i + 1])
            pos.fill_(i)
            run_step()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    for i in range(new_tokens):
        token.copy_(out_token)
        pos.fill_(prompt.numel() + i)
        run_step()
        tokens.append(out_token.clone())
    torch.cuda.synchronize()
    t2 = time.perf_counter()
    return torch.cat(tokens), t2 - t1, t1 - t0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--density", type=float, default=0.5, help="1.0 = dense nn.Linear (cuBLAS) baseline")
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--prompt", type=int, default=128)
    ap.add_argument("--new-tokens", type=int, default=256)
    ap.add_argument("--dense-lm-head", action="store_true")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--batched-prefill", action="store_true",
                    help="run the prompt in one pass (one GPU only): linear layers take the [tokens, hidden] batch")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    peer = None
    if world > 1:
        import torch.distributed as dist

        from .sharded import PeerGather

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
        cfg = LLAMA2_7B
        peer = PeerGather(max(world * cfg["hidden"], cfg["vocab"]), device)   # N partial vectors of the column-sharded layers, or the logits
    t0 = time.perf_counter()
    model = LlamaDecoder(args.density, layers=args.layers, device=device, max_len=args.prompt + args.new_tokens,
                         prune_lm_head=not args.dense_lm_head, peer=peer)
    torch.cuda.synchronize()
    build_s = time.perf_counter() - t0
    g = torch.Generator(device=device).manual_seed(4001)
    prompt = torch.randint(0, model.cfg["vocab"], (args.prompt,), generator=g, device=device)
    if world > 1:
        dist.barrier()
    if args.batched_prefill and world > 1:
        raise SystemExit("--batched-prefill runs on one GPU: the row-sharded layers multiply one vector at a time")
    tokens, gen_s, prompt_s = generate(model, prompt, args.new_tokens, use_graph=not args.no_graph,
                                       batched_prefill=args.batched_prefill)
    same = True
    if world > 1:
        t = torch.tensor([gen_s, prompt_s], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        gen_s, prompt_s = float(t[0]), float(t[1])
        ref = tokens.clone()
        dist.broadcast(ref, 0)
        agree = torch.tensor([int(torch.equal(ref, tokens))], device=device)
        dist.all_reduce(agree, op=dist.ReduceOp.MIN)
        same = bool(agree.item()) and peer.error_flag() == 0
    if rank == 0:
        print(json.dumps({
            "model": "llama-2-7b architecture, random init", "layers": args.layers, "density": args.density,
            "tensor_parallel": world, "ranks_agree": same,
            "lm_head": "dense" if args.dense_lm_head or args.density >= 1 else "pruned",
            "prompt_tokens": args.prompt, "new_tokens": args.new_tokens,
            "tokens_per_s": args.new_tokens / gen_s, "prompt_tokens_per_s": args.prompt / prompt_s,
            "build_seconds": build_s, "memory_GB": torch.cuda.max_memory_allocated() / 1e9,
            "cuda_graph": not args.no_graph, "batched_prefill": bool(args.batched_prefill), "first_tokens": tokens[:8].tolist(),
        }), flush=True)
    if world > 1:
        # in order: the model (its layers hold the exchange buffers), the buffers, then the process group
        torch.cuda.synchronize()
        dist.barrier()
        del model
        peer.close()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
