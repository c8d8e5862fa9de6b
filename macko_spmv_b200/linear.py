"""`MackoLinear`: a linear layer whose weight is stored in MACKO form, and helpers for the
compressed-checkpoint layout of the reference.

The reference's LLM scripts replace every `nn.Linear` of the attention and MLP blocks by a layer that
calls `multiply` once per input vector through `torch.vmap`
(python_scripts/util_run_pruned_llm.py:102-133) and store a compressed model as a state dict in which
each `<name>.weight` is replaced by `<name>.c_0 … <name>.c_4` = values, deltas, row_indices, rows, cols
(python_scripts/util_compress_llm.py:16-44). This module keeps that key layout, so checkpoints written
by either implementation load in the other, and routes batches itself: inputs of shape [..., in]
are flattened; one vector goes through `multiply` (decode), a few vectors share passes over the
compressed matrix (`multiply_batched`, 8 per pass), and large batches (prefill) run as a dense GEMM on a
decompressed copy.
"""
from __future__ import annotations

import torch
from torch import nn

COMPRESSED_KEYS = ("c_0", "c_1", "c_2", "c_3", "c_4")


class MackoLinear(nn.Module):
    """y = x @ W^T (+ bias) with W [out_features, in_features] held as a MACKO compressed matrix."""

    def __init__(self, compressed, bias: torch.Tensor | None = None):
        super().__init__()
        values, deltas, row_indices, rows, cols = compressed
        self.out_features = int(rows)
        self.in_features = int(cols)
        self.register_buffer("c_0", values)
        self.register_buffer("c_1", deltas)
        self.register_buffer("c_2", row_indices)
        self.bias = nn.Parameter(bias, requires_grad=False) if bias is not None else None
        self._frozen = None   # FrozenMatrix after freeze(): immutable weights, optional launch plan

    def freeze(self, plan="auto") -> "MackoLinear":
        """Declare the weight buffers final (call after loading / moving the module, before serving): the
        single-vector product may then read them ahead of stream order, and matrices with very uneven rows
        get a launch plan (see `macko_spmv_b200.freeze`). Writing c_0 / c_1 / c_2 afterwards (load_state_dict,
        .to(...)) requires another freeze()."""
        from . import freeze

        self._frozen = freeze(self.compressed, plan=plan)
        return self

    @classmethod
    def from_linear(cls, linear: nn.Linear) -> "MackoLinear":
        """Compress the (already pruned) fp16 weight of an `nn.Linear`."""
        from . import compress

        w = linear.weight.detach()
        if w.dtype != torch.float16:
            raise TypeError("MackoLinear stores fp16 weights; convert the layer with .half() first")
        bias = linear.bias.detach().clone() if linear.bias is not None else None
        return cls(compress(w.contiguous()), bias)

    @classmethod
    def from_state_dict_entry(cls, state_dict, prefix: str, device=None) -> "MackoLinear":
        """Build the layer from the `<prefix>.c_0 … c_4` entries of a compressed checkpoint."""
        parts = [state_dict[f"{prefix}.{k}"] for k in COMPRESSED_KEYS]
        tensors = [p.to(device) if device is not None else p for p in parts[:3]]
        bias = state_dict.get(f"{prefix}.bias")
        if bias is not None and device is not None:
            bias = bias.to(device)
        return cls((tensors[0], tensors[1], tensors[2], int(parts[3]), int(parts[4])), bias)

    @property
    def compressed(self):
        return (self.c_0, self.c_1, self.c_2, self.out_features, self.in_features)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from . import multiply, multiply_batched

        if x.shape[-1] != self.in_features:
            raise RuntimeError(f"expected last dimension {self.in_features}, got {tuple(x.shape)}")
        lead = x.shape[:-1]
        flat = x.reshape(-1, self.in_features)
        comp = self.compressed
        if flat.shape[0] == 1:
            fz = self._frozen
            if fz is not None and fz[0].data_ptr() != self.c_0.data_ptr():
                fz = self._frozen = None   # the buffers were replaced since freeze(): back to the safe path
            y = multiply(fz if fz is not None else comp, flat[0].contiguous()).unsqueeze(0)
        else:
            y = multiply_batched(comp, flat.contiguous())
        if self.bias is not None:
            y = y + self.bias
        return y.reshape(*lead, self.out_features)

    def extra_repr(self) -> str:
        stored = self.c_0.numel()
        dense = self.out_features * self.in_features
        return (f"in_features={self.in_features}, out_features={self.out_features}, "
                f"stored={stored} ({2.5 * stored / max(2 * dense, 1):.3f} of dense bytes)")


class RowShardedMackoLinear(nn.Module):
    """Tensor-parallel `MackoLinear`: this rank holds a contiguous block of output features (rows of W)
    in MACKO form; `forward` returns the full output on every rank.

    The product and the exchange are one kernel (`sharded.PeerGather`). With `copy_result=False` the returned
    tensor is a view of one of the exchange's slots: it must be consumed (in stream order) before the
    second-next product issued through the same `PeerGather`; the decode loop in `llama_decode` does exactly that.
    The reference has no multi-GPU layer; this is the layer its `fix()` would install under tensor
    parallelism."""

    def __init__(self, weight_block: torch.Tensor, row_lo: int, total_rows: int, peer, slot: int | None = None,
                 copy_result: bool = True):
        super().__init__()
        from . import compress, sharded

        self.slot = slot   # exchange slot of this layer's product (None: the alternating pair), see sharded.PeerGather
        # True: forward returns a tensor of its own. False: a view of the exchange slot, overwritten by the
        # second-next product through the same PeerGather (for callers that consume it at once, like the decode loop)
        self.copy_result = copy_result
        world = peer.world
        blocks = [sharded.row_block(total_rows, r, world) for r in range(world)]
        lo, hi = blocks[peer.rank]
        if lo != row_lo or weight_block.size(0) != hi - lo:
            raise ValueError(f"rank {peer.rank} must hold rows [{lo}, {hi}) of {total_rows}")
        values, deltas, row_indices, rows, cols = compress(weight_block.contiguous())
        self.register_buffer("c_0", values)
        self.register_buffer("c_1", deltas)
        self.register_buffer("c_2", row_indices)
        self.out_features, self.in_features = int(total_rows), int(cols)
        self.peer = peer
        self.shard = sharded.RowShard((values, deltas, row_indices, rows, cols), lo, hi, total_rows, blocks, peer.group)
        torch.cuda.synchronize(values.device)   # the compressor has finished: the block is final from here on
        self._c0_ptr = values.data_ptr()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.dim() != 1 or x.shape[0] != self.in_features:
            raise RuntimeError(f"expected a vector of {self.in_features} elements, got {tuple(x.shape)}")
        final = self.c_0.data_ptr() == self._c0_ptr   # buffers replaced since construction: no early matrix loads
        y = self.peer.multiply(self.shard, x.contiguous(), immutable=final, slot=self.slot)
        return y.clone() if self.copy_result else y


class ColumnShardedMackoLinear(nn.Module):
    """Tensor-parallel `MackoLinear` split by input features: this rank holds the columns
    [col_lo, col_lo + in_local) of W (all rows) in MACKO form and multiplies them with its slice of x; the
    partial results of all ranks are added. `forward(x_local)` returns the full output on every rank.

    Used where the input is already split (the attention output of a rank's heads, its slice of the MLP
    activation): no gather of x is needed, one exchange per layer. The exchange is the fused one of
    `sharded.PeerGather`: every rank's kernel stores its partial y into slot `rank` of an [N, out] buffer on
    all ranks (the buffer is addressed as one y of N * out rows of which this rank owns rows
    [rank * out, (rank + 1) * out)), and the N partial vectors are summed in rank order in fp32, so all ranks
    get the same bits. The reference has no multi-GPU layer."""

    def __init__(self, weight_columns: torch.Tensor, peer):
        super().__init__()
        from . import compress, sharded

        world, rank = peer.world, peer.rank
        values, deltas, row_indices, rows, cols = compress(weight_columns.contiguous())
        self.register_buffer("c_0", values)
        self.register_buffer("c_1", deltas)
        self.register_buffer("c_2", row_indices)
        self.out_features, self.in_local = int(rows), int(cols)
        self.peer = peer
        blocks = [(r * rows, (r + 1) * rows) for r in range(world)]
        self.shard = sharded.RowShard((values, deltas, row_indices, rows, cols), rank * rows, (rank + 1) * rows,
                                      world * rows, blocks, peer.group)
        torch.cuda.synchronize(values.device)   # the compressor has finished: the block is final from here on
        self._c0_ptr = values.data_ptr()

    def partials(self, x_local: torch.Tensor, defer_wait: bool = False) -> torch.Tensor:
        """The N partial output vectors [N, out] (rank order), not yet added: a view of the exchange slot, to be
        consumed (in stream order) before the second-next product through the same `PeerGather`.
        `defer_wait`: the rows of the other ranks are complete only behind a wait on the exchange's flag words
        (`torch.ops.macko_spmv.add_rmsnorm_peer` does it itself)."""
        if x_local.dim() != 1 or x_local.shape[0] != self.in_local:
            raise RuntimeError(f"expected this rank's {self.in_local} input features, got {tuple(x_local.shape)}")
        final = self.c_0.data_ptr() == self._c0_ptr
        parts = self.peer.multiply(self.shard, x_local.contiguous(), immutable=final, defer_wait=defer_wait)
        return parts.view(self.peer.world, self.out_features)

    def forward(self, x_local: torch.Tensor) -> torch.Tensor:
        # one reduction kernel: torch adds fp16 inputs in fp32 and rounds once, in rank order on every rank
        return self.partials(x_local).sum(dim=0)


def compress_state_dict(state_dict, select=lambda name: ("self_attn" in name or "mlp" in name) and name.endswith(".weight")):
    """Replace every selected 2-D fp16 `<name>.weight` by `<name>.c_0 … c_4`.

    The default selection is the reference's (attention and MLP projections,
    python_scripts/util_compress_llm.py:25-27). Tensors are compressed on the GPU and returned on the
    CPU, ready for `torch.save`; everything else is passed through unchanged.
    """
    from . import compress, move_to_device

    out = {}
    for name, tensor in state_dict.items():
        if select(name) and tensor.dim() == 2 and tensor.dtype == torch.float16:
            comp = move_to_device(compress(tensor.contiguous().to("cuda")), "cpu")
            prefix = name[: -len(".weight")]
            for key, part in zip(COMPRESSED_KEYS, comp):
                out[f"{prefix}.{key}"] = part
        else:
            out[name] = tensor
    return out


def compressed_prefixes(state_dict) -> list[str]:
    """Module paths that hold a compressed weight in `state_dict`."""
    return sorted({k[: -len(".c_0")] for k in state_dict if k.endswith(".c_0")})


def replace_linears(model: nn.Module, state_dict, device="cuda", freeze: bool = False) -> nn.Module:
    """Swap the modules named by the compressed entries of `state_dict` for `MackoLinear` layers
    (what `fix()` does in python_scripts/util_run_pruned_llm.py:123-133). `freeze=True` also declares the
    loaded weights final (`MackoLinear.freeze`)."""
    for prefix in compressed_prefixes(state_dict):
        parent_path, _, leaf = prefix.rpartition(".")
        parent = model.get_submodule(parent_path) if parent_path else model
        layer = MackoLinear.from_state_dict_entry(state_dict, prefix, device)
        setattr(parent, leaf, layer.freeze() if freeze else layer)
    return model
