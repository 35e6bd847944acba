"""Tensor-parallel dense SwiGLU block (the 27B sibling's FFN) over the ranks of one node.

The reference runs `DenseFfnBlock::forward` (crates/xabe-engine/src/block/dense_ffn.rs:9-16,
1047) on one device; its multi-GPU model is one replica per device.  This is the sharded form:

  * gate and up are split by OUTPUT rows (the intermediate dimension), down by its
    CONTRACTION dimension, both in units of 256 elements (one Q6_K superblock, eight Q8_0
    blocks), so every shard is a whole number of quantisation blocks and is read as is;
  * every rank normalises the replicated residual, runs its slice of the MLP with the same
    kernels as the one-GPU block and holds a partial [tokens][hidden] fp32 sum;
  * one all-reduce (NCCL over NVLink; gloo in the CPU tests) adds the partials, then the
    residual is added on every rank.

The order in which the all-reduce adds the ranks' partials is the library's, so a G-rank result
agrees with the one-rank result to rounding (rel-L2 far below 1e-3), not bit for bit.
One process per GPU.  The compute sits behind a small backend interface, as in `ep.py`.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

_BLOCK = {0: (256, 210), 1: (32, 34)}  # quant tag -> (elements, bytes) per block
UNIT = 256                             # shard granularity along the intermediate dimension


def shard_bounds(inter: int, rank: int, world: int) -> tuple[int, int]:
    """[i0, i1) of the intermediate dimension owned by `rank`: whole units of 256, as even as possible."""
    if inter % UNIT != 0:
        raise ValueError(f"intermediate size {inter} is not a multiple of {UNIT}")
    units = inter // UNIT
    if units < world:
        raise ValueError(f"{units} units of {UNIT} do not split over {world} ranks")
    return (rank * units // world) * UNIT, ((rank + 1) * units // world) * UNIT


def shard_rows(raw: torch.Tensor, rows: int, k: int, quant: int, r0: int, r1: int) -> torch.Tensor:
    """Rows [r0, r1) of a [rows][k] quantised matrix in file layout: a contiguous byte range (a view)."""
    elems, nbytes = _BLOCK[quant]
    row_bytes = k // elems * nbytes
    assert raw.numel() == rows * row_bytes
    return raw[r0 * row_bytes:r1 * row_bytes]


def shard_cols(raw: torch.Tensor, rows: int, k: int, quant: int, c0: int, c1: int) -> torch.Tensor:
    """Columns [c0, c1) of a [rows][k] quantised matrix: the blocks c0/elems .. c1/elems of every row,
    repacked contiguously (done once, when the weights are loaded)."""
    elems, nbytes = _BLOCK[quant]
    assert c0 % elems == 0 and c1 % elems == 0 and raw.numel() == rows * (k // elems) * nbytes
    v = raw.view(rows, k // elems, nbytes)
    return v[:, c0 // elems:c1 // elems, :].contiguous().view(-1)


class TpDenseFfnBlock:
    """`DenseFfnBlock` with the intermediate dimension sharded over `world` ranks."""

    def __init__(self, backend, rank: int, world: int, group=None):
        self.backend, self.rank, self.world, self.group = backend, rank, world, group

    def forward(self, residual: torch.Tensor, tokens: int, ffn_out: torch.Tensor, l_out: torch.Tensor) -> None:
        """residual, ffn_out, l_out: [max_tokens][hidden] f32; rows >= tokens are not written."""
        partial = self.backend.partial_mlp(residual, tokens)      # [max_tokens][hidden] f32, this rank's share
        live = partial[:tokens]
        if self.world > 1:
            dist.all_reduce(live, op=dist.ReduceOp.SUM, group=self.group)
        ffn_out[:tokens] = live
        torch.add(live, residual[:tokens], out=l_out[:tokens])


class CudaTpBackend:
    """The product backend: one shared-only C-ABI handle sized for this rank's slice."""

    def __init__(self, hidden: int, inter: int, max_tokens: int, rank: int, world: int, post_norm, gate, up, down,
                 eps: float = 1e-6):
        """gate, up, down: QuantTensor of the FULL matrices on this device (file layout)."""
        from .moe import MoeGeometry, MoeKernels, QuantTensor
        i0, i1 = shard_bounds(inter, rank, world)
        self.i0, self.i1 = i0, i1
        g = MoeGeometry(1, 1, hidden, i1 - i0, 64, max_tokens)
        self.k = MoeKernels(g, eps=eps, scope=MoeKernels.SCOPE_SHARED_ONLY)
        self.post_norm = post_norm
        self.gate = QuantTensor(shard_rows(gate.bytes, inter, hidden, gate.quant, i0, i1), gate.quant)
        self.up = QuantTensor(shard_rows(up.bytes, inter, hidden, up.quant, i0, i1), up.quant)
        self.down = QuantTensor(shard_cols(down.bytes, hidden, inter, down.quant, i0, i1), down.quant)
        self.out = torch.zeros(max_tokens, hidden, dtype=torch.float32, device=post_norm.device)

    def partial_mlp(self, residual, tokens):
        k = self.k
        k.set_valid_tokens(tokens)
        k.rms_norm(residual, self.post_norm)
        k.shared_expert(self.gate, self.up, self.down, None, self.out)
        return self.out
