"""Expert-parallel MoE block: experts sharded over ranks, tokens data-parallel.

The reference has no expert parallelism (its multi-GPU model is one full replica
per device, docs/ARCHITECTURE.md:25-30); this module is the sharded form of
`MoeBlock::forward` (crates/xabe-engine/src/block/moe.rs:1091-1329):

  1. every rank normalises, routes and picks the top-k for ITS tokens
  2. dispatch   all-to-all-v: each (token, k) pair sends the token's f16 row and
                the local expert id to the rank that owns expert e  (e // E_local)
  3. the owner runs expert_mlp for every row it received (weight 1)
  4. combine    all-to-all-v back, in the pair order of the sender
  5. the sender multiplies by the routing weights, sums ascending k, adds the
     gated shared expert and the residual

Per-row arithmetic on the owning rank is the same kernels with the same
reduction order as on one GPU, and the weighting and the ascending-k sum stay
on the sender, so a G-rank result is bit-identical to the 1-rank result.

One process per GPU; `torch.distributed` (NCCL over NVLink, or gloo on CPU for
the host-logic tests) carries the two exchanges.  The compute is behind a small
backend interface: `CudaEpBackend` is the product (C-ABI handles, no CPU path);
the tests plug in an oracle-backed one to check the exchange logic on CPU.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass
class EpPlan:
    order: torch.Tensor        # [pairs] flat (token, k) ids grouped by destination rank, ascending inside a rank
    send_counts: list[int]     # pairs per destination rank
    recv_counts: list[int]     # rows per source rank


def make_plan(topk_ids: torch.Tensor, experts_per_rank: int, world: int, group=None) -> EpPlan:
    """Groups the flat (token, k) pairs by owning rank and exchanges the counts."""
    flat = topk_ids.reshape(-1).to(torch.int64)
    dst = flat // experts_per_rank
    order = torch.argsort(dst, stable=True)
    send = torch.bincount(dst, minlength=world)
    if world == 1:
        return EpPlan(order, [int(send[0])], [int(send[0])])
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return EpPlan(order, [int(v) for v in send.tolist()], [int(v) for v in recv.tolist()])


def all_to_all_rows(send: torch.Tensor, send_counts: list[int], recv_counts: list[int], world: int,
                    group=None) -> torch.Tensor:
    """all-to-all-v of rows: `send` is grouped by destination, the result by source."""
    if world == 1:
        return send
    out = send.new_empty((sum(recv_counts),) + tuple(send.shape[1:]))
    dist.all_to_all_single(out, send.contiguous(), output_split_sizes=recv_counts, input_split_sizes=send_counts,
                           group=group)
    return out


class EpMoeBlock:
    """`MoeBlock` with the routed experts sharded over `world` ranks."""

    def __init__(self, backend, num_experts: int, experts_per_token: int, rank: int, world: int, group=None):
        if num_experts % world != 0:
            raise ValueError(f"{num_experts} experts do not split over {world} ranks")
        self.backend = backend
        self.num_experts, self.k = num_experts, experts_per_token
        self.rank, self.world, self.group = rank, world, group
        self.experts_per_rank = num_experts // world
        self.last_plan: EpPlan | None = None

    def forward(self, residual: torch.Tensor, tokens: int, ffn_out: torch.Tensor, l_out: torch.Tensor) -> None:
        b, K = self.backend, self.k
        rows, ids, weights = b.front(residual, tokens)             # [T,H], [T,K] int32, [T,K] f32
        plan = make_plan(ids[:tokens], self.experts_per_rank, self.world, self.group)
        self.last_plan = plan
        token_of = plan.order // K
        send_rows = rows[:tokens].index_select(0, token_of)
        send_eid = (ids[:tokens].reshape(-1).to(torch.int64).index_select(0, plan.order)
                    % self.experts_per_rank).to(torch.int32)
        recv_rows = all_to_all_rows(send_rows, plan.send_counts, plan.recv_counts, self.world, self.group)
        recv_eid = all_to_all_rows(send_eid, plan.send_counts, plan.recv_counts, self.world, self.group)
        out = b.experts(recv_rows, recv_eid)                        # [R,H] f32, unweighted
        back = all_to_all_rows(out, plan.recv_counts, plan.send_counts, self.world, self.group)
        w = weights[:tokens].reshape(-1).index_select(0, plan.order)
        contrib = torch.empty((tokens * K, back.shape[1]), dtype=torch.float32, device=back.device)
        contrib.index_copy_(0, plan.order, back * w[:, None])       # weight * value, as the down kernel stores it
        b.finish(contrib, residual, tokens, ffn_out, l_out)


class CudaEpBackend:
    """The product backend: two C-ABI handles per rank (front: routing, shared expert, combine;
    back: the local experts over received rows, k = 1)."""

    def __init__(self, geometry, experts_per_rank: int, max_rows: int, front_weights, local_gate, local_up,
                 local_down, eps: float = 1e-6, exact_decode: bool = False):
        from .moe import MoeGeometry, MoeKernels
        self.g = geometry
        self.front_k = MoeKernels(geometry, eps=eps)
        self.back_g = MoeGeometry(experts_per_rank, 1, geometry.hidden, geometry.intermediate, geometry.block_size,
                                  max_rows)
        self.back_k = MoeKernels(self.back_g, eps=eps)
        if exact_decode:
            self.front_k.set_exact_decode_regime(True)
            self.back_k.set_exact_decode_regime(True)
        self.fb = self.front_k.buffers()
        self.bb = self.back_k.buffers()
        self.w = front_weights                 # MoeLayerWeights: post_norm, router(+bias), shared expert, gate vector
        self.local = (local_gate, local_up, local_down)  # QuantTensor stacks of this rank's experts
        dev = self.fb.normed.device
        self.max_rows = max_rows
        self.ids_buf = torch.zeros(max_rows, 1, dtype=torch.int32, device=dev)
        self.ones = torch.ones(max_rows, 1, dtype=torch.float32, device=dev)
        self.rows_f32 = torch.zeros(max_rows, geometry.hidden, dtype=torch.float32, device=dev)

    def set_layer(self, front_weights, local_gate, local_up, local_down) -> None:
        self.w = front_weights
        self.local = (local_gate, local_up, local_down)

    def front(self, residual, tokens):
        k = self.front_k
        k.set_valid_tokens(tokens)
        k.rms_norm(residual, self.w.post_norm)
        k.router_logits(self.w.router, self.w.router_bias)
        k.route_and_dispatch()
        return self.fb.normed.to(torch.float16), self.fb.topk_ids, self.fb.topk_weights

    def experts(self, rows, local_expert):
        R = rows.shape[0]
        if R > self.max_rows:
            from .errors import TooManyTokens
            raise TooManyTokens(f"{R} received rows exceed the {self.max_rows} this rank was sized for")
        k = self.back_k
        k.set_valid_tokens(R)
        self.ids_buf[:R, 0] = local_expert
        self.rows_f32[:R] = rows.to(torch.float32)   # f16 -> f32 is exact; the kernels round back to the same f16
        k.build_dispatch(self.ids_buf, self.ones)
        k.grouped_forward_partial(self.local[0], self.local[1], self.local[2], self.rows_f32)
        return self.bb.partial[:R]

    def finish(self, contrib, residual, tokens, ffn_out, l_out):
        k = self.front_k
        self.fb.partial[: contrib.shape[0]] = contrib
        k.shared_expert(self.w.shared_gate, self.w.shared_up, self.w.shared_down)
        k.gate_and_combine(self.w.shared_gate_inp, residual, ffn_out, l_out)
