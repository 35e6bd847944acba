"""Expert-parallel MoE block: experts sharded over ranks, tokens data-parallel.

The reference has no expert parallelism (its multi-GPU model is one full replica
per device, docs/ARCHITECTURE.md:25-30); this module is the sharded form of
`MoeBlock::forward` (crates/xabe-engine/src/block/moe.rs:1091-1329):

  1. every rank normalises, routes and picks the top-k for ITS tokens
  2. dispatch   all-to-all-v: each (token, k) pair sends the token's f16 row and
                the local expert id to the rank that owns expert e  (e // E_local)
     (meanwhile every rank runs the shared expert over its own tokens)
  3. the owner runs expert_mlp for every row it received (weight 1)
  4. combine    all-to-all-v back, in the pair order of the sender
  5. the sender multiplies by the routing weights, sums ascending k, adds the
     gated shared expert and the residual (one kernel, reading the returned rows
     through the inverse of the send order)

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
    order: torch.Tensor | None # [pairs] flat (token, k) ids grouped by destination rank (None: order lives on the device)
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


def exchange_counts(send_counts: torch.Tensor, total: int, world: int, group=None) -> EpPlan:
    """The pair counts per destination live on the device; all_to_all_single wants host integers, so
    this is the one host read-back of a layer (send and receive counts together)."""
    if world == 1:
        return EpPlan(None, [total], [total])
    recv = torch.empty_like(send_counts)
    dist.all_to_all_single(recv, send_counts, group=group)
    both = torch.stack([send_counts, recv]).tolist()
    return EpPlan(None, [int(v) for v in both[0]], [int(v) for v in both[1]])


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

    def __init__(self, backend, num_experts: int, experts_per_token: int, rank: int, world: int, group=None,
                 overlap_shared: bool = True):
        if num_experts % world != 0:
            raise ValueError(f"{num_experts} experts do not split over {world} ranks")
        self.backend = backend
        self.num_experts, self.k = num_experts, experts_per_token
        self.rank, self.world, self.group = rank, world, group
        self.experts_per_rank = num_experts // world
        self.last_plan: EpPlan | None = None
        self._events = None
        # The shared expert needs only this rank's own tokens and its result is read by the last kernel of
        # the layer, so it runs on a stream of its own beside the exchange (CUDA backends only).
        self._side = None
        self._ev_fork = self._ev_join = None
        if overlap_shared and torch.cuda.is_available() and getattr(backend, "supports_streams", False):
            self._side = torch.cuda.Stream()
            self._ev_fork, self._ev_join = torch.cuda.Event(), torch.cuda.Event()

    def forward(self, residual: torch.Tensor, tokens: int, ffn_out: torch.Tensor, l_out: torch.Tensor) -> None:
        b = self.backend
        mark = self._mark
        mark("start")
        ids, weights = b.front(residual, tokens)                    # [T,K] int32, [T,K] f32
        mark("front")
        if getattr(b, "peer_memory", False):
            # rows, counts and completion flags travel by peer stores over NVLink: no library
            # collective, no host read-back; the three calls below only enqueue kernels
            self._shared_fork()
            b.p2p_send()
            if self._side is None:
                b.shared()
            mark("plan_pack")
            b.p2p_experts(mark if self._events is not None else None)
            mark("experts")
            self._shared_join()
            b.p2p_finish(residual, tokens, ffn_out, l_out)
            mark("finish")
            return
        # rows grouped by owner rank (by expert inside a rank), and how many go to each rank
        send_rows, send_eid, inverse, send_counts = b.plan_pack(self.experts_per_rank, self.world)
        self._shared_fork()
        if self._side is None:
            b.shared()   # needs only this rank's tokens: keeps the GPU busy while the host reads the counts back
        plan = exchange_counts(send_counts, tokens * self.k, self.world, self.group)
        self.last_plan = plan
        mark("plan_pack")
        send_rows, send_eid = send_rows[:tokens * self.k], send_eid[:tokens * self.k]
        recv_rows = all_to_all_rows(send_rows, plan.send_counts, plan.recv_counts, self.world, self.group)
        recv_eid = all_to_all_rows(send_eid, plan.send_counts, plan.recv_counts, self.world, self.group)
        mark("dispatch_exchange")
        out = b.experts(recv_rows, recv_eid)                        # [R,H] f32, unweighted
        mark("experts")
        back = all_to_all_rows(out, plan.recv_counts, plan.send_counts, self.world, self.group)
        mark("combine_exchange")
        self._shared_join()
        b.finish(back, inverse, residual, tokens, ffn_out, l_out)  # weight, sum ascending k, shared expert, residual
        mark("finish")

    def _shared_fork(self) -> None:
        """Starts the shared expert on the side stream, after everything enqueued so far (the front)."""
        if self._side is None:
            return
        main = torch.cuda.current_stream()
        self._ev_fork.record(main)
        self._side.wait_event(self._ev_fork)
        self.backend.shared(stream=self._side)
        self._ev_join.record(self._side)

    def _shared_join(self) -> None:
        if self._side is not None:
            torch.cuda.current_stream().wait_event(self._ev_join)

    # -- optional per-phase device timing (CUDA events on the current stream), for the benchmark
    def enable_phase_timing(self) -> None:
        self._events = []

    def _mark(self, name: str) -> None:
        if self._events is None:
            return
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self._events.append((name, ev))

    def phase_times_ms(self) -> dict:
        """Total device time per phase since enable_phase_timing(); synchronises."""
        torch.cuda.synchronize()
        out: dict = {}
        ev = self._events or []
        for (_, e0), (name, e1) in zip(ev, ev[1:]):
            if name != "start":
                ms = e0.elapsed_time(e1)
                out[name] = out.get(name, 0.0) + ms
                if ":" in name:     # a part of a phase ("experts:tables"): counted in the phase as well
                    phase = name.split(":")[0]
                    out[phase] = out.get(phase, 0.0) + ms
        self._events = []
        return out


class CudaEpBackend:
    """The product backend: two C-ABI handles per rank (front: routing, shared expert, combine;
    back: the local experts over received rows, k = 1).  Rows travel as f16 and are read in place by
    the expert kernels; expert outputs travel as f32 and are weighted and summed by the sender."""

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
        pairs = geometry.max_tokens * geometry.experts_per_token
        self.ids_buf = torch.zeros(max_rows, 1, dtype=torch.int32, device=dev)
        self.ones = torch.ones(max_rows, 1, dtype=torch.float32, device=dev)
        self.send_rows = torch.empty(pairs, geometry.hidden, dtype=torch.float16, device=dev)
        self.send_eid = torch.empty(pairs, dtype=torch.int32, device=dev)
        self.inverse = torch.empty(pairs, dtype=torch.int32, device=dev)
        self.send_counts = torch.zeros(geometry.num_experts, dtype=torch.int32, device=dev)
        # the owner applies no weights: set them to one, once (no live rows yet, so the tables stay empty)
        self.back_k.set_valid_tokens(0)
        self.back_k.build_dispatch(self.ids_buf, self.ones)

    def set_layer(self, front_weights, local_gate, local_up, local_down) -> None:
        self.w = front_weights
        self.local = (local_gate, local_up, local_down)

    def front(self, residual, tokens):
        k = self.front_k
        k.set_valid_tokens(tokens)
        k.rms_norm(residual, self.w.post_norm)
        k.router_logits(self.w.router, self.w.router_bias)
        k.route_and_dispatch()
        return self.fb.topk_ids, self.fb.topk_weights

    def plan_pack(self, experts_per_rank, world):
        self.front_k.ep_plan_pack(experts_per_rank, self.send_rows, self.send_eid, self.inverse, self.send_counts[:world])
        return self.send_rows, self.send_eid, self.inverse, self.send_counts[:world]

    def experts(self, rows, local_expert):
        R = rows.shape[0]
        if R > self.max_rows:
            from .errors import TooManyTokens
            raise TooManyTokens(f"{R} received rows exceed the {self.max_rows} this rank was sized for")
        k = self.back_k
        k.set_valid_tokens(R)
        self.ids_buf[:R, 0] = local_expert
        k.build_dispatch(self.ids_buf, None)
        k.grouped_forward_partial_f16(self.local[0], self.local[1], self.local[2], rows)
        return self.bb.partial[:R]

    supports_streams = True

    def shared(self, stream=None):
        self.front_k.shared_expert(self.w.shared_gate, self.w.shared_up, self.w.shared_down, stream=stream)

    def finish(self, back, inverse, residual, tokens, ffn_out, l_out):
        k = self.front_k
        k.ep_combine(back, inverse, self.w.shared_gate_inp, residual, ffn_out, l_out)


class SharedBuffer:
    """A zeroed device buffer of this rank that every rank of the node has mapped (CUDA IPC, peer access
    over NVLink).  `ptrs[r]` is rank r's buffer as this process sees it; `own` is a tensor over this rank's."""

    def __init__(self, shape, dtype: torch.dtype, rank: int, world: int, group=None):
        import ctypes as C

        from . import _lib
        from .moe import _check, _view
        lib = _lib.lib()
        nbytes = int(torch.empty((), dtype=dtype).element_size())
        for d in shape:
            nbytes *= int(d)
        own_ptr, handle = C.c_void_p(), (C.c_ubyte * 64)()
        _check(lib.xabe_ipc_alloc(nbytes, C.byref(own_ptr), handle))
        self._own_ptr, self._opened, self._lib = own_ptr.value, [], lib
        dev = torch.cuda.current_device()
        self.own = _view(own_ptr.value, tuple(shape), dtype, dev, self)
        self.ptrs = [own_ptr.value]
        if world > 1:
            gathered: list = [None] * world
            dist.all_gather_object(gathered, bytes(handle), group=group)
            self.ptrs = []
            for r, h in enumerate(gathered):
                if r == rank:
                    self.ptrs.append(own_ptr.value)
                    continue
                p = C.c_void_p()
                _check(lib.xabe_ipc_open((C.c_ubyte * 64).from_buffer_copy(h), C.byref(p)))
                self._opened.append(p.value)
                self.ptrs.append(p.value)

    def release(self) -> None:
        """Unmaps the peers' buffers and frees this rank's; call on every rank after a barrier."""
        for p in self._opened:
            self._lib.xabe_ipc_close(p)
        self._opened = []
        if self._own_ptr:
            self._lib.xabe_ipc_free(self._own_ptr)
            self._own_ptr = None


class PeerMemoryEpBackend(CudaEpBackend):
    """CudaEpBackend whose two exchanges are peer stores over NVLink (`csrc/ep_kernels.cuh`) instead of
    NCCL all-to-alls.  The owner-side handle sees `world` receive regions of `cap` rows each (cap = the
    most pairs one rank can send), most of them empty; rows that hold nothing carry expert id -1."""

    peer_memory = True

    def __init__(self, geometry, experts_per_rank: int, rank: int, world: int, front_weights, local_gate, local_up,
                 local_down, eps: float = 1e-6, exact_decode: bool = False, group=None, fused_return: bool = True):
        from . import _lib
        self.fused_return = fused_return
        cap = geometry.max_tokens * geometry.experts_per_token
        super().__init__(geometry, experts_per_rank, world * cap, front_weights, local_gate, local_up, local_down,
                         eps=eps, exact_decode=exact_decode)
        self.rank, self.world, self.cap, self.epr = rank, world, cap, experts_per_rank
        dev, H = self.fb.normed.device, geometry.hidden
        mk = lambda shape, dtype: SharedBuffer(shape, dtype, rank, world, group)
        self._shared = {"rows": mk((world * cap, H), torch.float16), "eid": mk((world * cap,), torch.int32),
                        "meta": mk((world * 2,), torch.int32), "flag_in": mk((world,), torch.int32),
                        "back": mk((cap, H), torch.float32), "flag_back": mk((world,), torch.int32)}
        self._own = {name: b.own for name, b in self._shared.items()}
        self.peers = _lib.EpPeersC()
        for name, b in self._shared.items():
            arr = getattr(self.peers, name)
            for r, p in enumerate(b.ptrs):
                arr[r] = p
        self.slot_ids = torch.full((world * cap, 1), -1, dtype=torch.int32, device=dev)
        self.result_dst = torch.zeros(world * cap, dtype=torch.int64, device=dev)
        self.step = 0
        self.back_k.set_valid_tokens(world * cap)     # every receive slot is a "token"; empty ones are skipped by id
        if world > 1:
            dist.barrier(group=group)                 # nobody writes into a peer before all mappings exist

    def p2p_send(self):
        self.step += 1
        self.front_k.ep_p2p_send(self.epr, self.world, self.rank, self.cap, self.peers, self.step, self.inverse)

    def p2p_experts(self, mark=None):
        """The owner's step.  `mark(name)` (optional) records a device event after each part, for the
        benchmark's per-phase timing."""
        mark = mark or (lambda name: None)
        k = self.back_k
        k.ep_p2p_receive(self.world, self.rank, self.cap, self.peers, self.step, self.slot_ids, self.result_dst)
        mark("experts:wait_rows+slots")
        k.build_dispatch(self.slot_ids, None)
        mark("experts:tables")
        if self.fused_return:   # the down projection's epilogue stores each result row at its sender
            k.set_result_destinations(self.result_dst)
        k.grouped_forward_partial_f16(self.local[0], self.local[1], self.local[2], self._own["rows"])
        mark("experts:gemms")
        k.ep_p2p_return(self.world, self.rank, self.cap, self.peers, self.step, self.result_dst)
        k.set_result_destinations(None)

    def p2p_finish(self, residual, tokens, ffn_out, l_out):
        k = self.front_k
        k.ep_p2p_wait_results(self.world, self.rank, self.peers, self.step)
        k.ep_combine(self._own["back"], self.inverse, self.w.shared_gate_inp, residual, ffn_out, l_out)
