"""Host-side mirror of the reference's MoE block interface over the C ABI.

Names, argument meaning and error behaviour follow the reference so that its
tests read the same here:

  MoeGeometry, ExpertQuant, QuantTensor, MoeKernels
      crates/xabe-cuda/src/kernels/moe.rs:4523-4598, 298-401, 448-464, 4969-6727
  MoeLayerWeights, MoeBlock
      crates/xabe-engine/src/block/moe.rs:634-800, 895-1330
  FfnBlock, DenseFfnBlock
      crates/xabe-engine/src/block/ffn.rs:27-228, block/dense_ffn.rs:1047

PyTorch supplies device memory and streams only; every computation is a call
into libxabe_moe_sm100.so.  There is no CPU path.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from enum import IntEnum

import numpy as np
import torch

from . import _lib
from .errors import InvalidArgument, check

DEFAULT_RMS_EPS = 1e-6  # crates/xabe-engine/src/block/moe.rs:179


class ExpertQuant(IntEnum):
    """ExpertQuant::code, moe.rs:319-327 (the two shipped formats)."""
    Q6K = 0
    Q8_0 = 1

    @property
    def block_elements(self) -> int:
        return 256 if self is ExpertQuant.Q6K else 32

    @property
    def file_block_bytes(self) -> int:
        return 210 if self is ExpertQuant.Q6K else 34


@dataclass(frozen=True)
class MoeGeometry:
    """moe.rs:4523-4540.  Fixed at construction; every buffer and grid derives from it."""
    num_experts: int
    experts_per_token: int
    hidden: int
    intermediate: int
    block_size: int
    max_tokens: int

    @staticmethod
    def qwen3_6(block_size: int, max_tokens: int) -> "MoeGeometry":
        return MoeGeometry(256, 8, 2048, 512, block_size, max_tokens)

    @staticmethod
    def qwen3_8_27b_dense(block_size: int, max_tokens: int) -> "MoeGeometry":
        """Dense sibling: hidden 5120, intermediate 17408 (crates/xabe-model/src/config.rs:307-395)."""
        return MoeGeometry(0, 0, 5120, 17408, block_size, max_tokens)

    def max_flat_pairs(self) -> int:
        return self.max_tokens * self.experts_per_token

    def sorted_capacity(self) -> int:
        return int(_lib.lib().xabe_moe_sorted_capacity(self._c()))

    def expert_block_capacity(self) -> int:
        return int(_lib.lib().xabe_moe_expert_block_capacity(self._c()))

    def stack_elements(self) -> int:
        return self.num_experts * self.intermediate * self.hidden

    def _c(self) -> _lib.GeometryC:
        return _lib.GeometryC(self.num_experts, self.experts_per_token, self.hidden, self.intermediate,
                              self.block_size, self.max_tokens)


def moe_block_size(tokens: int) -> int:
    """crates/xabe-engine/src/forward.rs:163-165."""
    return 32 if tokens <= 1152 else 64


@dataclass
class QuantTensor:
    """moe.rs:448-464: device bytes in GGUF file layout plus their format."""
    bytes: torch.Tensor  # uint8, on the device
    quant: ExpertQuant

    def _c(self) -> _lib.QuantTensorC:
        return _lib.QuantTensorC(self.bytes.data_ptr(), self.bytes.numel(), int(self.quant))


def _stream_ptr(stream) -> int:
    if stream is None:
        stream = torch.cuda.current_stream()
    return stream.cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _check(rc: int) -> None:
    if rc != 0:
        check(rc, _lib.lib().xabe_moe_last_error())


class MoeKernels:
    """The device kernel set (lower seam).  One instance per worker thread."""

    SCOPE_ROUTED, SCOPE_SHARED_ONLY = 0, 1

    def __init__(self, geometry: MoeGeometry, device: int | None = None, *, eps: float = DEFAULT_RMS_EPS,
                 scope: int = 0):
        self._h = C.c_void_p()
        self.geometry = geometry
        self.scope = scope
        if device is None:
            device = torch.cuda.current_device() if torch.cuda.is_available() else 0
        self.device = device
        L = _lib.lib()
        rc = L.xabe_moe_create(geometry._c(), device, scope, eps, C.byref(self._h))
        _check(rc)

    def close(self) -> None:
        if getattr(self, "_h", None) is not None and self._h.value:
            _lib.lib().xabe_moe_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- MoeKernels::set_valid_tokens, moe.rs:5473
    def set_valid_tokens(self, tokens: int, stream=None) -> None:
        _check(_lib.lib().xabe_moe_set_valid_tokens(self._h, _stream_ptr(stream), tokens))

    # -- LayerOpsKernels::rms_norm as the block calls it
    def rms_norm(self, x: torch.Tensor, weight: torch.Tensor, stream=None) -> None:
        _check(_lib.lib().xabe_moe_rms_norm(self._h, _stream_ptr(stream), x.data_ptr(), weight.data_ptr()))

    def router_logits(self, router: torch.Tensor, bias: torch.Tensor | None = None, stream=None) -> None:
        _check(_lib.lib().xabe_moe_router_logits(self._h, _stream_ptr(stream), router.data_ptr(), _ptr(bias)))

    # -- MoeKernels::route_and_dispatch, moe.rs:5498
    def route_and_dispatch(self, logits: torch.Tensor | None = None, stream=None) -> None:
        _check(_lib.lib().xabe_moe_route_and_dispatch(self._h, _stream_ptr(stream), _ptr(logits)))

    # -- MoeKernels::build_dispatch, moe.rs:5623
    def build_dispatch(self, topk_ids: torch.Tensor | None = None, topk_weights: torch.Tensor | None = None,
                       stream=None) -> None:
        _check(_lib.lib().xabe_moe_build_dispatch(self._h, _stream_ptr(stream), _ptr(topk_ids), _ptr(topk_weights)))

    # -- the last launch of MoeBlock::forward, block/moe.rs:1297-1326
    def gate_and_combine(self, shared_gate_inp: torch.Tensor, residual: torch.Tensor, ffn_out: torch.Tensor,
                         l_out: torch.Tensor, stream=None) -> None:
        _check(_lib.lib().xabe_moe_gate_and_combine(self._h, _stream_ptr(stream), shared_gate_inp.data_ptr(),
                                                    residual.data_ptr(), residual.numel(), ffn_out.data_ptr(),
                                                    ffn_out.numel(), l_out.data_ptr(), l_out.numel()))

    # -- expert parallelism (no counterpart in the reference): see include/xabe_moe.h
    def grouped_forward_partial_f16(self, gate: QuantTensor, up: QuantTensor, down: QuantTensor,
                                    rows_f16: torch.Tensor, stream=None) -> None:
        _check(_lib.lib().xabe_moe_grouped_forward_partial_f16(self._h, _stream_ptr(stream), gate._c(), up._c(),
                                                               down._c(), rows_f16.data_ptr(), rows_f16.shape[0]))

    def ep_pack(self, order: torch.Tensor, experts_per_rank: int, send_rows: torch.Tensor,
                send_local_expert: torch.Tensor, inverse: torch.Tensor, stream=None) -> None:
        _check(_lib.lib().xabe_moe_ep_pack(self._h, _stream_ptr(stream), order.data_ptr(), order.numel(),
                                           experts_per_rank, send_rows.data_ptr(), send_local_expert.data_ptr(),
                                           inverse.data_ptr()))

    def ep_plan_pack(self, experts_per_rank: int, send_rows: torch.Tensor, send_local_expert: torch.Tensor,
                     inverse: torch.Tensor, send_counts: torch.Tensor, stream=None) -> None:
        _check(_lib.lib().xabe_moe_ep_plan_pack(self._h, _stream_ptr(stream), experts_per_rank,
                                                send_rows.data_ptr(), send_local_expert.data_ptr(),
                                                inverse.data_ptr(), send_counts.data_ptr()))

    # -- expert-parallel exchange over peer memory: see include/xabe_moe.h (xabe_ep_peers)
    def ep_p2p_send(self, experts_per_rank: int, world: int, rank: int, cap: int, peers, step: int,
                    inverse: torch.Tensor, stream=None) -> None:
        _check(_lib.lib().xabe_moe_ep_p2p_send(self._h, _stream_ptr(stream), experts_per_rank, world, rank, cap,
                                               C.byref(peers), step, inverse.data_ptr()))

    def ep_p2p_receive(self, world: int, rank: int, cap: int, peers, step: int, ids_out: torch.Tensor,
                       result_dst: torch.Tensor, stream=None) -> None:
        _check(_lib.lib().xabe_moe_ep_p2p_receive(self._h, _stream_ptr(stream), world, rank, cap, C.byref(peers),
                                                  step, ids_out.data_ptr(), result_dst.data_ptr()))

    def ep_p2p_return(self, world: int, rank: int, cap: int, peers, step: int, result_dst: torch.Tensor,
                      stream=None) -> None:
        _check(_lib.lib().xabe_moe_ep_p2p_return(self._h, _stream_ptr(stream), world, rank, cap, C.byref(peers),
                                                 step, result_dst.data_ptr()))

    def set_result_destinations(self, table: torch.Tensor | None) -> None:
        _check(_lib.lib().xabe_moe_set_result_destinations(self._h, _ptr(table)))

    def ep_p2p_wait_results(self, world: int, rank: int, peers, step: int, stream=None) -> None:
        _check(_lib.lib().xabe_moe_ep_p2p_wait_results(self._h, _stream_ptr(stream), world, rank, C.byref(peers),
                                                       step))

    def ep_combine(self, back_rows: torch.Tensor, inverse: torch.Tensor, shared_gate_inp: torch.Tensor,
                   residual: torch.Tensor, ffn_out: torch.Tensor, l_out: torch.Tensor, stream=None) -> None:
        _check(_lib.lib().xabe_moe_ep_combine(self._h, _stream_ptr(stream), back_rows.data_ptr(),
                                              back_rows.shape[0], inverse.data_ptr(), shared_gate_inp.data_ptr(),
                                              residual.data_ptr(), residual.numel(), ffn_out.data_ptr(),
                                              ffn_out.numel(), l_out.data_ptr(), l_out.numel()))

    # -- MoeKernels::grouped_forward_partial, moe.rs:5727
    def grouped_forward_partial(self, gate: QuantTensor, up: QuantTensor, down: QuantTensor,
                                hidden_states: torch.Tensor | None = None, stream=None) -> None:
        _check(_lib.lib().xabe_moe_grouped_forward_partial(self._h, _stream_ptr(stream), gate._c(), up._c(),
                                                           down._c(), _ptr(hidden_states)))

    # -- MoeKernels::grouped_forward, moe.rs:6345
    def grouped_forward(self, gate: QuantTensor, up: QuantTensor, down: QuantTensor,
                        hidden_states: torch.Tensor | None, out: torch.Tensor, stream=None) -> None:
        _check(_lib.lib().xabe_moe_grouped_forward(self._h, _stream_ptr(stream), gate._c(), up._c(), down._c(),
                                                   _ptr(hidden_states), out.data_ptr()))

    # -- MoeKernels::shared_expert, moe.rs:6488
    def shared_expert(self, gate: QuantTensor, up: QuantTensor, down: QuantTensor,
                      hidden_states: torch.Tensor | None = None, out: torch.Tensor | None = None,
                      stream=None) -> None:
        _check(_lib.lib().xabe_moe_shared_expert(self._h, _stream_ptr(stream), gate._c(), up._c(), down._c(),
                                                 _ptr(hidden_states), _ptr(out)))

    def set_exact_decode_regime(self, on: bool) -> None:
        _check(_lib.lib().xabe_moe_set_exact_decode_regime(self._h, int(on)))

    # -- MoeKernels::disable_tensor_cores / tensor_cores_enabled, moe.rs:5416-5458
    def disable_tensor_cores(self) -> None:
        _check(_lib.lib().xabe_moe_disable_tensor_cores(self._h))

    def tensor_cores_enabled(self) -> bool:
        return bool(_lib.lib().xabe_moe_tensor_cores_enabled(self._h))

    def force_prefill_path(self, on: bool) -> None:
        """The tcgen05 kernels at every width (differential tests); choose before route_and_dispatch."""
        _check(_lib.lib().xabe_moe_force_prefill_path(self._h, int(on)))

    TUNE = {"pdl": 0, "stream_stages": 1, "stream_runs": 2, "rows_min_tokens": 3, "router_regw": 4,
            "force_tile_kernels": 5, "prefill_wide": 6, "fused_decode": 7, "dense_rows": 8}

    def set_tuning(self, key: str, value: int) -> None:
        """Per-handle launch-shape switches (XABE_TUNE_* of include/xabe_moe.h); results do not change."""
        _check(_lib.lib().xabe_moe_set_tuning(self._h, self.TUNE[key], int(value)))

    def set_peer_wait_limit(self, iterations: int) -> None:
        _check(_lib.lib().xabe_moe_set_peer_wait_limit(self._h, iterations))

    def device_status(self, stream=None) -> int:
        """The status word the kernels' bounded waits write (read and cleared); raises DeviceStatus when non-zero."""
        st = C.c_int(0)
        _check(_lib.lib().xabe_moe_device_status(self._h, _stream_ptr(stream), C.byref(st)))
        return st.value

    STAGES = ("rms_norm", "router_logits", "route_dispatch", "gate_up", "down", "combine")

    def stage_profile(self, on: bool) -> None:
        """StageProfile of the reference (crates/xabe-engine/src/forward.rs:783-855)."""
        _check(_lib.lib().xabe_moe_stage_profile(self._h, int(on)))

    def stage_times(self, stream=None) -> tuple[dict, int]:
        """Summed milliseconds per stage and the number of block calls they cover."""
        ms = (C.c_float * len(self.STAGES))()
        calls = C.c_int(0)
        _check(_lib.lib().xabe_moe_stage_times(self._h, _stream_ptr(stream), ms, C.byref(calls)))
        return dict(zip(self.STAGES, [float(v) for v in ms])), calls.value

    # -- MoeBuffers accessors as torch views over the handle's scratch
    def buffers(self) -> "MoeBuffers":
        v = _lib.BufferViewC()
        _check(_lib.lib().xabe_moe_buffers(self._h, C.byref(v)))
        return MoeBuffers(self, v)


def _view(ptr: int, shape, dtype: torch.dtype, device: int, owner) -> torch.Tensor:
    """A torch tensor over memory the handle owns (kept alive by `owner`)."""
    n = int(np.prod(shape))
    itemsize = torch.empty((), dtype=dtype).element_size()

    class _Mem:
        pass

    mem = _Mem()
    mem.__cuda_array_interface__ = {
        "shape": (n * itemsize,), "typestr": "|u1", "data": (int(ptr), False), "version": 2}
    mem._owner = owner
    t = torch.as_tensor(mem, device=f"cuda:{device}")
    return t.view(dtype).view(*shape)


class MoeBuffers:
    """moe.rs:4713-4864 plus the block intermediates (block/moe.rs:1022-1060)."""

    def __init__(self, kernels: MoeKernels, v: _lib.BufferViewC):
        g, d = kernels.geometry, kernels.device
        self.sorted_capacity = int(v.sorted_capacity)
        self.expert_block_capacity = int(v.expert_block_capacity)
        T, K, H, E = g.max_tokens, g.experts_per_token, g.hidden, g.num_experts
        mk = lambda p, shape, dt: _view(p, shape, dt, d, kernels) if p else None
        self.valid_tokens = mk(v.valid_tokens, (1,), torch.int32)
        self.topk_ids = mk(v.topk_ids, (T, K), torch.int32)
        self.topk_weights = mk(v.topk_weights, (T, K), torch.float32)
        self.sorted_token_ids = mk(v.sorted_token_ids, (self.sorted_capacity,), torch.int32)
        self.expert_ids = mk(v.expert_ids, (self.expert_block_capacity,), torch.int32)
        self.num_tokens_post_pad = mk(v.num_tokens_post_pad, (1,), torch.int32)
        self.partial = mk(v.partial, (T * K, H), torch.float32)
        self.normed = mk(v.normed, (T, H), torch.float32)
        self.logits = mk(v.logits, (T, E), torch.float32)
        self.routed = mk(v.routed, (T, H), torch.float32)
        self.shexp = mk(v.shexp, (T, H), torch.float32)
        self.gate = mk(v.gate, (T,), torch.float32)


def kernel_launch_count() -> int:
    """Kernels this library has launched in this process so far (see include/xabe_moe.h)."""
    return int(_lib.lib().xabe_kernel_launch_count())


def dequantize(t: QuantTensor, stream=None) -> torch.Tensor:
    """Standalone dequantisation (crates/xabe-cuda/src/kernels/dequant.rs), bit-identical to the scalar reference."""
    n = t.bytes.numel() // t.quant.file_block_bytes * t.quant.block_elements
    out = torch.empty(n, dtype=torch.float32, device=t.bytes.device)
    _check(_lib.lib().xabe_dequantize(_stream_ptr(stream), t._c(), out.data_ptr()))
    return out


def stream_read(data: torch.Tensor, sink: torch.Tensor, stream=None) -> None:
    """Benchmark calibration: one pure streaming read of `data`'s bytes (see include/xabe_moe.h)."""
    _check(_lib.lib().xabe_stream_read(_stream_ptr(stream), data.data_ptr(), data.numel() * data.element_size(),
                                       sink.data_ptr()))


def shared_expert_noalloc(gate: QuantTensor, up: QuantTensor, down: QuantTensor, hidden: int, intermediate: int,
                          hidden_states: torch.Tensor, tokens: int, out: torch.Tensor, stream=None) -> None:
    """Shared-expert MLP for callers that cannot allocate device memory (no handle, static scratch).

    Meant for a worker whose memory was all handed out at start-up, or for code that runs where the
    CUDA allocator must not be entered.  Limits: tokens <= 64, hidden <= 2048, intermediate <= 512.
    Calls share one static scratch array, so keep them on one stream; make the first call on a device
    before any stream capture.
    """
    _check(_lib.lib().xabe_shared_expert_noalloc(_stream_ptr(stream), gate._c(), up._c(), down._c(), hidden,
                                                 intermediate, hidden_states.data_ptr(), tokens, out.data_ptr()))


def shared_expert_noalloc_status(stream=None) -> int:
    """The status word of the static scratch after the last `shared_expert_noalloc` call on `stream`
    (0 = every bounded wait completed); synchronises the stream, allocates nothing."""
    st = C.c_int(-1)
    _check(_lib.lib().xabe_shared_expert_noalloc_status(_stream_ptr(stream), C.byref(st)))
    return st.value


class MoeLayerWeights:
    """One layer's MoE weights resident on the device (block/moe.rs:634-658).

    Quantized stacks are uploaded in GGUF file layout, unchanged.  Dense
    tensors arrive as float32; bf16 routers are widened on the host exactly
    (block/moe.rs:823-855) by `upload`'s caller handing float32.
    """

    def __init__(self, *, layer: int, post_norm, router, gate_exps, gate_quant, up_exps, up_quant, down_exps,
                 down_quant, shared_gate_inp, shared_gate, shared_gate_quant, shared_up, shared_up_quant,
                 shared_down, shared_down_quant, router_bias=None, device="cuda"):
        self.layer = layer
        dev = torch.device(device)

        def dense(x, name):
            t = torch.as_tensor(x)
            if t.dtype == torch.bfloat16:
                t = t.float()  # exact widening
            if t.dtype != torch.float32:
                from .errors import UnsupportedDenseType
                raise UnsupportedDenseType(
                    f"tensor `{name}` is {t.dtype}, and this block only widens f32 and bf16")
            return t.contiguous().to(dev)

        def quant(x, q, name):
            t = torch.as_tensor(x)
            if t.dtype != torch.uint8:
                raise InvalidArgument(f"`{name}` must be raw uint8 GGUF bytes")
            return QuantTensor(t.contiguous().view(-1).to(dev), ExpertQuant(q))

        self.post_norm = dense(post_norm, "post_attention_norm.weight")
        self.router = dense(router, "ffn_gate_inp.weight")
        self.router_bias = None if router_bias is None else dense(router_bias, "router bias")
        self.shared_gate_inp = dense(shared_gate_inp, "ffn_gate_inp_shexp.weight")
        self.gate_exps = quant(gate_exps, gate_quant, "ffn_gate_exps")
        self.up_exps = quant(up_exps, up_quant, "ffn_up_exps")
        self.down_exps = quant(down_exps, down_quant, "ffn_down_exps")
        self.shared_gate = quant(shared_gate, shared_gate_quant, "ffn_gate_shexp")
        self.shared_up = quant(shared_up, shared_up_quant, "ffn_up_shexp")
        self.shared_down = quant(shared_down, shared_down_quant, "ffn_down_shexp")

    def _c(self) -> _lib.LayerWeightsC:
        return _lib.LayerWeightsC(self.post_norm.data_ptr(), self.router.data_ptr(), _ptr(self.router_bias),
                                  self.gate_exps._c(),
                                  self.up_exps._c(), self.down_exps._c(), self.shared_gate_inp.data_ptr(),
                                  self.shared_gate._c(), self.shared_up._c(), self.shared_down._c())

    def device_bytes(self) -> int:
        return sum(t.bytes.numel() for t in (self.gate_exps, self.up_exps, self.down_exps, self.shared_gate,
                                             self.shared_up, self.shared_down)) + \
            4 * (self.post_norm.numel() + self.router.numel() + self.shared_gate_inp.numel())


class MoeBlock:
    """The MoE block (upper seam), block/moe.rs:895-1330."""

    def __init__(self, geometry: MoeGeometry, eps: float = DEFAULT_RMS_EPS, device: int | None = None):
        self.geometry = geometry
        self.eps = eps
        self.moe = MoeKernels(geometry, device, eps=eps, scope=MoeKernels.SCOPE_ROUTED)
        self._buffers = self.moe.buffers()

    @staticmethod
    def geometry_for(hidden: int, num_experts: int, experts_per_token: int, expert_intermediate: int,
                     block_size: int, max_tokens: int) -> MoeGeometry:
        """block/moe.rs:931-946 with the config fields spelled out."""
        return MoeGeometry(num_experts, experts_per_token, hidden, expert_intermediate, block_size, max_tokens)

    def set_exact_decode_regime(self, on: bool) -> None:
        self.moe.set_exact_decode_regime(on)

    def publish_tokens(self, tokens: int, stream=None) -> None:
        """block/moe.rs:1074-1089."""
        self.moe.set_valid_tokens(tokens, stream)

    # observable intermediates, block/moe.rs:1022-1060
    def normed(self) -> torch.Tensor:
        return self._buffers.normed

    def router_logits(self) -> torch.Tensor:
        return self._buffers.logits

    def routed(self) -> torch.Tensor:
        return self._buffers.routed

    def shared_ungated(self) -> torch.Tensor:
        return self._buffers.shexp

    def shared_gate(self) -> torch.Tensor:
        return self._buffers.gate

    def buffers(self) -> MoeBuffers:
        return self._buffers

    def forward(self, w: MoeLayerWeights, residual: torch.Tensor, tokens: int, ffn_out: torch.Tensor,
                l_out: torch.Tensor, stream=None) -> None:
        """block/moe.rs:1091-1329.  All three buffers are [max_tokens][hidden] on the device; ffn_out and
        l_out float32; the residual float32 (as in the reference) or bfloat16 (widened exactly inside)."""
        wc = w._c()
        if residual.dtype == torch.bfloat16:
            _check(_lib.lib().xabe_moe_block_forward_typed(self.moe._h, _stream_ptr(stream), C.byref(wc),
                                                           residual.data_ptr(), 1, residual.numel(), tokens,
                                                           ffn_out.data_ptr(), ffn_out.numel(), l_out.data_ptr(),
                                                           l_out.numel()))
            return
        if residual.dtype != torch.float32:
            raise InvalidArgument(f"residual must be float32 or bfloat16, got {residual.dtype}")
        _check(_lib.lib().xabe_moe_block_forward(self.moe._h, _stream_ptr(stream), C.byref(wc),
                                                 residual.data_ptr(), residual.numel(), tokens,
                                                 ffn_out.data_ptr(), ffn_out.numel(), l_out.data_ptr(),
                                                 l_out.numel()))

    def forward_host(self, w: MoeLayerWeights, residual: torch.Tensor, tokens: int,
                     ffn_out: torch.Tensor | None, l_out: torch.Tensor | None, stream=None) -> None:
        """The same block for HOST (pinned) buffers: copies in, runs, copies out, all on `stream`."""
        for t in (residual, ffn_out, l_out):
            if t is not None and t.is_cuda:
                raise InvalidArgument("forward_host takes host tensors")
        wc = w._c()
        _check(_lib.lib().xabe_moe_block_forward_host(self.moe._h, _stream_ptr(stream), C.byref(wc),
                                                      residual.data_ptr(), tokens, _ptr(ffn_out), _ptr(l_out)))


class DenseFfnBlock:
    """Dense SwiGLU MLP block of the 27B sibling (block/dense_ffn.rs:9-16, 1047)."""

    def __init__(self, geometry: MoeGeometry, eps: float = DEFAULT_RMS_EPS, device: int | None = None):
        self.geometry = geometry
        self.moe = MoeKernels(geometry, device, eps=eps, scope=MoeKernels.SCOPE_SHARED_ONLY)

    def forward(self, post_norm: torch.Tensor, gate: QuantTensor, up: QuantTensor, down: QuantTensor,
                residual: torch.Tensor, tokens: int, ffn_out: torch.Tensor, l_out: torch.Tensor,
                stream=None) -> None:
        _check(_lib.lib().xabe_dense_ffn_block_forward(
            self.moe._h, _stream_ptr(stream), post_norm.data_ptr(), gate._c(), up._c(), down._c(),
            residual.data_ptr(), residual.numel(), tokens, ffn_out.data_ptr(), ffn_out.numel(),
            l_out.data_ptr(), l_out.numel()))


class FfnBlock:
    """Two-variant dispatch `FfnBlock::{Moe, Dense}` (block/ffn.rs:27-47, 199-220)."""

    def __init__(self, inner: MoeBlock | DenseFfnBlock):
        self.inner = inner

    @staticmethod
    def new_moe(geometry: MoeGeometry, eps: float = DEFAULT_RMS_EPS) -> "FfnBlock":
        return FfnBlock(MoeBlock(geometry, eps))

    @staticmethod
    def new_dense(geometry: MoeGeometry, eps: float = DEFAULT_RMS_EPS) -> "FfnBlock":
        return FfnBlock(DenseFfnBlock(geometry, eps))

    def as_moe(self) -> MoeBlock | None:
        return self.inner if isinstance(self.inner, MoeBlock) else None

    def publish_tokens(self, tokens: int, stream=None) -> None:
        if isinstance(self.inner, MoeBlock):
            self.inner.publish_tokens(tokens, stream)
        else:
            self.inner.moe.set_valid_tokens(tokens, stream)

    def forward(self, weights, residual, tokens, ffn_out, l_out, stream=None) -> None:
        from .errors import MoeError
        if isinstance(self.inner, MoeBlock):
            if not isinstance(weights, MoeLayerWeights):
                raise MoeError("a `moe` feed-forward block was handed `dense` weights")  # FfnKindMismatch
            self.inner.forward(weights, residual, tokens, ffn_out, l_out, stream)
        else:
            if isinstance(weights, MoeLayerWeights):
                raise MoeError("a `dense` feed-forward block was handed `moe` weights")
            post_norm, gate, up, down = weights
            self.inner.forward(post_norm, gate, up, down, residual, tokens, ffn_out, l_out, stream)
