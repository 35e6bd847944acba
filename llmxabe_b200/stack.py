"""A stack of MoE blocks driven like the reference's `Forward::body`
(crates/xabe-engine/src/forward.rs:3497-3618), for models whose layers, as far
as this library is concerned, are MoE blocks only: one `MoeBlock` serves every
layer with that layer's weights, the block's `l_out` is the next layer's
residual, and the whole pass is launches only, so it is captured once as a CUDA
graph and replayed at any live token count (the count is a device scalar,
published before the replay as `Forward::prepare` does, forward.rs:3480-3484).

The mixers (attention / gated delta net), the embedding gather and the LM head
of `Forward::body` are outside this library; a caller that has them interleaves
`MoeBlock.forward` itself, exactly as the reference's loop does.
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, Sequence

import torch

from . import _lib
from .errors import InvalidArgument
from .moe import MoeBlock, MoeGeometry, MoeLayerWeights, DEFAULT_RMS_EPS, _check, _stream_ptr

# on_waypoint(layer, hidden_state): fired after each layer's block on the eager path
# (WaypointStage::Moe, forward.rs:3576-3577); a captured pass takes none.
Waypoint = Callable[[int, torch.Tensor], None]


class MoeStack:
    """`layers` MoE blocks sharing one handle and one pair of hidden-state buffers."""

    def __init__(self, geometry: MoeGeometry, layers: Sequence[MoeLayerWeights], eps: float = DEFAULT_RMS_EPS,
                 device: int | None = None):
        if not layers:
            raise InvalidArgument("a stack needs at least one layer")
        self.geometry = geometry
        self.layers = list(layers)
        self.block = MoeBlock(geometry, eps, device)
        dev = torch.device("cuda", torch.cuda.current_device() if device is None else device)
        shape = (geometry.max_tokens, geometry.hidden)
        # `hidden_state` and `mixer_out` of the reference, which alternate as residual and l_out
        self._hidden = [torch.zeros(shape, device=dev), torch.zeros(shape, device=dev)]
        self.ffn_out = torch.zeros(shape, device=dev)
        self._weights_c = (_lib.LayerWeightsC * len(self.layers))(*[w._c() for w in self.layers])
        self._graph: torch.cuda.CUDAGraph | None = None
        self.tokens = 0

    @property
    def hidden_in(self) -> torch.Tensor:
        """[max_tokens][hidden] f32: write the live rows here before a pass."""
        return self._hidden[0]

    @property
    def hidden_out(self) -> torch.Tensor:
        """[max_tokens][hidden] f32: the last layer's l_out after a pass."""
        return self._hidden[len(self.layers) % 2]

    def publish_tokens(self, tokens: int, stream=None) -> None:
        """Forward::prepare's `moe.publish_tokens` (forward.rs:3483): the device scalar a replay reads."""
        self.block.publish_tokens(tokens, stream)  # raises TooManyTokens past max_tokens
        self.tokens = tokens

    def body(self, stream=None, on_waypoint: Waypoint | None = None) -> None:
        """One pass over all layers at the published token count.  Without a waypoint callback this
        is ONE library call that enqueues every layer; with one, the layers are enqueued one by one
        and the callback sees each layer's l_out (the caller synchronises if it reads it)."""
        if on_waypoint is None:
            out = C.c_void_p()
            _check(_lib.lib().xabe_moe_stack_forward(self.block.moe._h, _stream_ptr(stream), self._weights_c,
                                                     len(self.layers), self._hidden[0].data_ptr(),
                                                     self._hidden[1].data_ptr(), self._hidden[0].numel(),
                                                     self.tokens, self.ffn_out.data_ptr(), self.ffn_out.numel(),
                                                     C.byref(out)))
            assert out.value == self.hidden_out.data_ptr()
            return
        for i, w in enumerate(self.layers):
            src, dst = self._hidden[i % 2], self._hidden[(i + 1) % 2]
            self.block.forward(w, src, self.tokens, self.ffn_out, dst, stream)
            on_waypoint(i, dst)

    def capture(self) -> None:
        """Captures `body` as a CUDA graph (the reference captures its decode bodies,
        forward.rs:2059,3145).  The count published at capture time is only the count of the
        warm-up pass: a replay runs at whatever `publish_tokens` set last."""
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.body()  # warm-up outside capture: attribute set-up and first-use work happen here
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.body()
        torch.cuda.synchronize()
        self._graph = graph

    def replay(self) -> None:
        if self._graph is None:
            raise InvalidArgument("capture() has not been called")
        self._graph.replay()

    def run(self, x: torch.Tensor, on_waypoint: Waypoint | None = None) -> torch.Tensor:
        """Convenience for tests: copies `x` [tokens][hidden] in, publishes its row count, runs one
        pass (the graph if captured and no waypoints are asked for) and returns the live rows of the
        final hidden state."""
        tokens = int(x.shape[0])
        self.publish_tokens(tokens)
        self._hidden[0][:tokens].copy_(x)
        if self._graph is not None and on_waypoint is None:
            self.replay()
        else:
            self.body(on_waypoint=on_waypoint)
        return self.hidden_out[:tokens]
