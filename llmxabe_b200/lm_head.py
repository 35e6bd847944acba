"""Host mirror of the reference's LM head kernel set
(crates/xabe-cuda/src/kernels/lm_head.rs): `LmHeadGeometry`, `HeadFormat`,
`HeadTensor`, `LmHeadKernels::{forward, argmax}`, over the C ABI.  No CPU path.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from enum import IntEnum

import torch

from . import _lib
from .moe import _check, _stream_ptr

MAX_BATCH_TILE = 8  # tokens one pass over the weights serves (lm_head.rs:125)


class HeadFormat(IntEnum):
    """The formats this build reads (lm_head.rs:1206-1226 lists more: the dense 16-bit and the
    community formats are not built).  Values are the quant tags of the C ABI."""
    Q6K = 0
    Q8_0 = 1

    def block_elements(self) -> int:
        return 256 if self is HeadFormat.Q6K else 32

    def block_bytes(self) -> int:
        return 210 if self is HeadFormat.Q6K else 34

    @staticmethod
    def from_ggml(name: str) -> "HeadFormat | None":
        """lm_head.rs:1243-1256."""
        return {"q8_0": HeadFormat.Q8_0, "q6_K": HeadFormat.Q6K}.get(name)


@dataclass(frozen=True)
class LmHeadGeometry:
    """lm_head.rs:1304-1314."""
    hidden: int
    vocab: int
    max_tokens: int

    @staticmethod
    def qwen3_6(max_tokens: int) -> "LmHeadGeometry":
        """lm_head.rs:1318-1324."""
        return LmHeadGeometry(2048, 248_320, max_tokens)

    def row_bytes_for(self, fmt: HeadFormat) -> int:
        return self.hidden // fmt.block_elements() * fmt.block_bytes()

    def weight_bytes_for(self, fmt: HeadFormat) -> int:
        return self.vocab * self.row_bytes_for(fmt)

    def elements(self) -> int:
        return self.vocab * self.hidden

    def weight_passes(self, tokens: int) -> int:
        """lm_head.rs:1380-1383."""
        return -(-tokens // MAX_BATCH_TILE)

    def weight_bytes_read(self, tokens: int, fmt: HeadFormat = HeadFormat.Q8_0) -> int:
        """lm_head.rs:1389-1391: the denominator of an honest GB/s figure."""
        return self.weight_passes(tokens) * self.weight_bytes_for(fmt)

    def _c(self) -> _lib.HeadGeometryC:
        return _lib.HeadGeometryC(self.hidden, self.vocab, self.max_tokens)


@dataclass
class HeadTensor:
    """lm_head.rs:1261-1300: the head's bytes in file layout, on the device, with their format."""
    bytes: torch.Tensor
    format: HeadFormat

    def _c(self) -> _lib.QuantTensorC:
        return _lib.QuantTensorC(self.bytes.data_ptr(), self.bytes.numel(), int(self.format))


class LmHeadKernels:
    """lm_head.rs:1493-2015.  One instance per worker thread."""

    def __init__(self, geometry: LmHeadGeometry, device: int | None = None):
        self._h = C.c_void_p()
        self.geometry = geometry
        if device is None:
            device = torch.cuda.current_device() if torch.cuda.is_available() else 0
        self.device = device
        _check(_lib.lib().xabe_lm_head_create(geometry._c(), device, C.byref(self._h)))

    def close(self) -> None:
        if getattr(self, "_h", None) is not None and self._h.value:
            _lib.lib().xabe_lm_head_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def forward(self, weight: HeadTensor, hidden_states: torch.Tensor, tokens: int, logits: torch.Tensor,
                stream=None) -> None:
        """lm_head.rs:1695-1937: logits[t][v] for the first `tokens` rows; `hidden_states`
        [max_tokens][hidden] f32, `logits` [max_tokens][vocab] f32, both on the device."""
        _check(_lib.lib().xabe_lm_head_forward(self._h, _stream_ptr(stream), weight._c(), hidden_states.data_ptr(),
                                               hidden_states.numel(), tokens, logits.data_ptr(), logits.numel()))

    def argmax(self, logits: torch.Tensor, tokens: int, out: torch.Tensor, stream=None) -> None:
        """lm_head.rs:1950-2015: out[t] (int32, device) = index of the largest logit of row t, ties
        to the lower index."""
        _check(_lib.lib().xabe_lm_head_argmax(self._h, _stream_ptr(stream), logits.data_ptr(), logits.numel(),
                                              tokens, out.data_ptr()))

    def device_status(self, stream=None) -> int:
        st = C.c_int(0)
        _check(_lib.lib().xabe_lm_head_device_status(self._h, _stream_ptr(stream), C.byref(st)))
        return st.value
