"""Host mirror of `xabe_gguf::GgufFile` (crates/xabe-gguf/src/file.rs) over the C ABI of
libxabe_gguf.so, and the step from a file to the device tensors of one MoE layer
(crates/xabe-model/src/weights.rs:173-212,403-413): tensors go to the GPU as the bytes of the
file, which is the layout the kernels read.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from enum import IntEnum

import numpy as np

from . import build as _build

_LIB = None


class GgufError(RuntimeError):
    """GgufError (crates/xabe-gguf/src/error.rs); `.kind` is the variant's name."""

    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = code
        self.kind = _KINDS.get(code, f"status {code}")


_KINDS = {1: "BadMagic", 2: "UnsupportedVersion", 3: "UnexpectedEof", 4: "NegativeCount", 5: "DuplicateKey",
          6: "UnknownValueType", 7: "NestedArray", 8: "BadAlignmentType", 9: "BadAlignment",
          10: "TooManyDimensions", 11: "ZeroDimension", 12: "DuplicateTensor", 13: "UnsupportedGgmlType",
          14: "UnalignedElementCount", 15: "OffsetOverflow", 16: "TensorOutOfBounds", 17: "Io", 18: "InvalidUtf8",
          19: "NotFound", 20: "TypeMismatch", 21: "InvalidArgument", 22: "Schema"}
_NOT_FOUND, _TYPE_MISMATCH = 19, 20


class GgmlType(IntEnum):
    """types.rs:36-60."""
    F32 = 0
    F16 = 1
    Q4_0 = 2
    Q8_0 = 8
    Q4K = 12
    Q5K = 13
    Q6K = 14
    BF16 = 30

    def block_size(self) -> int:
        return int(lib().xabe_ggml_block_size(int(self)))

    def type_size(self) -> int:
        return int(lib().xabe_ggml_type_size(int(self)))

    def type_name(self) -> str:
        return lib().xabe_ggml_type_name(int(self)).decode()

    def bytes_for_elements(self, n: int) -> int:
        out = C.c_uint64()
        _check(lib().xabe_ggml_bytes_for_elements(int(self), n, C.byref(out)))
        return out.value


class _TensorC(C.Structure):
    _fields_ = [("name", C.c_char_p), ("n_dims", C.c_uint32), ("dims", C.c_uint64 * 4), ("ggml_type", C.c_int32),
                ("offset", C.c_uint64), ("n_elements", C.c_uint64), ("n_bytes", C.c_uint64), ("data", C.c_void_p)]


class _MoeLayerC(C.Structure):
    _fields_ = [(n, _TensorC) for n in ("post_norm", "router", "gate_exps", "up_exps", "down_exps",
                                        "shared_gate_inp", "shared_gate", "shared_up", "shared_down")]


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        path = _build.GGUF_LIB
        if not os.path.exists(path):
            _build.build_gguf()
        L = C.CDLL(path)
        vp, u64, i32, cp = C.c_void_p, C.c_uint64, C.c_int32, C.c_char_p
        sig = {
            "xabe_gguf_last_error": (cp, []),
            "xabe_ggml_block_size": (u64, [i32]), "xabe_ggml_type_size": (u64, [i32]),
            "xabe_ggml_type_name": (cp, [i32]),
            "xabe_ggml_bytes_for_elements": (C.c_int, [i32, u64, C.POINTER(u64)]),
            "xabe_gguf_open": (C.c_int, [cp, C.POINTER(vp)]),
            "xabe_gguf_from_bytes": (C.c_int, [vp, C.c_size_t, C.POINTER(vp)]),
            "xabe_gguf_close": (None, [vp]),
            "xabe_gguf_version": (C.c_uint32, [vp]), "xabe_gguf_alignment": (C.c_uint32, [vp]),
            "xabe_gguf_n_kv": (u64, [vp]), "xabe_gguf_n_tensors": (u64, [vp]), "xabe_gguf_data_offset": (u64, [vp]),
            "xabe_gguf_tensor_at": (C.c_int, [vp, u64, C.POINTER(_TensorC)]),
            "xabe_gguf_find_tensor": (C.c_int, [vp, cp, C.POINTER(_TensorC)]),
            "xabe_gguf_key_at": (C.c_int, [vp, u64, C.POINTER(cp), C.POINTER(i32)]),
            "xabe_gguf_get_u32": (C.c_int, [vp, cp, C.POINTER(C.c_uint32)]),
            "xabe_gguf_get_u64": (C.c_int, [vp, cp, C.POINTER(u64)]),
            "xabe_gguf_get_f32": (C.c_int, [vp, cp, C.POINTER(C.c_float)]),
            "xabe_gguf_get_bool": (C.c_int, [vp, cp, C.POINTER(C.c_int)]),
            "xabe_gguf_get_str": (C.c_int, [vp, cp, C.POINTER(vp), C.POINTER(u64)]),
            "xabe_gguf_get_array": (C.c_int, [vp, cp, C.POINTER(i32), C.POINTER(u64), C.POINTER(vp)]),
            "xabe_gguf_get_array_str": (C.c_int, [vp, cp, u64, C.POINTER(vp), C.POINTER(u64)]),
            "xabe_gguf_moe_layer_tensors": (C.c_int, [vp, C.c_uint32, u64, u64, u64, C.POINTER(_MoeLayerC)]),
        }
        for name, (res, args) in sig.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _LIB = L
    return _LIB


def _check(rc: int) -> None:
    if rc != 0:
        raise GgufError(rc, lib().xabe_gguf_last_error().decode("utf-8", "replace"))


@dataclass(frozen=True)
class TensorInfo:
    """tensor.rs; `data` is a read-only numpy view of the tensor's bytes in the file."""
    name: str
    dims: tuple
    ggml_type: GgmlType
    offset: int
    n_elements: int
    n_bytes: int
    data: np.ndarray


_ARRAY_DTYPES = {0: np.uint8, 1: np.int8, 2: np.uint16, 3: np.int16, 4: np.uint32, 5: np.int32, 6: np.float32,
                 7: np.bool_, 10: np.uint64, 11: np.int64, 12: np.float64}


class GgufFile:
    """file.rs:62-260."""

    def __init__(self, handle: C.c_void_p, keepalive=None):
        self._h = handle
        self._keepalive = keepalive

    @staticmethod
    def open(path: str) -> "GgufFile":
        h = C.c_void_p()
        _check(lib().xabe_gguf_open(os.fsencode(path), C.byref(h)))
        return GgufFile(h)

    @staticmethod
    def from_bytes(data: bytes) -> "GgufFile":
        h = C.c_void_p()
        buf = (C.c_char * len(data)).from_buffer_copy(data) if data else None
        _check(lib().xabe_gguf_from_bytes(C.cast(buf, C.c_void_p) if buf is not None else None, len(data), C.byref(h)))
        return GgufFile(h)

    def close(self) -> None:
        if getattr(self, "_h", None) is not None and self._h.value:
            lib().xabe_gguf_close(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def version(self) -> int:
        return int(lib().xabe_gguf_version(self._h))

    def alignment(self) -> int:
        return int(lib().xabe_gguf_alignment(self._h))

    def n_kv(self) -> int:
        return int(lib().xabe_gguf_n_kv(self._h))

    def n_tensors(self) -> int:
        return int(lib().xabe_gguf_n_tensors(self._h))

    def data_offset(self) -> int:
        return int(lib().xabe_gguf_data_offset(self._h))

    def _info(self, t: _TensorC) -> TensorInfo:
        view = np.ctypeslib.as_array(C.cast(t.data, C.POINTER(C.c_uint8)), shape=(int(t.n_bytes),)) if t.n_bytes else \
            np.empty(0, dtype=np.uint8)
        view.flags.writeable = False
        # the view borrows the mapping: keep the file alive as long as the view is
        return TensorInfo(t.name.decode(), tuple(int(t.dims[i]) for i in range(t.n_dims)), GgmlType(t.ggml_type),
                          int(t.offset), int(t.n_elements), int(t.n_bytes), _Borrowed(view, self))

    def tensors(self) -> list:
        out = []
        for i in range(self.n_tensors()):
            t = _TensorC()
            _check(lib().xabe_gguf_tensor_at(self._h, i, C.byref(t)))
            out.append(self._info(t))
        return out

    def tensor(self, name: str) -> TensorInfo | None:
        t = _TensorC()
        rc = lib().xabe_gguf_find_tensor(self._h, name.encode(), C.byref(t))
        if rc == _NOT_FOUND:
            return None
        _check(rc)
        return self._info(t)

    def tensor_bytes(self, name: str) -> np.ndarray | None:
        info = self.tensor(name)
        return None if info is None else info.data

    def metadata_keys(self) -> list:
        keys = []
        for i in range(self.n_kv()):
            k = C.c_char_p()
            _check(lib().xabe_gguf_key_at(self._h, i, C.byref(k), None))
            keys.append(k.value.decode())
        return keys

    def _scalar(self, fn, ctype, key: str):
        out = ctype()
        rc = fn(self._h, key.encode(), C.byref(out))
        if rc in (_NOT_FOUND, _TYPE_MISMATCH):
            return None  # the reference's getters return None for a missing key or another type
        _check(rc)
        return out.value

    def get_u32(self, key: str):
        return self._scalar(lib().xabe_gguf_get_u32, C.c_uint32, key)

    def get_u64(self, key: str):
        return self._scalar(lib().xabe_gguf_get_u64, C.c_uint64, key)

    def get_f32(self, key: str):
        return self._scalar(lib().xabe_gguf_get_f32, C.c_float, key)

    def get_bool(self, key: str):
        v = self._scalar(lib().xabe_gguf_get_bool, C.c_int, key)
        return None if v is None else bool(v)

    def get_str(self, key: str):
        p, n = C.c_void_p(), C.c_uint64()
        rc = lib().xabe_gguf_get_str(self._h, key.encode(), C.byref(p), C.byref(n))
        if rc in (_NOT_FOUND, _TYPE_MISMATCH):
            return None
        _check(rc)
        return C.string_at(p.value, n.value).decode()

    def get_array(self, key: str):
        """A numpy copy of a numeric / bool array, a list of str for a string array, None otherwise."""
        tag, n, p = C.c_int32(), C.c_uint64(), C.c_void_p()
        rc = lib().xabe_gguf_get_array(self._h, key.encode(), C.byref(tag), C.byref(n), C.byref(p))
        if rc in (_NOT_FOUND, _TYPE_MISMATCH):
            return None
        _check(rc)
        if tag.value == 8:
            out = []
            for i in range(n.value):
                sp, sn = C.c_void_p(), C.c_uint64()
                _check(lib().xabe_gguf_get_array_str(self._h, key.encode(), i, C.byref(sp), C.byref(sn)))
                out.append(C.string_at(sp.value, sn.value).decode())
            return out
        dt = np.dtype(_ARRAY_DTYPES[tag.value])
        if n.value == 0:
            return np.empty(0, dtype=dt)
        raw = C.string_at(p.value, n.value * dt.itemsize)
        return np.frombuffer(raw, dtype=dt).copy()

    def moe_layer_tensors(self, layer: int, hidden: int, ff: int, experts: int) -> dict:
        """The nine tensors of MoE layer `layer` by role, shapes checked (weights.rs:403-413)."""
        m = _MoeLayerC()
        _check(lib().xabe_gguf_moe_layer_tensors(self._h, layer, hidden, ff, experts, C.byref(m)))
        return {name: self._info(getattr(m, name)) for name, _ in _MoeLayerC._fields_}


class _Borrowed(np.ndarray):
    """A numpy view that keeps its GgufFile (the owner of the mapping) alive."""

    def __new__(cls, view: np.ndarray, owner):
        obj = view.view(cls)
        obj._owner = owner
        return obj

    def __array_finalize__(self, obj):
        self._owner = getattr(obj, "_owner", None)


_QUANT_OF = {GgmlType.Q6K: 0, GgmlType.Q8_0: 1}


def load_moe_layer(f: GgufFile, layer: int, hidden: int, ff: int, experts: int, device="cuda"):
    """`MoeLayerWeights` of layer `layer` on `device`: expert and shared-expert tensors uploaded as the
    file's bytes (Q6_K or Q8_0, per tensor), f32 vectors as they are, the router widened to f32 the way
    the reference's loader does it (crates/xabe-engine/src/block/moe.rs:831-846: f32 as is, bf16 by a
    16-bit shift, which is exact) and, beyond the reference, a Q8_0 router dequantised with `q * d`."""
    import torch

    from .moe import ExpertQuant, MoeLayerWeights, QuantTensor, dequantize
    t = f.moe_layer_tensors(layer, hidden, ff, experts)

    def dense(info: TensorInfo) -> "torch.Tensor":
        if info.ggml_type == GgmlType.F32:
            return torch.from_numpy(np.frombuffer(info.data.tobytes(), dtype=np.float32).copy()).to(device)
        if info.ggml_type == GgmlType.BF16:
            u = np.frombuffer(info.data.tobytes(), dtype=np.uint16).astype(np.uint32) << 16
            return torch.from_numpy(u.view(np.float32).copy()).to(device)
        if info.ggml_type == GgmlType.Q8_0:
            q = QuantTensor(torch.from_numpy(np.array(info.data, dtype=np.uint8)).to(device), ExpertQuant.Q8_0)
            return dequantize(q)
        raise GgufError(22, f"{info.name}: {info.ggml_type.type_name()} is not a format this loader reads for a dense tensor")

    def quant(info: TensorInfo):
        if info.ggml_type not in _QUANT_OF:
            raise GgufError(22, f"{info.name}: {info.ggml_type.type_name()} is not an expert format this library reads (q6_K, q8_0)")
        return torch.from_numpy(np.array(info.data, dtype=np.uint8)).to(device), _QUANT_OF[info.ggml_type]

    ge, gq = quant(t["gate_exps"])
    ue, uq = quant(t["up_exps"])
    de, dq = quant(t["down_exps"])
    sg, sgq = quant(t["shared_gate"])
    su, suq = quant(t["shared_up"])
    sd, sdq = quant(t["shared_down"])
    return MoeLayerWeights(layer=layer, post_norm=dense(t["post_norm"]), router=dense(t["router"]), router_bias=None,
                           gate_exps=ge, gate_quant=gq, up_exps=ue, up_quant=uq, down_exps=de, down_quant=dq,
                           shared_gate_inp=dense(t["shared_gate_inp"]), shared_gate=sg, shared_gate_quant=sgq,
                           shared_up=su, shared_up_quant=suq, shared_down=sd, shared_down_quant=sdq, device=device)
