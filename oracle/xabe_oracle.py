"""ctypes binding of the CPU oracle (``oracle/libxabe_oracle.so``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()``
and by the CPU-baseline leg of ``bench.py``.  The product package never imports
it.  Parity of the oracle itself is pinned by the reference's known-answer
tests in ``tests/test_oracle_kats.py``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libxabe_oracle.so")

Q6K, Q8_0 = 0, 1
BLOCK_BYTES = {Q6K: 210, Q8_0: 34}
BLOCK_ELEMS = {Q6K: 256, Q8_0: 32}
INACTIVE_EXPERT = -1


def build(force: bool = False) -> str:
    """Compile the oracle with its Makefile when the library is missing or stale."""
    src = os.path.join(_HERE, "xabe_oracle.c")
    hdr = os.path.join(_HERE, "xabe_oracle.h")
    stale = (not os.path.exists(_SO)) or any(
        os.path.getmtime(p) > os.path.getmtime(_SO) for p in (src, hdr))
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B", "libxabe_oracle.so"], check=True,
                       capture_output=True)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_SO)
        _declare(_lib)
    return _lib


class _Rng(C.Structure):
    _fields_ = [("state", C.c_uint64)]


class _Cmp(C.Structure):
    _fields_ = [("max_abs_error", C.c_float), ("max_abs_error_index", C.c_uint64),
                ("max_rel_error", C.c_float), ("max_rel_error_index", C.c_uint64),
                ("cosine_similarity", C.c_float), ("non_finite_count", C.c_uint64),
                ("len", C.c_uint64), ("rel_l2", C.c_double)]


class _Layer(C.Structure):
    _fields_ = [("num_experts", C.c_uint32), ("top_k", C.c_uint32), ("hidden", C.c_uint32),
                ("inter", C.c_uint32), ("post_norm", C.c_void_p), ("router", C.c_void_p),
                ("router_bias", C.c_void_p),
                ("gate_exps", C.c_void_p), ("gate_quant", C.c_int),
                ("up_exps", C.c_void_p), ("up_quant", C.c_int),
                ("down_exps", C.c_void_p), ("down_quant", C.c_int),
                ("shared_gate_inp", C.c_void_p),
                ("shared_gate", C.c_void_p), ("shared_gate_quant", C.c_int),
                ("shared_up", C.c_void_p), ("shared_up_quant", C.c_int),
                ("shared_down", C.c_void_p), ("shared_down_quant", C.c_int),
                ("eps", C.c_float)]


class _Outputs(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in
                ("normed", "logits", "topk_ids", "topk_weights", "routed", "shexp", "gate",
                 "ffn_out", "l_out")]


def _declare(L):
    vp, sz, i32, f32 = C.c_void_p, C.c_size_t, C.c_int, C.c_float
    L.xo_rng_seed.argtypes = [C.POINTER(_Rng), C.c_uint64]
    L.xo_rng_next_u64.argtypes = [C.POINTER(_Rng)]
    L.xo_rng_next_u64.restype = C.c_uint64
    L.xo_rng_next_f32.argtypes = [C.POINTER(_Rng)]
    L.xo_rng_next_f32.restype = f32
    L.xo_rng_next_u32_below.argtypes = [C.POINTER(_Rng), C.c_uint32]
    L.xo_rng_next_u32_below.restype = C.c_uint32
    L.xo_rng_vec_f32.argtypes = [C.POINTER(_Rng), vp, sz, f32, f32]
    L.xo_f32_to_f16_bits.argtypes = [f32]
    L.xo_f32_to_f16_bits.restype = C.c_uint16
    L.xo_f16_bits_to_f32.argtypes = [C.c_uint16]
    L.xo_f16_bits_to_f32.restype = f32
    L.xo_dequantize_row.argtypes = [i32, vp, sz, vp]
    L.xo_dequantize_row.restype = i32
    L.xo_quantize_row.argtypes = [i32, vp, sz, vp]
    L.xo_quantize_row.restype = i32
    L.xo_rms_norm.argtypes = [vp, vp, f32, sz, vp]
    L.xo_rms_norm_dev.argtypes = [vp, vp, f32, sz, vp]
    L.xo_silu.argtypes = [f32]
    L.xo_silu.restype = f32
    L.xo_sigmoid.argtypes = [f32]
    L.xo_sigmoid.restype = f32
    L.xo_gemv.argtypes = [vp, sz, sz, vp, vp]
    L.xo_argmax.argtypes = [vp, sz]
    L.xo_argmax.restype = sz
    L.xo_lm_head.argtypes = [i32, vp, sz, sz, vp, sz, vp, i32]
    L.xo_lm_head.restype = i32
    L.xo_router_logits_dev.argtypes = [vp, vp, sz, sz, vp]
    L.xo_shared_gate_dot_dev.argtypes = [vp, vp, sz]
    L.xo_shared_gate_dot_dev.restype = f32
    L.xo_softmax_denominator_dev.argtypes = [vp, sz]
    L.xo_softmax_denominator_dev.restype = f32
    L.xo_route_batch.argtypes = [vp, sz, sz, sz, vp, vp]
    L.xo_moe_align_block_size.argtypes = [vp, sz, sz, sz, sz, vp, vp]
    L.xo_moe_align_block_size.restype = C.c_long
    L.xo_sorted_capacity.argtypes = [sz, sz, sz, sz]
    L.xo_sorted_capacity.restype = sz
    L.xo_expert_mlp.argtypes = [vp, vp, vp, vp, sz, sz, vp]
    L.xo_naive_forward.argtypes = [vp, sz, vp, vp, sz, vp, vp, vp, sz, sz, vp]
    L.xo_grouped_forward.argtypes = [vp, sz, vp, vp, sz, sz, vp, sz, vp, vp, vp, sz, sz, vp]
    L.xo_compare.argtypes = [vp, vp, sz, C.POINTER(_Cmp)]
    L.xo_moe_block_forward.argtypes = [C.POINTER(_Layer), vp, sz, i32, i32, C.POINTER(_Outputs)]
    L.xo_moe_block_forward.restype = i32
    L.xo_routed_forward_q.argtypes = [C.POINTER(_Layer), vp, sz, vp, vp, i32, vp]
    L.xo_routed_forward_q.restype = i32
    L.xo_mlp_forward_q.argtypes = [vp, i32, vp, i32, vp, i32, sz, sz, vp, sz, i32, vp]
    L.xo_mlp_forward_q.restype = i32
    L.xo_dense_block_forward.argtypes = [vp, f32, vp, i32, vp, i32, vp, i32, sz, sz, vp, sz,
                                         i32, i32, vp, vp]
    L.xo_dense_block_forward.restype = i32
    L.xo_max_threads.restype = i32


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint8)


class Xorshift64Star:
    """crates/xabe-kernels/src/rng.rs:12-56."""

    def __init__(self, seed: int):
        self._r = _Rng()
        lib().xo_rng_seed(C.byref(self._r), seed)

    def next_u64(self) -> int:
        return lib().xo_rng_next_u64(C.byref(self._r))

    def next_f32(self) -> float:
        return lib().xo_rng_next_f32(C.byref(self._r))

    def next_u32_below(self, bound: int) -> int:
        return lib().xo_rng_next_u32_below(C.byref(self._r), bound)

    def vec_f32(self, n: int, lo: float, hi: float) -> np.ndarray:
        out = np.empty(n, dtype=np.float32)
        lib().xo_rng_vec_f32(C.byref(self._r), _p(out), n, lo, hi)
        return out


def f32_to_f16_bits(x: float) -> int:
    return lib().xo_f32_to_f16_bits(x)


def f16_bits_to_f32(h: int) -> float:
    return lib().xo_f16_bits_to_f32(h)


def dequantize_row(quant: int, data) -> np.ndarray:
    b = _u8(data).reshape(-1)
    if b.size % BLOCK_BYTES[quant]:
        raise ValueError(f"{b.size} bytes is not a whole number of {BLOCK_BYTES[quant]} B blocks")
    out = np.empty(b.size // BLOCK_BYTES[quant] * BLOCK_ELEMS[quant], dtype=np.float32)
    rc = lib().xo_dequantize_row(quant, _p(b), b.size, _p(out))
    assert rc == 0
    return out


def quantize_row(quant: int, x) -> np.ndarray:
    x = _f32(x).reshape(-1)
    if x.size % BLOCK_ELEMS[quant]:
        raise ValueError("not a whole number of blocks")
    out = np.zeros(x.size // BLOCK_ELEMS[quant] * BLOCK_BYTES[quant], dtype=np.uint8)
    rc = lib().xo_quantize_row(quant, _p(x), x.size, _p(out))
    assert rc == 0
    return out


def rms_norm(x, w, eps: float, dev_order: bool = False) -> np.ndarray:
    x, w = _f32(x), _f32(w)
    out = np.empty_like(x)
    rows = x.reshape(-1, w.size)
    o = out.reshape(-1, w.size)
    fn = lib().xo_rms_norm_dev if dev_order else lib().xo_rms_norm
    for r in range(rows.shape[0]):
        fn(_p(rows[r]), _p(w), eps, w.size, _p(o[r]))
    return out


def silu(x: float) -> float:
    return lib().xo_silu(x)


def sigmoid(x: float) -> float:
    return lib().xo_sigmoid(x)


def gemv(w, x) -> np.ndarray:
    w, x = _f32(w), _f32(x)
    out = np.empty(w.shape[0], dtype=np.float32)
    lib().xo_gemv(_p(w), w.shape[0], w.shape[1], _p(x), _p(out))
    return out


def argmax(v) -> int:
    """gemv.rs:102-111: ties go to the lower index."""
    v = _f32(v)
    return int(lib().xo_argmax(_p(v), v.size))


def lm_head(quant: int, data, vocab: int, hidden: int, x, threads: int = 0) -> np.ndarray:
    """Logits [tokens][vocab] of the LM head: gemv_batch over rows dequantised from file bytes
    (crates/xabe-engine/tests/lm_head_differential.rs:17-19)."""
    data, x = _u8(data), _f32(x)
    x = x.reshape(-1, hidden)
    if data.size != vocab * (hidden // BLOCK_ELEMS[quant]) * BLOCK_BYTES[quant]:
        raise ValueError("weight bytes do not match vocab x hidden")
    out = np.empty((x.shape[0], vocab), dtype=np.float32)
    rc = lib().xo_lm_head(quant, _p(data), vocab, hidden, _p(x), x.shape[0], _p(out), threads)
    if rc != 0:
        raise ValueError(f"xo_lm_head failed ({rc})")
    return out


def router_logits_dev(w, x) -> np.ndarray:
    w, x = _f32(w), _f32(x)
    x2 = x.reshape(-1, w.shape[1])
    out = np.empty((x2.shape[0], w.shape[0]), dtype=np.float32)
    for t in range(x2.shape[0]):
        lib().xo_router_logits_dev(_p(w), _p(x2[t]), w.shape[0], w.shape[1], _p(out[t]))
    return out


def shared_gate_dot_dev(w, x) -> float:
    w, x = _f32(w), _f32(x)
    return lib().xo_shared_gate_dot_dev(_p(w), _p(x), w.size)


def softmax_denominator_dev(exps) -> float:
    e = _f32(exps)
    return lib().xo_softmax_denominator_dev(_p(e), e.size)


def route_batch(logits, k: int):
    lg = _f32(logits)
    lg = lg.reshape(-1, lg.shape[-1])
    ids = np.empty((lg.shape[0], k), dtype=np.int32)
    w = np.empty((lg.shape[0], k), dtype=np.float32)
    lib().xo_route_batch(_p(lg), lg.shape[0], lg.shape[1], k, _p(ids), _p(w))
    return ids, w


def sorted_capacity(num_experts: int, top_k: int, block_size: int, max_tokens: int) -> int:
    return lib().xo_sorted_capacity(num_experts, top_k, block_size, max_tokens)


@dataclass
class MoeDispatch:
    sorted_token_ids: np.ndarray
    expert_ids: np.ndarray
    num_tokens_post_pad: int


def moe_align_block_size(topk_ids, block_size: int, num_experts: int) -> MoeDispatch:
    ids = np.ascontiguousarray(topk_ids, dtype=np.int32)
    ids = ids.reshape(ids.shape[0], -1) if ids.ndim > 1 else ids.reshape(-1, 1)
    tokens, k = ids.shape
    if block_size <= 0:
        raise ValueError("block_size must be non-zero")
    cap = (tokens * k + min(num_experts, max(tokens * k, 1)) * (block_size - 1) + block_size)
    cap = (cap + block_size - 1) // block_size * block_size
    s = np.empty(cap, dtype=np.int32)
    e = np.empty(cap // block_size + 1, dtype=np.int32)
    n = lib().xo_moe_align_block_size(_p(ids), tokens, k, block_size, num_experts, _p(s), _p(e))
    if n < 0:
        raise ValueError("expert id out of range")
    return MoeDispatch(s[:n].copy(), e[: n // block_size].copy(), int(n))


def expert_mlp(gate, up, down, x) -> np.ndarray:
    gate, up, down, x = _f32(gate), _f32(up), _f32(down), _f32(x)
    inter, hidden = gate.shape
    out = np.empty(hidden, dtype=np.float32)
    lib().xo_expert_mlp(_p(gate), _p(up), _p(down), _p(x), hidden, inter, _p(out))
    return out


def naive_forward(hidden_states, ids, weights, gate, up, down) -> np.ndarray:
    hs, gate, up, down = _f32(hidden_states), _f32(gate), _f32(up), _f32(down)
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    w = _f32(weights)
    tokens, hidden = hs.shape
    inter = gate.shape[1]
    out = np.empty_like(hs)
    lib().xo_naive_forward(_p(hs), tokens, _p(ids), _p(w), ids.shape[1], _p(gate), _p(up),
                           _p(down), hidden, inter, _p(out))
    return out


def grouped_forward(hidden_states, dispatch: MoeDispatch, flat_weights, top_k, gate, up, down):
    hs, gate, up, down = _f32(hidden_states), _f32(gate), _f32(up), _f32(down)
    fw = _f32(flat_weights).reshape(-1)
    tokens, hidden = hs.shape
    inter = gate.shape[1]
    nb = dispatch.expert_ids.size
    bs = dispatch.sorted_token_ids.size // nb if nb else 1
    out = np.empty_like(hs)
    lib().xo_grouped_forward(_p(hs), tokens, _p(dispatch.sorted_token_ids),
                             _p(dispatch.expert_ids), nb, bs, _p(fw), top_k, _p(gate), _p(up),
                             _p(down), hidden, inter, _p(out))
    return out


@dataclass
class Comparison:
    max_abs_error: float
    max_abs_error_index: int
    max_rel_error: float
    max_rel_error_index: int
    cosine_similarity: float
    non_finite_count: int
    len: int
    rel_l2: float

    def __str__(self):
        return (f"cosine={self.cosine_similarity:.7f} max_abs={self.max_abs_error:.4e} "
                f"@[{self.max_abs_error_index}] max_rel={self.max_rel_error:.4e} "
                f"rel_l2={self.rel_l2:.4e} non_finite={self.non_finite_count}/{self.len}")


def compare(candidate, reference) -> Comparison:
    c, r = _f32(candidate).reshape(-1), _f32(reference).reshape(-1)
    assert c.size == r.size and c.size > 0
    out = _Cmp()
    lib().xo_compare(_p(c), _p(r), c.size, C.byref(out))
    return Comparison(out.max_abs_error, out.max_abs_error_index, out.max_rel_error,
                      out.max_rel_error_index, out.cosine_similarity, out.non_finite_count,
                      out.len, out.rel_l2)


class Layer:
    """One MoE layer's host-side weights in GGUF file layout (numpy arrays)."""

    def __init__(self, *, num_experts, top_k, hidden, inter, post_norm, router,
                 gate_exps, gate_quant, up_exps, up_quant, down_exps, down_quant,
                 shared_gate_inp, shared_gate, shared_gate_quant, shared_up, shared_up_quant,
                 shared_down, shared_down_quant, eps=1e-6, router_bias=None):
        self.keep = dict(post_norm=_f32(post_norm), router=_f32(router),
                         gate_exps=_u8(gate_exps), up_exps=_u8(up_exps), down_exps=_u8(down_exps),
                         shared_gate_inp=_f32(shared_gate_inp), shared_gate=_u8(shared_gate),
                         shared_up=_u8(shared_up), shared_down=_u8(shared_down))
        k = self.keep
        if router_bias is not None:
            k["router_bias"] = _f32(router_bias)
        self.c = _Layer(num_experts, top_k, hidden, inter, _p(k["post_norm"]), _p(k["router"]),
                        _p(k["router_bias"]) if router_bias is not None else None,
                        _p(k["gate_exps"]), gate_quant, _p(k["up_exps"]), up_quant,
                        _p(k["down_exps"]), down_quant, _p(k["shared_gate_inp"]),
                        _p(k["shared_gate"]), shared_gate_quant, _p(k["shared_up"]),
                        shared_up_quant, _p(k["shared_down"]), shared_down_quant, eps)
        self.num_experts, self.top_k, self.hidden, self.inter = num_experts, top_k, hidden, inter


def moe_block_forward(layer: Layer, residual, *, dev_order: bool = True, threads: int = 0) -> dict:
    x = _f32(residual)
    T, H = x.shape
    E, K = layer.num_experts, layer.top_k
    o = dict(normed=np.empty((T, H), np.float32), logits=np.empty((T, E), np.float32),
             topk_ids=np.empty((T, K), np.int32), topk_weights=np.empty((T, K), np.float32),
             routed=np.empty((T, H), np.float32), shexp=np.empty((T, H), np.float32),
             gate=np.empty(T, np.float32), ffn_out=np.empty((T, H), np.float32),
             l_out=np.empty((T, H), np.float32))
    outs = _Outputs(*[_p(o[n]) for n, _ in _Outputs._fields_])
    rc = lib().xo_moe_block_forward(C.byref(layer.c), _p(x), T, 1 if dev_order else 0, threads,
                                    C.byref(outs))
    if rc != 0:
        raise MemoryError("oracle allocation failed")
    return o


def routed_forward_q(layer: Layer, hidden_states, ids, weights, threads: int = 0) -> np.ndarray:
    x = _f32(hidden_states)
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    w = _f32(weights)
    out = np.empty_like(x)
    rc = lib().xo_routed_forward_q(C.byref(layer.c), _p(x), x.shape[0], _p(ids), _p(w), threads,
                                   _p(out))
    assert rc == 0
    return out


def mlp_forward_q(gate, gq, up, uq, down, dq, hidden, inter, x, threads: int = 0) -> np.ndarray:
    x = _f32(x)
    gate, up, down = _u8(gate), _u8(up), _u8(down)
    out = np.empty_like(x)
    rc = lib().xo_mlp_forward_q(_p(gate), gq, _p(up), uq, _p(down), dq, hidden, inter, _p(x),
                                x.shape[0], threads, _p(out))
    assert rc == 0
    return out


def dense_block_forward(post_norm, eps, gate, gq, up, uq, down, dq, hidden, inter, residual,
                        *, dev_order: bool = True, threads: int = 0):
    x = _f32(residual)
    pn = _f32(post_norm)
    gate, up, down = _u8(gate), _u8(up), _u8(down)
    ffn = np.empty_like(x)
    lo = np.empty_like(x)
    rc = lib().xo_dense_block_forward(_p(pn), eps, _p(gate), gq, _p(up), uq, _p(down), dq, hidden,
                                      inter, _p(x), x.shape[0], 1 if dev_order else 0, threads,
                                      _p(ffn), _p(lo))
    assert rc == 0
    return ffn, lo


def max_threads() -> int:
    return lib().xo_max_threads()
