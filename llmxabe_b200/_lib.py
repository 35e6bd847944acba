"""Loader for the C-ABI library.  There is no CPU path: if the CUDA library is
missing the import of anything that computes raises, loudly."""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

_LIB = None


class EpPeersC(C.Structure):
    _fields_ = [(n, C.c_void_p * 8) for n in ("rows", "eid", "meta", "flag_in", "back", "flag_back")]


class QuantTensorC(C.Structure):
    _fields_ = [("dev_bytes", C.c_void_p), ("n_bytes", C.c_size_t), ("quant", C.c_int32)]


class GeometryC(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("num_experts", "experts_per_token", "hidden", "intermediate",
                                          "block_size", "max_tokens")]


class LayerWeightsC(C.Structure):
    _fields_ = [("post_norm", C.c_void_p), ("router", C.c_void_p), ("router_bias", C.c_void_p),
                ("gate_exps", QuantTensorC), ("up_exps", QuantTensorC), ("down_exps", QuantTensorC),
                ("shared_gate_inp", C.c_void_p),
                ("shared_gate", QuantTensorC), ("shared_up", QuantTensorC), ("shared_down", QuantTensorC)]


class HeadGeometryC(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("hidden", "vocab", "max_tokens")]


class BufferViewC(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in
                ("valid_tokens", "topk_ids", "topk_weights", "sorted_token_ids", "expert_ids",
                 "num_tokens_post_pad", "partial", "normed", "logits", "routed", "shexp", "gate")] + \
               [("sorted_capacity", C.c_uint64), ("expert_block_capacity", C.c_uint64)]


# name -> (restype, argtypes); every symbol include/xabe_moe.h declares
_vp, _i, _sz, _f = C.c_void_p, C.c_int, C.c_size_t, C.c_float
SYMBOLS = {
    "xabe_moe_last_error": (C.c_char_p, []),
    "xabe_moe_abi_version": (_i, []),
    "xabe_kernel_launch_count": (C.c_uint64, []),
    "xabe_moe_sorted_capacity": (C.c_uint64, [C.POINTER(GeometryC)]),
    "xabe_moe_expert_block_capacity": (C.c_uint64, [C.POINTER(GeometryC)]),
    "xabe_moe_create": (_i, [C.POINTER(GeometryC), _i, _i, _f, C.POINTER(_vp)]),
    "xabe_moe_destroy": (None, [_vp]),
    "xabe_moe_set_valid_tokens": (_i, [_vp, _vp, _i]),
    "xabe_moe_rms_norm": (_i, [_vp, _vp, _vp, _vp]),
    "xabe_moe_router_logits": (_i, [_vp, _vp, _vp, _vp]),
    "xabe_moe_route_and_dispatch": (_i, [_vp, _vp, _vp]),
    "xabe_moe_build_dispatch": (_i, [_vp, _vp, _vp, _vp]),
    "xabe_moe_gate_and_combine": (_i, [_vp, _vp, _vp, _vp, _sz, _vp, _sz, _vp, _sz]),
    "xabe_moe_grouped_forward_partial_f16": (_i, [_vp, _vp, QuantTensorC, QuantTensorC, QuantTensorC, _vp, _sz]),
    "xabe_moe_ep_pack": (_i, [_vp, _vp, _vp, _sz, _i, _vp, _vp, _vp]),
    "xabe_moe_ep_plan_pack": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _vp]),
    "xabe_moe_ep_p2p_send": (_i, [_vp, _vp, _i, _i, _i, _i, _vp, _i, _vp]),
    "xabe_moe_ep_p2p_receive": (_i, [_vp, _vp, _i, _i, _i, _vp, _i, _vp, _vp]),
    "xabe_moe_ep_p2p_return": (_i, [_vp, _vp, _i, _i, _i, _vp, _i, _vp]),
    "xabe_ipc_alloc": (_i, [_sz, _vp, _vp]),
    "xabe_ipc_open": (_i, [_vp, _vp]),
    "xabe_ipc_close": (_i, [_vp]),
    "xabe_ipc_free": (_i, [_vp]),
    "xabe_moe_set_result_destinations": (_i, [_vp, _vp]),
    "xabe_moe_ep_p2p_wait_results": (_i, [_vp, _vp, _i, _i, _vp, _i]),
    "xabe_moe_ep_combine": (_i, [_vp, _vp, _vp, _sz, _vp, _vp, _vp, _sz, _vp, _sz, _vp, _sz]),
    "xabe_moe_grouped_forward_partial": (_i, [_vp, _vp, QuantTensorC, QuantTensorC, QuantTensorC, _vp]),
    "xabe_moe_grouped_forward": (_i, [_vp, _vp, QuantTensorC, QuantTensorC, QuantTensorC, _vp, _vp]),
    "xabe_moe_shared_expert": (_i, [_vp, _vp, QuantTensorC, QuantTensorC, QuantTensorC, _vp, _vp]),
    "xabe_moe_block_forward": (_i, [_vp, _vp, C.POINTER(LayerWeightsC), _vp, _sz, _i, _vp, _sz, _vp, _sz]),
    "xabe_moe_block_forward_host": (_i, [_vp, _vp, C.POINTER(LayerWeightsC), _vp, _i, _vp, _vp]),
    "xabe_moe_stack_forward": (_i, [_vp, _vp, C.POINTER(LayerWeightsC), _i, _vp, _vp, _sz, _i, _vp, _sz,
                                    C.POINTER(_vp)]),
    "xabe_dense_ffn_block_forward": (_i, [_vp, _vp, _vp, QuantTensorC, QuantTensorC, QuantTensorC, _vp, _sz,
                                          _i, _vp, _sz, _vp, _sz]),
    "xabe_moe_buffers": (_i, [_vp, C.POINTER(BufferViewC)]),
    "xabe_moe_set_exact_decode_regime": (_i, [_vp, _i]),
    "xabe_moe_disable_tensor_cores": (_i, [_vp]),
    "xabe_moe_tensor_cores_enabled": (_i, [_vp]),
    "xabe_moe_force_prefill_path": (_i, [_vp, _i]),
    "xabe_moe_set_tuning": (_i, [_vp, _i, _i]),
    "xabe_moe_set_peer_wait_limit": (_i, [_vp, C.c_uint32]),
    "xabe_moe_device_status": (_i, [_vp, _vp, C.POINTER(_i)]),
    "xabe_moe_stage_profile": (_i, [_vp, _i]),
    "xabe_moe_stage_times": (_i, [_vp, _vp, C.POINTER(C.c_float), C.POINTER(_i)]),
    "xabe_dequantize": (_i, [_vp, QuantTensorC, _vp]),
    "xabe_stream_read": (_i, [_vp, _vp, _sz, _vp]),
    "xabe_moe_block_forward_typed": (_i, [_vp, _vp, _vp, _vp, _i, _sz, _i, _vp, _sz, _vp, _sz]),
    "xabe_shared_expert_noalloc": (_i, [_vp, QuantTensorC, QuantTensorC, QuantTensorC, _i, _i, _vp, _i, _vp]),
    "xabe_shared_expert_noalloc_status": (_i, [_vp, C.POINTER(_i)]),
    "xabe_lm_head_create": (_i, [C.POINTER(HeadGeometryC), _i, C.POINTER(_vp)]),
    "xabe_lm_head_destroy": (None, [_vp]),
    "xabe_lm_head_forward": (_i, [_vp, _vp, QuantTensorC, _vp, _sz, _i, _vp, _sz]),
    "xabe_lm_head_argmax": (_i, [_vp, _vp, _vp, _sz, _i, _vp]),
    "xabe_lm_head_device_status": (_i, [_vp, _vp, C.POINTER(_i)]),
}


def library_path() -> str:
    return _build.LIB


def lib() -> C.CDLL:
    """The loaded C-ABI library.  Raises if it has not been built."""
    global _LIB
    if _LIB is None:
        path = library_path()
        if not os.path.exists(path):
            raise RuntimeError(
                f"{path} is missing: build it with `python -m llmxabe_b200.build` "
                "(nvcc, sm_100a). There is no CPU fallback for this path.")
        L = C.CDLL(path)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(L, name)  # AttributeError if the library lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _LIB = L
    return _LIB
