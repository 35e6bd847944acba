"""From a GGUF file to the block's output: a synthetic file with two MoE layers (mixed formats,
as a UD-Q6_K_XL file has them: Q6_K experts, Q8_0 shared expert, one bf16 router) is written to
disk, opened through libxabe_gguf.so, uploaded with `load_moe_layer` and run.

Gates: the file-loaded layer gives bit-identical outputs to the same tensors uploaded directly;
the bf16-router layer matches the oracle run on the widened router (ids exact, l_out rel-L2 <= 1e-3).
"""
import os

import numpy as np
import pytest

from gguf_builder import Builder
from helpers import bits, device_layer, oracle_layer, run_block

pytestmark = pytest.mark.gpu
H, F, E, K = 512, 256, 8, 2


def _bf16_bits(x: np.ndarray) -> np.ndarray:
    u = x.astype(np.float32).view(np.uint32)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def _add_layer(b, l, L, router_bf16):
    b.tensor(f"blk.{l}.post_attention_norm.weight", [H], "f32", L.post_norm.tobytes())
    if router_bf16:
        b.tensor(f"blk.{l}.ffn_gate_inp.weight", [H, E], "bf16", _bf16_bits(L.router).tobytes())
    else:
        b.tensor(f"blk.{l}.ffn_gate_inp.weight", [H, E], "f32", L.router.tobytes())
    b.tensor(f"blk.{l}.ffn_gate_exps.weight", [H, F, E], "q6_K", L.gate_exps.tobytes())
    b.tensor(f"blk.{l}.ffn_up_exps.weight", [H, F, E], "q6_K", L.up_exps.tobytes())
    b.tensor(f"blk.{l}.ffn_down_exps.weight", [F, H, E], "q6_K", L.down_exps.tobytes())
    b.tensor(f"blk.{l}.ffn_gate_inp_shexp.weight", [H], "f32", L.shared_gate_inp.tobytes())
    b.tensor(f"blk.{l}.ffn_gate_shexp.weight", [H, F], "q8_0", L.shared_gate.tobytes())
    b.tensor(f"blk.{l}.ffn_up_shexp.weight", [H, F], "q8_0", L.shared_up.tobytes())
    b.tensor(f"blk.{l}.ffn_down_shexp.weight", [F, H], "q8_0", L.shared_down.tobytes())


def test_a_layer_loaded_from_a_file_runs_like_the_same_tensors_uploaded_directly(tmp_path, oracle):
    import torch
    if not torch.cuda.is_available():
        pytest.fail("gpu-marked test collected without a CUDA device")
    from llmxabe_b200 import synth
    from llmxabe_b200.gguf import GgufFile, load_moe_layer
    from llmxabe_b200.moe import MoeBlock, MoeGeometry
    layers = [synth.moe_layer(seed=31, layer=i, num_experts=E, top_k=K, hidden=H, inter=F, shared_quant=synth.Q8_0)
              for i in range(2)]
    b = Builder().kv_str("general.architecture", "qwen35moe").kv_u32("qwen35moe.block_count", 2)
    b.kv_f32("qwen35moe.attention.layer_norm_rms_epsilon", 1e-6)
    _add_layer(b, 0, layers[0], router_bf16=False)
    _add_layer(b, 1, layers[1], router_bf16=True)
    path = os.path.join(tmp_path, "two_layers.gguf")
    with open(path, "wb") as fh:
        fh.write(b.build())
    f = GgufFile.open(path)
    assert f.get_u32("qwen35moe.block_count") == 2
    x = synth.activations(6, H, seed=31, layer=50)
    g = MoeGeometry(E, K, H, F, 32, 8)
    blk = MoeBlock(g, eps=f.get_f32("qwen35moe.attention.layer_norm_rms_epsilon"))
    # layer 0: f32 router -> the very same bytes as a direct upload
    got = run_block(blk, load_moe_layer(f, 0, H, F, E), x, 8)
    direct = run_block(blk, device_layer(layers[0]), x, 8)
    for name in ("logits", "topk_ids", "ffn_out", "l_out"):
        assert (bits(got[name]) == bits(direct[name])).all() if got[name].dtype == np.float32 else \
            (got[name] == direct[name]).all(), name
    # layer 1: bf16 router, widened exactly; the oracle sees the widened values
    got1 = run_block(blk, load_moe_layer(f, 1, H, F, E), x, 8)
    L1 = layers[1]
    L1.router = (_bf16_bits(L1.router).astype(np.uint32) << 16).view(np.float32).reshape(L1.router.shape)
    want1 = oracle.moe_block_forward(oracle_layer(oracle, L1), x, dev_order=True)
    assert (bits(got1["logits"]) == bits(want1["logits"])).all()
    assert (got1["topk_ids"] == want1["topk_ids"]).all()
    r = oracle.compare(got1["l_out"], want1["l_out"])
    print(f"gguf layer 1 l_out: {r}")
    assert r.non_finite_count == 0 and r.rel_l2 <= 1e-3
    assert blk.moe.device_status() == 0
