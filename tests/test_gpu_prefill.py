"""GPU parity of the prefill-shaped path (tcgen05 grouped GEMM, TMEM accumulators)
against the CPU oracle, through the same block entry point.

Gate: routing ids and tables exact; routed / shexp / ffn_out / l_out rel-L2 <= 1e-3 against the
oracle (max-abs printed).  The prefill kernels round the dequantised weights to f16, so their
outputs are also compared with the decode-shaped kernels' (exact codes) on the same input.
"""
import numpy as np
import pytest

from helpers import bits, device_layer, oracle_layer, run_block

pytestmark = pytest.mark.gpu
REL_L2 = 1e-3


@pytest.fixture(scope="module")
def torch_cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("gpu-marked test collected without a CUDA device")
    return torch


def _check(oracle, got, want, label):
    assert (bits(got["logits"]) == bits(want["logits"])).all(), f"{label}: logits"
    assert (got["topk_ids"] == want["topk_ids"]).all(), f"{label}: ids"
    for name in ("routed", "shexp", "ffn_out", "l_out"):
        r = oracle.compare(got[name], want[name])
        print(f"{label} {name}: {r}")
        assert r.non_finite_count == 0 and r.rel_l2 <= REL_L2, f"{label} {name}: {r}"
    assert got["untouched"]


@pytest.mark.parametrize("routed_quant,shared_quant,tokens,max_tokens",
                         [(0, 0, 600, 640), (1, 1, 513, 520), (0, 1, 1000, 1024)])
def test_small_geometry_prefill(torch_cuda, oracle, routed_quant, shared_quant, tokens, max_tokens):
    """H=512, I=256, E=8, K=2 at prefill width: hot experts span several 128-token tiles, tails are ragged."""
    from llmxabe_b200 import synth
    from llmxabe_b200.moe import MoeBlock, MoeGeometry
    L = synth.moe_layer(seed=5, num_experts=8, top_k=2, hidden=512, inter=256, routed_quant=routed_quant,
                        shared_quant=shared_quant, zipf=True)
    g = MoeGeometry(8, 2, 512, 256, 32, max_tokens)
    blk = MoeBlock(g)
    x = synth.activations(tokens, 512, seed=5, layer=tokens, bf16=True)
    got = run_block(blk, device_layer(L), x, max_tokens)
    assert blk.moe.device_status() == 0
    want = oracle.moe_block_forward(oracle_layer(oracle, L), x, dev_order=True)
    _check(oracle, got, want, f"prefill small q{routed_quant}/{shared_quant} T={tokens}")
    # the decode-shaped kernels on the same input (exact-regime switch of the reference, moe.rs:5450)
    blk.set_exact_decode_regime(True)
    dec = run_block(blk, device_layer(L), x, max_tokens)
    r = oracle.compare(got["l_out"], dec["l_out"])
    print(f"prefill vs decode kernels: {r}")
    assert r.rel_l2 <= REL_L2


def test_real_geometry_prefill_512(torch_cuda, oracle):
    """256 experts / top-8 / 2048 / 512, Q6_K, 512 bf16-rounded tokens, Zipf routing (the prefill shape at a quarter of its width)."""
    from llmxabe_b200 import synth
    from llmxabe_b200.moe import MoeBlock, MoeGeometry
    L = synth.moe_layer(seed=0, layer=0, zipf=True)
    g = MoeGeometry.qwen3_6(32, 512)
    blk = MoeBlock(g)
    x = synth.activations(512, 2048, seed=0, layer=2512, bf16=True)
    got = run_block(blk, device_layer(L), x, 512)
    assert blk.moe.device_status() == 0
    want = oracle.moe_block_forward(oracle_layer(oracle, L), x, dev_order=True)
    _check(oracle, got, want, "prefill real T=512")


def test_four_accumulator_kernel_matches_the_oracle(oracle):
    """k_prefill_gemm_wide (items of up to 512 columns, TMA-loaded activation tiles) is chosen by default only
    for the dense block at prefill width; the per-handle switch selects it here for a routed block and a dense block."""
    import torch
    from llmxabe_b200 import synth
    from llmxabe_b200.moe import DenseFfnBlock, MoeBlock, MoeGeometry, QuantTensor
    T = 700
    L = synth.moe_layer(seed=61, num_experts=4, top_k=2, hidden=512, inter=256, zipf=True)
    x = synth.activations(T, 512, seed=61)
    routed_blk = MoeBlock(MoeGeometry(4, 2, 512, 256, 32, T))
    routed_blk.moe.set_tuning("prefill_wide", 1)
    got = run_block(routed_blk, device_layer(L), x, T)
    want = oracle.moe_block_forward(oracle_layer(oracle, L), x, dev_order=True)
    assert (got["topk_ids"] == want["topk_ids"]).all() and got["untouched"]
    rel = np.linalg.norm(got["l_out"].astype(np.float64) - want["l_out"]) / np.linalg.norm(want["l_out"].astype(np.float64))
    assert rel <= 1e-3, rel
    # dense: 1100 tokens = two full items and a ragged one
    hidden, inter, tokens = 512, 768, 1100
    post_norm, gate, up, down = synth.dense_layer(seed=62, hidden=hidden, inter=inter, quant=0)
    xd = synth.activations(tokens, hidden, seed=62)
    want_ffn, _ = oracle.dense_block_forward(post_norm, 1e-6, gate, 0, up, 0, down, 0, hidden, inter, xd, dev_order=True)
    blk = DenseFfnBlock(MoeGeometry(1, 1, hidden, inter, 64, tokens))
    blk.moe.set_tuning("prefill_wide", 1)
    qt = [QuantTensor(torch.from_numpy(a).cuda(), 0) for a in (gate, up, down)]
    res = torch.from_numpy(xd).cuda()
    ffn = torch.zeros(tokens, hidden, device="cuda")
    lo = torch.zeros(tokens, hidden, device="cuda")
    blk.forward(torch.from_numpy(post_norm).cuda(), qt[0], qt[1], qt[2], res, tokens, ffn, lo)
    torch.cuda.synchronize()
    assert blk.moe.device_status() == 0
    got_ffn = ffn.cpu().numpy()
    rel = np.linalg.norm(got_ffn.astype(np.float64) - want_ffn) / np.linalg.norm(want_ffn.astype(np.float64))
    assert rel <= 1e-3, rel
