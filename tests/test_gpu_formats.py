"""Data formats either side of the block that the large configurations name: bf16 prefill activations
and a Q8_0 router tensor.

bf16 residual: widened exactly (a 16-bit shift, crates/xabe-kernels/src/quant.rs:1350-1358), so feeding the
bf16 rows through the typed entry point must give bit for bit what the f32 entry point gives on the widened
values, and `normed` must equal the oracle's on them.
Q8_0 router: the reference accepts f32 / bf16 routers only (block/moe.rs:831-846); a Q8_0 `ffn_gate_inp` is
dequantised with the `q * d` semantics of quant.rs:62-69 when the weights are uploaded, bit-identical to
the oracle's dequantisation, and the block then runs as usual.
"""
import numpy as np
import pytest

from helpers import bits, device_layer, oracle_layer, run_block

pytestmark = pytest.mark.gpu


def test_bf16_residual_equals_f32_entry_on_widened_values(oracle):
    import torch
    if not torch.cuda.is_available():
        pytest.fail("gpu-marked test collected without a CUDA device")
    from llmxabe_b200 import synth
    from llmxabe_b200.moe import MoeBlock, MoeGeometry
    T, MAXT = 37, 64
    L = synth.moe_layer(seed=31, num_experts=8, top_k=2, hidden=512, inter=256, zipf=True)
    x = synth.activations(T, 512, seed=31, bf16=True)           # f32 values exactly representable in bf16
    blk = MoeBlock(MoeGeometry(8, 2, 512, 256, 16, MAXT))
    w = device_layer(L)
    want = run_block(blk, w, x, MAXT)
    res16 = torch.zeros(MAXT, 512, dtype=torch.bfloat16, device="cuda")
    res16[:T] = torch.from_numpy(x).cuda().to(torch.bfloat16)
    assert (res16[:T].float().cpu().numpy().view(np.uint32) == x.view(np.uint32)).all()
    ffn = torch.full((MAXT, 512), 7.0, device="cuda")
    lo = torch.full((MAXT, 512), 7.0, device="cuda")
    blk.forward(w, res16, T, ffn, lo)
    torch.cuda.synchronize()
    assert (bits(lo[:T].cpu().numpy()) == bits(want["l_out"])).all()
    assert (bits(ffn[:T].cpu().numpy()) == bits(want["ffn_out"])).all()
    assert bool((lo[T:] == 7.0).all().item()) and bool((ffn[T:] == 7.0).all().item())
    normed = oracle.rms_norm(x, L.post_norm, L.eps, dev_order=True)
    assert (bits(blk.buffers().normed[:T].cpu().numpy()) == bits(normed)).all()


def test_q8_0_router_is_dequantised_bit_exactly_and_routes_like_the_oracle(oracle):
    import torch
    from llmxabe_b200 import synth
    from llmxabe_b200.moe import ExpertQuant, MoeBlock, MoeGeometry, QuantTensor, dequantize
    E, K, H, I, T = 8, 2, 512, 256, 21
    L = synth.moe_layer(seed=32, num_experts=E, top_k=K, hidden=H, inter=I, zipf=False)
    raw = synth.q8_0_bytes(E * H, 32, 0, 99)                     # a Q8_0 `ffn_gate_inp`, [E][H] row-major
    router_dev = dequantize(QuantTensor(torch.from_numpy(raw).cuda(), ExpertQuant(1))).view(E, H)
    router_ref = oracle.dequantize_row(1, raw).reshape(E, H)
    assert (bits(router_dev.cpu().numpy()) == bits(router_ref)).all()
    L.router = router_ref * np.float32(20.0)                     # spread the logits (scaled once, on the host, for both sides)
    w = device_layer(L)
    x = synth.activations(T, H, seed=32)
    got = run_block(MoeBlock(MoeGeometry(E, K, H, I, 16, T)), w, x, T)
    want = oracle.moe_block_forward(oracle_layer(oracle, L), x, dev_order=True)
    assert (got["topk_ids"] == want["topk_ids"]).all()
    assert (bits(got["logits"]) == bits(want["logits"])).all()
    rel = np.linalg.norm(got["l_out"].astype(np.float64) - want["l_out"]) / np.linalg.norm(want["l_out"].astype(np.float64))
    assert rel <= 1e-3


def test_unknown_dtype_tag_is_rejected_before_any_launch():
    import ctypes as C
    import torch
    from llmxabe_b200 import _lib, synth
    from llmxabe_b200.errors import MoeError
    from llmxabe_b200.moe import MoeBlock, MoeGeometry, _check
    L = synth.moe_layer(seed=33, num_experts=8, top_k=2, hidden=512, inter=256, zipf=False)
    blk = MoeBlock(MoeGeometry(8, 2, 512, 256, 16, 4))
    w = device_layer(L)
    wc = w._c()
    res = torch.zeros(4, 512, device="cuda")
    out = torch.full((4, 512), 3.0, device="cuda")
    with pytest.raises(MoeError):
        _check(_lib.lib().xabe_moe_block_forward_typed(blk.moe._h, torch.cuda.current_stream().cuda_stream,
                                                       C.byref(wc), res.data_ptr(), 7, res.numel(), 2,
                                                       out.data_ptr(), out.numel(), out.data_ptr(), out.numel()))
    torch.cuda.synchronize()
    assert bool((out == 3.0).all().item())


def test_streaming_read_calibration_runs():
    import torch
    from llmxabe_b200.moe import stream_read
    data = torch.randint(0, 255, (1 << 20,), dtype=torch.uint8, device="cuda")
    sink = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream_read(data, sink)
    torch.cuda.synchronize()
