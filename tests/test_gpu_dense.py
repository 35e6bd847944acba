"""Dense SwiGLU block (the 27B sibling) on the GPU against the CPU oracle, and its tensor-parallel form.

DenseFfnBlock::forward (crates/xabe-engine/src/block/dense_ffn.rs:9-16): l_out = down(silu(gate n) * (up n)) + x
with n = rmsnorm(x); oracle recipe of crates/xabe-engine/tests/dense_ffn_differential.rs:46-49.
Gate: rel-L2 <= 1e-3 on ffn_out and l_out (max-abs printed on failure); normed rows bit-identical;
rows >= tokens never written.
"""
import os
import socket
import sys

import numpy as np
import pytest

from helpers import bits

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REL_L2 = 1e-3


def _rel_l2(got, want):
    return float(np.linalg.norm(got.astype(np.float64) - want) / max(np.linalg.norm(want.astype(np.float64)), 1e-30))


def _dense_inputs(hidden, inter, quant, tokens, seed):
    from llmxabe_b200 import synth
    post_norm, gate, up, down = synth.dense_layer(seed=seed, hidden=hidden, inter=inter, quant=quant)
    post_norm = (post_norm * (1.0 + 0.1 * np.sin(np.arange(hidden, dtype=np.float32)))).astype(np.float32)
    x = synth.activations(tokens, hidden, seed=seed)
    return post_norm, gate, up, down, x


def _run_dense(torch, hidden, inter, quant, post_norm, gate, up, down, x, max_tokens):
    from llmxabe_b200.moe import DenseFfnBlock, MoeGeometry, QuantTensor
    T = x.shape[0]
    blk = DenseFfnBlock(MoeGeometry(1, 1, hidden, inter, 64, max_tokens))
    qt = [QuantTensor(torch.from_numpy(a).cuda(), quant) for a in (gate, up, down)]
    res = torch.zeros(max_tokens, hidden, device="cuda")
    res[:T] = torch.from_numpy(x).cuda()
    canary = 4321.0
    ffn = torch.full((max_tokens, hidden), canary, device="cuda")
    lo = torch.full((max_tokens, hidden), canary, device="cuda")
    blk.forward(torch.from_numpy(post_norm).cuda(), qt[0], qt[1], qt[2], res, T, ffn, lo)
    torch.cuda.synchronize()
    assert blk.moe.device_status() == 0
    untouched = bool((ffn[T:] == canary).all().item() and (lo[T:] == canary).all().item())
    return ffn[:T].cpu().numpy(), lo[:T].cpu().numpy(), blk.moe.buffers().normed[:T].cpu().numpy(), untouched


@pytest.mark.parametrize("hidden,inter,quant,tokens,max_tokens", [
    (512, 1024, 0, 1, 1), (512, 1024, 0, 3, 8), (512, 1024, 0, 64, 64), (512, 1024, 0, 300, 320),
    (512, 1024, 1, 5, 8), (1024, 768, 1, 130, 130),
])
def test_dense_block_matches_the_oracle(oracle, hidden, inter, quant, tokens, max_tokens):
    import torch
    if not torch.cuda.is_available():
        pytest.fail("gpu-marked test collected without a CUDA device")
    post_norm, gate, up, down, x = _dense_inputs(hidden, inter, quant, tokens, seed=40 + tokens)
    want_ffn, want_lo = oracle.dense_block_forward(post_norm, 1e-6, gate, quant, up, quant, down, quant, hidden,
                                                   inter, x, dev_order=True)
    ffn, lo, normed, untouched = _run_dense(torch, hidden, inter, quant, post_norm, gate, up, down, x, max_tokens)
    want_normed = oracle.rms_norm(x, post_norm, 1e-6, dev_order=True)
    assert (bits(normed) == bits(want_normed)).all()
    assert untouched
    for name, got, want in (("ffn_out", ffn, want_ffn), ("l_out", lo, want_lo)):
        r = _rel_l2(got, want)
        assert r <= REL_L2, f"{name}: rel-L2 {r:.3e}, max-abs {np.abs(got - want).max():.3e}"


def test_dense_block_at_the_27b_geometry(oracle):
    """hidden 5120, intermediate 17408, Q6_K, three tokens: contraction lengths the decode kernels
    do not serve, so the tensor-core kernels run at decode width."""
    import torch
    hidden, inter, quant, tokens = 5120, 17408, 0, 3
    post_norm, gate, up, down, x = _dense_inputs(hidden, inter, quant, tokens, seed=77)
    want_ffn, want_lo = oracle.dense_block_forward(post_norm, 1e-6, gate, quant, up, quant, down, quant, hidden,
                                                   inter, x, dev_order=True)
    ffn, lo, _, untouched = _run_dense(torch, hidden, inter, quant, post_norm, gate, up, down, x, 4)
    assert untouched
    r = _rel_l2(ffn, want_ffn)
    assert r <= REL_L2, f"ffn_out: rel-L2 {r:.3e}, max-abs {np.abs(ffn - want_ffn).max():.3e}"
    assert _rel_l2(lo, want_lo) <= REL_L2


def _tp_forward(torch, rank, world, hidden, inter, quant, post_norm, gate, up, down, x, max_tokens):
    from llmxabe_b200.moe import QuantTensor
    from llmxabe_b200.tp import CudaTpBackend, TpDenseFfnBlock
    qt = [QuantTensor(torch.from_numpy(a).cuda(), quant) for a in (gate, up, down)]
    backend = CudaTpBackend(hidden, inter, max_tokens, rank, world, torch.from_numpy(post_norm).cuda(), *qt)
    blk = TpDenseFfnBlock(backend, rank, world)
    T = x.shape[0]
    res = torch.zeros(max_tokens, hidden, device="cuda")
    res[:T] = torch.from_numpy(x).cuda()
    ffn = torch.full((max_tokens, hidden), 4321.0, device="cuda")
    lo = torch.full((max_tokens, hidden), 4321.0, device="cuda")
    blk.forward(res, T, ffn, lo)
    torch.cuda.synchronize()
    assert backend.k.device_status() == 0
    assert bool((ffn[T:] == 4321.0).all().item() and (lo[T:] == 4321.0).all().item())
    return ffn[:T].cpu().numpy(), lo[:T].cpu().numpy()


def test_one_rank_tensor_parallel_equals_the_dense_block():
    import torch
    hidden, inter, quant, tokens = 512, 1024, 0, 9
    post_norm, gate, up, down, x = _dense_inputs(hidden, inter, quant, tokens, seed=5)
    ffn0, lo0, _, _ = _run_dense(torch, hidden, inter, quant, post_norm, gate, up, down, x, 16)
    ffn1, lo1 = _tp_forward(torch, 0, 1, hidden, inter, quant, post_norm, gate, up, down, x, 16)
    assert (bits(ffn0) == bits(ffn1)).all() and (bits(lo0) == bits(lo1)).all()


def _rank_main(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    hidden, inter, quant, tokens = 512, 1536, 0, 20
    post_norm, gate, up, down, x = _dense_inputs(hidden, inter, quant, tokens, seed=6)
    _, lo = _tp_forward(torch, rank, world, hidden, inter, quant, post_norm, gate, up, down, x, 32)
    np.save(os.path.join(out_dir, f"l_out_{rank}.npy"), lo)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_tensor_parallel_matches_the_oracle(tmp_path, oracle):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_rank_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    hidden, inter, quant, tokens = 512, 1536, 0, 20
    post_norm, gate, up, down, x = _dense_inputs(hidden, inter, quant, tokens, seed=6)
    _, want_lo = oracle.dense_block_forward(post_norm, 1e-6, gate, quant, up, quant, down, quant, hidden, inter, x,
                                            dev_order=True)
    l0, l1 = np.load(tmp_path / "l_out_0.npy"), np.load(tmp_path / "l_out_1.npy")
    assert (bits(l0) == bits(l1)).all()          # every rank holds the same all-reduced result
    assert _rel_l2(l0, want_lo) <= REL_L2
