"""Expert-parallel block on the GPU.

World 1 (always runs): EpMoeBlock over CudaEpBackend must reproduce MoeBlock.forward bit for bit --
same kernels, same reduction order, the routing weight applied after the (identity) exchange.
World 2 (runs when two devices are visible): two NCCL ranks, experts sharded 128 + 128, tokens split;
the concatenated result must equal the one-GPU block bit for bit as well.
"""
import os
import socket
import sys

import numpy as np
import pytest

from helpers import bits, device_layer, run_block

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _slice_stack(qt, first, count, num_experts):
    from llmxabe_b200.moe import QuantTensor
    per = qt.bytes.numel() // num_experts
    return QuantTensor(qt.bytes[first * per:(first + count) * per].clone(), qt.quant)


def _ep_forward(torch, L, x_np, rank, world, exact, peer_memory=False, live=None, layers=1):
    """One rank's share of the block.  `live`: tokens of this rank that are live (default: all);
    `layers`: how many times the block is applied in a row (the exchange's step counter advances)."""
    from llmxabe_b200.ep import CudaEpBackend, EpMoeBlock, PeerMemoryEpBackend
    from llmxabe_b200.moe import MoeGeometry
    E, K, H = L.num_experts, L.top_k, L.hidden
    w = device_layer(L)
    per = x_np.shape[0] // world
    mine = x_np[rank * per:(rank + 1) * per]
    g = MoeGeometry(E, K, H, L.inter, 16, per)
    epr = E // world
    stacks = (_slice_stack(w.gate_exps, rank * epr, epr, E), _slice_stack(w.up_exps, rank * epr, epr, E),
              _slice_stack(w.down_exps, rank * epr, epr, E))
    if peer_memory:
        backend = PeerMemoryEpBackend(g, epr, rank, world, w, *stacks, exact_decode=exact,
                                      fused_return=peer_memory != "push")
    else:
        backend = CudaEpBackend(g, epr, x_np.shape[0] * K, w, *stacks, exact_decode=exact)
    blk = EpMoeBlock(backend, E, K, rank, world)
    res = torch.from_numpy(mine.copy()).cuda()
    n = per if live is None else live
    ffn = torch.zeros(per, H, device="cuda")
    lo = torch.zeros(per, H, device="cuda")
    for _ in range(layers):
        blk.forward(res, n, ffn, lo)
    torch.cuda.synchronize()
    assert backend.front_k.device_status() == 0 and backend.back_k.device_status() == 0
    return ffn.cpu().numpy()[:n], lo.cpu().numpy()[:n]


@pytest.mark.parametrize("tokens", [1, 24])
def test_one_rank_expert_parallel_equals_the_plain_block(tokens):
    import torch
    if not torch.cuda.is_available():
        pytest.fail("gpu-marked test collected without a CUDA device")
    from llmxabe_b200 import synth
    from llmxabe_b200.moe import MoeBlock, MoeGeometry
    L = synth.moe_layer(seed=21, num_experts=8, top_k=2, hidden=512, inter=256, zipf=True)
    x = synth.activations(tokens, 512, seed=21)
    plain = run_block(MoeBlock(MoeGeometry(8, 2, 512, 256, 16, tokens)), device_layer(L), x, tokens)
    ffn, lo = _ep_forward(torch, L, x, 0, 1, exact=False)
    assert (bits(lo) == bits(plain["l_out"])).all() and (bits(ffn) == bits(plain["ffn_out"])).all()


@pytest.mark.parametrize("mode", ["fused", "push"])
@pytest.mark.parametrize("tokens,live", [(1, 1), (24, 24), (24, 17)])
def test_one_rank_peer_memory_exchange_equals_the_plain_block(tokens, live, mode):
    """The NVLink exchange kernels with a single rank (its own buffers are the "peers"): every kernel of
    the path runs, and repeating the layer advances the step counter the flags compare against."""
    import torch
    from llmxabe_b200 import synth
    from llmxabe_b200.moe import MoeBlock, MoeGeometry
    L = synth.moe_layer(seed=23, num_experts=8, top_k=2, hidden=512, inter=256, zipf=True)
    x = synth.activations(tokens, 512, seed=23)
    plain = run_block(MoeBlock(MoeGeometry(8, 2, 512, 256, 16, tokens)), device_layer(L), x[:live], tokens)
    ffn, lo = _ep_forward(torch, L, x, 0, 1, exact=False, peer_memory=mode, live=live, layers=3)
    assert (bits(lo) == bits(plain["l_out"])).all() and (bits(ffn) == bits(plain["ffn_out"])).all()


def test_a_peer_wait_that_runs_out_reports_status_and_moves_nothing():
    """The failure path of the peer-memory exchange without harming the GPU: the owner waits for a step
    number no sender has announced, with a limit of a few thousand 200 ns iterations.  The wait gives up
    and returns, the status word reads 3, every receive slot is reported empty (so no expert runs and
    nothing is stored into a peer), and the next normal layer is still bit-identical to the plain block."""
    import torch
    from llmxabe_b200 import errors, synth
    from llmxabe_b200.ep import EpMoeBlock, PeerMemoryEpBackend
    from llmxabe_b200.moe import MoeBlock, MoeGeometry
    tokens = 24
    L = synth.moe_layer(seed=24, num_experts=8, top_k=2, hidden=512, inter=256, zipf=True)
    x = synth.activations(tokens, 512, seed=24)
    w = device_layer(L)
    g = MoeGeometry(8, 2, 512, 256, 16, tokens)
    backend = PeerMemoryEpBackend(g, 8, 0, 1, w, w.gate_exps, w.up_exps, w.down_exps)
    blk = EpMoeBlock(backend, 8, 2, 0, 1)
    res = torch.from_numpy(x).cuda()
    ffn = torch.zeros(tokens, 512, device="cuda")
    lo = torch.zeros(tokens, 512, device="cuda")
    blk.forward(res, tokens, ffn, lo)           # a normal layer first: the regions now hold live rows
    torch.cuda.synchronize()
    assert backend.back_k.device_status() == 0
    backend.back_k.set_peer_wait_limit(4000)    # under a millisecond
    backend.slot_ids.fill_(7)
    backend.result_dst.fill_(1)
    backend.back_k.ep_p2p_receive(1, 0, backend.cap, backend.peers, backend.step + 1, backend.slot_ids,
                                  backend.result_dst)
    torch.cuda.synchronize()
    assert bool((backend.slot_ids == -1).all().item()), "a timed-out step must report every slot empty"
    assert bool((backend.result_dst == 0).all().item()), "and no destination pointers"
    with pytest.raises(errors.DeviceStatus, match="status 3"):
        backend.back_k.device_status()
    assert backend.back_k.device_status() == 0  # reading cleared it
    backend.back_k.set_peer_wait_limit(0)
    plain = run_block(MoeBlock(g), w, x, tokens)
    blk.forward(res, tokens, ffn, lo)
    torch.cuda.synchronize()
    assert backend.front_k.device_status() == 0 and backend.back_k.device_status() == 0
    assert (bits(lo.cpu().numpy()) == bits(plain["l_out"])).all()
    for b in backend._shared.values():
        b.release()


def _rank_main(rank, world, port, out_dir, peer_memory=False):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    from llmxabe_b200 import synth
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    L = synth.moe_layer(seed=22, num_experts=8, top_k=2, hidden=512, inter=256, zipf=True)
    x = synth.activations(32, 512, seed=22)
    ffn, lo = _ep_forward(torch, L, x, rank, world, exact=True, peer_memory=peer_memory, layers=2 if peer_memory else 1)
    np.save(os.path.join(out_dir, f"l_out_{rank}.npy"), lo)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("peer_memory", [False, "fused", "push"])
def test_two_rank_expert_parallel_equals_the_plain_block(tmp_path, peer_memory):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from llmxabe_b200 import synth
    from llmxabe_b200.moe import MoeBlock, MoeGeometry
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_rank_main, args=(2, port, str(tmp_path), peer_memory), nprocs=2, join=True)
    L = synth.moe_layer(seed=22, num_experts=8, top_k=2, hidden=512, inter=256, zipf=True)
    x = synth.activations(32, 512, seed=22)
    blk = MoeBlock(MoeGeometry(8, 2, 512, 256, 16, 32))
    blk.set_exact_decode_regime(True)
    plain = run_block(blk, device_layer(L), x, 32)
    got = np.concatenate([np.load(tmp_path / f"l_out_{r}.npy") for r in range(2)])
    assert (bits(got) == bits(plain["l_out"])).all()
