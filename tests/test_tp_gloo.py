"""Tensor-parallel dense block on CPU: two gloo ranks, the intermediate dimension split 3 + 3 units.

An oracle-backed backend stands in for the GPU one, so this checks the sharding itself
(llmxabe_b200.tp: row slices of gate/up, block-column slices of down, the all-reduce, the residual)
against the unsharded oracle block.  The ranks' partial sums are added in a different order than the
oracle's single left fold, hence a tolerance (1e-5 relative), not bit identity.
"""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HIDDEN, INTER, TOKENS, QUANT = 512, 1536, 7, 0


class OracleTpBackend:
    def __init__(self, oracle, torch, rank, world, post_norm, gate, up, down):
        from llmxabe_b200.tp import shard_bounds, shard_cols, shard_rows
        self.o, self.torch, self.post_norm = oracle, torch, post_norm
        i0, i1 = shard_bounds(INTER, rank, world)
        self.inter = i1 - i0
        t = torch.from_numpy
        self.gate = shard_rows(t(gate), INTER, HIDDEN, QUANT, i0, i1).numpy()
        self.up = shard_rows(t(up), INTER, HIDDEN, QUANT, i0, i1).numpy()
        self.down = shard_cols(t(down), HIDDEN, INTER, QUANT, i0, i1).numpy()

    def partial_mlp(self, residual, tokens):
        o = self.o
        normed = o.rms_norm(residual[:tokens].numpy(), self.post_norm, 1e-6, dev_order=True)
        out = o.mlp_forward_q(self.gate, QUANT, self.up, QUANT, self.down, QUANT, HIDDEN, self.inter, normed)
        full = np.zeros((residual.shape[0], HIDDEN), np.float32)
        full[:tokens] = out
        return self.torch.from_numpy(full)


def _inputs():
    from llmxabe_b200 import synth
    post_norm, gate, up, down = synth.dense_layer(seed=3, hidden=HIDDEN, inter=INTER, quant=QUANT)
    return post_norm, gate, up, down, synth.activations(TOKENS, HIDDEN, seed=3)


def _rank_main(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from llmxabe_b200.tp import TpDenseFfnBlock
    from oracle import xabe_oracle as oracle
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    post_norm, gate, up, down, x = _inputs()
    blk = TpDenseFfnBlock(OracleTpBackend(oracle, torch, rank, world, post_norm, gate, up, down), rank, world)
    res = torch.zeros(TOKENS + 2, HIDDEN)
    res[:TOKENS] = torch.from_numpy(x)
    ffn = torch.full((TOKENS + 2, HIDDEN), 9.0)
    lo = torch.full((TOKENS + 2, HIDDEN), 9.0)
    blk.forward(res, TOKENS, ffn, lo)
    assert bool((ffn[TOKENS:] == 9.0).all()) and bool((lo[TOKENS:] == 9.0).all())
    np.save(os.path.join(out_dir, f"l_out_{rank}.npy"), lo[:TOKENS].numpy())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_rank_tensor_parallel_dense_block_matches_the_unsharded_oracle(tmp_path, oracle):
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_rank_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    post_norm, gate, up, down, x = _inputs()
    _, want = oracle.dense_block_forward(post_norm, 1e-6, gate, QUANT, up, QUANT, down, QUANT, HIDDEN, INTER, x,
                                         dev_order=True)
    l0, l1 = np.load(tmp_path / "l_out_0.npy"), np.load(tmp_path / "l_out_1.npy")
    assert (l0.view(np.uint32) == l1.view(np.uint32)).all()
    rel = np.linalg.norm(l0.astype(np.float64) - want) / np.linalg.norm(want.astype(np.float64))
    assert rel <= 1e-5, rel


def test_shard_bounds_cover_the_27b_intermediate_size_in_whole_units():
    from llmxabe_b200.tp import shard_bounds
    for world in (1, 2, 4, 8):
        edges = [shard_bounds(17408, r, world) for r in range(world)]
        assert edges[0][0] == 0 and edges[-1][1] == 17408
        assert all(a[1] == b[0] for a, b in zip(edges, edges[1:]))
        assert all((hi - lo) % 256 == 0 and hi > lo for lo, hi in edges)
