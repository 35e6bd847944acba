"""Expert-parallel exchange logic on CPU: two gloo ranks, experts sharded 4 + 4, tokens split in two.

The product's compute backend needs a GPU; here an oracle-backed backend stands in so that the
dispatch / combine plumbing of llmxabe_b200.ep (pair grouping by owner rank, all-to-all-v both
ways, inverse permutation, weighting and ascending-k sum on the sender) is checked end to end
against the single-process oracle block: every output must be bit-identical.
"""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


class OracleBackend:
    """CPU stand-in for CudaEpBackend, built on the oracle (test infrastructure only)."""

    def __init__(self, oracle, L, first_expert, experts_per_rank):
        import torch
        self.torch, self.o, self.L = torch, oracle, L
        n = L.hidden * L.inter
        bb = {0: 210, 1: 34}
        be = {0: 256, 1: 32}

        def mats(stack, quant):
            per = n // be[quant] * bb[quant]
            return [oracle.dequantize_row(quant, stack[(first_expert + e) * per:(first_expert + e + 1) * per])
                    for e in range(experts_per_rank)]
        self.gate = [m.reshape(L.inter, L.hidden) for m in mats(L.gate_exps, L.routed_quant)]
        self.up = [m.reshape(L.inter, L.hidden) for m in mats(L.up_exps, L.routed_quant)]
        self.down = [m.reshape(L.hidden, L.inter) for m in mats(L.down_exps, L.down_quant)]

    def front(self, residual, tokens):
        o, L, t = self.o, self.L, self.torch
        x = residual[:tokens].numpy()
        self.normed = o.rms_norm(x, L.post_norm, L.eps, dev_order=True)
        logits = o.router_logits_dev(L.router, self.normed)
        if L.router_bias is not None:
            logits = logits + L.router_bias[None, :]
        self.ids, self.w = o.route_batch(logits.astype(np.float32), L.top_k)
        return t.from_numpy(self.ids), t.from_numpy(self.w)

    def plan_pack(self, experts_per_rank, world):
        t = self.torch
        K = self.L.top_k
        flat_ids = self.ids.reshape(-1)
        order = np.lexsort((np.arange(flat_ids.size), flat_ids))  # by expert, ascending flat id inside an expert
        rows = self.normed[order // K]
        eid = (flat_ids[order] % experts_per_rank).astype(np.int32)
        inverse = np.empty(order.size, np.int32)
        inverse[order] = np.arange(order.size, dtype=np.int32)
        counts = np.bincount(flat_ids // experts_per_rank, minlength=world).astype(np.int32)
        return t.from_numpy(rows.copy()), t.from_numpy(eid), t.from_numpy(inverse), t.from_numpy(counts)

    def shared(self):
        o, L = self.o, self.L
        self.shexp = o.mlp_forward_q(L.shared_gate, L.shared_quant, L.shared_up, L.shared_quant, L.shared_down,
                                     L.shared_quant, L.hidden, L.inter, self.normed)

    def experts(self, rows, local_expert):
        out = np.empty((rows.shape[0], self.L.hidden), np.float32)
        for r in range(rows.shape[0]):
            e = int(local_expert[r])
            out[r] = self.o.expert_mlp(self.gate[e], self.up[e], self.down[e], rows[r].numpy())
        return self.torch.from_numpy(out)

    def finish(self, back, inverse, residual, tokens, ffn_out, l_out):
        o, L = self.o, self.L
        K, H = L.top_k, L.hidden
        contrib = back.numpy()[inverse.numpy()] * self.w.reshape(-1)[:, None]  # weight * value, flat (token, k) order
        c = contrib.reshape(tokens, K, H)
        routed = np.zeros((tokens, H), np.float32)
        for k in range(K):
            routed = routed + c[:, k]
        shexp = self.shexp
        for t in range(tokens):
            g = np.float32(o.sigmoid(o.shared_gate_dot_dev(L.shared_gate_inp, self.normed[t])))
            v = routed[t] + shexp[t] * g
            ffn_out[t] = self.torch.from_numpy(v)
            l_out[t] = self.torch.from_numpy(v + residual[t].numpy())


def _rank_main(rank, world, port, tokens_total, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    from llmxabe_b200 import synth
    from llmxabe_b200.ep import EpMoeBlock
    from oracle import xabe_oracle as oracle
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    L = synth.moe_layer(seed=9, num_experts=8, top_k=2, hidden=512, inter=256, zipf=True)
    x = synth.activations(tokens_total, 512, seed=9)
    per = tokens_total // world
    mine = torch.from_numpy(x[rank * per:(rank + 1) * per].copy())
    backend = OracleBackend(oracle, L, rank * (8 // world), 8 // world)
    blk = EpMoeBlock(backend, 8, 2, rank, world)
    ffn = torch.zeros(per, 512)
    lo = torch.zeros(per, 512)
    blk.forward(mine, per, ffn, lo)
    np.save(os.path.join(out_dir, f"l_out_{rank}.npy"), lo.numpy())
    np.save(os.path.join(out_dir, f"ffn_{rank}.npy"), ffn.numpy())
    np.save(os.path.join(out_dir, f"counts_{rank}.npy"),
            np.array([blk.last_plan.send_counts, blk.last_plan.recv_counts]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_rank_expert_parallel_block_is_bit_identical_to_one_rank(tmp_path, oracle):
    import torch.multiprocessing as mp
    from helpers import oracle_layer
    from llmxabe_b200 import synth
    world, tokens = 2, 24
    port = _free_port()
    mp.spawn(_rank_main, args=(world, port, tokens, str(tmp_path)), nprocs=world, join=True)
    L = synth.moe_layer(seed=9, num_experts=8, top_k=2, hidden=512, inter=256, zipf=True)
    x = synth.activations(tokens, 512, seed=9)
    want = oracle.moe_block_forward(oracle_layer(oracle, L), x, dev_order=True)
    got_l = np.concatenate([np.load(tmp_path / f"l_out_{r}.npy") for r in range(world)])
    got_f = np.concatenate([np.load(tmp_path / f"ffn_{r}.npy") for r in range(world)])
    assert (got_l.view(np.uint32) == want["l_out"].view(np.uint32)).all()
    assert (got_f.view(np.uint32) == want["ffn_out"].view(np.uint32)).all()
    c0, c1 = np.load(tmp_path / "counts_0.npy"), np.load(tmp_path / "counts_1.npy")
    # what rank 0 sends to rank 1 is what rank 1 receives from rank 0, and every pair is sent once
    assert c0[0][1] == c1[1][0] and c1[0][0] == c0[1][1]
    assert c0[0].sum() == (tokens // world) * 2 and c1[0].sum() == (tokens // world) * 2


def test_plan_groups_pairs_by_owner_in_ascending_flat_order():
    import torch
    from llmxabe_b200.ep import make_plan
    ids = torch.tensor([[5, 0], [1, 7], [6, 2]], dtype=torch.int32)  # 8 experts, 4 per rank, world 1 view
    plan = make_plan(ids, 8, 1)
    assert plan.order.tolist() == [0, 1, 2, 3, 4, 5] and plan.send_counts == [6]
    dst = (ids.reshape(-1).long() // 4)
    order = torch.argsort(dst, stable=True)
    assert order.tolist() == [1, 2, 5, 0, 3, 4]
