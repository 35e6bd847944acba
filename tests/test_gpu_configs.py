"""GPU parity at the benchmark configurations' own shapes, through the C ABI, against the CPU oracle.

What each group covers (256 experts / top-8 / hidden 2048 / intermediate 512 unless said otherwise):
  * a 2048-token bf16 prefill chunk with Zipf-skewed routing: the hottest expert holds more than 500
    tokens, so an expert spans several 128-token tiles of the tensor-core kernels;
  * the per-tensor formats of the shipped model file (docs/MODEL.md:124-141): routed gate/up Q6_K with
    routed down Q8_0 and a Q8_0 shared expert (blocks 0-38), and all-Q8_0 (block 39);
  * every token width at which this library switches kernels (8|9, 15|16, 31|32, 255|256, 511|512) and
    the speculative-verify widths 2, 4, 8, 12 (crates/xabe-engine/tests/serving_speculative_identity.rs:37-41),
    the width list of docs/TESTING.md:426-460, with handles wider than the live token count;
  * one layer of the 40-layer expert-parallel stack: Q8_0 router dequantised at upload, Q8_0 shared
    expert, 16384 tokens on the device, a seeded sample of rows checked, through both exchange backends;
  * the dense 27B block (hidden 5120, intermediate 17408) at 64 tokens and, by sampled rows, at 4096.

Gates, as in crates/xabe-engine/tests/moe_differential.rs:73-93,1097-1576: ids and dispatch tables
exact, routing weights <= 1e-6, outputs rel-L2 <= 1e-3 with max-abs printed, rows at and past the live
token count untouched.
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


def _check_block(oracle, got, want, g, label, tables=True):
    assert (bits(got["normed"]) == bits(want["normed"])).all(), f"{label}: normed not bit-identical"
    assert (bits(got["logits"]) == bits(want["logits"])).all(), f"{label}: logits not bit-identical"
    assert (got["topk_ids"] == want["topk_ids"]).all(), f"{label}: expert ids differ"
    assert np.abs(got["topk_weights"] - want["topk_weights"]).max() <= 1e-6, f"{label}: routing weights"
    if tables:
        d = oracle.moe_align_block_size(want["topk_ids"], g.block_size, g.num_experts)
        n = int(got["num_tokens_post_pad"][0])
        assert n == d.num_tokens_post_pad, f"{label}: post-pad count"
        assert (got["sorted_token_ids"][:n] == d.sorted_token_ids).all(), f"{label}: sorted_token_ids"
        assert (got["expert_ids"][: n // g.block_size] == d.expert_ids).all(), f"{label}: expert_ids"
    assert np.abs(got["gate"] - want["gate"]).max() <= 2e-6, f"{label}: shared gate"
    for name in ("routed", "shexp", "ffn_out", "l_out"):
        r = oracle.compare(got[name], want[name])
        print(f"{label} {name}: {r}")
        assert r.non_finite_count == 0 and r.rel_l2 <= REL_L2, f"{label} {name}: {r}"
    assert got["untouched"], f"{label}: rows past the live tokens were written"


# ---------------------------------------------------------------------------------------------
# layers (host generation of a 256-expert layer takes seconds, so each layout is built once)
# ---------------------------------------------------------------------------------------------
LAYOUTS = {
    # name: (routed gate/up, routed down, shared)
    "q6k": (0, 0, 0),
    "shipped_0_38": (0, 1, 1),   # Q6_K gate/up, Q8_0 down, Q8_0 shared
    "shipped_39": (1, 1, 1),     # all Q8_0
}


@pytest.fixture(scope="module")
def layers(torch_cuda, oracle):
    from llmxabe_b200 import synth
    cache = {}

    def get(name):
        if name not in cache:
            rq, dq, sq = LAYOUTS[name]
            L = synth.moe_layer(seed=0, layer=0, routed_quant=rq, down_quant=dq, shared_quant=sq, zipf=True)
            cache[name] = (L, oracle_layer(oracle, L), device_layer(L))
        return cache[name]
    return get


def _run(oracle, layers, layout, tokens, max_tokens, block_size, x_layer, bf16=False, exact=False):
    from llmxabe_b200 import synth
    from llmxabe_b200.moe import MoeBlock, MoeGeometry
    L, ol, w = layers(layout)
    g = MoeGeometry.qwen3_6(block_size, max_tokens)
    blk = MoeBlock(g)
    if exact:
        blk.set_exact_decode_regime(True)
    x = synth.activations(tokens, 2048, seed=0, layer=x_layer, bf16=bf16)
    got = run_block(blk, w, x, max_tokens)
    assert blk.moe.device_status() == 0
    want = oracle.moe_block_forward(ol, x, dev_order=True)
    return g, got, want


def test_prefill_chunk_of_2048_tokens_with_a_hot_expert(torch_cuda, oracle, layers):
    """2048 bf16-rounded tokens, Zipf routing (about 64 tokens per expert, the hottest above 500)."""
    g, got, want = _run(oracle, layers, "q6k", 2048, 2048, 32, x_layer=4048, bf16=True)
    counts = np.bincount(want["topk_ids"].reshape(-1), minlength=256)
    print(f"tokens per expert: max {counts.max()}, mean {counts.mean():.1f}, active {(counts > 0).sum()}")
    assert counts.max() > 500, "the input was meant to put an expert on the multi-tile path"
    _check_block(oracle, got, want, g, "prefill T=2048")


def test_prefill_chunk_as_bf16_rows(torch_cuda, oracle, layers):
    """The same entry point fed bf16 rows (a 16-bit shift widens them exactly): equal to the f32 feed."""
    torch = torch_cuda
    from llmxabe_b200 import synth
    from llmxabe_b200.moe import MoeBlock, MoeGeometry
    _, _, w = layers("q6k")
    T = 640
    x = synth.activations(T, 2048, seed=0, layer=4640, bf16=True)
    blk = MoeBlock(MoeGeometry.qwen3_6(32, T))
    f32 = run_block(blk, w, x, T)
    ffn = torch.zeros(T, 2048, device="cuda")
    lo = torch.zeros(T, 2048, device="cuda")
    blk.forward(w, torch.from_numpy(x).cuda().to(torch.bfloat16), T, ffn, lo)
    torch.cuda.synchronize()
    assert (bits(ffn.cpu().numpy()) == bits(f32["ffn_out"])).all()
    assert (bits(lo.cpu().numpy()) == bits(f32["l_out"])).all()


@pytest.mark.parametrize("layout", ["shipped_0_38", "shipped_39"])
@pytest.mark.parametrize("tokens,max_tokens,block_size", [(1, 1, 16), (3, 3, 16), (64, 64, 16), (2048, 2048, 32)])
def test_shipped_file_layouts(torch_cuda, oracle, layers, layout, tokens, max_tokens, block_size):
    """Routed gate/up and down in different formats, shared expert in Q8_0 (blocks 0-38), all-Q8_0 (block 39)."""
    g, got, want = _run(oracle, layers, layout, tokens, max_tokens, block_size, x_layer=5000 + tokens,
                        bf16=tokens >= 512)
    _check_block(oracle, got, want, g, f"{layout} T={tokens}")


# every width at which a different kernel (or launch structure) takes over, both sides of it
SWITCH_WIDTHS = [(2, 2), (4, 4), (8, 8), (9, 9), (12, 12), (15, 15), (16, 16), (17, 17), (31, 31), (32, 32),
                 (63, 64), (65, 65), (128, 128), (255, 255), (256, 256), (511, 511),
                 # handles wider than the live count: the launch shape of the wider handle, fewer live rows
                 (5, 9), (9, 16), (15, 32), (17, 256), (100, 511), (300, 512)]


@pytest.mark.parametrize("tokens,max_tokens", SWITCH_WIDTHS)
def test_kernel_switch_widths_at_the_real_geometry(torch_cuda, oracle, layers, tokens, max_tokens):
    block_size = 16 if max_tokens <= 64 else 32
    g, got, want = _run(oracle, layers, "q6k", tokens, max_tokens, block_size, x_layer=6000 + tokens)
    _check_block(oracle, got, want, g, f"width T={tokens}/{max_tokens}")


def test_rows_are_bit_identical_across_the_kernel_switches(torch_cuda, oracle, layers):
    """Batched rows equal the rows run alone on both sides of 8|9 and 15|16 (and up to 511, below the
    tensor-core switch): each handle width picks different kernels, a row's floats do not move."""
    from llmxabe_b200 import synth
    from llmxabe_b200.moe import MoeBlock, MoeGeometry
    _, _, w = layers("q6k")
    x = synth.activations(511, 2048, seed=0, layer=7511)
    ref = {}
    alone = MoeBlock(MoeGeometry.qwen3_6(16, 1))
    for t in (0, 7, 8, 14, 15, 16, 30, 31, 254, 255, 510):
        ref[t] = run_block(alone, w, x[t:t + 1], 1)
    for width in (8, 9, 15, 16, 17, 31, 32, 255, 256, 511):
        got = run_block(MoeBlock(MoeGeometry.qwen3_6(16 if width <= 64 else 32, width)), w, x[:width], width)
        for t, one in ref.items():
            if t >= width:
                continue
            for name in ("logits", "routed", "shexp", "ffn_out", "l_out"):
                assert (bits(one[name][0]) == bits(got[name][t])).all(), (name, t, width)


@pytest.mark.parametrize("tokens,max_tokens", [(257, 257), (301, 512), (2, 256), (1030, 1030)])
def test_router_kernels_agree_bit_for_bit(torch_cuda, oracle, layers, tokens, max_tokens):
    """Three router launches serve the prefill widths (token rows broadcast from shared memory; expert rows
    held in registers, sixteen per CTA with one CTA per SM or eight with two): identical logits, equal to
    the oracle's."""
    from llmxabe_b200 import synth
    from llmxabe_b200.moe import MoeBlock, MoeGeometry
    _, ol, w = layers("q6k")
    x = synth.activations(tokens, 2048, seed=0, layer=7700 + tokens)
    want = oracle.moe_block_forward(ol, x, dev_order=True)["logits"]
    for mode in (2, 1, 0):
        blk = MoeBlock(MoeGeometry.qwen3_6(32, max_tokens))
        blk.moe.set_tuning("router_regw", mode)
        got = run_block(blk, w, x, max_tokens)
        assert blk.moe.device_status() == 0
        assert (bits(got["logits"]) == bits(want)).all(), f"router_regw={mode}"
        assert got["untouched"]


# (tokens, max_tokens, launches per layer: default [the router normalises its rows at one or two tokens],
#  last stage folded into the down launch, front fused as well)
FUSION_WIDTHS = [(1, 1, 5, 5, 3), (2, 2, 5, 5, 3), (3, 4, 6, 5, 3), (8, 8, 6, 5, 3), (12, 15, 7, 6, 3), (16, 16, 7, 7, 4),
                 (64, 64, 7, 7, 5), (200, 256, 7, 7, 5)]


@pytest.mark.parametrize("tokens,max_tokens,launches_default,launches_tail,launches_both", FUSION_WIDTHS)
def test_fused_decode_launches_equal_the_unfused_ones(torch_cuda, oracle, layers, tokens, max_tokens,
                                                      launches_default, launches_tail, launches_both):
    """By default the router of a handle of one or two tokens normalises its input rows itself (no RMSNorm
    launch: five launches per layer instead of six).  Per-handle switches also fold the gate-and-combine
    stage of handles under 16 tokens into the down projection's launch, and run norm, router, routing
    and dispatch as ONE launch: with both, three launches per layer.  Every waypoint and table must be
    bit-identical to the one-kernel-per-stage path, whichever combination runs."""
    from llmxabe_b200 import synth
    from llmxabe_b200.moe import MoeBlock, MoeGeometry, kernel_launch_count
    torch = torch_cuda
    _, _, w = layers("q6k")
    g = MoeGeometry.qwen3_6(16, max_tokens)
    x = synth.activations(tokens, 2048, seed=0, layer=8000 + tokens)
    plain_blk = MoeBlock(g)
    plain_blk.moe.set_tuning("fused_decode", 0)
    plain = run_block(plain_blk, w, x, max_tokens)
    plain2 = run_block(plain_blk, w, x[: max(1, tokens - 1)], max_tokens)
    for mode, launches in ((4, launches_default), (1, launches_tail), (3, launches_both)):
        blk = MoeBlock(g)
        blk.moe.set_tuning("fused_decode", mode)
        fused = run_block(blk, w, x, max_tokens)
        assert blk.moe.device_status() == 0
        for name in ("normed", "logits", "topk_weights", "gate", "routed", "shexp", "ffn_out", "l_out"):
            assert (bits(fused[name]) == bits(plain[name])).all(), (mode, name)
        for name in ("topk_ids", "sorted_token_ids", "expert_ids", "num_tokens_post_pad"):
            assert (fused[name] == plain[name]).all(), (mode, name)
        assert fused["untouched"]
        # a second step on the same handle (the arrival counters must have returned to zero), fewer live rows
        again = run_block(blk, w, x[: max(1, tokens - 1)], max_tokens)
        assert (bits(again["l_out"]) == bits(plain2["l_out"])).all() and again["untouched"], mode
        # launches per step, counted at the launch sites (the token count is already published)
        res = torch.zeros(max_tokens, 2048, device="cuda")
        out = torch.zeros(max_tokens, 2048, device="cuda")
        n0 = kernel_launch_count()
        blk.forward(w, res, max(1, tokens - 1), out, out.clone())
        assert kernel_launch_count() - n0 == launches, mode
        torch.cuda.synchronize()


def test_exact_decode_regime_holds_rows_across_the_tensor_core_switch(torch_cuda, oracle, layers):
    """With the exact-decode switch (moe.rs:5450) a 512-token handle keeps the decode kernels, so its
    rows equal the rows run alone; without it the tensor-core kernels differ by the weight rounding only."""
    from llmxabe_b200 import synth
    from llmxabe_b200.moe import MoeBlock, MoeGeometry
    _, _, w = layers("q6k")
    x = synth.activations(512, 2048, seed=0, layer=7512)
    blk = MoeBlock(MoeGeometry.qwen3_6(32, 512))
    blk.set_exact_decode_regime(True)
    exact = run_block(blk, w, x, 512)
    alone = MoeBlock(MoeGeometry.qwen3_6(16, 1))
    for t in (0, 100, 511):
        one = run_block(alone, w, x[t:t + 1], 1)
        assert (bits(one["l_out"][0]) == bits(exact["l_out"][t])).all(), t
    fast = run_block(MoeBlock(MoeGeometry.qwen3_6(32, 512)), w, x, 512)
    r = oracle.compare(fast["l_out"], exact["l_out"])
    print(f"tensor-core kernels vs decode kernels at 512 tokens: {r}")
    assert r.rel_l2 <= REL_L2


# ---------------------------------------------------------------------------------------------
# one layer of the expert-parallel prefill stack at its real size
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("backend_name", ["nccl_path", "peer_memory"])
def test_expert_parallel_layer_at_16384_tokens(torch_cuda, oracle, backend_name):
    """Q6_K routed experts, Q8_0 shared expert, Q8_0 router (dequantised with q * d at upload), 16384
    tokens on the device, one rank.  256 seeded rows are checked against the oracle (a token's output
    depends on its own row only), ids exact, outputs rel-L2 <= 1e-3."""
    torch = torch_cuda
    from llmxabe_b200 import synth
    from llmxabe_b200.ep import CudaEpBackend, EpMoeBlock, PeerMemoryEpBackend
    from llmxabe_b200.moe import ExpertQuant, MoeGeometry, QuantTensor, dequantize
    E, K, H, I, T = 256, 8, 2048, 512, 16384
    L = synth.moe_layer(seed=3, layer=0, routed_quant=0, shared_quant=1, zipf=True)
    router_q8 = synth.q8_0_bytes(E * H, 3, 0, 11)
    router_dev = dequantize(QuantTensor(torch.from_numpy(router_q8).cuda(), ExpertQuant.Q8_0)).view(E, H)
    router_host = oracle.dequantize_row(1, router_q8).reshape(E, H)
    assert (bits(router_dev.cpu().numpy()) == bits(router_host)).all(), "router dequantisation is bit-exact"
    L.router = router_host
    w = device_layer(L)
    ol = oracle_layer(oracle, L)
    g = MoeGeometry(E, K, H, I, 64, T)
    stacks = (w.gate_exps, w.up_exps, w.down_exps)
    if backend_name == "peer_memory":
        backend = PeerMemoryEpBackend(g, E, 0, 1, w, *stacks)
    else:
        backend = CudaEpBackend(g, E, T * K, w, *stacks)
    blk = EpMoeBlock(backend, E, K, 0, 1)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(163)
    x = torch.randn(T, H, device="cuda", generator=gen)
    ffn = torch.zeros(T, H, device="cuda")
    lo = torch.zeros(T, H, device="cuda")
    blk.forward(x, T, ffn, lo)
    torch.cuda.synchronize()
    assert backend.front_k.device_status() == 0 and backend.back_k.device_status() == 0
    rows = np.sort(np.random.default_rng(16384).choice(T, size=256, replace=False))
    idx = torch.from_numpy(rows).cuda()
    want = oracle.moe_block_forward(ol, x[idx].cpu().numpy(), dev_order=True)
    fb = backend.front_k.buffers()
    assert (fb.topk_ids[idx].cpu().numpy() == want["topk_ids"]).all(), "expert ids of the sampled rows"
    assert np.abs(fb.topk_weights[idx].cpu().numpy() - want["topk_weights"]).max() <= 1e-6
    for name, t in (("ffn_out", ffn), ("l_out", lo)):
        r = oracle.compare(t[idx].cpu().numpy(), want[name])
        print(f"ep layer ({backend_name}) {name}, 256 of {T} rows: {r}")
        assert r.non_finite_count == 0 and r.rel_l2 <= REL_L2, f"{name}: {r}"
    # every row was produced: nothing left at the zero the outputs started from
    assert bool((lo.abs().sum(dim=1) > 0).all().item())
    if backend_name == "peer_memory":
        for b in backend._shared.values():
            b.release()


# ---------------------------------------------------------------------------------------------
# dense 27B block
# ---------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def dense_27b(torch_cuda):
    torch = torch_cuda
    from llmxabe_b200 import synth
    from llmxabe_b200.moe import QuantTensor
    hidden, inter = 5120, 17408
    post_norm, gate, up, down = synth.dense_layer(seed=78, hidden=hidden, inter=inter, quant=0)
    dev = [QuantTensor(torch.from_numpy(a).cuda(), 0) for a in (gate, up, down)]
    return hidden, inter, post_norm, (gate, up, down), dev


def _dense_forward(torch, dense_27b, x, max_tokens):
    from llmxabe_b200.moe import DenseFfnBlock, MoeGeometry
    hidden, inter, post_norm, _, dev = dense_27b
    T = x.shape[0]
    blk = DenseFfnBlock(MoeGeometry(1, 1, hidden, inter, 64, max_tokens))
    res = torch.zeros(max_tokens, hidden, device="cuda")
    res[:T] = torch.from_numpy(x).cuda()
    ffn = torch.full((max_tokens, hidden), 4321.0, device="cuda")
    lo = torch.full((max_tokens, hidden), 4321.0, device="cuda")
    blk.forward(torch.from_numpy(post_norm).cuda(), dev[0], dev[1], dev[2], res, T, ffn, lo)
    torch.cuda.synchronize()
    assert blk.moe.device_status() == 0
    assert bool((ffn[T:] == 4321.0).all().item() and (lo[T:] == 4321.0).all().item())
    return ffn[:T].cpu().numpy(), lo[:T].cpu().numpy()


@pytest.mark.parametrize("tokens,max_tokens", [(1, 1), (64, 64), (40, 64)])
def test_dense_27b_block_at_decode_widths(torch_cuda, oracle, dense_27b, tokens, max_tokens):
    from llmxabe_b200 import synth
    hidden, inter, post_norm, (gate, up, down), _ = dense_27b
    x = synth.activations(tokens, hidden, seed=78, layer=tokens)
    want_ffn, want_lo = oracle.dense_block_forward(post_norm, 1e-6, gate, 0, up, 0, down, 0, hidden, inter, x,
                                                   dev_order=True)
    ffn, lo = _dense_forward(torch_cuda, dense_27b, x, max_tokens)
    for name, got, want in (("ffn_out", ffn, want_ffn), ("l_out", lo, want_lo)):
        r = oracle.compare(got, want)
        print(f"dense 27B T={tokens} {name}: {r}")
        assert r.non_finite_count == 0 and r.rel_l2 <= REL_L2, f"{name}: {r}"


def test_dense_27b_rows_are_batch_invariant_and_agree_with_the_tensor_core_path(torch_cuda, oracle, dense_27b):
    """Decode widths of the dense block run k_dense_rows (slices of the contraction streamed with the
    activations, one accumulator tile per eight tokens).  A token's row must not depend on its batch:
    the 64-token handle's rows equal the rows run alone bit for bit; and the tcgen05 kernels, which the
    per-handle switch brings back, agree to the weight rounding."""
    torch = torch_cuda
    from llmxabe_b200 import synth
    from llmxabe_b200.moe import DenseFfnBlock, MoeGeometry
    hidden, inter, post_norm, _, dev = dense_27b
    x = synth.activations(64, hidden, seed=78, layer=64)
    ffn64, lo64 = _dense_forward(torch, dense_27b, x, 64)
    for tk in (0, 7, 8, 33, 63):
        ffn1, lo1 = _dense_forward(torch, dense_27b, x[tk:tk + 1], 1)
        assert (bits(ffn1[0]) == bits(ffn64[tk])).all() and (bits(lo1[0]) == bits(lo64[tk])).all(), tk
    ffn20, _ = _dense_forward(torch, dense_27b, x[:20], 24)
    assert (bits(ffn20) == bits(ffn64[:20])).all()
    blk = DenseFfnBlock(MoeGeometry(1, 1, hidden, inter, 64, 64))
    blk.moe.set_tuning("dense_rows", 0)
    res = torch.from_numpy(x).cuda()
    ffn = torch.zeros(64, hidden, device="cuda")
    lo = torch.zeros(64, hidden, device="cuda")
    blk.forward(torch.from_numpy(post_norm).cuda(), dev[0], dev[1], dev[2], res, 64, ffn, lo)
    torch.cuda.synchronize()
    r = oracle.compare(ffn.cpu().numpy(), ffn64)
    print(f"dense 27B, 64 tokens, tensor-core kernels vs k_dense_rows: {r}")
    assert r.rel_l2 <= REL_L2


def test_dense_27b_block_at_4096_tokens_by_sampled_rows(torch_cuda, oracle, dense_27b):
    """The prefill width of the dense block: all 4096 rows computed on the device, 48 seeded rows
    compared with the oracle (a row depends on its own input only)."""
    from llmxabe_b200 import synth
    hidden, inter, post_norm, (gate, up, down), _ = dense_27b
    T = 4096
    x = synth.activations(T, hidden, seed=78, layer=4096)
    ffn, lo = _dense_forward(torch_cuda, dense_27b, x, T)
    rows = np.sort(np.random.default_rng(4096).choice(T, size=48, replace=False))
    want_ffn, want_lo = oracle.dense_block_forward(post_norm, 1e-6, gate, 0, up, 0, down, 0, hidden, inter,
                                                   x[rows], dev_order=True)
    for name, got, want in (("ffn_out", ffn[rows], want_ffn), ("l_out", lo[rows], want_lo)):
        r = oracle.compare(got, want)
        print(f"dense 27B T=4096, 48 rows, {name}: {r}")
        assert r.non_finite_count == 0 and r.rel_l2 <= REL_L2, f"{name}: {r}"
    assert np.isfinite(ffn).all() and float(np.abs(ffn).sum(axis=1).min()) > 0
