"""GPU parity of the whole MoE block against the CPU oracle, through the C ABI.

Gates (stated here, asserted below):
  normed, router logits      bit-identical to the oracle's device-order restatement
  top-k ids, dispatch tables exact
  routing weights, gate      <= 1e-6 / 2e-6 absolute
  routed, shexp, ffn_out, l_out   rel-L2 <= 1e-3 against the oracle (max-abs printed);
                             the expert products use f16 activations with exact
                             integer codes and fp32 scales and accumulation
  batched vs alone           bit-identical rows
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


def _compare_block(oracle, got, want, g, tokens, label):
    assert (bits(got["normed"]) == bits(want["normed"])).all(), f"{label}: normed not bit-identical"
    assert (bits(got["logits"]) == bits(want["logits"])).all(), f"{label}: logits not bit-identical"
    assert (got["topk_ids"] == want["topk_ids"]).all(), f"{label}: expert ids differ"
    assert np.abs(got["topk_weights"] - want["topk_weights"]).max() <= 1e-6
    d = oracle.moe_align_block_size(want["topk_ids"], g.block_size, g.num_experts)
    n = int(got["num_tokens_post_pad"][0])
    assert n == d.num_tokens_post_pad
    assert (got["sorted_token_ids"][:n] == d.sorted_token_ids).all()
    assert (got["expert_ids"][: n // g.block_size] == d.expert_ids).all()
    assert np.abs(got["gate"] - want["gate"]).max() <= 2e-6
    for name in ("routed", "shexp", "ffn_out", "l_out"):
        r = oracle.compare(got[name], want[name])
        print(f"{label} {name}: {r}")
        assert r.non_finite_count == 0
        assert r.rel_l2 <= REL_L2, f"{label} {name}: {r}"
    assert got["untouched"], f"{label}: rows past the live tokens were written"


# (max_tokens, tokens) per launch structure: one, several, exactly a bucket, bucket + tail
SMALL_WIDTHS = [(1, 1), (2, 2), (4, 3), (8, 6), (16, 16), (19, 19), (40, 37), (64, 64)]


@pytest.mark.parametrize("routed_quant,shared_quant", [(0, 0), (1, 1), (0, 1)])
def test_small_geometry_block(torch_cuda, oracle, routed_quant, shared_quant):
    """H=512, I=256, E=8, K=2, bucket 32: the shape of tests/moe_quant_formats_differential.rs:64-68."""
    from llmxabe_b200 import synth
    from llmxabe_b200.moe import MoeBlock, MoeGeometry
    L = synth.moe_layer(seed=3, num_experts=8, top_k=2, hidden=512, inter=256, routed_quant=routed_quant,
                        shared_quant=shared_quant, zipf=True)
    ol = oracle_layer(oracle, L)
    w = device_layer(L)
    for max_tokens, tokens in SMALL_WIDTHS:
        g = MoeGeometry(8, 2, 512, 256, 32, max_tokens)
        blk = MoeBlock(g)
        x = synth.activations(tokens, 512, seed=3, layer=tokens)
        got = run_block(blk, w, x, max_tokens)
        want = oracle.moe_block_forward(ol, x, dev_order=True)
        _compare_block(oracle, got, want, g, tokens, f"small q{routed_quant}/{shared_quant} T={tokens}")
        assert blk.moe.device_status() == 0


def test_reference_synthetic_weight_recipe(torch_cuda, oracle):
    """Weights built by quantize_q6_k / quantize_q8_0 from the seeded stacks of
    tests/moe_quant_formats_differential.rs:151-161,229-277, widths (1,1),(2,2),(4,3),(8,6)."""
    torch = torch_cuda
    from llmxabe_b200.moe import ExpertQuant, MoeGeometry, MoeKernels, QuantTensor
    H, I, E, K = 512, 256, 8, 2

    def stack(seed, out_dim, in_dim):
        rng = oracle.Xorshift64Star(seed)
        parts = []
        for e in range(E):
            parts.append(rng.vec_f32(out_dim * in_dim, -1.0, 1.0) * np.float32(0.02 * (1.0 + e)))
        return np.concatenate(parts)

    for quant in (0, 1):
        packs = [oracle.quantize_row(quant, stack(s, *dims))
                 for s, dims in ((0x6A7E0001, (I, H)), (0x0BE00002, (I, H)), (0xD0E00003, (H, I)))]
        dev = [QuantTensor(torch.from_numpy(p).cuda(), ExpertQuant(quant)) for p in packs]
        dummy = np.zeros(1, np.float32)
        ol = oracle.Layer(num_experts=E, top_k=K, hidden=H, inter=I, post_norm=np.ones(H, np.float32),
                          router=np.zeros((E, H), np.float32), gate_exps=packs[0], gate_quant=quant,
                          up_exps=packs[1], up_quant=quant, down_exps=packs[2], down_quant=quant,
                          shared_gate_inp=dummy, shared_gate=dummy.view(np.uint8), shared_gate_quant=quant,
                          shared_up=dummy.view(np.uint8), shared_up_quant=quant,
                          shared_down=dummy.view(np.uint8), shared_down_quant=quant)
        for max_tokens, tokens in [(1, 1), (2, 2), (4, 3), (8, 6)]:
            k = MoeKernels(MoeGeometry(E, K, H, I, 32, max_tokens))
            rng = oracle.Xorshift64Star(0xAC170004)
            hs = np.stack([rng.vec_f32(H, -1.0, 1.0) for _ in range(tokens)])
            rng = oracle.Xorshift64Star(0x0F170005)
            logits = np.stack([rng.vec_f32(E, -1.0, 1.0) for _ in range(tokens)])
            flat_h = np.zeros((max_tokens, H), np.float32)
            flat_h[:tokens] = hs
            flat_l = np.zeros((max_tokens, E), np.float32)
            flat_l[:tokens] = logits
            k.set_valid_tokens(tokens)
            k.route_and_dispatch(torch.from_numpy(flat_l).cuda())
            out = torch.zeros(max_tokens, H, device="cuda")
            k.grouped_forward(dev[0], dev[1], dev[2], torch.from_numpy(flat_h).cuda(), out)
            torch.cuda.synchronize()
            ids, w = oracle.route_batch(logits, K)
            want = oracle.routed_forward_q(ol, hs, ids, w)
            r = oracle.compare(out.cpu().numpy()[:tokens], want)
            print(f"recipe quant={quant} n={tokens}/{max_tokens}: {r}")
            assert r.rel_l2 <= REL_L2 and r.cosine_similarity > 1 - 1e-6, str(r)
            assert (out.cpu().numpy()[tokens:] == 0).all()


@pytest.fixture(scope="module")
def real_layer(oracle):
    from llmxabe_b200 import synth
    L = synth.moe_layer(seed=0, layer=0, zipf=True)  # 256/8/2048/512, all Q6_K, Zipf-skewed routing
    return L, oracle_layer(oracle, L)


@pytest.fixture(scope="module")
def real_device_layer(torch_cuda, real_layer):
    return device_layer(real_layer[0])


@pytest.mark.parametrize("max_tokens,tokens,block_size", [(1, 1, 16), (3, 3, 16), (64, 64, 16), (64, 37, 32)])
def test_real_geometry_block(torch_cuda, oracle, real_layer, real_device_layer, max_tokens, tokens, block_size):
    """The one-token and the 3- / 64-token decode shapes: 256 experts, top-8, hidden 2048, intermediate 512, Q6_K, seed 0."""
    from llmxabe_b200 import synth
    from llmxabe_b200.moe import MoeBlock, MoeGeometry
    L, ol = real_layer
    g = MoeGeometry.qwen3_6(block_size, max_tokens)
    blk = MoeBlock(g)
    x = synth.activations(tokens, 2048, seed=0, layer=100 + tokens)
    got = run_block(blk, real_device_layer, x, max_tokens)
    want = oracle.moe_block_forward(ol, x, dev_order=True)
    _compare_block(oracle, got, want, g, tokens, f"real T={tokens}")
    assert blk.moe.device_status() == 0
    # the CPU reference's own sequential order agrees with the device order to rounding
    seq = oracle.moe_block_forward(ol, x[: min(tokens, 4)], dev_order=False)
    assert np.abs(seq["logits"] - want["logits"][: min(tokens, 4)]).max() < 1e-4


def test_batched_rows_are_bit_identical_to_rows_run_alone(torch_cuda, oracle, real_layer, real_device_layer):
    """The serving contract: a sequence's output does not depend on its batch (1, 3 and 64 concurrent sequences)."""
    from llmxabe_b200 import synth
    from llmxabe_b200.moe import MoeBlock, MoeGeometry
    x = synth.activations(64, 2048, seed=0, layer=164)
    big = run_block(MoeBlock(MoeGeometry.qwen3_6(16, 64)), real_device_layer, x, 64)
    three = run_block(MoeBlock(MoeGeometry.qwen3_6(16, 3)), real_device_layer, x[:3], 3)
    alone_blk = MoeBlock(MoeGeometry.qwen3_6(16, 1))
    for name in ("ffn_out", "l_out", "routed", "shexp"):
        assert (bits(three[name]) == bits(big[name][:3])).all(), name
    for t in (0, 1, 2, 17, 63):
        one = run_block(alone_blk, real_device_layer, x[t:t + 1], 1)
        for name in ("ffn_out", "l_out", "routed", "shexp", "logits"):
            assert (bits(one[name][0]) == bits(big[name][t])).all(), (name, t)
    # handles of 16 and 32 tokens (the narrowest that run gate/up through k_gateup_rows) give the same rows
    for width in (16, 32):
        mid = run_block(MoeBlock(MoeGeometry.qwen3_6(16, width)), real_device_layer, x[:width], width)
        for name in ("ffn_out", "l_out", "routed", "shexp"):
            assert (bits(mid[name]) == bits(big[name][:width])).all(), (name, width)
    # and a different bucket width does not change a row either
    wide = run_block(MoeBlock(MoeGeometry.qwen3_6(32, 64)), real_device_layer, x, 64)
    assert (bits(wide["l_out"]) == bits(big["l_out"])).all()
    # run twice: deterministic
    again = run_block(MoeBlock(MoeGeometry.qwen3_6(16, 64)), real_device_layer, x, 64)
    assert (bits(again["l_out"]) == bits(big["l_out"])).all()


def test_host_buffer_entry_point_matches_the_device_one(torch_cuda, real_device_layer):
    torch = torch_cuda
    from llmxabe_b200 import synth
    from llmxabe_b200.moe import MoeBlock, MoeGeometry
    x = synth.activations(8, 2048, seed=0, layer=108)
    blk = MoeBlock(MoeGeometry.qwen3_6(16, 8))
    dev = run_block(blk, real_device_layer, x, 8)
    hx = torch.from_numpy(x).pin_memory()
    hf = torch.empty(8, 2048).pin_memory()
    hl = torch.empty(8, 2048).pin_memory()
    blk.forward_host(real_device_layer, hx, 8, hf, hl)
    torch.cuda.synchronize()
    assert (bits(hl.numpy()) == bits(dev["l_out"])).all() and (bits(hf.numpy()) == bits(dev["ffn_out"])).all()


def test_error_paths_mirror_the_reference(torch_cuda, real_device_layer):
    torch = torch_cuda
    from llmxabe_b200 import errors
    from llmxabe_b200.moe import ExpertQuant, MoeBlock, MoeGeometry, MoeKernels, QuantTensor
    blk = MoeBlock(MoeGeometry.qwen3_6(16, 4))
    buf = torch.zeros(4, 2048, device="cuda")
    with pytest.raises(errors.TooManyTokens):
        blk.forward(real_device_layer, buf, 5, buf.clone(), buf.clone())
    with pytest.raises(errors.BufferLength):
        blk.forward(real_device_layer, buf[:3], 3, buf.clone(), buf.clone())
    w = real_device_layer
    short = QuantTensor(w.gate_exps.bytes[:-210], ExpertQuant.Q6K)
    with pytest.raises(errors.WrongElementCount):
        blk.moe.grouped_forward_partial(short, w.up_exps, w.down_exps)
    ragged = QuantTensor(w.gate_exps.bytes[:-16], ExpertQuant.Q6K)
    with pytest.raises(errors.RaggedWeights):
        blk.moe.grouped_forward_partial(ragged, w.up_exps, w.down_exps)
    shared_only = MoeKernels(MoeGeometry.qwen3_6(16, 4), scope=MoeKernels.SCOPE_SHARED_ONLY)
    with pytest.raises(errors.SharedOnlyBuffers):
        shared_only.route_and_dispatch(torch.zeros(4, 256, device="cuda"))
