"""GPU parity of the discrete half of the path: dequantisation, routing and
the dispatch tables must equal the oracle bit for bit (ids, ordering, tables)
or within 1e-6 (routing weights), as the reference gates them
(crates/xabe-engine/tests/moe_differential.rs:315-543,
crates/xabe-engine/tests/dequant_differential.rs:1-18)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch_cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("gpu-marked test collected without a CUDA device")
    return torch


@pytest.mark.parametrize("quant,nblocks", [(0, 4096), (1, 8192), (0, 1), (1, 1)])
def test_dequantisation_is_bit_identical(torch_cuda, oracle, quant, nblocks):
    torch = torch_cuda
    from llmxabe_b200.moe import ExpertQuant, QuantTensor, dequantize
    rng = np.random.default_rng(17 + quant)
    bb = 210 if quant == 0 else 34
    raw = rng.integers(0, 256, size=(nblocks, bb), dtype=np.uint8)
    # super-scales across the whole half range, subnormals included, no inf/nan
    d = (rng.standard_normal(nblocks) * 10.0 ** rng.uniform(-7, 1, nblocks)).astype(np.float16)
    off = 208 if quant == 0 else 0
    raw[:, off:off + 2] = d.view(np.uint8).reshape(nblocks, 2)
    want = oracle.dequantize_row(quant, raw.reshape(-1))
    got = dequantize(QuantTensor(torch.from_numpy(raw.reshape(-1)).cuda(), ExpertQuant(quant)))
    torch.cuda.synchronize()
    assert (got.cpu().numpy().view(np.uint32) == want.view(np.uint32)).all()


def test_ragged_tensor_is_rejected(torch_cuda):
    torch = torch_cuda
    from llmxabe_b200.errors import RaggedWeights
    from llmxabe_b200.moe import ExpertQuant, QuantTensor, dequantize
    with pytest.raises(RaggedWeights):
        dequantize(QuantTensor(torch.zeros(211, dtype=torch.uint8, device="cuda"), ExpertQuant.Q6K))


def _route(torch, kernels, logits_np, tokens):
    g = kernels.geometry
    flat = np.full((g.max_tokens, g.num_experts), -1.0e30, np.float32)
    flat[:tokens] = logits_np
    kernels.set_valid_tokens(tokens)
    kernels.route_and_dispatch(torch.from_numpy(flat).cuda())
    torch.cuda.synchronize()
    b = kernels.buffers()
    return b


def _check_tables(oracle, b, ids, g, tokens):
    want = oracle.moe_align_block_size(ids, g.block_size, g.num_experts)
    n = int(b.num_tokens_post_pad.cpu().item())
    assert n == want.num_tokens_post_pad
    s = b.sorted_token_ids.cpu().numpy()
    e = b.expert_ids.cpu().numpy()
    assert (s[:n] == want.sorted_token_ids).all()
    assert (e[: n // g.block_size] == want.expert_ids).all()
    # the fill covers the whole capacity (crates/xabe-cuda/src/kernels/moe.rs:2060-2065)
    assert (s[n:] == tokens * g.experts_per_token).all()
    assert (e[n // g.block_size:] == -1).all()


@pytest.mark.parametrize("block_size,tokens,max_tokens", [(16, 37, 64), (32, 64, 64), (16, 1, 1), (8, 3, 3),
                                                           (64, 300, 512), (32, 2048, 2048)])
def test_routing_and_dispatch_match_the_oracle_exactly(torch_cuda, oracle, block_size, tokens, max_tokens):
    torch = torch_cuda
    from llmxabe_b200.moe import MoeGeometry, MoeKernels
    g = MoeGeometry.qwen3_6(block_size, max_tokens)
    k = MoeKernels(g)
    rng = oracle.Xorshift64Star(0x5EED0A01)  # tests/moe_differential.rs:86
    logits = np.stack([rng.vec_f32(g.num_experts, -8.0, 8.0) for _ in range(tokens)])
    b = _route(torch, k, logits, tokens)
    ids, w = oracle.route_batch(logits, g.experts_per_token)
    got_ids = b.topk_ids.cpu().numpy()[:tokens]
    got_w = b.topk_weights.cpu().numpy()[:tokens]
    assert (got_ids == ids).all()
    assert np.abs(got_w - w).max() <= 1e-6  # tests/moe_differential.rs:367-376
    _check_tables(oracle, b, ids, g, tokens)
    assert k.device_status() == 0
    # a shorter step after a longer one never sees the longer step's ids
    if tokens > 2:
        b = _route(torch, k, logits[:2], 2)
        _check_tables(oracle, b, ids[:2], g, 2)


def test_an_exact_tie_resolves_to_the_lowest_indices(torch_cuda, oracle, kats):
    torch = torch_cuda
    from llmxabe_b200.moe import MoeGeometry, MoeKernels
    c = kats["router_all_tie"]
    g = MoeGeometry.qwen3_6(16, 64)
    k = MoeKernels(g)
    logits = np.full((c["tokens"], g.num_experts), c["value"], np.float32)
    for _ in range(4):
        b = _route(torch, k, logits, c["tokens"])
        assert (b.topk_ids.cpu().numpy()[:c["tokens"]] == np.array(c["ids"])).all()
        assert np.abs(b.topk_weights.cpu().numpy()[:c["tokens"]] - c["weight"]).max() < c["tol"]


def test_dispatch_docstring_example_through_the_device(torch_cuda, oracle, kats):
    """crates/xabe-kernels/src/moe/dispatch.rs:138-169, with logits crafted so the top-3 come out in the listed order."""
    torch = torch_cuda
    from llmxabe_b200.moe import MoeGeometry, MoeKernels
    c = kats["dispatch_docstring"]
    topk = np.array(c["topk"])
    g = MoeGeometry(c["num_experts"], 3, 256, 256, c["block_size"], 4)
    k = MoeKernels(g)
    logits = np.full((4, c["num_experts"]), -20.0, np.float32)
    for t in range(4):
        for j, e in enumerate(topk[t]):
            logits[t, e] = 3.0 - j
    b = _route(torch, k, logits, 4)
    assert (b.topk_ids.cpu().numpy() == topk).all()
    assert b.sorted_token_ids.cpu().numpy()[:16].tolist() == c["sorted_token_ids"]
    assert b.expert_ids.cpu().numpy()[:4].tolist() == c["expert_ids"]
    assert int(b.num_tokens_post_pad.cpu().item()) == c["num_tokens_post_pad"]


@pytest.mark.parametrize("seed,tokens,top_k,num_experts,block_size", [(42, 37, 8, 256, 32), (43, 20, 4, 16, 8)])
def test_seeded_dispatch_recipes(torch_cuda, oracle, seed, tokens, top_k, num_experts, block_size):
    """The seeds of dispatch.rs:172-244, fed as logits whose top-k order is a seeded choice of distinct experts."""
    torch = torch_cuda
    from llmxabe_b200.moe import MoeGeometry, MoeKernels
    rng = oracle.Xorshift64Star(seed)
    g = MoeGeometry(num_experts, top_k, 256, 256, block_size, tokens)
    k = MoeKernels(g)
    logits = np.stack([rng.vec_f32(num_experts, -6.0, 6.0) for _ in range(tokens)])
    b = _route(torch, k, logits, tokens)
    ids, _ = oracle.route_batch(logits, top_k)
    assert (b.topk_ids.cpu().numpy() == ids).all()
    _check_tables(oracle, b, ids, g, tokens)


def test_zero_tokens_is_a_no_op(torch_cuda):
    torch = torch_cuda
    from llmxabe_b200.moe import MoeGeometry, MoeKernels
    g = MoeGeometry.qwen3_6(16, 8)
    k = MoeKernels(g)
    k.set_valid_tokens(0)
    k.route_and_dispatch(torch.zeros(8, 256, device="cuda"))
    torch.cuda.synchronize()
    b = k.buffers()
    assert int(b.num_tokens_post_pad.cpu().item()) == 0
    assert (b.expert_ids.cpu().numpy() == -1).all()
