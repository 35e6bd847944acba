"""Pins the CPU oracle against the reference's own known-answer tests.

Every case is a fact transcribed from a unit test of the reference project
(file:line in tests/golden/reference_kats.json); none needs a GPU.
"""
import itertools

import numpy as np
import pytest


def test_rng_zero_seed_is_remapped(oracle, kats):
    a = oracle.Xorshift64Star(0)
    b = oracle.Xorshift64Star(int(kats["rng_zero_seed"]["state"], 16))
    assert [a.next_u64() for _ in range(8)] == [b.next_u64() for _ in range(8)]
    assert oracle.Xorshift64Star(0).next_u64() != 0


def test_rng_first_output_matches_the_published_transition(oracle):
    # xorshift64*: x^=x>>12; x^=x<<25; x^=x>>27; out = x*0x2545F4914F6CDD1D  (rng.rs:26-33)
    x = 42
    x ^= x >> 12
    x ^= (x << 25) & (2**64 - 1)
    x ^= x >> 27
    assert oracle.Xorshift64Star(42).next_u64() == (x * 0x2545F4914F6CDD1D) % 2**64
    r = oracle.Xorshift64Star(7)
    assert all(0.0 <= r.next_f32() < 1.0 for _ in range(10000))
    r = oracle.Xorshift64Star(99)
    assert all(r.next_u32_below(7) < 7 for _ in range(10000))


@pytest.mark.parametrize("i", range(7))
def test_router_small_vectors(oracle, kats, i):
    c = kats["router"][i]
    ids, w = oracle.route_batch(np.array([c["logits"]], np.float32), c["k"])
    ids, w = ids[0], w[0]
    if "ids" in c:
        assert ids.tolist() == c["ids"]
    if "sorted_ids" in c:
        assert sorted(ids.tolist()) == c["sorted_ids"]
    if "weight_sum_tol" in c:
        assert abs(float(w.sum()) - 1.0) < c["weight_sum_tol"]
    if c.get("weights_strictly_decreasing"):
        assert all(w[j] > w[j + 1] for j in range(len(w) - 1))


def test_router_top8_of_256(oracle, kats):
    c = kats["router_seeded"]
    logits = oracle.Xorshift64Star(c["seed"]).vec_f32(c["num_experts"], c["lo"], c["hi"])
    ids, w = oracle.route_batch(logits[None, :], c["k"])
    assert len(set(ids[0].tolist())) == c["k"]
    assert abs(float(w[0].sum()) - 1.0) < c["weight_sum_tol"]
    # selection is the k largest logits, in descending order
    order = np.argsort(-logits, kind="stable")[: c["k"]]
    assert ids[0].tolist() == order.tolist()


def test_router_all_tie(oracle, kats):
    c = kats["router_all_tie"]
    logits = np.full((c["tokens"], c["num_experts"]), c["value"], np.float32)
    ids, w = oracle.route_batch(logits, c["k"])
    assert (ids == np.array(c["ids"])).all()
    assert np.abs(w - c["weight"]).max() < c["tol"]


def test_dispatch_docstring_example(oracle, kats):
    c = kats["dispatch_docstring"]
    d = oracle.moe_align_block_size(c["topk"], c["block_size"], c["num_experts"])
    assert d.sorted_token_ids.tolist() == c["sorted_token_ids"]
    assert d.expert_ids.tolist() == c["expert_ids"]
    assert d.num_tokens_post_pad == c["num_tokens_post_pad"]


@pytest.mark.parametrize("i", range(2))
def test_dispatch_seeded(oracle, kats, i):
    c = kats["dispatch_seeded"][i]
    rng = oracle.Xorshift64Star(c["seed"])
    topk = np.array([[rng.next_u32_below(c["num_experts"]) for _ in range(c["top_k"])]
                     for _ in range(c["tokens"])], np.int32)
    d = oracle.moe_align_block_size(topk, c["block_size"], c["num_experts"])
    sentinel = c["tokens"] * c["top_k"]
    valid = d.sorted_token_ids[d.sorted_token_ids != sentinel]
    assert sorted(valid.tolist()) == list(range(sentinel))
    flat = topk.reshape(-1)
    for b, e in enumerate(d.expert_ids):
        for s in d.sorted_token_ids[b * c["block_size"]:(b + 1) * c["block_size"]]:
            if s != sentinel:
                assert e != oracle.INACTIVE_EXPERT and flat[s] == e


def test_dispatch_small_cases(oracle, kats):
    a, b, c = kats["dispatch_small"]
    d = oracle.moe_align_block_size(a["topk"], a["block_size"], a["num_experts"])
    assert all(d.sorted_token_ids[s] == 3 for s in a["sentinel_slots"])
    d = oracle.moe_align_block_size(b["topk"], b["block_size"], b["num_experts"])
    assert d.num_tokens_post_pad == b["num_tokens_post_pad"] and d.expert_ids.tolist() == b["expert_ids"]
    d = oracle.moe_align_block_size(c["topk"], c["block_size"], c["num_experts"])
    assert d.num_tokens_post_pad == 4 and (d.sorted_token_ids != 4).all()
    with pytest.raises(ValueError):  # dispatch.rs:281-285
        oracle.moe_align_block_size([[0]], 0, 1)
    with pytest.raises(ValueError):  # dispatch.rs:287-291
        oracle.moe_align_block_size([[5]], 4, 4)


def test_capacity_formulas(oracle, kats):
    for c in kats["capacity"]:
        cap = oracle.sorted_capacity(c["num_experts"], c["top_k"], c["block_size"], c["max_tokens"])
        assert cap == c["sorted_capacity"]
        assert cap // c["block_size"] == c["expert_block_capacity"]
    c = kats["capacity_bruteforce"]
    numel = c["max_tokens"] * c["top_k"]
    worst = 0
    for a, b, cc in itertools.product(range(numel + 1), repeat=3):
        if a + b + cc > numel:
            continue
        parts = [a, b, cc, numel - a - b - cc]
        worst = max(worst, sum(-(-n // c["block_size"]) * c["block_size"] for n in parts))
    assert oracle.sorted_capacity(c["num_experts"], c["top_k"], c["block_size"], c["max_tokens"]) >= worst


def _random_experts(oracle, rng, n, hidden, inter, r):
    g, u, d = [], [], []
    for _ in range(n):
        g.append(rng.vec_f32(inter * hidden, -r, r).reshape(inter, hidden))
        u.append(rng.vec_f32(inter * hidden, -r, r).reshape(inter, hidden))
        d.append(rng.vec_f32(hidden * inter, -r, r).reshape(hidden, inter))
    return np.stack(g), np.stack(u), np.stack(d)


def test_grouped_matches_naive(oracle, kats):
    c = kats["gemm_equivalence"]
    rng = oracle.Xorshift64Star(c["seed"])
    g, u, d = _random_experts(oracle, rng, c["num_experts"], c["hidden"], c["intermediate"], c["w_range"])
    hs = np.stack([rng.vec_f32(c["hidden"], -1.0, 1.0) for _ in range(c["tokens"])])
    logits = np.stack([rng.vec_f32(c["num_experts"], -3.0, 3.0) for _ in range(c["tokens"])])
    ids, w = oracle.route_batch(logits, c["top_k"])
    disp = oracle.moe_align_block_size(ids, c["block_size"], c["num_experts"])
    grouped = oracle.grouped_forward(hs, disp, w, c["top_k"], g, u, d)
    naive = oracle.naive_forward(hs, ids, w, g, u, d)
    r = oracle.compare(grouped, naive)
    assert r.max_abs_error < c["max_abs"] and r.cosine_similarity > c["min_cos"], str(r)


def test_single_expert_reduces_to_shared_expert(oracle, kats):
    c = kats["gemm_single_expert"]
    rng = oracle.Xorshift64Star(c["seed"])
    g, u, d = _random_experts(oracle, rng, c["num_experts"], c["hidden"], c["intermediate"], 0.3)
    hs = np.stack([rng.vec_f32(c["hidden"], -1.0, 1.0) for _ in range(c["tokens"])])
    ids = np.zeros((c["tokens"], 1), np.int32)
    w = np.ones((c["tokens"], 1), np.float32)
    disp = oracle.moe_align_block_size(ids, 4, c["num_experts"])
    grouped = oracle.grouped_forward(hs, disp, w, 1, g, u, d)
    naive = oracle.naive_forward(hs, ids, w, g, u, d)
    for t in range(c["tokens"]):
        direct = oracle.expert_mlp(g[0], u[0], d[0], hs[t])
        assert oracle.compare(grouped[t], direct).max_abs_error < c["max_abs"]
        assert oracle.compare(naive[t], direct).max_abs_error < c["max_abs"]


def test_zero_routing_weight_contributes_nothing(oracle, kats):
    c = kats["gemm_zero_weight"]
    h, i = c["hidden"], c["intermediate"]
    g = np.ones((1, i, h), np.float32)
    d = np.ones((1, h, i), np.float32)
    x = np.ones((1, h), np.float32)
    assert (oracle.expert_mlp(g[0], g[0], d[0], x[0]) != 0).any()
    out = oracle.naive_forward(x, np.zeros((1, 1), np.int32), np.zeros((1, 1), np.float32), g, g, d)
    assert (out == 0).all()


def test_gemv_vectors(oracle, kats):
    for c in kats["gemv"]:
        out = oracle.gemv(np.array(c["w"], np.float32), np.array(c["x"], np.float32))
        assert out.tolist() == [float(v) for v in c["out"]]


def test_block_sizes(oracle, kats):
    assert oracle.BLOCK_BYTES[oracle.Q8_0] == kats["block_bytes"]["q8_0"]
    assert oracle.BLOCK_BYTES[oracle.Q6K] == kats["block_bytes"]["q6_k"]


def test_q6k_hand_built_superblock(oracle, kats):
    c = kats["q6k_hand_built"]
    blk = np.zeros(210, np.uint8)
    blk[0] = c["ql0"]
    blk[128] = c["qh0"]
    blk[192:208] = c["scales"]
    h = oracle.f32_to_f16_bits(c["d"])
    blk[208], blk[209] = h & 0xFF, h >> 8
    y = oracle.dequantize_row(oracle.Q6K, blk)
    assert abs(y[0] - c["y0"]) < c["tol"]
    # every other code is raw 0 -> q = -32 at scale 1, d = 2: -64
    assert (y[1:] == -64.0).all()


def test_q6k_element_map_matches_the_documented_layout(oracle):
    """Independent numpy decode of the Q6_K bit layout (quant.rs:175-198)."""
    rng = np.random.default_rng(5)
    blk = rng.integers(0, 256, 210, dtype=np.uint8)
    blk[208:210] = np.frombuffer(np.float16(0.37).tobytes(), np.uint8)
    y = oracle.dequantize_row(oracle.Q6K, blk)
    d = np.float32(np.float16(0.37))
    sc = blk[192:208].view(np.int8)
    for r in range(256):
        half, grp, l = r // 128, (r % 128) // 32, r % 32
        b = blk[half * 64 + (grp & 1) * 32 + l]
        nib = (b & 0xF) if grp < 2 else (b >> 4)
        hi = (blk[128 + half * 32 + l] >> (2 * grp)) & 3
        q = int(nib | (hi << 4)) - 32
        s = sc[half * 8 + 2 * grp + l // 16]
        want = np.float32(np.float32(d * np.float32(s)) * np.float32(q))
        assert y[r] == want, r


def test_q6k_round_trips(oracle, kats):
    c = kats["q6k_round_trip"]
    x = np.array([oracle.Xorshift64Star(c["seed"]).vec_f32(256, c["lo"], c["hi"])]).reshape(-1)
    y = oracle.dequantize_row(oracle.Q6K, oracle.quantize_row(oracle.Q6K, x))
    r = oracle.compare(y, x)
    assert r.max_abs_error < c["max_abs"] and r.cosine_similarity > c["min_cos"], str(r)
    c = kats["q6k_large"]
    x = oracle.Xorshift64Star(c["seed"]).vec_f32(256, c["lo"], c["hi"])
    y = oracle.dequantize_row(oracle.Q6K, oracle.quantize_row(oracle.Q6K, x))
    assert np.isfinite(y).all() and oracle.compare(y, x).cosine_similarity > c["min_cos"]
    z = np.zeros(256, np.float32)  # quant.rs:643-648
    assert (oracle.dequantize_row(oracle.Q6K, oracle.quantize_row(oracle.Q6K, z)) == 0).all()


def test_q8_0_cases(oracle, kats):
    c = kats["q8_0_round_trip"]
    x = oracle.Xorshift64Star(c["seed"]).vec_f32(32, c["lo"], c["hi"])
    y = oracle.dequantize_row(oracle.Q8_0, oracle.quantize_row(oracle.Q8_0, x))
    step = np.abs(x).max() / 127.0
    assert oracle.compare(y, x).max_abs_error <= step / 2 + 1e-5
    z = np.zeros(32, np.float32)  # quant.rs:600-605
    assert (oracle.dequantize_row(oracle.Q8_0, oracle.quantize_row(oracle.Q8_0, z)) == 0).all()
    c = kats["q8_0_saturate"]
    x = np.zeros(32, np.float32)
    x[0], x[1] = c["x0"], c["x1"]
    q = oracle.quantize_row(oracle.Q8_0, x)[2:].view(np.int8)
    assert q[0] == c["q0"] and q[1] == c["q1"]
    # int8 fields read signed (quant.rs:1340-1347): with d = 1.0 every value is -1
    blk = np.full(34, 255, np.uint8)
    h = oracle.f32_to_f16_bits(1.0)
    blk[0], blk[1] = h & 0xFF, h >> 8
    assert (oracle.dequantize_row(oracle.Q8_0, blk) == -1.0).all()


def test_ragged_rows_are_rejected(oracle, kats):
    c = kats["ragged_rows"]
    with pytest.raises(ValueError):
        oracle.dequantize_row(oracle.Q6K, np.zeros(c["q6k_bytes"], np.uint8))
    with pytest.raises(ValueError):
        oracle.dequantize_row(oracle.Q8_0, np.zeros(c["q8_0_bytes"], np.uint8))


def _rt(oracle, x):
    return oracle.f16_bits_to_f32(oracle.f32_to_f16_bits(x))


def test_f16_conversions(oracle, kats):
    for v in kats["f16_exact"]["values"]:
        assert _rt(oracle, v) == v
    assert np.signbit(np.float32(_rt(oracle, -0.0)))
    assert _rt(oracle, 1.0 + 2.0 ** -11) == 1.0
    assert _rt(oracle, 1.0 + 2.0 ** -10 + 2.0 ** -11) == 1.0 + 2.0 ** -9
    assert _rt(oracle, 1e30) == float("inf") and _rt(oracle, -1e30) == float("-inf")
    assert np.float32(_rt(oracle, 1e-10)).view(np.uint32) == 0
    assert np.float32(_rt(oracle, -1e-10)).view(np.uint32) == 0x80000000
    assert _rt(oracle, 2.0 ** -24) == 2.0 ** -24 and _rt(oracle, 2.0 ** -20) == 2.0 ** -20


def test_f16_agrees_with_numpy_everywhere(oracle, kats):
    c = kats["f16_half_ulp"]
    x = oracle.Xorshift64Star(c["seed"]).vec_f32(20000, c["lo"], c["hi"])
    x = np.concatenate([x, x * 1e-4, x * 1e-6, x * 1e4, x * 3e4]).astype(np.float32)
    want = x.astype(np.float16).view(np.uint16)
    got = np.array([oracle.f32_to_f16_bits(float(v)) for v in x], np.uint16)
    assert (got == want).all()
    allh = np.arange(65536, dtype=np.uint16)
    back = np.array([oracle.f16_bits_to_f32(int(h)) for h in allh], np.float32)
    ref = allh.view(np.float16).astype(np.float32)
    ok = (back.view(np.uint32) == ref.view(np.uint32)) | (np.isnan(back) & np.isnan(ref))
    assert ok.all()
    nz = x[:20000][x[:20000] != 0]
    rt = nz.astype(np.float16).astype(np.float32)
    assert np.abs((rt - nz) / nz).max() <= 2.0 ** -11


def test_norm_and_activations(oracle):
    rng = oracle.Xorshift64Star(11)
    x = rng.vec_f32(2048, -3, 3)
    w = rng.vec_f32(2048, 0.5, 1.5)
    y = oracle.rms_norm(x, w, 1e-6)
    want = x.astype(np.float64) / np.sqrt((x.astype(np.float64) ** 2).mean() + 1e-6) * w
    assert np.abs(y - want).max() < 1e-5
    yd = oracle.rms_norm(x, w, 1e-6, dev_order=True)
    assert np.abs(yd - want).max() < 1e-5
    assert (oracle.rms_norm(np.zeros(2048, np.float32), w, 1e-6) == 0).all()
    for v in (-3.0, -0.5, 0.0, 0.7, 5.0):
        assert abs(oracle.silu(v) - v / (1 + np.exp(-v))) < 1e-6
        assert abs(oracle.sigmoid(v) - 1 / (1 + np.exp(-v))) < 1e-6


def test_device_order_logits_agree_with_sequential_to_rounding(oracle):
    rng = oracle.Xorshift64Star(12)
    w = rng.vec_f32(256 * 2048, -0.05, 0.05).reshape(256, 2048)
    x = rng.vec_f32(2048, -2, 2)
    a = oracle.gemv(w, x)
    b = oracle.router_logits_dev(w, x)[0]
    exact = w.astype(np.float64) @ x.astype(np.float64)
    assert np.abs(a - exact).max() < 2e-5 and np.abs(b - exact).max() < 2e-5
    g = oracle.shared_gate_dot_dev(w[0], x)
    assert g == b[0]  # same lanes, same tree
