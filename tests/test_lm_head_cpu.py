"""CPU checks of the LM head's reference arithmetic and geometry: the oracle against the
reference's own known answers (crates/xabe-kernels/src/gemv.rs tests,
crates/xabe-cuda/src/kernels/lm_head.rs tests), no GPU needed."""
import numpy as np
import pytest


def test_gemv_multiplies_row_major(oracle):
    """gemv.rs `gemv_multiplies_row_major`: [[1,2,3],[4,5,6]] @ [1,10,100] = [321, 654]."""
    out = oracle.gemv(np.array([[1, 2, 3], [4, 5, 6]], dtype=np.float32), np.array([1, 10, 100], dtype=np.float32))
    assert out.tolist() == [321.0, 654.0]


def test_argmax_ties_go_to_the_lower_index(oracle):
    """gemv.rs:102-111."""
    assert oracle.argmax([1.0, 5.0, 5.0, 2.0]) == 1
    assert oracle.argmax([3.0]) == 0
    assert oracle.argmax([-1.0, -1.0, -1.0]) == 0
    assert oracle.argmax([0.0, 1.0, 2.0, 9.0]) == 3


@pytest.mark.parametrize("quant_name", ["Q8_0", "Q6K"])
def test_lm_head_is_gemv_batch_over_dequantised_rows(oracle, quant_name):
    """tests/lm_head_differential.rs:17-19: the reference logits are gemv_batch over rows dequantised
    from the file bytes, each dot product bit-identical to gemv of that row (gemv.rs:61-88)."""
    quant = getattr(oracle, quant_name)
    rng = np.random.default_rng(5)
    vocab, hidden, tokens = 9, 512, 3
    w = (rng.standard_normal((vocab, hidden)) * 0.05).astype(np.float32)
    data = np.concatenate([oracle.quantize_row(quant, r) for r in w])
    x = rng.standard_normal((tokens, hidden)).astype(np.float32)
    got = oracle.lm_head(quant, data, vocab, hidden, x, threads=2)
    rb = data.size // vocab
    wd = np.stack([oracle.dequantize_row(quant, data[i * rb:(i + 1) * rb]) for i in range(vocab)])
    for t in range(tokens):
        assert np.array_equal(got[t], oracle.gemv(wd, x[t]))


def test_geometry_figures_of_the_real_head():
    """lm_head.rs tests `the_real_geometry_costs_the_540_mb_per_token_the_model_docs_claim`,
    `the_batch_tiling_reads_the_weights_once_per_tile_not_once_per_token`; module docs :1-6."""
    from llmxabe_b200.lm_head import HeadFormat, LmHeadGeometry
    g = LmHeadGeometry.qwen3_6(8)
    assert (g.hidden, g.vocab) == (2048, 248_320)
    assert g.row_bytes_for(HeadFormat.Q8_0) == 2176
    assert g.weight_bytes_for(HeadFormat.Q8_0) == 540_344_320
    assert g.elements() == 508_559_360
    assert g.row_bytes_for(HeadFormat.Q6K) == 1680
    assert [g.weight_passes(t) for t in (1, 8, 9, 37)] == [1, 1, 2, 5]
    assert g.weight_bytes_read(37) == 5 * 540_344_320
    assert HeadFormat.from_ggml("q8_0") is HeadFormat.Q8_0 and HeadFormat.from_ggml("q6_K") is HeadFormat.Q6K
    assert HeadFormat.from_ggml("bf16") is None


@pytest.mark.parametrize("kw,reason", [
    (dict(hidden=0), "zero dimension"),
    (dict(vocab=0), "zero dimension"),
    (dict(max_tokens=0), "zero dimension"),
    (dict(hidden=2048 + 32), "multiple of 256"),
    (dict(hidden=8192), "at most 4096"),
])
def test_head_geometry_is_validated_not_assumed(kw, reason):
    """lm_head.rs test `geometry_is_validated_not_assumed`: rejected before any device call."""
    from llmxabe_b200.errors import UnsupportedGeometry
    from llmxabe_b200.lm_head import LmHeadGeometry, LmHeadKernels
    base = dict(hidden=2048, vocab=1024, max_tokens=8)
    base.update(kw)
    with pytest.raises(UnsupportedGeometry, match=reason):
        LmHeadKernels(LmHeadGeometry(**base), device=0)
