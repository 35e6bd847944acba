"""GPU parity of the LM head (xabe_lm_head_forward / _argmax) against the CPU oracle.

Gates (the reference's, crates/xabe-engine/tests/lm_head_differential.rs:17-19,114-137):
  logits           rel-L2 <= 2e-5 against gemv over dequantised rows (the reference measures
                   4e-6 for its fp32 path; here an activation keeps 22 bits), max-abs printed
  argmax           exact, every token
  batched vs alone bit-identical logits per token (one pass serves up to eight tokens)
  rows past the live tokens untouched
"""
import numpy as np
import pytest

from helpers import bits

pytestmark = pytest.mark.gpu
REL_L2 = 2e-5


@pytest.fixture(scope="module")
def torch_cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("gpu-marked test collected without a CUDA device")
    return torch


def _head(torch, quant, vocab, hidden, max_tokens, seed):
    from llmxabe_b200 import synth
    from llmxabe_b200.lm_head import HeadFormat, HeadTensor, LmHeadGeometry, LmHeadKernels
    data = synth.quant_bytes(quant, vocab * hidden, seed, 77, 3)
    fmt = HeadFormat.Q6K if quant == synth.Q6K else HeadFormat.Q8_0
    k = LmHeadKernels(LmHeadGeometry(hidden, vocab, max_tokens))
    return data, HeadTensor(torch.from_numpy(data).cuda(), fmt), k


def _run(torch, k, w, x_np, max_tokens, vocab):
    T, H = x_np.shape
    x = torch.zeros(max_tokens, H, device="cuda")
    x[:T] = torch.from_numpy(x_np).cuda()
    canary = -777.0
    logits = torch.full((max_tokens, vocab), canary, device="cuda")
    k.forward(w, x, T, logits)
    ids = torch.full((max_tokens,), -1, dtype=torch.int32, device="cuda")
    k.argmax(logits, T, ids)
    torch.cuda.synchronize()
    assert bool((logits[T:] == canary).all().item()), "rows past the live tokens were written"
    assert bool((ids[T:] == -1).all().item())
    return logits[:T].cpu().numpy(), ids[:T].cpu().numpy()


@pytest.mark.parametrize("quant_name,vocab,tokens", [("Q8_0", 1000, 1), ("Q8_0", 2048, 5), ("Q8_0", 777, 11),
                                                     ("Q6K", 640, 3)])
def test_logits_and_argmax_match_the_oracle(torch_cuda, oracle, quant_name, vocab, tokens):
    torch = torch_cuda
    from llmxabe_b200 import synth
    quant = getattr(synth, quant_name)
    hidden, max_tokens = 2048, 16
    data, w, k = _head(torch, quant, vocab, hidden, max_tokens, seed=21)
    x = synth.activations(tokens, hidden, seed=21, layer=vocab)
    got, ids = _run(torch, k, w, x, max_tokens, vocab)
    want = oracle.lm_head(getattr(oracle, quant_name), data, vocab, hidden, x)
    r = oracle.compare(got, want)
    print(f"lm_head {quant_name} vocab={vocab} T={tokens}: {r}")
    assert r.non_finite_count == 0 and r.rel_l2 <= REL_L2, str(r)
    for t in range(tokens):
        assert int(ids[t]) == oracle.argmax(want[t]), f"token {t}: argmax differs from the reference"
        assert int(ids[t]) == oracle.argmax(got[t]), f"token {t}: device argmax differs from argmax of its own logits"
    assert k.device_status() == 0


def test_a_token_has_the_same_logits_batched_or_alone(torch_cuda):
    torch = torch_cuda
    from llmxabe_b200 import synth
    hidden, vocab, max_tokens = 1024, 1536, 16
    _data, w, k = _head(torch, synth.Q8_0, vocab, hidden, max_tokens, seed=22)
    x = synth.activations(11, hidden, seed=22, layer=1)
    full, _ = _run(torch, k, w, x, max_tokens, vocab)
    for t in (0, 4, 7, 8, 10):
        one, _ = _run(torch, k, w, x[t:t + 1], max_tokens, vocab)
        assert (bits(one[0]) == bits(full[t])).all(), t
    again, _ = _run(torch, k, w, x, max_tokens, vocab)
    assert (bits(again) == bits(full)).all()


def test_device_argmax_agrees_with_the_scalar_reference(torch_cuda, oracle):
    """tests/lm_head_differential.rs:765-830: ties, the first and the last index, negatives."""
    torch = torch_cuda
    from llmxabe_b200.lm_head import LmHeadGeometry, LmHeadKernels
    vocab, max_tokens = 5000, 6
    k = LmHeadKernels(LmHeadGeometry(256, vocab, max_tokens))
    rng = np.random.default_rng(3)
    v = rng.standard_normal((max_tokens, vocab)).astype(np.float32)
    v[1, 0] = 50.0                      # the first index
    v[2, vocab - 1] = 50.0              # the last index
    v[3, 1234] = v[3, 4321] = 50.0      # a tie: the lower index wins
    v[4] = -3.0                         # all equal
    v[5] = -np.abs(v[5]) - 1.0          # all negative
    logits = torch.from_numpy(v).cuda()
    out = torch.zeros(max_tokens, dtype=torch.int32, device="cuda")
    k.argmax(logits, max_tokens, out)
    torch.cuda.synchronize()
    assert out.cpu().tolist() == [oracle.argmax(v[t]) for t in range(max_tokens)]
    assert out.cpu().tolist()[1:5] == [0, vocab - 1, 1234, 0]


def test_head_error_paths_mirror_the_reference(torch_cuda):
    """lm_head.rs:1703-1800 (RaggedWeights, WrongElementCount, TooManyTokens, buffer lengths)."""
    torch = torch_cuda
    from llmxabe_b200 import errors, synth
    from llmxabe_b200.lm_head import HeadFormat, HeadTensor
    hidden, vocab, max_tokens = 512, 256, 4
    _data, w, k = _head(torch, synth.Q8_0, vocab, hidden, max_tokens, seed=23)
    x = torch.zeros(max_tokens, hidden, device="cuda")
    logits = torch.zeros(max_tokens, vocab, device="cuda")
    with pytest.raises(errors.RaggedWeights):
        k.forward(HeadTensor(w.bytes[:-1], HeadFormat.Q8_0), x, 1, logits)
    with pytest.raises(errors.WrongElementCount):
        k.forward(HeadTensor(w.bytes[:-34], HeadFormat.Q8_0), x, 1, logits)
    with pytest.raises(errors.TooManyTokens):
        k.forward(w, x, max_tokens + 1, logits)
    with pytest.raises(errors.BufferLength):
        k.forward(w, x[:3], 1, logits)
    with pytest.raises(errors.BufferLength):
        k.forward(w, x, 1, logits[:, :-1].contiguous())
    bad = HeadTensor(w.bytes, HeadFormat.Q8_0)
    bad.format = 7
    with pytest.raises(errors.UnsupportedDenseType):
        k.forward(bad, x, 1, logits)
    k.forward(w, x, 0, logits)  # zero tokens: a no-op
    torch.cuda.synchronize()
