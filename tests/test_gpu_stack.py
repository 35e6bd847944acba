"""GPU tests of the MoE stack driver (the MoE half of the reference's Forward::body,
crates/xabe-engine/src/forward.rs:3497-3618) through xabe_moe_stack_forward.

Gates:
  each layer's l_out     rel-L2 <= 1e-3 against the oracle block run on the hidden state that
                         layer actually received (the reference's waypoint comparison), expert ids exact
  one-call pass, graph replay   bit-identical to the layer-by-layer eager pass
  replay at a smaller published count   live rows bit-identical to the same rows of the full
                         batch, rows past the count untouched
"""
import copy

import pytest

from helpers import bits, device_layer, oracle_layer

pytestmark = pytest.mark.gpu
REL_L2 = 1e-3
N_LAYERS = 4
MAX_TOKENS = 16  # wide enough for the handle to pick k_gateup_rows


@pytest.fixture(scope="module")
def torch_cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("gpu-marked test collected without a CUDA device")
    return torch


@pytest.fixture(scope="module")
def small_stack(torch_cuda):
    from llmxabe_b200 import synth
    from llmxabe_b200.moe import MoeGeometry
    from llmxabe_b200.stack import MoeStack
    host = [synth.moe_layer(seed=11, layer=i, num_experts=8, top_k=2, hidden=512, inter=256,
                            shared_quant=synth.Q8_0 if i == 2 else synth.Q6K, zipf=True) for i in range(N_LAYERS)]
    dev = [device_layer(L, layer=i) for i, L in enumerate(host)]
    g = MoeGeometry(8, 2, 512, 256, 32, MAX_TOKENS)
    return host, dev, g, MoeStack(g, dev)


def test_each_layer_matches_the_oracle_on_the_hidden_state_it_received(torch_cuda, oracle, small_stack):
    torch = torch_cuda
    from llmxabe_b200 import synth
    host, _dev, _g, stack = small_stack
    tokens = 11
    x = synth.activations(tokens, 512, seed=11, layer=99)
    seen = []

    def waypoint(layer, hidden):
        torch.cuda.synchronize()
        ids = stack.block.buffers().topk_ids[:tokens].cpu().numpy().copy()
        seen.append((layer, hidden[:tokens].cpu().numpy().copy(), ids))

    out = stack.run(torch.from_numpy(x).cuda(), on_waypoint=waypoint)
    torch.cuda.synchronize()
    assert [s[0] for s in seen] == list(range(N_LAYERS))
    assert (bits(out.cpu().numpy()) == bits(seen[-1][1])).all()
    fed = x
    for layer, got, ids in seen:
        want = oracle.moe_block_forward(oracle_layer(oracle, host[layer]), fed, dev_order=True)
        assert (ids == want["topk_ids"]).all(), f"layer {layer}: expert ids differ"
        r = oracle.compare(got, want["l_out"])
        print(f"stack layer {layer} l_out: {r}")
        assert r.non_finite_count == 0 and r.rel_l2 <= REL_L2, f"layer {layer}: {r}"
        fed = got
    assert stack.block.moe.device_status() == 0


def test_one_call_pass_and_graph_replay_equal_the_eager_pass(torch_cuda, small_stack):
    torch = torch_cuda
    from llmxabe_b200 import synth
    _host, _dev, _g, stack = small_stack
    x = torch.from_numpy(synth.activations(MAX_TOKENS, 512, seed=11, layer=98)).cuda()
    eager = stack.run(x, on_waypoint=lambda layer, hidden: None).clone()
    one_call = stack.run(x).clone()
    assert (bits(one_call.cpu().numpy()) == bits(eager.cpu().numpy())).all()
    stack.capture()
    replayed = stack.run(x).clone()
    torch.cuda.synchronize()
    assert (bits(replayed.cpu().numpy()) == bits(eager.cpu().numpy())).all()
    # the same graph at a smaller published count: the live rows are those of the full batch
    # (a row does not depend on its batch), the rows past the count are never written
    canary = 4321.0
    for buf in stack._hidden:
        buf.fill_(canary)
    stack.ffn_out.fill_(canary)
    few = stack.run(x[:3]).clone()
    torch.cuda.synchronize()
    assert (bits(few.cpu().numpy()) == bits(eager[:3].cpu().numpy())).all()
    for buf in stack._hidden:
        assert bool((buf[3:] == canary).all().item())
    assert bool((stack.ffn_out[3:] == canary).all().item())
    assert stack.block.moe.device_status() == 0


def test_every_layer_is_checked_before_the_first_launch(torch_cuda, small_stack):
    torch = torch_cuda
    from llmxabe_b200 import _lib, errors
    from llmxabe_b200.moe import ExpertQuant, QuantTensor
    from llmxabe_b200.stack import MoeStack
    _host, dev, g, _stack = small_stack
    bad = copy.copy(dev[2])
    bad.down_exps = QuantTensor(dev[2].down_exps.bytes[:-210], ExpertQuant.Q6K)
    stack = MoeStack(g, [dev[0], dev[1], bad, dev[3]])
    canary = 777.0
    stack.hidden_out.fill_(canary)
    stack._hidden[1].fill_(canary)
    stack.publish_tokens(4)
    with pytest.raises(errors.WrongElementCount):
        stack.body()
    torch.cuda.synchronize()
    assert bool((stack._hidden[1] == canary).all().item()), "a layer ran before the bad one was found"
    with pytest.raises(errors.TooManyTokens):
        stack.publish_tokens(MAX_TOKENS + 1)
    # the two hidden-state buffers must be distinct
    h = stack._hidden[0]
    rc = _lib.lib().xabe_moe_stack_forward(stack.block.moe._h, torch.cuda.current_stream().cuda_stream,
                                           stack._weights_c, 2, h.data_ptr(), h.data_ptr(), h.numel(), 4,
                                           stack.ffn_out.data_ptr(), stack.ffn_out.numel(), None)
    assert rc != 0 and b"distinct" in _lib.lib().xabe_moe_last_error()
