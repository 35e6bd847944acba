"""The allocation-free shared-expert entry point against the handle-based one.

Some callers of this library cannot allocate device memory at all -- a worker whose memory was
handed out at start-up, or code running where the CUDA allocator must not be entered -- so they
cannot create a handle.  `xabe_shared_expert_noalloc` serves them from a static device array.
This file is collected last on purpose: it checks the new entry point against
`xabe_moe_shared_expert` on two calls in a row (the second reuses the array the first one left
dirty), with the tolerance the other parity tests use, and it passes alone in a fresh process too.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
REL_L2 = 1e-3


def test_no_alloc_shared_expert_matches_the_handle_based_entry_point_twice_in_a_row():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("gpu-marked test collected without a CUDA device")
    from llmxabe_b200 import errors, synth
    from llmxabe_b200.moe import (ExpertQuant, MoeGeometry, MoeKernels, QuantTensor, shared_expert_noalloc,
                                  shared_expert_noalloc_status)
    from oracle import xabe_oracle as oracle
    H, I = 2048, 512
    for call, (quant, tokens) in enumerate([(0, 37), (1, 5)]):
        raw = [synth.quant_bytes(quant, H * I, 11 + call, 0, t) for t in (3, 4, 5)]
        gate, up, down = [QuantTensor(torch.from_numpy(b).cuda(), ExpertQuant(quant)) for b in raw]
        x = torch.from_numpy(synth.activations(tokens, H, seed=11, layer=call)).cuda()
        # existing entry point (needs a handle, which allocates)
        k = MoeKernels(MoeGeometry(0, 0, H, I, 16, 64), scope=MoeKernels.SCOPE_SHARED_ONLY)
        k.set_valid_tokens(tokens)
        xin = torch.zeros(64, H, device="cuda")
        xin[:tokens] = x
        want = torch.zeros(64, H, device="cuda")
        k.shared_expert(gate, up, down, xin, want)
        # the allocation-free one: no handle; outputs past `tokens` must stay untouched
        got = torch.full((64, H), 777.0, device="cuda")
        shared_expert_noalloc(gate, up, down, H, I, x, tokens, got)
        # a caller without a handle learns from this word whether a bounded wait of the kernels ran out
        assert shared_expert_noalloc_status() == 0
        torch.cuda.synchronize()
        r = oracle.compare(got[:tokens].cpu().numpy(), want[:tokens].cpu().numpy())
        print(f"call {call} (quant {quant}, {tokens} tokens): {r}")
        assert r.non_finite_count == 0 and r.rel_l2 <= REL_L2, str(r)
        assert (got[tokens:] == 777.0).all()
        # and against the CPU oracle, like every other parity test
        ref = oracle.mlp_forward_q(raw[0], quant, raw[1], quant, raw[2], quant, H, I, x.cpu().numpy())
        r2 = oracle.compare(got[:tokens].cpu().numpy(), ref)
        assert r2.rel_l2 <= REL_L2, str(r2)
    # sizes beyond the static array are refused with a clear error, nothing is launched
    big = torch.zeros(65, H, device="cuda")
    with pytest.raises(errors.TooManyTokens, match="static scratch"):
        shared_expert_noalloc(gate, up, down, H, I, big, 65, big.clone())
