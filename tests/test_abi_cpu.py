"""CPU checks of the boundary: the library loads, exports every symbol the
header declares, validates geometry before touching a device, and fails
loudly (no fallback) when there is no GPU."""
import ctypes as C
import os
import re

import pytest

from conftest import ROOT


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "xabe_moe.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(xabe_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from llmxabe_b200 import _lib, build
    build.build()
    L = C.CDLL(_lib.library_path())
    names = _declared_functions()
    assert len(names) >= 18
    for n in names:
        assert hasattr(L, n), f"{n} is declared in include/xabe_moe.h but not exported"
    assert set(names) == set(_lib.SYMBOLS), "the ctypes table and the header disagree"


def test_capacity_formulas_through_the_abi(kats):
    from llmxabe_b200.moe import MoeGeometry
    for c in kats["capacity"]:
        g = MoeGeometry(c["num_experts"], c["top_k"], 2048, 512, c["block_size"], c["max_tokens"])
        assert g.sorted_capacity() == c["sorted_capacity"]
        assert g.expert_block_capacity() == c["expert_block_capacity"]
        if "max_flat_pairs" in c:
            assert g.max_flat_pairs() == c["max_flat_pairs"]


@pytest.mark.parametrize("kw,reason", [
    (dict(block_size=0), "block_size must be non-zero"),
    (dict(experts_per_token=0), "experts_per_token must be non-zero"),
    (dict(experts_per_token=9, num_experts=8), "must not exceed num_experts"),
    (dict(max_tokens=0), "max_tokens must be non-zero"),
    (dict(hidden=0), "must be non-zero"),
    (dict(hidden=2048 + 128), "hidden must be a multiple"),
    (dict(intermediate=384), "intermediate must be a multiple"),
    (dict(block_size=128), "block_size exceeds"),
    (dict(max_tokens=2_000_000), "max_tokens exceeds"),
])
def test_geometry_is_validated_before_any_device_call(kw, reason):
    """MoeKernels::new rejects these (crates/xabe-cuda/src/kernels/moe.rs:5043-5111)."""
    from llmxabe_b200.errors import UnsupportedGeometry
    from llmxabe_b200.moe import MoeGeometry, MoeKernels
    base = dict(num_experts=256, experts_per_token=8, hidden=2048, intermediate=512, block_size=16,
                max_tokens=64)
    base.update(kw)
    with pytest.raises(UnsupportedGeometry, match=reason):
        MoeKernels(MoeGeometry(**base), device=0)


def test_no_gpu_means_a_loud_driver_error_not_a_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from llmxabe_b200.errors import Driver
    from llmxabe_b200.moe import MoeGeometry, MoeKernels
    with pytest.raises(Driver):
        MoeKernels(MoeGeometry.qwen3_6(16, 64), device=0)


def test_product_package_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "llmxabe_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert "xabe_oracle" not in src and "from oracle" not in src and "import oracle" not in src, f


def test_synthetic_generator_is_deterministic_and_well_formed(oracle):
    import numpy as np
    from llmxabe_b200 import synth
    a = synth.moe_layer(num_experts=8, top_k=2, hidden=512, inter=256, zipf=True)
    b = synth.moe_layer(num_experts=8, top_k=2, hidden=512, inter=256, zipf=True)
    assert (a.gate_exps == b.gate_exps).all() and (a.router == b.router).all()
    assert a.gate_exps.size == 8 * 256 * 512 // 256 * 210
    sb = a.gate_exps.reshape(-1, 210)
    sc = sb[:, 192:208].view(np.int8)
    assert sc.min() >= -32 and sc.max() <= 31
    d = sb[:, 208:210].copy().view(np.float16).astype(np.float32)
    assert (d >= 0).all() and d.mean() < 4e-4
    w = oracle.dequantize_row(oracle.Q6K, a.gate_exps[:210 * 64])
    assert np.isfinite(w).all() and np.abs(w).max() < 2.0
    q8 = synth.q8_0_bytes(32 * 100, 0, 0, 1)
    w8 = oracle.dequantize_row(oracle.Q8_0, q8)
    assert np.isfinite(w8).all()
    x = synth.activations(4, 512, bf16=True)
    assert ((x.view(np.uint32) & 0xFFFF) == 0).all()
