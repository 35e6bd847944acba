"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations (they stand in for the real GGUF model file, which
is not available offline).

Every tensor is generated from a counter-based stream keyed by
(seed, layer, tensor id), so any process or rank can materialise exactly the
bytes it needs and the CPU oracle sees the same bytes as the GPU.

Distributions:
  Q6_K superblock (210 B): ql 128 B uniform u8, qh 64 B uniform u8, 16 int8
      scales uniform in [-32, 31], d = fp16(|N(0,1)| * 2e-4)
  Q8_0 block (34 B): d = fp16(|N(0,1)| * 2e-4 * Q8_0_SCALE_MATCH), qs uniform int8
      (the factor makes Q8_0 weights as large as the Q6_K ones: rms(sc*q)
      of Q6_K is 18.5^2 = 341, rms(q) of Q8_0 is 74)
  router fp32 ~ N(0, 0.02); post-norm weight = 1; shared-gate vector ~ N(0, 0.02)
  activations ~ N(0, 1)
  Zipf routing skew: bias_e = ZIPF_C * (-1.1 * ln(rank_e)) over a seeded
      permutation of the experts, added to the router logits
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

Q6K, Q8_0 = 0, 1
Q8_0_SCALE_MATCH = 4.6
ZIPF_S = 1.1
ZIPF_C = 0.25  # at 2048 tokens: every expert active, the hottest takes > 500 tokens
DEFAULT_EPS = 1e-6

_T_GATE, _T_UP, _T_DOWN, _T_SGATE, _T_SUP, _T_SDOWN, _T_ROUTER, _T_SGINP, _T_X, _T_PERM = range(10)


def _gen(seed: int, layer: int, tensor: int) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=[seed & (2**64 - 1), (layer << 8) | tensor]))


def q6k_bytes(n_elements: int, seed: int, layer: int, tensor: int) -> np.ndarray:
    assert n_elements % 256 == 0
    nsb = n_elements // 256
    g = _gen(seed, layer, tensor)
    out = np.empty((nsb, 210), dtype=np.uint8)
    out[:, :192] = g.integers(0, 256, size=(nsb, 192), dtype=np.uint8)
    out[:, 192:208] = g.integers(-32, 32, size=(nsb, 16), dtype=np.int8).view(np.uint8)
    d = (np.abs(g.standard_normal(nsb, dtype=np.float32)) * np.float32(2e-4)).astype(np.float16)
    out[:, 208:210] = d.view(np.uint8).reshape(nsb, 2)
    return out.reshape(-1)


def q8_0_bytes(n_elements: int, seed: int, layer: int, tensor: int) -> np.ndarray:
    assert n_elements % 32 == 0
    nb = n_elements // 32
    g = _gen(seed, layer, tensor)
    out = np.empty((nb, 34), dtype=np.uint8)
    d = (np.abs(g.standard_normal(nb, dtype=np.float32)) * np.float32(2e-4 * Q8_0_SCALE_MATCH)).astype(np.float16)
    out[:, 0:2] = d.view(np.uint8).reshape(nb, 2)
    out[:, 2:34] = g.integers(-128, 128, size=(nb, 32), dtype=np.int8).view(np.uint8)
    return out.reshape(-1)


def quant_bytes(quant: int, n_elements: int, seed: int, layer: int, tensor: int) -> np.ndarray:
    return (q6k_bytes if quant == Q6K else q8_0_bytes)(n_elements, seed, layer, tensor)


@dataclass
class SynthLayer:
    num_experts: int
    top_k: int
    hidden: int
    inter: int
    post_norm: np.ndarray
    router: np.ndarray
    router_bias: np.ndarray | None
    gate_exps: np.ndarray
    up_exps: np.ndarray
    down_exps: np.ndarray
    routed_quant: int
    down_quant: int
    shared_gate_inp: np.ndarray
    shared_gate: np.ndarray
    shared_up: np.ndarray
    shared_down: np.ndarray
    shared_quant: int
    eps: float = DEFAULT_EPS


def zipf_bias(num_experts: int, seed: int, layer: int, c: float = ZIPF_C, s: float = ZIPF_S) -> np.ndarray:
    perm = _gen(seed, layer, _T_PERM).permutation(num_experts)
    rank = np.empty(num_experts, dtype=np.float64)
    rank[perm] = np.arange(1, num_experts + 1)
    return (c * (-s * np.log(rank))).astype(np.float32)


def moe_layer(*, seed: int = 0, layer: int = 0, num_experts: int = 256, top_k: int = 8, hidden: int = 2048,
              inter: int = 512, routed_quant: int = Q6K, down_quant: int | None = None,
              shared_quant: int = Q6K, zipf: bool = False) -> SynthLayer:
    """One MoE layer of the benchmark family (defaults: the 256/8/2048/512 geometry, all Q6_K)."""
    down_quant = routed_quant if down_quant is None else down_quant
    n = num_experts * inter * hidden
    g = _gen(seed, layer, _T_ROUTER)
    router = (g.standard_normal((num_experts, hidden), dtype=np.float32) * np.float32(0.02))
    sg = _gen(seed, layer, _T_SGINP).standard_normal(hidden, dtype=np.float32) * np.float32(0.02)
    return SynthLayer(
        num_experts=num_experts, top_k=top_k, hidden=hidden, inter=inter,
        post_norm=np.ones(hidden, dtype=np.float32), router=router,
        router_bias=zipf_bias(num_experts, seed, layer) if zipf else None,
        gate_exps=quant_bytes(routed_quant, n, seed, layer, _T_GATE),
        up_exps=quant_bytes(routed_quant, n, seed, layer, _T_UP),
        down_exps=quant_bytes(down_quant, n, seed, layer, _T_DOWN),
        routed_quant=routed_quant, down_quant=down_quant,
        shared_gate_inp=sg,
        shared_gate=quant_bytes(shared_quant, inter * hidden, seed, layer, _T_SGATE),
        shared_up=quant_bytes(shared_quant, inter * hidden, seed, layer, _T_SUP),
        shared_down=quant_bytes(shared_quant, inter * hidden, seed, layer, _T_SDOWN),
        shared_quant=shared_quant)


def activations(tokens: int, hidden: int, *, seed: int = 0, layer: int = 0, bf16: bool = False) -> np.ndarray:
    """[tokens][hidden] ~ N(0,1) float32 (optionally rounded through bf16, as the prefill config feeds them)."""
    x = _gen(seed, layer, _T_X).standard_normal((tokens, hidden), dtype=np.float32)
    if bf16:
        u = x.view(np.uint32)
        u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16  # round to nearest even on the top 16 bits
        x = u.astype(np.uint32).view(np.float32)
    return x


def dense_layer(*, seed: int = 0, layer: int = 0, hidden: int = 5120, inter: int = 17408, quant: int = Q6K):
    """Dense SwiGLU MLP of the 27B sibling: (post_norm, gate, up, down)."""
    n = hidden * inter
    return (np.ones(hidden, dtype=np.float32), quant_bytes(quant, n, seed, layer, _T_SGATE),
            quant_bytes(quant, n, seed, layer, _T_SUP), quant_bytes(quant, n, seed, layer, _T_SDOWN))


# ---------------------------------------------------------------------------
# The same distributions generated ON the device (torch), for benchmark layers
# that are only ever checked through size-independent properties: a 667 MB
# layer takes milliseconds instead of ten seconds of host time.  Not
# bit-identical to the numpy generator above.
# ---------------------------------------------------------------------------
def _device_quant_bytes(torch, quant: int, n_elements: int, gen, device):
    if quant == Q6K:
        nsb = n_elements // 256
        out = torch.empty((nsb, 210), dtype=torch.uint8, device=device)
        out[:, :192] = torch.randint(0, 256, (nsb, 192), dtype=torch.uint8, device=device, generator=gen)
        out[:, 192:208] = torch.randint(-32, 32, (nsb, 16), dtype=torch.int8, device=device,
                                        generator=gen).view(torch.uint8)
        d = (torch.randn(nsb, device=device, generator=gen).abs() * 2e-4).to(torch.float16)
        out[:, 208:210] = d.view(torch.uint8).view(nsb, 2)
        return out.view(-1)
    nb = n_elements // 32
    out = torch.empty((nb, 34), dtype=torch.uint8, device=device)
    d = (torch.randn(nb, device=device, generator=gen).abs() * (2e-4 * Q8_0_SCALE_MATCH)).to(torch.float16)
    out[:, 0:2] = d.view(torch.uint8).view(nb, 2)
    out[:, 2:34] = torch.randint(-128, 128, (nb, 32), dtype=torch.int8, device=device,
                                 generator=gen).view(torch.uint8)
    return out.view(-1)


def moe_layer_on_device(*, seed: int = 0, layer: int = 0, num_experts: int = 256, top_k: int = 8,
                        hidden: int = 2048, inter: int = 512, routed_quant: int = Q6K,
                        down_quant: int | None = None, shared_quant: int = Q6K, zipf: bool = False,
                        device="cuda"):
    """A `MoeLayerWeights` whose tensors are generated on `device` (see the note above)."""
    import torch
    from .moe import MoeLayerWeights
    down_quant = routed_quant if down_quant is None else down_quant
    gen = torch.Generator(device=device)
    gen.manual_seed((seed * 1000003 + layer) & 0x7FFFFFFF)
    n = num_experts * inter * hidden
    q = lambda quant, count: _device_quant_bytes(torch, quant, count, gen, device)
    bias = torch.from_numpy(zipf_bias(num_experts, seed, layer)) if zipf else None
    return MoeLayerWeights(
        layer=layer, post_norm=torch.ones(hidden, device=device),
        router=torch.randn(num_experts, hidden, device=device, generator=gen) * 0.02, router_bias=bias,
        gate_exps=q(routed_quant, n), gate_quant=routed_quant, up_exps=q(routed_quant, n),
        up_quant=routed_quant, down_exps=q(down_quant, n), down_quant=down_quant,
        shared_gate_inp=torch.randn(hidden, device=device, generator=gen) * 0.02,
        shared_gate=q(shared_quant, inter * hidden), shared_gate_quant=shared_quant,
        shared_up=q(shared_quant, inter * hidden), shared_up_quant=shared_quant,
        shared_down=q(shared_quant, inter * hidden), shared_down_quant=shared_quant, device=device)
