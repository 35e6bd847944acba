"""sm_100a kernel set for the per-layer MoE FFN block of nixabe/llmxabe,
behind the reference's own MoeKernels / MoeBlock interface.

Importing the package does not load CUDA; the first computation does, and
raises if libxabe_moe_sm100.so is missing (there is no CPU path).
"""
__all__ = ["moe", "synth", "build"]
