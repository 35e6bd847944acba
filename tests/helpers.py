"""Shared test plumbing: one synthetic layer as oracle weights and as device weights."""
import numpy as np


def oracle_layer(oracle, L):
    return oracle.Layer(num_experts=L.num_experts, top_k=L.top_k, hidden=L.hidden, inter=L.inter,
                        post_norm=L.post_norm, router=L.router, router_bias=L.router_bias,
                        gate_exps=L.gate_exps, gate_quant=L.routed_quant, up_exps=L.up_exps,
                        up_quant=L.routed_quant, down_exps=L.down_exps, down_quant=L.down_quant,
                        shared_gate_inp=L.shared_gate_inp, shared_gate=L.shared_gate,
                        shared_gate_quant=L.shared_quant, shared_up=L.shared_up,
                        shared_up_quant=L.shared_quant, shared_down=L.shared_down,
                        shared_down_quant=L.shared_quant, eps=L.eps)


def device_layer(L, layer=0):
    import torch
    from llmxabe_b200.moe import MoeLayerWeights
    t = torch.from_numpy
    return MoeLayerWeights(layer=layer, post_norm=t(L.post_norm), router=t(L.router),
                           router_bias=None if L.router_bias is None else t(L.router_bias),
                           gate_exps=t(L.gate_exps), gate_quant=L.routed_quant, up_exps=t(L.up_exps),
                           up_quant=L.routed_quant, down_exps=t(L.down_exps), down_quant=L.down_quant,
                           shared_gate_inp=t(L.shared_gate_inp), shared_gate=t(L.shared_gate),
                           shared_gate_quant=L.shared_quant, shared_up=t(L.shared_up),
                           shared_up_quant=L.shared_quant, shared_down=t(L.shared_down),
                           shared_down_quant=L.shared_quant)


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def run_block(block, w, x_np, max_tokens):
    """Runs MoeBlock.forward on `x_np` rows; returns numpy waypoints of the live rows."""
    import torch
    T, H = x_np.shape
    res = torch.zeros(max_tokens, H, device="cuda")
    res[:T] = torch.from_numpy(x_np).cuda()
    canary = 12345.0
    ffn = torch.full((max_tokens, H), canary, device="cuda")
    lo = torch.full((max_tokens, H), canary, device="cuda")
    block.forward(w, res, T, ffn, lo)
    torch.cuda.synchronize()
    b = block.buffers()
    out = dict(normed=b.normed[:T], logits=b.logits[:T], topk_ids=b.topk_ids[:T],
               topk_weights=b.topk_weights[:T], routed=b.routed[:T], shexp=b.shexp[:T], gate=b.gate[:T],
               ffn_out=ffn[:T], l_out=lo[:T], sorted_token_ids=b.sorted_token_ids,
               expert_ids=b.expert_ids, num_tokens_post_pad=b.num_tokens_post_pad)
    out = {k: v.detach().cpu().numpy().copy() for k, v in out.items()}
    out["untouched"] = bool((ffn[T:] == canary).all().item() and (lo[T:] == canary).all().item())
    return out
