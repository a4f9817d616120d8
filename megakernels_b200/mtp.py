"""Host-side (PyTorch) multi-token-prediction head: fills the draft head's KV cache for prompt tokens.

During speculative cycles the kernel maintains the draft head's cache itself.  For tokens fed
outside such cycles (the prompt, plain `run` launches) the cache entry of position i needs the final
hidden state h_i and the token x_{i+1} that followed, which is only known one step later; this class
computes those entries in one batch, exactly as the reference does with its own `MTP` class
(`qwen3.5-0.8b/qwen_mk/mtp.py:39-82`, used from `qwen_mk/engine.py:178-196`):

    u_i = fc([rmsnorm(embed(x_{i+1})), rmsnorm(h_i)])
    k_i, v_i = k/v projection of rmsnorm(u_i), with per-head norm and partial RoPE at position i

It is not on the decode hot path; the math runs in fp32 on the device through plain torch ops.
"""

import torch


def rmsnorm(x, w, eps):
    """Weights are offsets from 1 (`qwen_mk/reference.py:12-15`)."""
    x = x.float()
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * (1.0 + w.float())


def apply_rope(x, cos, sin, rotary_dim):
    half = rotary_dim // 2
    x1, x2, rest = x[..., :half], x[..., half:rotary_dim], x[..., rotary_dim:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin, rest], dim=-1)


class MTP:
    def __init__(self, cfg, weights, embed_rows, cos, sin, write_kv):
        """`weights`: name -> fp32 tensor as the kernel sees it (dequantised for int8);
        `embed_rows(tokens)` -> fp32 embedding rows; `write_kv(positions, k, v)` stores [n, kv_heads, D]."""
        self.cfg, self.w = cfg, weights
        self.embed_rows, self.cos, self.sin, self.write_kv = embed_rows, cos, sin, write_kv

    def layer_input(self, h, next_tokens):
        c, w = self.cfg, self.w
        e = rmsnorm(self.embed_rows(next_tokens), w["pre_fc_norm_embedding.weight"], c.eps)
        g = rmsnorm(h, w["pre_fc_norm_hidden.weight"], c.eps)
        return torch.cat([e, g], dim=-1) @ w["fc.weight"].t()

    @torch.no_grad()
    def fill_kv(self, h, next_tokens, start):
        """Cache entries for positions start .. start + n - 1 from final hidden states `h` [n, hidden]
        (after the final norm) and the tokens that followed them."""
        c, w, p = self.cfg, self.w, "layers.0.self_attn."
        n = h.shape[0]
        pos = torch.arange(start, start + n, device=h.device)
        x = rmsnorm(self.layer_input(h, next_tokens), w["layers.0.input_layernorm.weight"], c.eps)
        k = (x @ w[p + "k_proj.weight"].t()).view(n, c.n_kv_heads, c.head_dim)
        v = (x @ w[p + "v_proj.weight"].t()).view(n, c.n_kv_heads, c.head_dim)
        k = rmsnorm(k, w[p + "k_norm.weight"], c.eps)
        k = apply_rope(k, self.cos[pos][:, None], self.sin[pos][:, None], c.rotary_dim)
        self.write_kv(pos, k, v)
