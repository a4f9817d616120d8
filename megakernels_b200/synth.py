"""Seeded random-init weights in the reference's checkpoint naming.

The reference loads a Hugging Face snapshot into a dict keyed by names such as
`layers.3.self_attn.q_proj.weight` (`qwen3.5-0.8b/qwen_mk/weights.py:69-90`) and the MTP head
into names without the `mtp.` prefix (`qwen_mk/mtp.py:26-36`).  No checkpoint is available
offline, so these factories produce the same dicts from a seed: every tensor is drawn on the
CPU, in the fixed order listed here, from one `torch.Generator`, as N(0, std) in fp32 and cast
to bf16.  The CPU generator makes the values independent of the machine they are drawn on.

`init="baseline"` draws everything from N(0, 0.02), norm offsets and conv taps included.
`init="realistic"` keeps N(0, 0.02) for the matrices but gives the DeltaNet output norm a gain
near 1, conv taps near 0.5 and a spread of decay rates, so that the recurrent branch carries
signal of the same order as the attention branch.
"""

import torch


def _draw(gen, shape, std, mean=0.0, dtype=torch.bfloat16):
    t = torch.empty(shape, dtype=torch.float32)
    t.normal_(mean, std, generator=gen)
    return t.to(dtype)


def _attn_layer(gen, cfg, p, std, out):
    H, D = cfg.hidden, cfg.head_dim
    out[p + "self_attn.q_proj.weight"] = _draw(gen, (2 * cfg.n_heads * D, H), std)
    out[p + "self_attn.k_proj.weight"] = _draw(gen, (cfg.n_kv_heads * D, H), std)
    out[p + "self_attn.v_proj.weight"] = _draw(gen, (cfg.n_kv_heads * D, H), std)
    out[p + "self_attn.q_norm.weight"] = _draw(gen, (D,), std)
    out[p + "self_attn.k_norm.weight"] = _draw(gen, (D,), std)
    out[p + "self_attn.o_proj.weight"] = _draw(gen, (H, cfg.n_heads * D), std)


def _mlp(gen, cfg, p, std, out):
    H, I = cfg.hidden, cfg.intermediate
    out[p + "mlp.gate_proj.weight"] = _draw(gen, (I, H), std)
    out[p + "mlp.up_proj.weight"] = _draw(gen, (I, H), std)
    out[p + "mlp.down_proj.weight"] = _draw(gen, (H, I), std)


def make_weights(cfg, seed=0, std=0.02, init="baseline"):
    """Main-model weights: dict name -> CPU tensor (bf16; `A_log` fp32 like the checkpoint)."""
    assert init in ("baseline", "realistic"), init
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    H = cfg.hidden
    w = {"embed_tokens.weight": _draw(gen, (cfg.vocab, H), std)}
    nh, dk, dv = cfg.lin_heads, cfg.lin_k_dim, cfg.lin_v_dim
    for i, kind in enumerate(cfg.layer_types):
        p = f"layers.{i}."
        w[p + "input_layernorm.weight"] = _draw(gen, (H,), std)
        w[p + "post_attention_layernorm.weight"] = _draw(gen, (H,), std)
        if kind == "linear_attention":
            q = p + "linear_attn."
            w[q + "in_proj_qkv.weight"] = _draw(gen, (cfg.conv_dim, H), std)
            w[q + "in_proj_z.weight"] = _draw(gen, (nh * dv, H), std)
            w[q + "in_proj_b.weight"] = _draw(gen, (nh, H), std)
            w[q + "in_proj_a.weight"] = _draw(gen, (nh, H), std)
            if init == "baseline":
                w[q + "conv1d.weight"] = _draw(gen, (cfg.conv_dim, 1, cfg.conv_k), std)
                w[q + "A_log"] = _draw(gen, (nh,), std).float()
                w[q + "dt_bias"] = _draw(gen, (nh,), std)
                w[q + "norm.weight"] = _draw(gen, (dv,), std)
            else:
                w[q + "conv1d.weight"] = _draw(gen, (cfg.conv_dim, 1, cfg.conv_k), 0.2, mean=0.5)
                w[q + "A_log"] = _draw(gen, (nh,), 1.0, mean=-1.0).float()
                w[q + "dt_bias"] = _draw(gen, (nh,), 1.0)
                w[q + "norm.weight"] = _draw(gen, (dv,), 0.1, mean=1.0)
            w[q + "out_proj.weight"] = _draw(gen, (H, nh * dv), std)
        else:
            _attn_layer(gen, cfg, p, std, w)
        _mlp(gen, cfg, p, std, w)
    w["norm.weight"] = _draw(gen, (H,), std)
    if not cfg.tied:
        w["lm_head.weight"] = _draw(gen, (cfg.vocab, H), std)
    return w


def make_mtp_weights(cfg, seed=1, std=0.02):
    """MTP head weights (one gated-attention decoder layer plus the 2H -> H fusion projection)."""
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    H = cfg.hidden
    w = {"fc.weight": _draw(gen, (H, 2 * H), std),
         "pre_fc_norm_embedding.weight": _draw(gen, (H,), std),
         "pre_fc_norm_hidden.weight": _draw(gen, (H,), std)}
    p = "layers.0."
    w[p + "input_layernorm.weight"] = _draw(gen, (H,), std)
    w[p + "post_attention_layernorm.weight"] = _draw(gen, (H,), std)
    _attn_layer(gen, cfg, p, std, w)
    _mlp(gen, cfg, p, std, w)
    w["norm.weight"] = _draw(gen, (H,), std)
    return w


def make_prompt(cfg, n, seed=0):
    """`n` uniform-random token ids in [0, vocab)."""
    gen = torch.Generator(device="cpu")
    gen.manual_seed(1000 + seed)
    return torch.randint(0, cfg.vocab, (n,), generator=gen).tolist()
