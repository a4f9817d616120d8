"""Seeded synthetic weights of the 27B shape in the reference's checkpoint naming.

The reference loads `amd/Qwen3.8-27B-Quark-AWQ-MXFP4` into a `Weights` object
(`qwen3.8-27b-gfx942/mk/reference.py:86-155`): `.t` maps names to bf16 tensors (MXFP4 matrices dequantised
exactly), `.q` maps a linear layer's base name to its raw `(packed e2m1 [N, K/2], e8m0 [N, K/32])` pair,
`.L(i, name)` and `W[name]` look tensors up.  No checkpoint can be downloaded where this library is tested,
so `SynthWeights` builds an object with the same attributes from a seed: every tensor is N(0, 0.02) drawn on
the CPU from one generator in the fixed order below, cast to bf16; the twelve linear layers of every decoder
layer are then quantised to MXFP4 (`stage/quant.py`) and `.t` holds their exact dequantisation, so the
reference decoder and the kernel see the same numbers.  Embedding and LM head stay bf16 (untied).

`init="realistic"` gives the DeltaNet output norm a gain near 1, conv taps near 0.5 and a spread of decay
rates so that the recurrent branch carries signal (with everything at N(0, 0.02) it is numerically tiny).
"""

import torch

from ..stage import quant
from .dims import CONV_K, DK, DV, HD, FULL

P = "model.language_model."
LIN = ("in_proj_qkv", "in_proj_z", "in_proj_b", "in_proj_a", "out_proj", "q_proj", "k_proj", "v_proj", "o_proj",
       "gate_proj", "up_proj", "down_proj")


class SynthWeights:
    def __init__(self, shape=FULL, layers=None, seed=0, std=0.02, init="baseline", device="cpu", fmt="mxfp4",
                 draw_device="cpu", keep_dequant=True):
        """`draw_device="cuda"` draws on the GPU (values then depend on the GPU's generator: for benchmarks at
        full depth, where 27 G normals on the CPU would take minutes); `keep_dequant=False` drops the
        dequantised copies of the MXFP4 matrices, which only the reference decoder needs."""
        assert fmt in ("mxfp4", "bf16") and init in ("baseline", "realistic")
        s = shape
        self.shape, self.fmt, self.device = s, fmt, device
        self.layers = layers if layers is not None else s.layers
        self.t, self.q = {}, {}
        gen = torch.Generator(device=draw_device)
        gen.manual_seed(seed)

        def draw(*shp, mean=0.0, sd=std, dtype=torch.bfloat16):
            t = torch.empty(*shp, dtype=torch.float32, device=draw_device)
            t.normal_(mean, sd, generator=gen)
            return t.to(dtype)

        def linear(name, n, k):
            w = draw(n, k)
            if fmt == "mxfp4":
                pk, sc = quant.quantize_mxfp4(w.to(device))
                self.q[name] = (pk, sc)
                if not keep_dequant:
                    return
                w = quant.dequantize_mxfp4(pk, sc)
            self.t[name + ".weight"] = w.to(device)

        H = s.hidden
        self.t[P + "embed_tokens.weight"] = draw(s.vocab, H).to(device)
        for i in range(self.layers):
            L = f"{P}layers.{i}."
            self.t[L + "input_layernorm.weight"] = draw(H).to(device)
            self.t[L + "post_attention_layernorm.weight"] = draw(H).to(device)
            if s.is_attn(i):
                a = L + "self_attn."
                linear(a + "q_proj", 2 * s.nq * HD, H)
                linear(a + "k_proj", s.nkv * HD, H)
                linear(a + "v_proj", s.nkv * HD, H)
                self.t[a + "q_norm.weight"] = draw(HD).to(device)
                self.t[a + "k_norm.weight"] = draw(HD).to(device)
                linear(a + "o_proj", H, s.nq * HD)
            else:
                g = L + "linear_attn."
                linear(g + "in_proj_qkv", s.conv_dim, H)
                linear(g + "in_proj_z", s.val_dim, H)
                linear(g + "in_proj_b", s.nvh, H)
                linear(g + "in_proj_a", s.nvh, H)
                if init == "baseline":
                    self.t[g + "conv1d.weight"] = draw(s.conv_dim, 1, CONV_K).to(device)
                    self.t[g + "A_log"] = draw(s.nvh, dtype=torch.float32).to(device)
                    self.t[g + "dt_bias"] = draw(s.nvh).to(device)
                    self.t[g + "norm.weight"] = draw(DV).to(device)
                else:
                    self.t[g + "conv1d.weight"] = draw(s.conv_dim, 1, CONV_K, mean=0.5, sd=0.2).to(device)
                    self.t[g + "A_log"] = draw(s.nvh, mean=-1.0, sd=1.0, dtype=torch.float32).to(device)
                    self.t[g + "dt_bias"] = draw(s.nvh, sd=1.0).to(device)
                    self.t[g + "norm.weight"] = draw(DV, mean=1.0, sd=0.1).to(device)
                linear(g + "out_proj", H, s.val_dim)
            m = L + "mlp."
            linear(m + "gate_proj", s.ffn, H)
            linear(m + "up_proj", s.ffn, H)
            linear(m + "down_proj", H, s.ffn)
        self.t[P + "norm.weight"] = draw(H).to(device)
        self.t["lm_head.weight"] = draw(s.vocab, H).to(device)

    def __getitem__(self, k):
        return self.t[k]

    def L(self, i, name):
        return self.t[f"{P}layers.{i}.{name}"]

    def raw(self, i, name):
        """(packed, scales) of linear layer `name` ('linear_attn.out_proj', ...) of layer i."""
        return self.q[f"{P}layers.{i}.{name}"]


def make_prompt(vocab, n, seed=0):
    gen = torch.Generator(device="cpu")
    gen.manual_seed(1000 + seed)
    return torch.randint(0, vocab, (n,), generator=gen).tolist()
