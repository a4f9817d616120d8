"""Seeded synthetic weights of the 35B-A3B model in the layout of the reference's `Weights`
(`qwen3.6-35b-a3b-gfx942/mk/reference.py:61-151`): `.t` holds dense matrices as fp32 (FP8 ones dequantised
exactly), `.raw[name] = (e4m3fn, block scales)`, `.ex[(layer, proj)]` / `.exs[...]` the routed experts stacked
as [experts, N, K] in the checkpoint's format, `.fp8` the names of FP8 matrices; `.L`, `.is_fp8`, `.expert`
as there.  Which matrices are FP8 follows the checkpoint the reference loads: every projection and expert
matrix; the router, the shared-expert gate, in_proj_a / in_proj_b, the embedding and the LM head stay bf16.

`router="uniform"` leaves the router rows N(0, std): on normalised inputs every expert is equally likely.
`router="zipf"` skews the load: the model has no router bias, so expert e's row is scaled by (e + 1)^-0.6 and its
logits spread accordingly; the top 8 then fall on the low-numbered experts with a frequency that decays like a
Zipf law of exponent about 1.2 (`expert_load` measures it)."""

import torch

from ..stage import quant
from .dims import CONV_K, DV, HD, FULL

P = "model.language_model."


class SynthWeights:
    def __init__(self, shape=FULL, layers=None, seed=0, std=0.02, init="baseline", device="cpu", fmt="fp8",
                 draw_device=None, router="uniform", keep_dense=True):
        """`keep_dense=False` drops the fp32 dequantised copies of the FP8 matrices (only the decoder needs them)."""
        assert fmt in ("fp8", "bf16") and init in ("baseline", "realistic") and router in ("uniform", "zipf")
        s = shape
        self.shape, self.fmt, self.device = s, fmt, device
        self.layers = layers if layers is not None else s.layers
        self.t, self.raw, self.fp8, self.ex, self.exs = {}, {}, set(), {}, {}
        draw_device = draw_device if draw_device is not None else "cpu"
        gen = torch.Generator(device=draw_device)
        gen.manual_seed(seed)

        def draw(*shp, mean=0.0, sd=std):
            t = torch.empty(*shp, dtype=torch.float32, device=draw_device)
            t.normal_(mean, sd, generator=gen)
            return t

        def dense(name, n, k, quantised=True):
            w = draw(n, k).to(torch.bfloat16).to(device)
            key = name + ".weight"
            if quantised and fmt == "fp8":
                q, sc = quant.quantize_fp8_block(w)
                self.raw[key] = (q, sc)
                self.fp8.add(key)
                if keep_dense:
                    self.t[key] = quant.dequantize_fp8_block(q, sc)
            else:
                self.t[key] = w.float()

        def small(name, *shp, mean=0.0, sd=std):
            self.t[name] = draw(*shp, mean=mean, sd=sd).to(torch.bfloat16).float().to(device)

        H = s.hidden
        self.t[P + "embed_tokens.weight"] = draw(s.vocab, H).to(torch.bfloat16).to(device)
        for i in range(self.layers):
            L = f"{P}layers.{i}."
            small(L + "input_layernorm.weight", H)
            small(L + "post_attention_layernorm.weight", H)
            if s.is_attn(i):
                a = L + "self_attn."
                dense(a + "q_proj", 2 * s.nq * HD, H)
                dense(a + "k_proj", s.nkv * HD, H)
                dense(a + "v_proj", s.nkv * HD, H)
                small(a + "q_norm.weight", HD)
                small(a + "k_norm.weight", HD)
                dense(a + "o_proj", H, s.nq * HD)
            else:
                g = L + "linear_attn."
                dense(g + "in_proj_qkv", s.conv_dim, H)
                dense(g + "in_proj_z", s.val_dim, H)
                dense(g + "in_proj_b", s.nvh, H, quantised=False)
                dense(g + "in_proj_a", s.nvh, H, quantised=False)
                if init == "baseline":
                    small(g + "conv1d.weight", s.conv_dim, 1, CONV_K)
                    self.t[g + "A_log"] = draw(s.nvh).to(device)
                    small(g + "dt_bias", s.nvh)
                    small(g + "norm.weight", DV)
                else:
                    small(g + "conv1d.weight", s.conv_dim, 1, CONV_K, mean=0.5, sd=0.2)
                    self.t[g + "A_log"] = draw(s.nvh, mean=-1.0, sd=1.0).to(device)
                    small(g + "dt_bias", s.nvh, sd=1.0)
                    small(g + "norm.weight", DV, mean=1.0, sd=0.1)
                dense(g + "out_proj", H, s.val_dim)
            m = L + "mlp."
            gate = draw(s.experts, H, sd=std if init == "baseline" else 0.2)
            if router == "zipf":
                # row e scaled by (rank + 1)^(-0.6): the chance to reach the top 8 falls roughly as rank^-1.2
                rank = torch.arange(s.experts, device=draw_device, dtype=torch.float32)
                gate = gate * (rank + 1.0).pow(-0.6)[:, None] * 4.0
            self.t[m + "gate.weight"] = gate.to(torch.bfloat16).float().to(device)
            small(m + "shared_expert_gate.weight", 1, H)
            for pj, (n, k) in (("gate_proj", (s.fi, H)), ("up_proj", (s.fi, H)), ("down_proj", (H, s.fi))):
                w = draw(s.experts * n, k).to(torch.bfloat16).to(device)
                if fmt == "fp8":
                    assert n % 128 == 0 or s.experts == 1, "expert rows must be whole 128-row blocks to stack"
                    q, sc = quant.quantize_fp8_block(w)
                    self.ex[(i, pj)] = q.reshape(s.experts, n, k)
                    self.exs[(i, pj)] = sc.reshape(s.experts, n // 128, -1)
                else:
                    self.ex[(i, pj)] = w.reshape(s.experts, n, k)
            se = m + "shared_expert."
            dense(se + "gate_proj", s.sfi, H)
            dense(se + "up_proj", s.sfi, H)
            dense(se + "down_proj", H, s.sfi)
        small(P + "norm.weight", H)
        self.t["lm_head.weight"] = draw(s.vocab, H).to(torch.bfloat16).to(device)

    def __getitem__(self, k):
        return self.t[k]

    def L(self, i, name):
        return self.t[f"{P}layers.{i}.{name}"]

    def is_fp8(self, i, name):
        return f"{P}layers.{i}.{name}" in self.fp8

    def expert(self, i, e):
        """fp32 (gate [FI, H], up [FI, H], down [H, FI]) of routed expert e of layer i."""
        out = []
        for pj in ("gate_proj", "up_proj", "down_proj"):
            w = self.ex[(i, pj)][e]
            out.append(quant.dequantize_fp8_block(w, self.exs[(i, pj)][e]) if self.fmt == "fp8" else w.float())
        return out


def make_prompt(vocab, n, seed=0):
    gen = torch.Generator(device="cpu")
    gen.manual_seed(2000 + seed)
    return torch.randint(0, vocab, (n,), generator=gen).tolist()


def expert_load(idx, experts):
    """Share of the routed slots each expert received: idx = expert ids of any shape."""
    return torch.bincount(idx.flatten().long().cpu(), minlength=experts).float() / idx.numel()
