"""Seeded synthetic weights of the 26B-A4B model with the accessors of the reference's `Weights`
(`gemma4-26b-a4b-gfx942/mk/reference.py:64-117`): `.t[name]`, `.L(i, name)`, `.lin(i, name) -> (weight, row scale
or None)`, `.expert(i, e) -> (gate, up, down) pairs`, `.embed`, `.fmt`.  fmt "fp8": every projection and expert
matrix is e4m3fn with one bf16 scale per output row, as the FP8-dynamic checkpoint the reference loads; the
router, the norms, the embedding (tied LM head) stay bf16.  The routed experts are also kept stacked
(`.ex[(i, proj)]` [experts, N, K], `.exs[...]` [experts, N]) for the packer; `.t` holds views of them under the
checkpoint's per-expert names."""

import torch

from ..stage import quant
from .dims import FULL

L = "model.language_model.layers.{}."


class SynthWeights:
    def __init__(self, shape=FULL, layers=None, seed=0, std=0.02, init="baseline", device="cpu", fmt="fp8", draw_device=None,
                 router="uniform"):
        assert fmt in ("fp8", "bf16") and init in ("baseline", "realistic") and router in ("uniform", "zipf")
        s = shape
        self.shape, self.fmt, self.device = s, fmt, device
        self.layers = layers if layers is not None else s.layers
        self.t, self.ex, self.exs = {}, {}, {}
        draw_device = draw_device if draw_device is not None else "cpu"
        gen = torch.Generator(device=draw_device)
        gen.manual_seed(seed)

        def draw(*shp, mean=0.0, sd=std):
            t = torch.empty(*shp, dtype=torch.float32, device=draw_device)
            t.normal_(mean, sd, generator=gen)
            return t

        def vec(name, *shp, mean=0.0, sd=std):
            self.t[name] = draw(*shp, mean=mean, sd=sd).to(torch.bfloat16).to(device)

        def dense(name, n, k):
            w = draw(n, k).to(torch.bfloat16).to(device)
            if fmt == "fp8":
                q, sc = quant.quantize_fp8_row(w)
                self.t[name + ".weight"], self.t[name + ".weight_scale"] = q, sc.reshape(-1, 1)
            else:
                self.t[name + ".weight"] = w

        H = s.hidden
        real = init == "realistic"
        self.t["model.language_model.embed_tokens.weight"] = draw(s.vocab, H).to(torch.bfloat16).to(device)
        for i in range(self.layers):
            p = L.format(i)
            nkv, hd = s.attn_dims(i)
            for n in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm", "pre_feedforward_layernorm_2",
                      "post_feedforward_layernorm_1", "post_feedforward_layernorm_2", "post_feedforward_layernorm"):
                # plain (not zero-centred) norm weights: around 1 in a trained model
                vec(p + n + ".weight", H, mean=1.0 if real else 0.0, sd=0.1 if real else std)
            self.t[p + "layer_scalar"] = (draw(1, mean=1.0, sd=0.05) if real else draw(1, mean=1.0, sd=std)).to(torch.bfloat16).to(device)
            a = p + "self_attn."
            dense(a + "q_proj", s.nq * hd, H)
            dense(a + "k_proj", nkv * hd, H)
            if not s.is_full(i):
                dense(a + "v_proj", nkv * hd, H)
            # attention scores are q . k with scaling 1: norm weights around 1/4 keep them O(1) over 256 or 512 dims, as
            # trained weights do; around 1 the softmax is one-hot and amplifies single bf16 roundings of the cache
            vec(a + "q_norm.weight", hd, mean=0.25 if real else 0.0, sd=0.025 if real else std)
            vec(a + "k_norm.weight", hd, mean=0.25 if real else 0.0, sd=0.025 if real else std)
            dense(a + "o_proj", H, s.nq * hd)
            vec(p + "router.scale", H, mean=1.0 if real else 0.0, sd=0.1 if real else std)
            # router logits of deviation ~3 on the realistic initialisation: boundary gaps far above the arithmetic noise
            proj = draw(s.experts, H, sd=3.0 if real else std)
            if router == "zipf":
                rank = torch.arange(s.experts, device=draw_device, dtype=torch.float32)
                proj = proj * (rank + 1.0).pow(-0.6)[:, None] * 4.0
            self.t[p + "router.proj.weight"] = proj.to(torch.bfloat16).to(device)
            vec(p + "router.per_expert_scale", s.experts, mean=1.0, sd=0.1 if real else std)
            dense(p + "mlp.gate_proj", s.ffn, H)
            dense(p + "mlp.up_proj", s.ffn, H)
            dense(p + "mlp.down_proj", H, s.ffn)
            for pj, (n, k) in (("gate_proj", (s.eff, H)), ("up_proj", (s.eff, H)), ("down_proj", (H, s.eff))):
                w = draw(s.experts * n, k).to(torch.bfloat16).to(device)
                if fmt == "fp8":
                    q, sc = quant.quantize_fp8_row(w)
                    self.ex[(i, pj)], self.exs[(i, pj)] = q.reshape(s.experts, n, k), sc.reshape(s.experts, n)
                    for e in range(s.experts):
                        self.t[f"{p}experts.{e}.{pj}.weight"] = self.ex[(i, pj)][e]
                        self.t[f"{p}experts.{e}.{pj}.weight_scale"] = self.exs[(i, pj)][e].reshape(-1, 1)
                else:
                    self.ex[(i, pj)] = w.reshape(s.experts, n, k)
            if fmt == "bf16":
                self.t[p + "experts.gate_up_proj"] = torch.cat([self.ex[(i, "gate_proj")], self.ex[(i, "up_proj")]], dim=1)
                self.t[p + "experts.down_proj"] = self.ex[(i, "down_proj")]
        vec("model.language_model.norm.weight", H, mean=1.0 if real else 0.0, sd=0.1 if real else std)

    def __getitem__(self, k):
        return self.t[k]

    def L(self, i, name):
        return self.t[L.format(i) + name]

    def lin(self, i, name):
        """name: e.g. 'self_attn.q_proj', 'mlp.down_proj' -> (weight, row scale or None)."""
        return self.L(i, name + ".weight"), self.t.get(L.format(i) + name + ".weight_scale")

    def expert(self, i, e):
        eff = self.shape.eff
        if self.fmt == "bf16":
            gu = self.L(i, "experts.gate_up_proj")[e]
            return (gu[:eff], None), (gu[eff:], None), (self.L(i, "experts.down_proj")[e], None)
        return tuple(self.lin(i, f"experts.{e}.{n}") for n in ("gate_proj", "up_proj", "down_proj"))

    @property
    def embed(self):
        return self.t["model.language_model.embed_tokens.weight"]


def make_prompt(vocab, n, seed=0):
    gen = torch.Generator(device="cpu")
    gen.manual_seed(3000 + seed)
    return torch.randint(0, vocab, (n,), generator=gen).tolist()
