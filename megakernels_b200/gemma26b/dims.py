"""Shape of the 26B-A4B model.  Defaults are the reference's constants (`gemma4-26b-a4b-gfx942/mk/dims.py:8-38`);
every width can be overridden so tests run reduced shapes through the same code."""

import math
from dataclasses import dataclass, replace

import torch


@dataclass(frozen=True)
class Shape:
    hidden: int = 2816
    layers: int = 30            # layer i is full attention iff i % 6 == 5
    vocab: int = 262144
    nq: int = 16
    nkv_s: int = 8              # sliding-window layers
    hd_s: int = 256
    window: int = 1024          # key j is visible to query i iff i - window < j <= i
    theta_s: float = 1e4        # rotation over all hd_s dims
    nkv_f: int = 2              # full-attention layers: V is the k projection
    hd_f: int = 512
    theta_f: float = 1e6
    rot_f: int = 64             # rotated angle pairs (d, d + hd_f / 2), d < rot_f
    ffn: int = 2112             # dense GeGLU MLP
    experts: int = 128
    topk: int = 8
    eff: int = 704              # expert intermediate
    softcap: float = 30.0
    eps: float = 1e-6

    def with_(self, **kw):
        return replace(self, **kw)

    @property
    def embed_scale(self):
        """sqrt(hidden) rounded to bf16, as the serving stacks do (`dims.py:13`)."""
        return float(torch.tensor(math.sqrt(self.hidden), dtype=torch.bfloat16))

    def is_full(self, i):
        return i % 6 == 5

    def attn_dims(self, i):
        """(kv heads, head dim) of layer i."""
        return (self.nkv_f, self.hd_f) if self.is_full(i) else (self.nkv_s, self.hd_s)

    def qkv_n(self, i):
        nkv, hd = self.attn_dims(i)
        return self.nq * hd + (1 if self.is_full(i) else 2) * nkv * hd

    @property
    def n_full(self):
        return sum(self.is_full(i) for i in range(self.layers))

    @property
    def n_slide(self):
        return self.layers - self.n_full


FULL = Shape()
