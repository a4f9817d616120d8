"""Shape of the 35B-A3B MoE hybrid.  Defaults are the reference's constants
(`qwen3.6-35b-a3b-gfx942/mk/dims.py:6-40`); every width can be overridden so tests run reduced shapes
through the same code."""

from dataclasses import dataclass, replace

DK = DV = 128
HD = 256
ROT = 64
CONV_K = 4


@dataclass(frozen=True)
class Shape:
    hidden: int = 2048
    vocab: int = 248320
    layers: int = 40            # layer i is full attention iff i % 4 == 3
    nkh: int = 16               # DeltaNet key heads; value head h uses key head h // (nvh / nkh)
    nvh: int = 32
    nq: int = 16
    nkv: int = 2
    experts: int = 256
    topk: int = 8
    fi: int = 512               # expert intermediate
    sfi: int = 512              # shared expert intermediate
    theta: float = 1e7
    eps: float = 1e-6

    def with_(self, **kw):
        return replace(self, **kw)

    @property
    def key_dim(self):
        return self.nkh * DK

    @property
    def val_dim(self):
        return self.nvh * DV

    @property
    def conv_dim(self):
        return 2 * self.key_dim + self.val_dim

    @property
    def qkvz_n(self):
        """Rows of the FP8 part of the DeltaNet in-projection: [q | k | v | z]."""
        return self.conv_dim + self.val_dim

    @property
    def inp_n(self):
        """... plus the bf16 rows [b | a]."""
        return self.qkvz_n + 2 * self.nvh

    @property
    def qkv_n(self):
        return 2 * self.nq * HD + 2 * self.nkv * HD

    def is_attn(self, i):
        return i % 4 == 3

    @property
    def n_gdn(self):
        return sum(not self.is_attn(i) for i in range(self.layers))

    @property
    def n_attn(self):
        return self.layers - self.n_gdn


FULL = Shape()
