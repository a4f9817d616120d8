"""Shape of the 27B dense Gated-DeltaNet / gated-attention hybrid, and what one tensor-parallel rank holds.

Defaults are the reference's constants (`qwen3.8-27b-gfx942/mk/dims.py:3-31`); every width can be
overridden so that tests run reduced shapes through the same code.  `Dims(shape, tp)` restates the
reference's per-rank widths (`dims.py:38-64`) and extends them to tp = 4 and 8: a rank takes 1 / tp of the
DeltaNet key and value heads, of the query heads and of the FFN columns; with more ranks than KV heads
each KV head is held by tp / n_kv consecutive ranks.
"""

from dataclasses import dataclass, replace

DK = DV = 128       # DeltaNet head dims (the kernel's recurrence is built for 128 x 128 states)
HD = 256            # attention head dim
ROT = 64
CONV_K = 4


@dataclass(frozen=True)
class Shape:
    hidden: int = 5120
    ffn: int = 17408
    vocab: int = 248320
    layers: int = 64            # layer i is full attention iff i % 4 == 3
    nkh: int = 16               # DeltaNet key heads
    nvh: int = 48               # DeltaNet value heads
    nq: int = 24
    nkv: int = 4
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
    def inp_n(self):
        return self.conv_dim + self.val_dim + 2 * self.nvh

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


class Dims:
    """Widths of rank `rank` of `tp`."""

    def __init__(self, shape=FULL, tp=1):
        s = shape
        assert tp in (1, 2, 4, 8), "tensor parallel sizes 1, 2, 4, 8"
        assert s.nkh % tp == 0 and s.nvh % tp == 0 and s.nq % tp == 0 and s.ffn % tp == 0 and s.vocab % tp == 0, (s, tp)
        self.shape, self.tp = s, tp
        self.nkh, self.nvh = s.nkh // tp, s.nvh // tp
        self.key_dim, self.val_dim = self.nkh * DK, self.nvh * DV
        self.conv_dim = 2 * self.key_dim + self.val_dim
        self.inp_n = self.conv_dim + self.val_dim + 2 * self.nvh
        self.q_off, self.k_off, self.v_off = 0, self.key_dim, 2 * self.key_dim
        self.z_off = self.conv_dim
        self.b_off = self.conv_dim + self.val_dim
        self.a_off = self.b_off + self.nvh
        self.nq = s.nq // tp
        self.nkv = max(1, s.nkv // tp)
        self.kv_rep = max(1, tp // s.nkv)          # ranks that hold the same KV head
        self.qkv_n = 2 * self.nq * HD + 2 * self.nkv * HD
        self.ffn = s.ffn // tp
        self.vocab = s.vocab // tp

    def kv_heads(self, rank):
        """Global KV heads of `rank`."""
        if self.kv_rep > 1:
            return [rank // self.kv_rep]
        return list(range(rank * self.nkv, (rank + 1) * self.nkv))

    def vocab_off(self, rank):
        return rank * self.vocab
