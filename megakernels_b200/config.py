"""Model configuration for the hybrid Gated-DeltaNet / gated-attention decoders.

`Config` carries the same fields, with the same meaning, as the reference's
`qwen3.5-0.8b/qwen_mk/weights.py:13-33` so that code written against the reference's
`Megakernel.cfg` keeps working.  `Config.from_json` reads a Hugging Face `config.json`
the same way (`weights.py:35-58`); `qwen35_08b()` builds the 0.8B shape without one.
"""

import json
from dataclasses import dataclass, field, replace


@dataclass
class Config:
    hidden: int
    n_layers: int
    layer_types: list
    intermediate: int
    vocab: int
    eps: float
    # gated full attention
    n_heads: int
    n_kv_heads: int
    head_dim: int
    rotary_dim: int
    rope_theta: float
    # gated deltanet
    lin_heads: int
    lin_k_dim: int
    lin_v_dim: int
    conv_k: int
    eos_token_id: int
    tied: bool = True

    @classmethod
    def from_json(cls, path):
        with open(path) as f:
            c = json.load(f)
        t = c.get("text_config", c)
        rope = t["rope_parameters"]
        if t["linear_num_key_heads"] != t["linear_num_value_heads"]:
            raise ValueError("this shape needs as many DeltaNet key heads as value heads")
        return cls(
            hidden=t["hidden_size"], n_layers=t["num_hidden_layers"], layer_types=list(t["layer_types"]),
            intermediate=t["intermediate_size"], vocab=t["vocab_size"], eps=t["rms_norm_eps"],
            n_heads=t["num_attention_heads"], n_kv_heads=t["num_key_value_heads"], head_dim=t["head_dim"],
            rotary_dim=int(t["head_dim"] * rope.get("partial_rotary_factor", 1.0)), rope_theta=rope["rope_theta"],
            lin_heads=t["linear_num_value_heads"], lin_k_dim=t["linear_key_head_dim"],
            lin_v_dim=t["linear_value_head_dim"], conv_k=t["linear_conv_kernel_dim"],
            eos_token_id=t["eos_token_id"], tied=t.get("tie_word_embeddings", c.get("tie_word_embeddings", True)),
        )

    def with_(self, **kw):
        return replace(self, **kw)

    @property
    def conv_dim(self):
        return 2 * self.lin_heads * self.lin_k_dim + self.lin_heads * self.lin_v_dim

    @property
    def gdn_in_rows(self):
        """Rows of the concatenated DeltaNet input projection: qkv | z | b | a."""
        return self.conv_dim + self.lin_heads * self.lin_v_dim + 2 * self.lin_heads

    @property
    def attn_in_rows(self):
        """Rows of the concatenated attention input projection: per-head [q | gate], then k, then v."""
        return 2 * self.n_heads * self.head_dim + 2 * self.n_kv_heads * self.head_dim


def layer_pattern(n_layers, period=4):
    """[DeltaNet x (period-1), FullAttn] repeated."""
    return ["full_attention" if (i + 1) % period == 0 else "linear_attention" for i in range(n_layers)]


def qwen35_08b(n_layers=24, vocab=151936):
    """The 0.8B hybrid: hidden 1024, 16+16 DeltaNet heads of 128, 8 q / 2 kv heads of 256,
    RoPE on 64 dims (theta 1e7), SwiGLU 3584, tied embeddings."""
    return Config(hidden=1024, n_layers=n_layers, layer_types=layer_pattern(n_layers), intermediate=3584,
                  vocab=vocab, eps=1e-6, n_heads=8, n_kv_heads=2, head_dim=256, rotary_dim=64, rope_theta=1e7,
                  lin_heads=16, lin_k_dim=128, lin_v_dim=128, conv_k=4, eos_token_id=vocab - 1, tied=True)
