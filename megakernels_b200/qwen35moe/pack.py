"""Packing of the 35B-A3B model's weights into the stage-machine kernel's tile layouts.

Mirrors the reference's `Packed(W, device, layers)` (`qwen3.6-35b-a3b-gfx942/mk/pack.py`).  Per layer:

    DeltaNet layer:  qkvz = [in_proj_qkv | in_proj_z] (FP8)     ba = [in_proj_b | in_proj_a] (bf16)   out = out_proj
    attention layer: qkv  = [q_proj | k_proj | v_proj] (FP8)                                           o   = o_proj
    every layer:     router = [gate | shared_expert_gate] (bf16, 257 rows)
                     ex_gu[e] = [gate_proj_e | up_proj_e] with gate / up rows paired inside a tile, ex_down[e]
                     sh_gu, sh_down: the shared expert, same geometry as one routed expert

FP8 matrices keep their 128 x 128 block scales: the packer puts the scales of a chunk's columns behind the
chunk (one per 128 columns for the upper and one for the lower eight rows of a tile).  The routed experts of a
layer are packed as one tall matrix with a single K split, so expert e's tiles are the contiguous byte range
[e * stride, (e + 1) * stride) the kernel indexes with the routing list.
"""

import torch

from ..qwen27b.pack import pick_splits
from ..stage import pack as tile
from .dims import HD

FP8_KC = 1024
LM_KC = 2048


class Packed:
    def __init__(self, W, device="cuda", layers=None, consume=False):
        """`consume=True` frees W's expert tensors layer by layer while packing (full-depth benchmarks)."""
        s = W.shape
        self.shape, self.fmt = s, W.fmt
        self.layers = layers if layers is not None else W.layers
        self.tp, self.rank = 1, 0
        dev = torch.device(device)
        self.device = dev
        self.mats, self.small, self.keep = {}, {}, []
        fp8 = W.fmt == "fp8"
        lay = "model.language_model.layers.{}."

        def get(i, name):
            """(weight, block scales or None) of a projection: FP8 raw when the checkpoint has it, else bf16."""
            key = lay.format(i) + name + ".weight"
            if key in W.raw:
                q, sc = W.raw[key]
                return q.to(dev), sc.to(dev)
            return W.t[key].to(dev).to(torch.bfloat16), None

        def cat(parts):
            w = torch.cat([p[0] for p in parts])
            if parts[0][1] is None:
                return w, None
            assert all(p[0].shape[0] % 128 == 0 for p in parts[:-1]), "stacked FP8 matrices must be whole 128-row blocks"
            return w, torch.cat([p[1] for p in parts])

        def pack(key, pair, prefer_kc, row_order=None, splits=None):
            w, sc = pair
            fmt = tile.FMT_BF16 if sc is None and w.dtype == torch.bfloat16 else tile.FMT_FP8
            S = splits if splits is not None else pick_splits(w.shape[1], tile.STEP_K[fmt], prefer_kc)
            t, meta = tile.pack_matrix(fmt, S, w, block_scales=sc, row_order=row_order)
            self.mats[key] = (t, meta)
            self.keep.append(t)
            return meta

        for i in range(self.layers):
            if s.is_attn(i):
                a = "self_attn."
                pack((i, "qkv"), cat([get(i, a + "q_proj"), get(i, a + "k_proj"), get(i, a + "v_proj")]), FP8_KC)
                pack((i, "o"), get(i, a + "o_proj"), FP8_KC)
            else:
                g = "linear_attn."
                pack((i, "qkvz"), cat([get(i, g + "in_proj_qkv"), get(i, g + "in_proj_z")]), FP8_KC)
                pack((i, "ba"), cat([get(i, g + "in_proj_b"), get(i, g + "in_proj_a")]), FP8_KC)
                pack((i, "out"), get(i, g + "out_proj"), FP8_KC)
            m = "mlp."
            pack((i, "router"), cat([get(i, m + "gate"), get(i, m + "shared_expert_gate")]), FP8_KC)
            # routed experts: one tall matrix per projection, a single K split
            E = s.experts
            gate, up, down = W.ex[(i, "gate_proj")], W.ex[(i, "up_proj")], W.ex[(i, "down_proj")]
            gu = torch.cat([gate, up], dim=1).to(dev)                                  # [E, 2 FI, H]
            order = (tile.glu_row_order(s.fi)[None, :] + torch.arange(E)[:, None] * 2 * s.fi).reshape(-1)
            if fp8:
                gus = torch.cat([W.exs[(i, "gate_proj")], W.exs[(i, "up_proj")]], dim=1).to(dev)
                gu_pair = (gu.reshape(E * 2 * s.fi, -1), gus.reshape(E * 2 * s.fi // 128, -1))
                down_pair = (down.to(dev).reshape(E * s.hidden, -1), W.exs[(i, "down_proj")].to(dev).reshape(E * s.hidden // 128, -1))
            else:
                gu_pair = (gu.reshape(E * 2 * s.fi, -1).to(torch.bfloat16), None)
                down_pair = (down.to(dev).reshape(E * s.hidden, -1).to(torch.bfloat16), None)
            meta = pack((i, "ex_gu"), gu_pair, FP8_KC, row_order=order, splits=1)
            self._per_expert(meta, E)
            meta = pack((i, "ex_down"), down_pair, FP8_KC, splits=1)
            self._per_expert(meta, E)
            del gu, gu_pair, down_pair
            if consume:
                for pj in ("gate_proj", "up_proj", "down_proj"):
                    W.ex.pop((i, pj), None)
                    W.exs.pop((i, pj), None)
                torch.cuda.empty_cache()
            se = m + "shared_expert."
            pack((i, "sh_gu"), cat([get(i, se + "gate_proj"), get(i, se + "up_proj")]), FP8_KC, row_order=tile.glu_row_order(s.sfi), splits=1)
            pack((i, "sh_down"), get(i, se + "down_proj"), FP8_KC, splits=1)
            assert s.sfi == s.fi, "the shared expert rides the routed stages as one more group: same geometry"
            names = ["input_layernorm.weight", "post_attention_layernorm.weight"]
            names += ["self_attn.q_norm.weight", "self_attn.k_norm.weight"] if s.is_attn(i) else \
                     ["linear_attn.A_log", "linear_attn.dt_bias", "linear_attn.conv1d.weight", "linear_attn.norm.weight"]
            for n in names:
                t = W.L(i, n).to(dev).float()
                if n == "linear_attn.conv1d.weight":
                    t = t[:, 0, :]
                t = t.contiguous()
                self.small[(i, n)] = t
                self.keep.append(t)
        lm = W["lm_head.weight"].to(dev).to(torch.bfloat16).contiguous()
        t, meta = tile.pack_matrix(tile.FMT_BF16, pick_splits(s.hidden, tile.STEP_K[tile.FMT_BF16], LM_KC), lm)
        self.lm_head = (t, meta)
        self.embed = W["model.language_model.embed_tokens.weight"].to(dev).to(torch.bfloat16).contiguous()
        self.final_norm = W["model.language_model.norm.weight"].to(dev).float().contiguous()
        self.keep += [t, self.embed, self.final_norm]

    @staticmethod
    def _per_expert(meta, E):
        """Turn the meta of a tall stack of E equal matrices into that of one expert plus the stride between experts."""
        assert meta["tiles"] % E == 0 and meta["bytes"] % E == 0 and meta["splits"] == 1
        meta["stride"] = meta["bytes"] // E
        meta["tiles"] //= E
        meta["rows"] //= E
        meta["bytes"] = meta["stride"]
        meta["experts"] = E

    def weight_bytes(self, batch=1):
        """Bytes of weights one decode step streams: (dense layers' matrices, routed experts at `batch` sequences
        with disjoint choices -- the upper bound -- and the shared expert, LM head)."""
        dense = sum(m["bytes"] for (k, (_, m)) in self.mats.items() if not k[1].startswith("ex_"))
        routed = sum(m["stride"] * min(self.shape.experts, batch * self.shape.topk) for (k, (_, m)) in self.mats.items() if k[1].startswith("ex_"))
        return dense, routed, self.lm_head[1]["bytes"]
