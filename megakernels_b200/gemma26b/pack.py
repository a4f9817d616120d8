"""Packing of the 26B-A4B model's weights into the stage-machine kernel's tile layouts.

Mirrors the reference's `Packed(W, device, layers)` (`gemma4-26b-a4b-gfx942/mk/pack.py`).  Per layer:

    qkv    = [q_proj | k_proj | v_proj] (sliding) or [q_proj | k_proj] (full: V is the k projection)      o = o_proj
    router = router.proj (bf16)
    d_gu   = [mlp.gate_proj | mlp.up_proj] with gate / up rows paired inside a tile      d_down = mlp.down_proj
    ex_gu[e], ex_down[e]: the routed experts, one tall matrix per projection with a single K split, so that expert e's
    tiles are the byte range [e * stride, (e + 1) * stride) the kernel indexes with the routing list

FP8 matrices come with one scale per output row; the scales travel as fp32 arrays in the packed row order and are
applied to the accumulators (`y = (x @ W^T) * scale`, `mk/reference.py:150-157`).
"""

import torch

from ..qwen27b.pack import pick_splits
from ..stage import pack as tile

FP8_KC = 1024
LM_KC = 2816


class Packed:
    def __init__(self, W, device="cuda", layers=None, consume=False):
        s = W.shape
        self.shape, self.fmt = s, W.fmt
        self.layers = layers if layers is not None else W.layers
        self.tp, self.rank = 1, 0
        dev = torch.device(device)
        self.device = dev
        self.mats, self.scales, self.small, self.keep = {}, {}, {}, []

        def cat(parts):
            w = torch.cat([p[0] for p in parts]).to(dev)
            if parts[0][1] is None:
                return w, None
            return w, torch.cat([p[1].reshape(-1) for p in parts]).to(dev)

        def pack(key, pair, row_order=None, splits=None):
            w, sc = pair
            w = w.to(dev)
            fmt = tile.FMT_FP8 if w.dtype == torch.float8_e4m3fn else tile.FMT_BF16
            if fmt == tile.FMT_BF16:
                w = w.to(torch.bfloat16)
            S = splits if splits is not None else pick_splits(w.shape[1], tile.STEP_K[fmt], FP8_KC)
            t, meta = tile.pack_matrix(fmt, S, w, row_order=row_order)
            self.mats[key] = (t, meta)
            self.keep.append(t)
            if sc is not None:
                rs = sc.to(dev).float().reshape(-1)
                if row_order is not None:
                    rs = rs[row_order.to(dev)]
                pad = meta["tiles"] * 16 - rs.numel()
                if pad:
                    rs = torch.cat([rs, torch.zeros(pad, device=dev)])
                self.scales[key] = rs.contiguous()
                self.keep.append(self.scales[key])
            else:
                self.scales[key] = None
            return meta

        E = s.experts
        for i in range(self.layers):
            a = "self_attn."
            parts = [W.lin(i, a + "q_proj"), W.lin(i, a + "k_proj")] + ([] if s.is_full(i) else [W.lin(i, a + "v_proj")])
            pack((i, "qkv"), cat(parts))
            pack((i, "o"), W.lin(i, a + "o_proj"))
            pack((i, "router"), (W.L(i, "router.proj.weight"), None))
            pack((i, "d_gu"), cat([W.lin(i, "mlp.gate_proj"), W.lin(i, "mlp.up_proj")]), row_order=tile.glu_row_order(s.ffn))
            pack((i, "d_down"), W.lin(i, "mlp.down_proj"))
            gu = torch.cat([W.ex[(i, "gate_proj")], W.ex[(i, "up_proj")]], dim=1).to(dev)              # [E, 2 eff, H]
            order = (tile.glu_row_order(s.eff)[None, :] + torch.arange(E)[:, None] * 2 * s.eff).reshape(-1)
            if W.fmt == "fp8":
                gus = torch.cat([W.exs[(i, "gate_proj")], W.exs[(i, "up_proj")]], dim=1).to(dev)       # [E, 2 eff]
                gu_pair, down_pair = (gu.reshape(E * 2 * s.eff, -1), gus.reshape(-1)), \
                                     (W.ex[(i, "down_proj")].reshape(E * s.hidden, -1), W.exs[(i, "down_proj")].reshape(-1))
            else:
                gu_pair, down_pair = (gu.reshape(E * 2 * s.eff, -1), None), (W.ex[(i, "down_proj")].reshape(E * s.hidden, -1), None)
            self._per_expert(pack((i, "ex_gu"), gu_pair, row_order=order, splits=1), E)
            self._per_expert(pack((i, "ex_down"), down_pair, splits=1), E)
            del gu, gu_pair, down_pair
            if consume:
                for pj in ("gate_proj", "up_proj", "down_proj"):
                    W.ex.pop((i, pj), None)
                    W.exs.pop((i, pj), None)
                torch.cuda.empty_cache()
            for n in ("input_layernorm.weight", "post_attention_layernorm.weight", "pre_feedforward_layernorm.weight",
                      "pre_feedforward_layernorm_2.weight", "post_feedforward_layernorm_1.weight", "post_feedforward_layernorm_2.weight",
                      "post_feedforward_layernorm.weight", "self_attn.q_norm.weight", "self_attn.k_norm.weight", "router.scale",
                      "router.per_expert_scale"):
                t = W.L(i, n).to(dev).float().contiguous()
                self.small[(i, n)] = t
                self.keep.append(t)
            self.small[(i, "layer_scalar")] = float(W.L(i, "layer_scalar").float())
        emb = W.embed.to(dev).to(torch.bfloat16).contiguous()
        t, meta = tile.pack_matrix(tile.FMT_BF16, pick_splits(s.hidden, tile.STEP_K[tile.FMT_BF16], LM_KC), emb)
        self.lm_head = (t, meta)                                   # tied: the LM head is the embedding table, tiled
        self.embed = emb
        self.final_norm = W["model.language_model.norm.weight"].to(dev).float().contiguous()
        self.keep += [t, self.embed, self.final_norm]

    @staticmethod
    def _per_expert(meta, E):
        assert meta["tiles"] % E == 0 and meta["bytes"] % E == 0 and meta["splits"] == 1
        meta["stride"] = meta["bytes"] // E
        meta["tiles"] //= E
        meta["rows"] //= E
        meta["bytes"] = meta["stride"]
        meta["experts"] = E

    def weight_bytes(self):
        """(dense matrices of all layers, one routed expert's gate/up + down per layer summed over layers, LM head)."""
        dense = sum(m["bytes"] for (k, (_, m)) in self.mats.items() if not k[1].startswith("ex_"))
        expert = sum(m["stride"] for (k, (_, m)) in self.mats.items() if k[1].startswith("ex_"))
        return dense, expert, self.lm_head[1]["bytes"]
