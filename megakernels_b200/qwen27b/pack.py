"""Packing of the 27B model's weights into the stage-machine kernel's tile layouts, per tensor-parallel rank.

Mirrors the reference's `Packed(W, device, layers, tp, rank)` (`qwen3.8-27b-gfx942/mk/pack.py:103-149`).  Per
layer the GEMVs are, as there (`pack.py:3-9`):

    DeltaNet layer:  inp  = [in_proj_qkv | in_proj_z | in_proj_b | in_proj_a]   out = out_proj
    attention layer: qkv  = [q_proj | k_proj | v_proj]                         o   = o_proj
    every layer:     gu   = [gate_proj | up_proj] (a tile pairs 8 gate rows with their up rows)   down = down_proj

Sharding follows vLLM's layout as the reference does (`pack.py:27-78`): column-parallel matrices keep the
rank's slice of every logical row segment (q | k | v of in_proj_qkv and conv1d by heads; q heads with their
gates; KV heads; the FFN slice), row-parallel matrices (out_proj, o_proj, down_proj) their K slice, norms are
replicated, the LM head is split by vocabulary rows.  Two differences from the reference: tp may be 4 or 8
(with more ranks than KV heads a KV head is held by consecutive ranks), and the embedding table is kept whole
on every rank, so a step needs no embedding exchange.
"""

import math

import torch

from ..stage import pack as tile
from ..stage import quant
from .dims import DK, DV, HD, Dims

L = "model.language_model.layers.{}."
MXFP4_KC = 1024         # preferred input columns per K split of an MXFP4 matrix
LM_KC = 2560            # ... of the bf16 LM head


def rows_of_heads(n_heads, head_rows, tp, rank):
    per = n_heads // tp
    return slice(rank * per * head_rows, (rank + 1) * per * head_rows)


def pick_splits(K, step_k, prefer, limit=3072):
    """Number of K splits: columns per split a whole number of tile steps and at most `limit`; among those the
    one whose steps group into the largest ring chunks, then the one closest to `prefer` columns (as a ratio)."""
    best, best_key = None, None
    for s in range(1, K // step_k + 1):
        if K % s or (K // s) % step_k or K // s > limit:
            continue
        steps = K // s // step_k
        cs = next(c for c in (8, 4, 2, 1) if steps % c == 0)
        key = (-cs, abs(math.log2(K // s / prefer)))
        if best_key is None or key < best_key:
            best, best_key = s, key
    if best is None:
        raise ValueError(f"K = {K} has no split into multiples of {step_k} up to {limit}")
    return best


class Packed:
    """All kernel-side weights of TP rank `rank` (of `tp`) on one device."""

    def __init__(self, W, device="cuda", layers=None, tp=1, rank=0, pack_device=None):
        """`pack_device="cpu"` tiles the weights on the host and uploads the result."""
        s = W.shape
        self.shape, self.tp, self.rank, self.fmt = s, tp, rank, W.fmt
        self.layers = layers if layers is not None else W.layers
        d = self.d = Dims(s, tp)
        self.device = torch.device(device)
        self.mats, self.small, self.keep = {}, {}, []
        final = self.device
        dev = torch.device(pack_device) if pack_device is not None else final      # where the packing arithmetic runs

        def lin(i, name):
            """(codes-or-bf16 [N, K], scales or None) of one linear layer, on the device."""
            if self.fmt == "mxfp4":
                pk, sc = W.raw(i, name)
                return quant.mxfp4_codes(pk.to(dev)), sc.to(dev)
            return W.L(i, name + ".weight").to(dev), None

        def cat_rows(parts):
            ws = torch.cat([p[0] for p in parts])
            ss = torch.cat([p[1] for p in parts]) if parts[0][1] is not None else None
            return ws, ss

        def rows(pair, sl):
            return pair[0][sl], (pair[1][sl] if pair[1] is not None else None)

        def cols(pair, frac_lo, frac_hi):
            w, sc = pair
            K = w.shape[1]
            lo, hi = K * frac_lo // tp, K * frac_hi // tp
            return w[:, lo:hi], (sc[:, lo // 32: hi // 32] if sc is not None else None)

        def pack(i, name, pair, prefer_kc, row_order=None):
            w, sc = pair
            fmt = tile.FMT_MXFP4 if self.fmt == "mxfp4" else tile.FMT_BF16
            S = pick_splits(w.shape[1], tile.STEP_K[fmt], prefer_kc)
            t, meta = tile.pack_matrix(fmt, S, w, scales=sc, row_order=row_order)
            t = t.to(final)
            self.mats[(i, name)] = (t, meta)
            self.keep.append(t)

        for i in range(self.layers):
            if s.is_attn(i):
                a = "self_attn."
                q = rows(lin(i, a + "q_proj"), rows_of_heads(s.nq, 2 * HD, tp, rank))
                kvh = d.kv_heads(rank)
                kv_sl = slice(kvh[0] * HD, (kvh[-1] + 1) * HD)
                k, v = rows(lin(i, a + "k_proj"), kv_sl), rows(lin(i, a + "v_proj"), kv_sl)
                pack(i, "qkv", cat_rows([q, k, v]), MXFP4_KC)
                pack(i, "o", cols(lin(i, a + "o_proj"), rank, rank + 1), MXFP4_KC)
            else:
                g = "linear_attn."
                qkv = lin(i, g + "in_proj_qkv")
                seg = []
                off = 0
                for n_heads, hr in ((s.nkh, DK), (s.nkh, DK), (s.nvh, DV)):
                    sl = rows_of_heads(n_heads, hr, tp, rank)
                    seg.append(rows(qkv, slice(off + sl.start, off + sl.stop)))
                    off += n_heads * hr
                z = rows(lin(i, g + "in_proj_z"), rows_of_heads(s.nvh, DV, tp, rank))
                b = rows(lin(i, g + "in_proj_b"), rows_of_heads(s.nvh, 1, tp, rank))
                a_ = rows(lin(i, g + "in_proj_a"), rows_of_heads(s.nvh, 1, tp, rank))
                pack(i, "inp", cat_rows(seg + [z, b, a_]), MXFP4_KC)
                pack(i, "out", cols(lin(i, g + "out_proj"), rank, rank + 1), MXFP4_KC)
            m = "mlp."
            ffn_sl = slice(rank * d.ffn, (rank + 1) * d.ffn)
            gu = cat_rows([rows(lin(i, m + "gate_proj"), ffn_sl), rows(lin(i, m + "up_proj"), ffn_sl)])
            pack(i, "gu", gu, MXFP4_KC, row_order=tile.glu_row_order(d.ffn))
            pack(i, "down", cols(lin(i, m + "down_proj"), rank, rank + 1), MXFP4_KC)
            # small tensors
            names = ["input_layernorm.weight", "post_attention_layernorm.weight"]
            names += ["self_attn.q_norm.weight", "self_attn.k_norm.weight"] if s.is_attn(i) else \
                     ["linear_attn.A_log", "linear_attn.dt_bias", "linear_attn.conv1d.weight", "linear_attn.norm.weight"]
            for n in names:
                t = W.L(i, n).to(dev).float()
                if n == "linear_attn.conv1d.weight":
                    t = t[:, 0, :]
                    parts, off = [], 0
                    for n_heads, hr in ((s.nkh, DK), (s.nkh, DK), (s.nvh, DV)):
                        sl = rows_of_heads(n_heads, hr, tp, rank)
                        parts.append(t[off + sl.start: off + sl.stop])
                        off += n_heads * hr
                    t = torch.cat(parts)
                elif n in ("linear_attn.A_log", "linear_attn.dt_bias"):
                    t = t[rows_of_heads(s.nvh, 1, tp, rank)]
                t = t.contiguous().to(final)
                self.small[(i, n)] = t
                self.keep.append(t)
        lm = W["lm_head.weight"].to(dev)[rank * d.vocab: (rank + 1) * d.vocab]
        t, meta = tile.pack_matrix(tile.FMT_BF16, pick_splits(s.hidden, tile.STEP_K[tile.FMT_BF16], LM_KC), lm.contiguous())
        t = t.to(final)
        self.lm_head = (t, meta)
        self.embed = W["model.language_model.embed_tokens.weight"].to(final).contiguous()
        self.final_norm = W["model.language_model.norm.weight"].to(final).float().contiguous()
        self.keep += [t, self.embed, self.final_norm]

    def weight_bytes(self):
        """Bytes of weights one decode step streams on this rank: (layers, LM head)."""
        body = sum(m["bytes"] for (_, m) in self.mats.values())
        return body, self.lm_head[1]["bytes"]
