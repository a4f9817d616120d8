"""Host side of the 26B-A4B engine: buffers, the stage program, one launch per decode step (or per generation).

Keeps the interface of the reference's `Engine` (`gemma4-26b-a4b-gfx942/mk/runner.py`): `Engine(PK, M, maxlen, layers,
device)`, `.step(tok[M]) -> fp32 logits [M, vocab]` (soft-capped; a view, overwritten by the next step), `.reset()`.
Additions: `.generate(tok, n)` / `.prefill(prompts)` in one launch and state accessors for tests.

Stage program of one step (the reference's layer, `mk/reference.py:218-307, 327-345`):

    embed (x 53, rounded to bf16) | per layer:
        qkv GEMV | attention (sliding window of 1024, or full with V = k projection) | o GEMV -> a |
        h1 = h + rms(a) w | dense gate/up GEMV (GeGLU) , router GEMV | routing tables , experts' gate/up GEMVs |
        dense down GEMV -> d , experts' down GEMVs combined -> e | y = rms(d) w1 + rms(e) w2 | h = (h1 + rms(y) w3) scalar
    | LM head (the embedding table) with the logit soft cap

`|` is a grid barrier, `,` separates stages that share one.
"""

import torch

from ..qwen27b.runner import KV_BLOCK, attn_chunk
from ..stage import desc as D
from ..stage.runtime import Program, Runtime
from .pack import Packed


def rope_table(theta, head_dim, pairs, maxlen, device):
    """cos, sin [maxlen, pairs] fp32 of the first `pairs` angle pairs (d, d + head_dim / 2), angles in fp64
    (`gemma4-26b-a4b-gfx942/mk/reference.py:168-185`)."""
    i = torch.arange(pairs, dtype=torch.float64)
    inv = theta ** (-2 * i / head_dim)
    ang = torch.arange(maxlen, dtype=torch.float64)[:, None] * inv[None, :]
    return ang.cos().float().to(device).contiguous(), ang.sin().float().to(device).contiguous()


class Engine:
    def __init__(self, PK: Packed, M: int, maxlen: int = 4096, layers=None, device="cuda", lm_head: bool = True, spin_limit_ms=2000):
        if not 1 <= M <= D.MAX_BATCH:
            raise ValueError(f"M must lie in [1, {D.MAX_BATCH}]")
        if not torch.cuda.is_available():
            raise RuntimeError("the megakernel needs a CUDA device; there is no CPU path")
        self.PK, self.M = PK, M
        self.layers = layers if layers is not None else PK.layers
        s = self.shape = PK.shape
        dev = torch.device(device)
        if dev.index is None:
            dev = torch.device("cuda", torch.cuda.current_device())
        torch.cuda.set_device(dev)
        self.device = dev
        self.maxlen = -(-maxlen // KV_BLOCK) * KV_BLOCK
        nb = self.maxlen // KV_BLOCK
        grid = self.grid = torch.cuda.get_device_properties(dev).multi_processor_count
        H = s.hidden
        pr = self.prog = Program(dev, M, grid)
        z = pr.zeros
        self.h, self.ssq = z(M, H), z(M, H // 16)
        ymax = max(s.qkv_n(i) for i in range(max(self.layers, 6)))
        y2w = s.nq * max(s.hd_s, s.hd_f)
        self.y, self.y2 = z(M, ymax), z(M, y2w)
        self.a, self.d, self.e, self.yv = z(M, H), z(M, H), z(M, H), z(M, H)
        self.ssq_a, self.ssq_d, self.ssq_e, self.ssq_y = (z(M, H // 16) for _ in range(4))
        self.act_d = z(M, s.ffn)
        gmax = D.query("MAX_GROUPS")
        self.act_e = z(gmax, M, s.eff)
        self.router = z(M, s.experts)
        self.route_ids = z(max(self.layers, 1), M, s.topk, dtype=torch.int32)      # every layer's chosen experts, rank order
        self.logits = z(M, s.vocab)
        self.keys = z(M, grid, dtype=torch.int64)
        g = torch.Generator().manual_seed(0)
        self.bt = (torch.randperm(M * nb, generator=g) + 1).reshape(M, nb).to(torch.int32).to(dev)
        pr.hold(self.bt)
        n_full = sum(s.is_full(i) for i in range(self.layers))
        n_slide = self.layers - n_full
        self.ks = z(n_slide, M * nb + 1, s.nkv_s, KV_BLOCK, s.hd_s, dtype=torch.bfloat16)
        self.vs = z(n_slide, M * nb + 1, s.nkv_s, KV_BLOCK, s.hd_s, dtype=torch.bfloat16)
        self.kf = z(n_full, M * nb + 1, s.nkv_f, KV_BLOCK, s.hd_f, dtype=torch.bfloat16)
        self.vf = z(n_full, M * nb + 1, s.nkv_f, KV_BLOCK, s.hd_f, dtype=torch.bfloat16)
        tabs = {False: rope_table(s.theta_s, s.hd_s, s.hd_s // 2, self.maxlen, dev), True: rope_table(s.theta_f, s.hd_f, s.rot_f, self.maxlen, dev)}
        for c, sn in tabs.values():
            pr.hold(c), pr.hold(sn)
        geo = {}
        for full in (False, True):
            nkv, hd = (s.nkv_f, s.hd_f) if full else (s.nkv_s, s.hd_s)
            span = self.maxlen if full else min(self.maxlen, s.window)
            cp = attn_chunk(span, M * nkv, grid)
            mc = -(-span // cp) + 1
            qpk = s.nq // nkv
            tag = "f" if full else "s"
            part = pr.region(f"attn_{tag}.part", M * nkv * mc * (-(-qpk * (hd + 2) // 4) * 4) + grid * 16 * qpk * 128, torch.float32)
            cnt = pr.region(f"attn_{tag}.cnt", M * nkv, torch.int32)
            geo[full] = (cp, mc, part, cnt)
        plain = dict(norm_off=0.0, eps=s.eps)                      # this model's norm weights are the factors themselves

        pr.embed(PK.embed, self.h, self.ssq, self.keys if lm_head else None, H, s.vocab, scale=s.embed_scale, keys_valid=lm_head)
        si = fi = 0
        for i in range(self.layers):
            sm = lambda n: PK.small[(i, n)]                        # noqa: E731
            full = s.is_full(i)
            nkv, hd = s.attn_dims(i)
            cp, mc, a_part, a_cnt = geo[full]
            kc_, vc_ = (self.kf[fi], self.vf[fi]) if full else (self.ks[si], self.vs[si])
            cos, sin = tabs[full]

            def gemv(key, x, out, **kw):
                w, meta = PK.mats[(i, key)]
                # counters and partial tiles are shared by name between layers: the two layer types differ in size
                pr.gemv(key + (".f" if full else ".s"), w, meta, x, out, row_scale=PK.scales[(i, key)], **kw)

            gemv("qkv", self.h, self.y, x_stride=H, out_stride=ymax, n_valid=s.qkv_n(i), prologue=D.MKS_P_NORM, x_ssq=self.ssq,
                 norm_w=sm("input_layernorm.weight"), k_total=H, **plain)
            pr.add(D.desc(D.MKS_OP_ATTN, 0,
                          i=dict(NQ=s.nq, NKV=nkv, HD=hd, ROT=hd, A_Q_OFF=0, A_Q_HSTRIDE=hd, A_GATE_OFF=-1, A_K_OFF=s.nq * hd,
                                 A_V_OFF=-1 if full else s.nq * hd + nkv * hd, A_Y_STRIDE=ymax, A_Y2_STRIDE=y2w,
                                 WINDOW=0 if full else s.window, CHUNK_POS=cp, MAX_PAGES=nb, KV_F32=0, NORM_PLAIN=1, V_NORM=1,
                                 ROPE_PAIRS=s.rot_f if full else hd // 2, Q_BF16=1, MAX_CHUNKS=mc),
                          f=dict(EPS=s.eps, SCALE=1.0),
                          p=dict(A_Y=self.y.data_ptr(), A_Y2=self.y2.data_ptr(), Q_NORM=sm("self_attn.q_norm.weight").data_ptr(),
                                 K_NORM=sm("self_attn.k_norm.weight").data_ptr(), K_CACHE=kc_.data_ptr(), V_CACHE=vc_.data_ptr(),
                                 BLOCK_TABLE=self.bt.data_ptr(), ROPE_COS=cos.data_ptr(), ROPE_SIN=sin.data_ptr(),
                                 A_PART=a_part.data_ptr(), A_CNT=a_cnt.data_ptr())))
            gemv("o", self.y2, self.a, x_stride=y2w, out_stride=H, n_valid=H, out_ssq=self.ssq_a)
            # h1 = h + rms(a) w
            pr.add(D.desc(D.MKS_OP_VEC, 0, i=dict(VEC_N=H), f=dict(EPS=s.eps, NORM_OFF=0.0),
                          p=dict(VEC_BASE=self.h.data_ptr(), VEC_A=self.a.data_ptr(), VEC_A_SSQ=self.ssq_a.data_ptr(),
                                 VEC_A_W=sm("post_attention_layernorm.weight").data_ptr(), VEC_OUT=self.h.data_ptr(),
                                 VEC_OUT_SSQ=self.ssq.data_ptr())))
            gemv("d_gu", self.h, self.act_d, x_stride=H, out_stride=s.ffn, n_valid=s.ffn, prologue=D.MKS_P_NORM, x_ssq=self.ssq,
                 norm_w=sm("pre_feedforward_layernorm.weight"), k_total=H, epilogue=D.MKS_E_GLU, act=D.MKS_ACT_GELU_TANH,
                 no_barrier=True, **plain)
            gemv("router", self.h, self.router, x_stride=H, out_stride=s.experts, n_valid=s.experts, prologue=D.MKS_P_NORM,
                 x_ssq=self.ssq, norm_w=sm("router.scale"), k_total=H, in_scale=H ** -0.5, **plain)
            pr.add(D.desc(D.MKS_OP_ROUTE, D.MKS_FLAG_NO_BARRIER,
                          i=dict(EXPERTS=s.experts, TOPK=s.topk, LOGIT_STRIDE=s.experts, ROUTE_KIND=1),
                          p=dict(LOGITS=self.router.data_ptr(), EXPERT_SCALE=sm("router.per_expert_scale").data_ptr(),
                                 ROUTE_OUT=self.route_ids[i].data_ptr())))
            meta = PK.mats[(i, "ex_gu")][1]
            gemv("ex_gu", self.h, self.act_e, x_stride=H, out_stride=s.eff, out_gstride=M * s.eff, n_valid=s.eff,
                 prologue=D.MKS_P_NORM, x_ssq=self.ssq, norm_w=sm("pre_feedforward_layernorm_2.weight"), k_total=H,
                 epilogue=D.MKS_E_GLU, act=D.MKS_ACT_GELU_TANH, groups=-1, w_gstride=meta["stride"],
                 rs_gstride=meta["tiles"] * 16, **plain)
            gemv("d_down", self.act_d, self.d, x_stride=s.ffn, out_stride=H, n_valid=H, out_ssq=self.ssq_d, no_barrier=True)
            meta = PK.mats[(i, "ex_down")][1]
            gemv("ex_down", self.act_e, self.e, x_stride=s.eff, x_gstride=M * s.eff, out_stride=H, n_valid=H, out_ssq=self.ssq_e,
                 groups=-1, w_gstride=meta["stride"], rs_gstride=meta["tiles"] * 16, reduce_groups=True)
            # y = rms(d) w1 + rms(e) w2 ;  h = (h1 + rms(y) w3) * layer scalar
            pr.add(D.desc(D.MKS_OP_VEC, 0, i=dict(VEC_N=H), f=dict(EPS=s.eps, NORM_OFF=0.0),
                          p=dict(VEC_A=self.d.data_ptr(), VEC_A_SSQ=self.ssq_d.data_ptr(), VEC_A_W=sm("post_feedforward_layernorm_1.weight").data_ptr(),
                                 VEC_B=self.e.data_ptr(), VEC_B_SSQ=self.ssq_e.data_ptr(), VEC_B_W=sm("post_feedforward_layernorm_2.weight").data_ptr(),
                                 VEC_OUT=self.yv.data_ptr(), VEC_OUT_SSQ=self.ssq_y.data_ptr())))
            pr.add(D.desc(D.MKS_OP_VEC, 0, i=dict(VEC_N=H), f=dict(EPS=s.eps, NORM_OFF=0.0, SCALE=PK.small[(i, "layer_scalar")]),
                          p=dict(VEC_BASE=self.h.data_ptr(), VEC_A=self.yv.data_ptr(), VEC_A_SSQ=self.ssq_y.data_ptr(),
                                 VEC_A_W=sm("post_feedforward_layernorm.weight").data_ptr(), VEC_OUT=self.h.data_ptr(),
                                 VEC_OUT_SSQ=self.ssq.data_ptr())))
            if full:
                fi += 1
            else:
                si += 1
        if lm_head:
            w, meta = PK.lm_head
            pr.gemv("lm", w, meta, self.h, self.logits, x_stride=H, out_stride=s.vocab, prologue=D.MKS_P_NORM, x_ssq=self.ssq,
                    norm_w=PK.final_norm, k_total=H, epilogue=D.MKS_E_LOGITS, n_valid=s.vocab, keys=self.keys, row_base=0,
                    softcap=s.softcap, **plain)
        self.lm_head = lm_head
        self.rt = Runtime(pr, spin_limit_ms=spin_limit_ms)
        self.pos = self.rt.pos

    # ------------------------------------------------------------------------------------------------
    def reset(self):
        self.rt.reset()

    def step(self, tok: torch.Tensor, valid=None, stream=None):
        self.rt.tok[: self.M].copy_(tok.to(device=self.device, dtype=torch.int32))
        self.rt.launch(1, stream=stream, row_valid=self._rows(valid))
        return self.logits

    def _rows(self, valid):
        """valid[m] False marks a padding row of one step (the reference's `valid` / slot < 0 rows): its state, caches
        and position are left alone, it selects no routed expert, and its logits are undefined."""
        if valid is None:
            return None
        if not hasattr(self, "rowv"):
            self.rowv = torch.ones(8, dtype=torch.int32, device=self.device)
        self.rowv[: self.M].copy_(torch.as_tensor(valid).to(device=self.device, dtype=torch.int32))
        return self.rowv

    def generate(self, tok: torch.Tensor, n_steps: int):
        if not self.lm_head:
            raise RuntimeError("generate needs the LM head")
        out = torch.zeros(n_steps, self.M, dtype=torch.int32, device=self.device)
        self.rt.tok[: self.M].copy_(tok.to(device=self.device, dtype=torch.int32))
        self.rt.launch(n_steps, tokens_out=out)
        return out

    def prefill(self, prompts):
        if len(prompts) != self.M or len({len(p) for p in prompts}) != 1 or not prompts[0]:
            raise ValueError(f"prefill takes {self.M} prompts of one common, non-zero length")
        toks = torch.tensor(prompts, dtype=torch.int32).t().contiguous().to(self.device)
        self.rt.tok[: self.M].copy_(toks[0])
        self.rt.launch(toks.shape[0], tokens_in=toks)
        self._prompt = toks
        return self.logits

    def check(self):
        self.rt.check()

    def kv_rows(self, full, li, m, n):
        """K, V of layer `li` of its type for positions [0, n) of sequence m: [kv heads, n, head dim] fp32."""
        kc, vc = (self.kf, self.vf) if full else (self.ks, self.vs)
        pos = torch.arange(n, device=self.device)
        blk, off = self.bt[m].long()[pos // KV_BLOCK], pos % KV_BLOCK
        return kc[li][blk, :, off].transpose(0, 1).float(), vc[li][blk, :, off].transpose(0, 1).float()

    def bytes_per_step(self, context, distinct_experts=None):
        """Algorithmic bytes of one decode step: dense weights and the LM head once, `distinct_experts` routed experts
        per layer (default M x top-k, the most a step can touch), the KV cache read at `context` positions (at most
        the window on sliding layers) per sequence."""
        s = self.shape
        dense, expert, head = self.PK.weight_bytes()
        n = distinct_experts if distinct_experts is not None else min(s.experts, self.M * s.topk)
        kv = self.kf.shape[0] * 2 * s.nkv_f * s.hd_f * 2 * context + self.ks.shape[0] * 2 * s.nkv_s * s.hd_s * 2 * min(context, s.window)
        return dense + expert * n + head + self.M * kv
