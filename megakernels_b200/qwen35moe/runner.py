"""Host side of the 35B-A3B engine: buffers, the stage program, one launch per decode step (or per generation).

Keeps the interface of the reference's `Engine` (`qwen3.6-35b-a3b-gfx942/mk/runner.py`): `Engine(PK, M, maxlen,
layers, device)`, `.step(tok[M]) -> fp32 logits [M, vocab]` (a view, overwritten by the next step), `.reset()`.
Additions: `.generate(tok, n)` / `.prefill(prompts)` in one launch, state accessors in the reference decoder's
layouts, `.routing(i)` for tests.

Stage program of one step (the reference's schedule, `mk/kernel.py`):

    embed | per layer: in-proj GEMV(s) | mixer | out-proj GEMV (+h) | router GEMV | routing tables |
            experts' gate/up GEMVs (routed list + shared expert) | experts' down GEMVs, combined (+h) | ... | LM head

The routed stages take their matrices from the list the routing stage leaves in every CTA's shared memory: the
distinct experts of the step's M x 8 choices in ascending id, the shared expert as one more group; the down
stage adds the groups' products with the routing weights (and the shared expert's sigmoid gate) per sequence, in
group order, into the residual stream.
"""

import torch

from ..stage import desc as D
from ..stage.runtime import Program, Runtime
from ..qwen27b.runner import KV_BLOCK, attn_chunk, rope_tables
from .dims import DK, DV, HD, ROT
from .pack import Packed


class Engine:
    def __init__(self, PK: Packed, M: int, maxlen: int = 4096, layers=None, device="cuda", lm_head: bool = True,
                 spin_limit_ms=2000, exact_inputs=False, kv_dtype="bf16"):
        """`exact_inputs=True` feeds the FP8 GEMVs fp32-exact inputs as two fp16 pieces (M <= 4) and keeps the conv
        history unrounded: the arithmetic of the reference's exact mode.  The default rounds GEMV inputs and the
        conv history to bf16, the model's own dtype."""
        if not 1 <= M <= D.MAX_BATCH:
            raise ValueError(f"M must lie in [1, {D.MAX_BATCH}]")
        if exact_inputs and M > 4:
            raise ValueError("two-piece inputs occupy two MMA columns per sequence: M <= 4")
        if kv_dtype not in ("bf16", "fp32"):
            raise ValueError("kv_dtype: 'bf16' or 'fp32'")
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
        ymax = max(s.inp_n, s.qkv_n)
        y2w = max(s.val_dim, s.nq * HD)
        self.y, self.y2 = z(M, ymax), z(M, y2w)
        self.logits = z(M, s.vocab)
        self.keys = z(M, grid, dtype=torch.int64)
        rw = -(-(s.experts + 1) // 16) * 16
        self.router = z(M, rw)                                     # router logits | shared-expert gate logit
        self.route_ids = z(max(self.layers, 1), M, s.topk, dtype=torch.int32)      # every layer's chosen experts, rank order
        gmax = D.query("MAX_GROUPS")
        self.act = z(gmax, M, s.fi)                                # experts' activations, one slab per routed group
        cos, sin = rope_tables(s.theta, self.maxlen, dev)
        pr.hold(cos), pr.hold(sin)
        g = torch.Generator().manual_seed(0)
        self.bt = (torch.randperm(M * nb, generator=g) + 1).reshape(M, nb).to(torch.int32).to(dev)
        pr.hold(self.bt)
        n_att = sum(s.is_attn(i) for i in range(self.layers))
        n_gdn = self.layers - n_att
        kvt = torch.bfloat16 if kv_dtype == "bf16" else torch.float32
        self.k_cache = z(n_att, M * nb + 1, s.nkv, KV_BLOCK, HD, dtype=kvt)
        self.v_cache = z(n_att, M * nb + 1, s.nkv, KV_BLOCK, HD, dtype=kvt)
        self.conv = z(n_gdn, M, s.conv_dim, 4)
        self.ssm = z(n_gdn, M, s.nvh, DV, DK)
        qpk = s.nq // s.nkv
        cp = self.chunk_pos = attn_chunk(self.maxlen, M * s.nkv, grid)
        max_chunks = -(-self.maxlen // cp)
        a_part = pr.region("attn.part", M * s.nkv * max_chunks * (-(-qpk * (HD + 2) // 4) * 4) + grid * 16 * qpk * 128, torch.float32)
        a_cnt = pr.region("attn.cnt", M * s.nkv, torch.int32)
        pieces = 2 if exact_inputs else 1
        pc = lambda meta: pieces                                              # noqa: E731

        pr.embed(PK.embed, self.h, self.ssq, self.keys if lm_head else None, H, s.vocab, keys_valid=lm_head)
        gi = ai = 0
        for i in range(self.layers):
            sm = lambda n: PK.small[(i, n)]                        # noqa: E731
            norm_in = dict(prologue=D.MKS_P_NORM, x_ssq=self.ssq, norm_w=sm("input_layernorm.weight"), eps=s.eps, k_total=H)
            if s.is_attn(i):
                w, meta = PK.mats[(i, "qkv")]
                pr.gemv("qkv", w, meta, self.h, self.y, x_stride=H, out_stride=ymax, n_valid=s.qkv_n, pieces=pc(meta), **norm_in)
                pr.add(D.desc(D.MKS_OP_ATTN, 0,
                              i=dict(NQ=s.nq, NKV=s.nkv, HD=HD, ROT=ROT, A_Q_OFF=0, A_Q_HSTRIDE=2 * HD, A_GATE_OFF=HD,
                                     A_K_OFF=2 * s.nq * HD, A_V_OFF=2 * s.nq * HD + s.nkv * HD, A_Y_STRIDE=ymax, A_Y2_STRIDE=y2w,
                                     WINDOW=0, CHUNK_POS=cp, MAX_PAGES=nb, KV_F32=int(kv_dtype == "fp32"), NORM_PLAIN=0, V_NORM=0,
                                     ROPE_PAIRS=ROT // 2, Q_BF16=int(not exact_inputs), MAX_CHUNKS=max_chunks),
                              f=dict(EPS=s.eps, SCALE=HD ** -0.5),
                              p=dict(A_Y=self.y.data_ptr(), A_Y2=self.y2.data_ptr(), Q_NORM=sm("self_attn.q_norm.weight").data_ptr(),
                                     K_NORM=sm("self_attn.k_norm.weight").data_ptr(), K_CACHE=self.k_cache[ai].data_ptr(),
                                     V_CACHE=self.v_cache[ai].data_ptr(), BLOCK_TABLE=self.bt.data_ptr(), ROPE_COS=cos.data_ptr(),
                                     ROPE_SIN=sin.data_ptr(), A_PART=a_part.data_ptr(), A_CNT=a_cnt.data_ptr())))
                w, meta = PK.mats[(i, "o")]
                pr.gemv("o", w, meta, self.y2, self.h, x_stride=y2w, out_stride=H, epilogue=D.MKS_E_RESID, out_ssq=self.ssq,
                        n_valid=H, pieces=pc(meta))
                ai += 1
            else:
                w, meta = PK.mats[(i, "qkvz")]
                pr.gemv("qkvz", w, meta, self.h, self.y, x_stride=H, out_stride=ymax, n_valid=s.qkvz_n, pieces=pc(meta),
                        no_barrier=True, **norm_in)
                w, meta = PK.mats[(i, "ba")]
                pr.gemv("ba", w, meta, self.h, self.y[:, s.qkvz_n:], x_stride=H, out_stride=ymax, n_valid=2 * s.nvh, pieces=pc(meta), **norm_in)
                pr.add(D.desc(D.MKS_OP_GDN, 0,
                              i=dict(NKH=s.nkh, NVH=s.nvh, Q_OFF=0, K_OFF=s.key_dim, V_OFF=2 * s.key_dim, Z_OFF=s.conv_dim,
                                     B_OFF=s.qkvz_n, A_OFF=s.qkvz_n + s.nvh, CONV_DIM=s.conv_dim, Y_STRIDE=ymax, Y2_STRIDE=y2w,
                                     CONV_BF16=int(not exact_inputs), L2_CLAMP=0),
                              f=dict(EPS=s.eps),
                              p=dict(Y=self.y.data_ptr(), Y2=self.y2.data_ptr(), CONV_W=sm("linear_attn.conv1d.weight").data_ptr(),
                                     A_LOG=sm("linear_attn.A_log").data_ptr(), DT_BIAS=sm("linear_attn.dt_bias").data_ptr(),
                                     GDN_NORM=sm("linear_attn.norm.weight").data_ptr(), CONV_STATE=self.conv[gi].data_ptr(),
                                     SSM_STATE=self.ssm[gi].data_ptr())))
                w, meta = PK.mats[(i, "out")]
                pr.gemv("out", w, meta, self.y2, self.h, x_stride=y2w, out_stride=H, epilogue=D.MKS_E_RESID, out_ssq=self.ssq,
                        n_valid=H, pieces=pc(meta))
                gi += 1
            # ---- mixture of experts
            norm_post = dict(prologue=D.MKS_P_NORM, x_ssq=self.ssq, norm_w=sm("post_attention_layernorm.weight"), eps=s.eps, k_total=H)
            w, meta = PK.mats[(i, "router")]
            pr.gemv("router", w, meta, self.h, self.router, x_stride=H, out_stride=rw, n_valid=s.experts + 1, pieces=pc(meta), **norm_post)
            pr.add(D.desc(D.MKS_OP_ROUTE, D.MKS_FLAG_NO_BARRIER,
                          i=dict(EXPERTS=s.experts, TOPK=s.topk, LOGIT_STRIDE=rw, ROUTE_KIND=0),
                          p=dict(LOGITS=self.router.data_ptr(), ROUTE_OUT=self.route_ids[i].data_ptr())))
            w, meta = PK.mats[(i, "ex_gu")]
            ws, _ = PK.mats[(i, "sh_gu")]
            pr.gemv("ex_gu", w, meta, self.h, self.act, x_stride=H, out_stride=s.fi, out_gstride=M * s.fi, epilogue=D.MKS_E_GLU,
                    n_valid=s.fi, groups=-1, w_gstride=meta["stride"], w_shared=ws, pieces=pc(meta), **norm_post)
            w, meta = PK.mats[(i, "ex_down")]
            ws, _ = PK.mats[(i, "sh_down")]
            pr.gemv("ex_down", w, meta, self.act, self.h, x_stride=s.fi, x_gstride=M * s.fi, out_stride=H, epilogue=D.MKS_E_RESID,
                    out_ssq=self.ssq, n_valid=H, groups=-1, w_gstride=meta["stride"], w_shared=ws, reduce_groups=True, pieces=pc(meta))
        if lm_head:
            w, meta = PK.lm_head
            pr.gemv("lm", w, meta, self.h, self.logits, x_stride=H, out_stride=s.vocab, prologue=D.MKS_P_NORM, x_ssq=self.ssq,
                    norm_w=PK.final_norm, eps=s.eps, k_total=H, epilogue=D.MKS_E_LOGITS, n_valid=s.vocab, keys=self.keys, row_base=0,
                    pieces=pieces)
        self.lm_head = lm_head
        self.rt = Runtime(pr, spin_limit_ms=spin_limit_ms)
        self.pos = self.rt.pos

    # ------------------------------------------------------------------------------------------------
    def reset(self):
        for t in (self.conv, self.ssm):
            t.zero_()
        self.rt.reset()

    def step(self, tok: torch.Tensor, valid=None, stream=None):
        """One decode step for all M rows.  tok: [M] int.  Returns fp32 logits [M, vocab] (a view, overwritten by
        the next step)."""
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
        """`n_steps` decode steps in one launch, every later step fed the greedy choice of the one before.
        Returns the chosen ids [n_steps, M] (int32, on the device)."""
        if not self.lm_head:
            raise RuntimeError("generate needs the LM head")
        out = torch.zeros(n_steps, self.M, dtype=torch.int32, device=self.device)
        self.rt.tok[: self.M].copy_(tok.to(device=self.device, dtype=torch.int32))
        self.rt.launch(n_steps, tokens_out=out)
        return out

    def prefill(self, prompts):
        """The prompts (M lists of one length) position by position in one launch; returns the last logits."""
        if len(prompts) != self.M or len({len(p) for p in prompts}) != 1 or not prompts[0]:
            raise ValueError(f"prefill takes {self.M} prompts of one common, non-zero length")
        toks = torch.tensor(prompts, dtype=torch.int32).t().contiguous().to(self.device)
        self.rt.tok[: self.M].copy_(toks[0])
        self.rt.launch(toks.shape[0], tokens_in=toks)
        self._prompt = toks
        return self.logits

    def check(self):
        self.rt.check()

    def hidden(self):
        return self.h

    # ---- state in the reference decoder's layouts (tests) ---------------------------------------------
    def ssm_state(self, gi):
        return self.ssm[gi]

    def conv_window(self, gi, m):
        p = int(self.pos[m])
        slots = [(p - 3 + j) % 4 for j in range(3)]
        return self.conv[gi][m][:, slots]

    def kv_rows(self, ai, m, n):
        pos = torch.arange(n, device=self.device)
        blk, off = self.bt[m].long()[pos // KV_BLOCK], pos % KV_BLOCK
        return self.k_cache[ai][blk, :, off].transpose(0, 1).float(), self.v_cache[ai][blk, :, off].transpose(0, 1).float()

    def bytes_per_step(self, context, distinct_experts=None):
        """Algorithmic bytes of one decode step: dense weights and the LM head once, `distinct_experts` routed
        experts per layer (default: M x top-k, the most a step can touch), SSM state read + written and the KV cache
        read at `context` positions per sequence."""
        s = self.shape
        dense, _, head = self.PK.weight_bytes()
        n = distinct_experts if distinct_experts is not None else min(s.experts, self.M * s.topk)
        routed = sum(m["stride"] * n for (k, (_, m)) in self.PK.mats.items() if k[1].startswith("ex_"))
        state = 2 * 4 * self.ssm.shape[0] * s.nvh * DV * DK
        kv = self.k_cache.shape[0] * 2 * s.nkv * HD * self.k_cache.element_size() * context
        return dense + routed + head + self.M * (state + kv)
