"""Host side of the 27B engine: buffers, the stage program, one launch per decode step (or per generation).

Keeps the interface of the reference's `Engine` (`qwen3.8-27b-gfx942/mk/runner.py:26-49,198-213`):
`Engine(PK, M, maxlen, layers, device, block, group)`, `.step(tok[M]) -> fp32 logits [M, vocab of this rank]`
(a view, overwritten by the next step), `.reset()`, attributes `PK, M, maxlen, layers, d, logits, pos, bt`.
Additions: `.generate(tok, n)` runs n steps in one launch with the greedy choice made on the GPU, and
`.hidden()` / state accessors in the reference decoder's layouts for tests.

Stage program of one step (the reference's schedule, `mk/kernel.py:267` and its docstring `:1-16`):

    embed | per layer: in-proj GEMV | mixer | out-proj GEMV (+h) | gate/up GEMV | down GEMV (+h) | ... | LM head

Every `|` is a grid barrier.  Caches: KV pages of 64 positions handed out in a shuffled order, page 0 being
the null page (`runner.py:27-34,103-112`); DeltaNet conv history as a ring of four inputs per channel; SSM
state fp32 [value head][v][k].
"""

import math

import torch

from ..stage import desc as D
from ..stage.runtime import PeerMailbox, Program, Runtime
from .dims import DK, DV, HD, ROT, Dims
from .pack import Packed

KV_BLOCK = 64


def rope_tables(theta, maxlen, device):
    """cos, sin [maxlen, ROT / 2] fp32, angles in fp64 as the reference computes them
    (`qwen3.8-27b-gfx942/mk/reference.py:226-232`)."""
    inv = theta ** (-torch.arange(0, ROT, 2, dtype=torch.float64) / ROT)
    ang = torch.arange(maxlen, dtype=torch.float64)[:, None] * inv[None, :]
    return ang.cos().float().to(device).contiguous(), ang.sin().float().to(device).contiguous()


def attn_chunk(maxlen, tasks_per_pos, grid):
    """Positions per attention task: about one task per CTA at the longest context."""
    cp = -(-maxlen * tasks_per_pos // grid)
    cp = -(-cp // 16) * 16
    return max(16, min(D.query("ATTN_MAX_CHUNK"), cp))


class Engine:
    def __init__(self, PK: Packed, M: int, maxlen: int = 4096, layers=None, device="cuda", block: int = KV_BLOCK,
                 group=None, lm_head: bool = True, spin_limit_ms=2000, mailbox=None, kv_layout="pages", kv_block=KV_BLOCK):
        """`kv_layout="serving"` keeps the KV cache as [page][position][kv head][head dim] with `kv_block` positions per
        page (a power of two), the layout a serving stack's paged attention uses; the default is this kernel's own
        [page][kv head][64][head dim]."""
        if block != KV_BLOCK:
            raise ValueError(f"KV pages hold {KV_BLOCK} positions (kv_block sets the page size of the serving layout)")
        if kv_layout not in ("pages", "serving") or kv_block < 8 or kv_block & (kv_block - 1):
            raise ValueError("kv_layout: 'pages' or 'serving'; kv_block: a power of two >= 8")
        if kv_layout == "pages":
            kv_block = KV_BLOCK
        self.kv_layout, self.kv_block = kv_layout, kv_block
        if not 1 <= M <= D.MAX_BATCH:
            raise ValueError(f"M must lie in [1, {D.MAX_BATCH}]")
        if not torch.cuda.is_available():
            raise RuntimeError("the megakernel needs a CUDA device; there is no CPU path")
        self.PK, self.M = PK, M
        self.layers = layers if layers is not None else PK.layers
        s, d = PK.shape, PK.d
        self.d, self.shape = d, s
        tp, rank = PK.tp, PK.rank
        dev = torch.device(device)
        if dev.index is None:
            dev = torch.device("cuda", torch.cuda.current_device())
        torch.cuda.set_device(dev)
        self.device = dev
        KB = self.kv_block
        self.maxlen = -(-maxlen // max(KB, KV_BLOCK)) * max(KB, KV_BLOCK)
        nb = self.maxlen // KB
        grid = torch.cuda.get_device_properties(dev).multi_processor_count
        self.grid = grid
        H = s.hidden
        pr = self.prog = Program(dev, M, grid)
        z = pr.zeros
        self.h, self.ssq = z(M, H), z(M, H // 16)
        ymax = max(d.inp_n, d.qkv_n)
        y2w = max(d.val_dim, d.nq * HD)
        self.y, self.y2, self.act = z(M, ymax), z(M, y2w), z(M, d.ffn)
        self.logits = z(M, d.vocab)
        self.keys = z(M, grid, dtype=torch.int64)
        cos, sin = rope_tables(s.theta, self.maxlen, dev)
        pr.hold(cos), pr.hold(sin)
        g = torch.Generator().manual_seed(0)
        self.bt = (torch.randperm(M * nb, generator=g) + 1).reshape(M, nb).to(torch.int32).to(dev)
        pr.hold(self.bt)
        n_att = sum(s.is_attn(i) for i in range(self.layers))
        n_gdn = self.layers - n_att
        kv_shape = (M * nb + 1, d.nkv, KB, HD) if kv_layout == "pages" else (M * nb + 1, KB, d.nkv, HD)
        self.k_cache = z(n_att, *kv_shape, dtype=torch.bfloat16)
        self.v_cache = z(n_att, *kv_shape, dtype=torch.bfloat16)
        kv_fields = {} if kv_layout == "pages" else dict(KV_BLOCK=KB, KV_S_PAGE=KB * d.nkv * HD, KV_S_HEAD=HD, KV_S_POS=d.nkv * HD)
        self.conv = z(n_gdn, M, d.conv_dim, 4)
        self.ssm = z(n_gdn, M, d.nvh, DV, DK)
        qpk = d.nq // d.nkv
        cp = self.chunk_pos = attn_chunk(self.maxlen, M * d.nkv, grid)
        max_chunks = -(-self.maxlen // cp)
        a_part = pr.region("attn.part", M * d.nkv * max_chunks * (-(-qpk * (HD + 2) // 4) * 4) + grid * 16 * qpk * 128, torch.float32)
        a_cnt = pr.region("attn.cnt", M * d.nkv, torch.int32)
        ar = tp > 1

        pr.embed(PK.embed, self.h, self.ssq, self.keys if lm_head else None, H, s.vocab, keys_valid=lm_head)
        gi = ai = 0
        for i in range(self.layers):
            sm = lambda n: PK.small[(i, n)]
            if s.is_attn(i):
                w, meta = PK.mats[(i, "qkv")]
                pr.gemv("qkv", w, meta, self.h, self.y, x_stride=H, out_stride=ymax, prologue=D.MKS_P_NORM, x_ssq=self.ssq,
                        norm_w=sm("input_layernorm.weight"), eps=s.eps, k_total=H, n_valid=d.qkv_n)
                pr.add(D.desc(D.MKS_OP_ATTN, 0,
                              i=dict(NQ=d.nq, NKV=d.nkv, HD=HD, ROT=ROT, A_Q_OFF=0, A_Q_HSTRIDE=2 * HD, A_GATE_OFF=HD,
                                     A_K_OFF=2 * d.nq * HD, A_V_OFF=2 * d.nq * HD + d.nkv * HD, A_Y_STRIDE=ymax, A_Y2_STRIDE=y2w,
                                     WINDOW=0, CHUNK_POS=cp, MAX_PAGES=nb, KV_F32=0, NORM_PLAIN=0, V_NORM=0, ROPE_PAIRS=ROT // 2,
                                     Q_BF16=1, MAX_CHUNKS=max_chunks, **kv_fields),
                              f=dict(EPS=s.eps, SCALE=HD ** -0.5),
                              p=dict(A_Y=self.y.data_ptr(), A_Y2=self.y2.data_ptr(), Q_NORM=sm("self_attn.q_norm.weight").data_ptr(),
                                     K_NORM=sm("self_attn.k_norm.weight").data_ptr(), K_CACHE=self.k_cache[ai].data_ptr(),
                                     V_CACHE=self.v_cache[ai].data_ptr(), BLOCK_TABLE=self.bt.data_ptr(), ROPE_COS=cos.data_ptr(),
                                     ROPE_SIN=sin.data_ptr(), A_PART=a_part.data_ptr(), A_CNT=a_cnt.data_ptr())))
                w, meta = PK.mats[(i, "o")]
                pr.gemv("o", w, meta, self.y2, self.h, x_stride=y2w, out_stride=H, epilogue=D.MKS_E_RESID, out_ssq=self.ssq,
                        n_valid=H, allreduce=ar)
                ai += 1
            else:
                w, meta = PK.mats[(i, "inp")]
                pr.gemv("inp", w, meta, self.h, self.y, x_stride=H, out_stride=ymax, prologue=D.MKS_P_NORM, x_ssq=self.ssq,
                        norm_w=sm("input_layernorm.weight"), eps=s.eps, k_total=H, n_valid=d.inp_n)
                pr.add(D.desc(D.MKS_OP_GDN, 0,
                              i=dict(NKH=d.nkh, NVH=d.nvh, Q_OFF=d.q_off, K_OFF=d.k_off, V_OFF=d.v_off, Z_OFF=d.z_off, B_OFF=d.b_off,
                                     A_OFF=d.a_off, CONV_DIM=d.conv_dim, Y_STRIDE=ymax, Y2_STRIDE=y2w, CONV_BF16=1, L2_CLAMP=0),
                              f=dict(EPS=s.eps),
                              p=dict(Y=self.y.data_ptr(), Y2=self.y2.data_ptr(), CONV_W=sm("linear_attn.conv1d.weight").data_ptr(),
                                     A_LOG=sm("linear_attn.A_log").data_ptr(), DT_BIAS=sm("linear_attn.dt_bias").data_ptr(),
                                     GDN_NORM=sm("linear_attn.norm.weight").data_ptr(), CONV_STATE=self.conv[gi].data_ptr(),
                                     SSM_STATE=self.ssm[gi].data_ptr())))
                w, meta = PK.mats[(i, "out")]
                pr.gemv("out", w, meta, self.y2, self.h, x_stride=y2w, out_stride=H, epilogue=D.MKS_E_RESID, out_ssq=self.ssq,
                        n_valid=H, allreduce=ar)
                gi += 1
            w, meta = PK.mats[(i, "gu")]
            pr.gemv("gu", w, meta, self.h, self.act, x_stride=H, out_stride=d.ffn, prologue=D.MKS_P_NORM, x_ssq=self.ssq,
                    norm_w=sm("post_attention_layernorm.weight"), eps=s.eps, k_total=H, epilogue=D.MKS_E_GLU, n_valid=d.ffn)
            w, meta = PK.mats[(i, "down")]
            pr.gemv("down", w, meta, self.act, self.h, x_stride=d.ffn, out_stride=H, epilogue=D.MKS_E_RESID, out_ssq=self.ssq,
                    n_valid=H, allreduce=ar)
        if lm_head:
            w, meta = PK.lm_head
            pr.gemv("lm", w, meta, self.h, self.logits, x_stride=H, out_stride=d.vocab, prologue=D.MKS_P_NORM, x_ssq=self.ssq,
                    norm_w=PK.final_norm, eps=s.eps, k_total=H, epilogue=D.MKS_E_LOGITS, n_valid=d.vocab, keys=self.keys,
                    row_base=rank * d.vocab)
        self.lm_head = lm_head
        # `mailbox`: an object with `.addresses` (every rank's mailbox as this device sees it) made by the caller
        self.peer = mailbox if mailbox is not None else (PeerMailbox(group, rank, tp, dev) if tp > 1 else None)
        self.rt = Runtime(pr, mailbox=self.peer, tp=tp, rank=rank, spin_limit_ms=spin_limit_ms)
        self.pos = self.rt.pos

    # ------------------------------------------------------------------------------------------------
    def reset(self):
        for t in (self.conv, self.ssm):
            t.zero_()
        self.rt.reset()

    def step(self, tok: torch.Tensor, valid=None, stream=None):
        """One decode step for all M rows.  tok: [M] int.  Returns fp32 logits [M, vocab of this rank] (a view,
        overwritten by the next step)."""
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
        """`n_steps` decode steps in one launch: step 0 feeds `tok`, every later step the greedy choice of the
        step before.  Returns the chosen ids [n_steps, M] (int32, on the device)."""
        if not self.lm_head:
            raise RuntimeError("generate needs the LM head")
        out = torch.zeros(n_steps, self.M, dtype=torch.int32, device=self.device)
        self.rt.tok[: self.M].copy_(tok.to(device=self.device, dtype=torch.int32))
        self.rt.launch(n_steps, tokens_out=out)
        return out

    def prefill(self, prompts):
        """Feeds the prompts (M lists of equal length) position by position in ONE launch and returns the logits
        after the last position: what the reference does with one `step` per position (`mk/reference.py:378-386`)."""
        if len(prompts) != self.M or len({len(p) for p in prompts}) != 1 or not prompts[0]:
            raise ValueError(f"prefill takes {self.M} prompts of one common, non-zero length")
        toks = torch.tensor(prompts, dtype=torch.int32).t().contiguous().to(self.device)      # [L, M]
        self.rt.tok[: self.M].copy_(toks[0])
        self.rt.launch(toks.shape[0], tokens_in=toks)
        self._prompt = toks                                  # alive until the launch has run
        return self.logits

    def check(self):
        self.rt.check()

    def hidden(self):
        """The residual stream after the last layer, fp32 [M, hidden]."""
        return self.h

    # ---- state in the reference decoder's layouts (tests) ---------------------------------------------
    def ssm_state(self, gi):
        """[M, value heads of this rank, v, k] fp32: the layout of `State.ssm[gi]` (`mk/reference.py:251`)."""
        return self.ssm[gi]

    def conv_window(self, gi, m):
        """Last three conv inputs of sequence m as [conv_dim, 3], oldest first (`State.conv`, `reference.py:250`)."""
        p = int(self.pos[m])
        slots = [(p - 3 + j) % 4 for j in range(3)]
        return self.conv[gi][m][:, slots]

    def kv_rows(self, ai, m, n):
        """K, V of attention layer ai for positions [0, n) of sequence m: [kv heads, n, 256] fp32."""
        pos = torch.arange(n, device=self.device)
        blk, off = self.bt[m].long()[pos // self.kv_block], pos % self.kv_block
        if self.kv_layout == "pages":
            return self.k_cache[ai][blk, :, off].transpose(0, 1).float(), self.v_cache[ai][blk, :, off].transpose(0, 1).float()
        return self.k_cache[ai][blk, off].transpose(0, 1).float(), self.v_cache[ai][blk, off].transpose(0, 1).float()

    def bytes_per_step(self, context):
        """Algorithmic bytes one decode step moves on this rank: weights once, SSM state read + written and the KV
        cache read at `context` positions, per sequence."""
        body, head = self.PK.weight_bytes()
        d = self.d
        state = 2 * 4 * self.ssm.shape[0] * d.nvh * DV * DK
        kv = self.k_cache.shape[0] * 2 * d.nkv * HD * 2 * context
        return body + head + self.M * (state + kv)
