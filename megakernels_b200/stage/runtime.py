"""Program builder and launcher shared by the large-shape engines.

`Program` collects stage records (`desc.StageDesc`) and the device buffers they point at; `Runtime`
uploads the program and launches decode steps through `mk_stage_launch`.  PyTorch allocates the device
memory and provides the stream; every launch goes through the C ABI of `include/mk_stage.h`.  There is no
fallback: without the CUDA library and a GPU the constructors raise.
"""

import ctypes

import torch

from .. import _lib
from . import desc as D
from . import pack as P


class Program:
    """Stage records plus everything that must stay alive while they are used."""

    def __init__(self, device, batch, grid):
        self.device, self.batch, self.grid = torch.device(device), batch, grid
        self.stages, self.names, self.keep, self.shared = [], [], [], {}

    # ---- memory -------------------------------------------------------------------------------------
    def zeros(self, *shape, dtype=torch.float32):
        t = torch.zeros(*shape, dtype=dtype, device=self.device)
        self.keep.append(t)
        return t

    def hold(self, t):
        t = t.contiguous()
        self.keep.append(t)
        return t

    def region(self, name, n, dtype):
        """One zeroed buffer per name, grown to the largest request (stages of the same kind in different
        layers never run at the same time, so they share counters and partial tiles)."""
        cur = self.shared.get(name)
        if cur is None:
            cur = self.shared[name] = torch.zeros(n, dtype=dtype, device=self.device)
        if cur.numel() < n or cur.dtype != dtype:
            raise ValueError(f"region {name!r} was created with {cur.numel()} elements, a later stage asks for {n}")
        return cur

    # ---- stages -------------------------------------------------------------------------------------
    def add(self, d, name=None):
        self.stages.append(d)
        self.names.append(name if name is not None else {D.MKS_OP_EMBED: "embed", D.MKS_OP_GDN: "deltanet", D.MKS_OP_ATTN: "attention",
                                                         D.MKS_OP_ROUTE: "route", D.MKS_OP_VEC: "vector"}.get(d.op, "gemv"))
        return d

    def embed(self, table, h, h_ssq, keys, hidden, vocab, scale=0.0, keys_valid=True):
        return self.add(D.desc(D.MKS_OP_EMBED, 0, i=dict(HIDDEN=hidden, VOCAB=vocab, KEYS_VALID=int(keys_valid)), f=dict(SCALE=scale),
                               p=dict(TABLE=table.data_ptr(), H=h.data_ptr(), H_SSQ=h_ssq.data_ptr(), E_KEYS=keys.data_ptr() if keys is not None else 0)))

    def gemv(self, name, w, meta, x, out, *, x_stride, out_stride, prologue=D.MKS_P_PLAIN, x_ssq=None, norm_w=None, norm_off=1.0,
             eps=1e-6, k_total=None, epilogue=D.MKS_E_STORE, out_ssq=None, n_valid=None, act=D.MKS_ACT_SILU, groups=1,
             w_gstride=0, x_gstride=0, out_gstride=0, reduce_groups=False, allreduce=False, row_scale=None, rs_gstride=0,
             w_shared=None, rs_shared=None, keys=None, row_base=0, softcap=0.0, pieces=1, no_barrier=False, in_scale=0.0,
             max_groups=None):
        T, S = meta["tiles"], meta["splits"]
        dyn = groups < 0
        gmax = (max_groups or D.query("MAX_GROUPS")) if dyn else groups
        arrivals = gmax * S if reduce_groups else S
        cnt = part = None
        if arrivals > 1:
            ncnt = T if reduce_groups else gmax * T
            cnt = self.region(name + ".cnt", ncnt, torch.int32)
            part = self.region(name + ".part", ncnt * arrivals * 128, torch.float32)
        ptr = lambda t: t.data_ptr() if t is not None else 0
        i = dict(FMT=meta["fmt"], TILES=T, SPLITS=S, GROUPS=groups, UNIT_STEPS=meta["unit_steps"], CHUNK_STEPS=meta["chunk_steps"],
                 CHUNK_BYTES=meta["chunk_bytes"], KC=meta["kc"], PROLOGUE=prologue, EPILOGUE=epilogue,
                 N_VALID=n_valid if n_valid is not None else meta["rows"], X_STRIDE=x_stride, X_GSTRIDE=x_gstride,
                 OUT_STRIDE=out_stride, OUT_GSTRIDE=out_gstride, REDUCE_GROUPS=int(reduce_groups), ALLREDUCE=int(allreduce), ACT=act,
                 K_TOTAL=k_total if k_total is not None else meta["kc"] * S, BLOCK_SCALES=int(meta["block_scaled"]), PIECES=pieces)
        in_bound = 0.0
        if prologue == D.MKS_P_NORM and norm_w is not None:
            # |x_i| / rms(x) <= sqrt(K): a bound on every normed value, with a margin for the roundings
            kt = k_total if k_total is not None else meta["kc"] * S
            in_bound = 1.02 * (kt ** 0.5) * float((norm_w.float() + norm_off).abs().max()) * (in_scale if in_scale else 1.0)
        f = dict(EPS=eps, NORM_OFF=norm_off, SOFTCAP=softcap, IN_SCALE=in_scale, IN_BOUND=in_bound)
        p = dict(W=ptr(w), W_GSTRIDE=w_gstride, W_SHARED=ptr(w_shared), ROW_SCALE=ptr(row_scale), RS_GSTRIDE=rs_gstride,
                 RS_SHARED=ptr(rs_shared), X=ptr(x), X_SSQ=ptr(x_ssq), NORM_W=ptr(norm_w), OUT=ptr(out), OUT_SSQ=ptr(out_ssq),
                 CNT=ptr(cnt), PART=ptr(part), KEYS=ptr(keys), ROW_BASE=row_base, W_BYTES=meta["bytes"])
        return self.add(D.desc(D.MKS_OP_GEMV, D.MKS_FLAG_NO_BARRIER if no_barrier else 0, i=i, f=f, p=p), name=name)

    def host_array(self):
        arr = (D.StageDesc * len(self.stages))(*self.stages)
        return arr


def pack_to(fmt, splits, device, w, **kw):
    """pack_matrix on `device`; returns (tensor kept by the caller, meta)."""
    t, meta = P.pack_matrix(fmt, splits, w.to(device), **{k: (v.to(device) if torch.is_tensor(v) else v) for k, v in kw.items()})
    return t, meta


class PeerMailbox:
    """Every rank's all-reduce mailbox, visible to every other rank of the node: allocated with
    `mk_peer_alloc`, handles exchanged over `group` (any torch.distributed group; gloo is enough), opened with
    `mk_peer_open`.  Follows the hand-shake of the reference's peer buffer
    (`qwen3.8-27b-gfx942/mk/peer.py:26-126`), with CUDA IPC in the place of hipIpc."""

    def __init__(self, group, rank, tp, device):
        import torch.distributed as dist
        self.lib = D.lib()
        self.rank, self.tp = rank, tp
        dev = torch.device(device).index
        nbytes = D.query("MAILBOX_BYTES")
        ptr = ctypes.c_uint64()
        handle = (ctypes.c_uint8 * 64)()
        _lib.check(self.lib.mk_peer_alloc(dev, nbytes, ctypes.byref(ptr), handle))
        self.own = ptr.value
        handles = [None] * tp
        dist.all_gather_object(handles, bytes(handle), group=group)
        self.addresses, self._opened = [0] * tp, []
        for r in range(tp):
            if r == rank:
                self.addresses[r] = self.own
                continue
            h = (ctypes.c_uint8 * 64)(*handles[r])
            p = ctypes.c_uint64()
            _lib.check(self.lib.mk_peer_open(dev, h, ctypes.byref(p)))
            self.addresses[r] = p.value
            self._opened.append(p.value)
        dist.barrier(group=group)

    def close(self):
        for p in self._opened:
            self.lib.mk_peer_close(p)
        self._opened = []
        if self.own:
            self.lib.mk_peer_free(self.own)
            self.own = 0


class Runtime:
    """Uploads a program and launches steps.  Owns tok / pos / barrier / status words."""

    def __init__(self, program, mailbox=None, tp=1, rank=0, spin_limit_ms=2000):
        if not torch.cuda.is_available():
            raise RuntimeError("the stage-machine megakernel needs a CUDA device; there is no CPU path")
        self.lib = D.lib()
        self.prog = program
        dev = program.device
        self.device, self.M, self.grid = dev, program.batch, program.grid
        host = program.host_array()
        _lib.check(self.lib.mk_stage_validate(host, len(program.stages), self.M))
        nb, na = ctypes.c_int64(), ctypes.c_int64()
        _lib.check(self.lib.mk_stage_count(host, len(program.stages), ctypes.byref(nb), ctypes.byref(na)))
        self.barriers_per_step, self.allreduces_per_step = nb.value, na.value
        self.xs_bytes = int(self.lib.mk_stage_scratch_bytes(host, len(program.stages), self.M))
        raw = bytes(host)
        self.program_dev = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(dev)
        self.n_stages = len(program.stages)
        z = lambda n, dt: torch.zeros(n, dtype=dt, device=dev)
        self.tok, self.pos = z(D.MAX_BATCH, torch.int32), z(D.MAX_BATCH, torch.int32)
        self.bar, self.status = z(1, torch.int64), z(4, torch.int32)
        self.bar_base = 0
        self.ar_base = 0
        self.tp, self.rank, self.mailbox = tp, rank, mailbox
        self.spin_limit_ns = int(spin_limit_ms * 1e6)
        self.launches = 0

    def reset(self):
        self.pos.zero_()
        for t in self.prog.shared.values():
            if t.dtype == torch.int32:
                t.zero_()

    def launch(self, n_steps=1, tokens_out=None, prof=None, stream=None, n_stages=None, prof_cta=0, tokens_in=None, row_valid=None):
        """`n_stages` runs only a prefix of the program (one step; for stage-by-stage checks in tests)."""
        full = n_stages is None
        n_stages = self.n_stages if full else n_stages
        assert full or n_steps == 1
        a = D.StageArgs(program=self.program_dev.data_ptr(), n_stages=n_stages, batch=self.M, n_steps=n_steps,
                        device=self.device.index, tok=self.tok.data_ptr(), pos=self.pos.data_ptr(),
                        tokens_out=tokens_out.data_ptr() if tokens_out is not None else 0, barrier=self.bar.data_ptr(),
                        barrier_base=self.bar_base, status=self.status.data_ptr(), spin_limit_ns=self.spin_limit_ns,
                        prof=prof.data_ptr() if prof is not None else 0, tp=self.tp, rank=self.rank, ar_base=self.ar_base,
                        grid=self.grid, prof_cta=prof_cta, xs_bytes=self.xs_bytes,
                        tokens_in=tokens_in.data_ptr() if tokens_in is not None else 0,
                        n_tokens_in=tokens_in.shape[0] if tokens_in is not None else 0,
                        row_valid=row_valid.data_ptr() if row_valid is not None else 0)
        if self.tp > 1:
            for r in range(self.tp):
                a.mailbox[r] = self.mailbox.addresses[r]
        st = stream if stream is not None else torch.cuda.current_stream(self.device)
        _lib.check(self.lib.mk_stage_launch(ctypes.byref(a), ctypes.c_void_p(st.cuda_stream)))
        nb, na = self.barriers_per_step, self.allreduces_per_step
        if not full:
            nb = sum(1 for d in self.prog.stages[:n_stages] if not d.flags & D.MKS_FLAG_NO_BARRIER)
            na = sum(1 for d in self.prog.stages[:n_stages] if d.op == D.MKS_OP_GEMV and d.i[D.MKS_I_ALLREDUCE])
        self.bar_base += nb * n_steps * self.grid
        self.ar_base += na * n_steps
        self.launches += 1

    def check(self):
        """Synchronise and raise if a device-side wait ran out in any launch so far."""
        st = self.status.tolist()
        if st[0] != 0:
            raise _lib.MkError(_lib.MK_ERR_TIMEOUT, f"a device-side wait ran out (site {st[1]}, CTA {st[2]}, thread {st[3]})")
