"""Python driver for the B200 decode megakernel: packs weights, owns state, launches steps.

The class keeps the interface of the reference's `Megakernel`
(`qwen3.5-0.8b/qwen_mk/engine.py:49-327`): the same constructor arguments, `run`, `prefill`,
`generate`, `reset`, and the attributes its session, benchmark and test code read (`cfg`, `grid`,
`pos`, `epoch`, `conv_hist`, `state`, `state_bak`, `k_cache`, `v_cache`, `weight_bytes`,
`last_step_ns`, `embed`, `final_norm`).  Differences, all additions:

* `model` may be a `(Config, weights dict)` pair instead of a checkpoint path, because no
  checkpoint can be downloaded where this library is tested;
* `quant="int8"` is per output channel (see `quant.py`) and covers the embedding table;
* the KV cache is paged (`KV_BLOCK` positions per page, `block_table` maps logical to physical
  pages) and its element type is selectable (`kv_dtype`);
* `batch=B` (int8 engines, B <= 8) keeps B independent sequences, each with its own recurrent
  state, conv history, KV pages and position, and `run_batch` advances them side by side with one
  pass over the weights per step;
* PyTorch only allocates device memory and provides the stream; every launch goes through the C
  ABI in `include/mk_b200.h`.
"""

import ctypes
import os

import torch

from . import _lib
from . import mtp as mtp_mod
from .config import Config
from .pack import as_bytes, pack_down_cols, pack_out_cols, pack_rows
from .quant import is_gemv_weight, quantize_int8_rows, roundtrip_int8_rows

# Steps per launch.  A step takes well under a millisecond on a B200, so this only bounds the size
# of the per-launch output buffers.
MAX_STEPS_PER_LAUNCH = 1024


def rope_tables(cfg, max_seq, device):
    """cos / sin [max_seq, rotary_dim / 2] in fp32 (definition: `qwen_mk/reference.py:18-23`)."""
    idx = torch.arange(0, cfg.rotary_dim, 2, dtype=torch.int64).float()
    inv_freq = 1.0 / (cfg.rope_theta ** (idx / cfg.rotary_dim))
    ang = torch.arange(max_seq, dtype=torch.float32)[:, None] * inv_freq[None, :]
    return ang.cos().to(device), ang.sin().to(device)


class Megakernel:
    def __init__(self, model, max_seq=8192, device="cuda", quant="bf16", mtp=False,
                 draft_vocab=0, kv_dtype="fp32", spin_limit_ms=2000, draft_ids=None, batch=1, pack_device=None):
        """`mtp` loads the multi-token-prediction head for speculative decoding (`run_spec`); its drafts
        come from the `draft_vocab` most frequent tokens listed in `draft_ids` (0: the whole vocabulary).
        `pack_device="cpu"` quantises and tiles the weights on the host and uploads the result (a handful of copies
        instead of a few hundred small GPU kernels; slower for large models)."""
        if quant not in ("bf16", "int8"):
            raise ValueError(f"quant must be 'bf16' or 'int8', got {quant!r}")
        if kv_dtype not in ("bf16", "fp32"):
            raise ValueError(f"kv_dtype must be 'bf16' or 'fp32', got {kv_dtype!r}")
        if not 1 <= batch <= _lib.MAX_BATCH:
            raise ValueError(f"batch must lie in [1, {_lib.MAX_BATCH}], got {batch}")
        if batch > 1 and quant != "int8":
            raise ValueError("batched decoding is built for int8 weights only")
        if not torch.cuda.is_available():
            raise RuntimeError("the decode megakernel needs a CUDA device; there is no CPU path")
        self.batch = batch
        self.lib = _lib.load()
        self.quant, self.kv_dtype = quant, kv_dtype
        self.spin_limit_ns = int(spin_limit_ms * 1e6)
        device = torch.device(device)
        if device.index is None:
            device = torch.device(device.type, torch.cuda.current_device())
        torch.cuda.set_device(device)
        self.device = device
        wm = None
        if isinstance(model, (tuple, list)):
            self.cfg, w = model[0], model[1]
            wm = model[2] if len(model) > 2 else None
        else:
            from . import weights as _weights
            self.cfg, w = _weights.load(model, "cpu")
            if mtp:
                wm = _weights.load_mtp(model, "cpu")
        if mtp and not wm:
            raise ValueError("mtp=True needs the MTP head's weights (a third element of `model`, or `mtp.*` tensors in the snapshot)")
        cfg = self.cfg
        assert isinstance(cfg, Config) or hasattr(cfg, "layer_types")
        self._check_shape(cfg)
        self.KV_BLOCK = _lib.query("KV_BLOCK")
        self.GDN_SLICE = 16                                  # value columns per recurrence task
        self.GDN_TASKS = cfg.lin_heads * cfg.lin_v_dim // self.GDN_SLICE
        self.TASK_CHANNELS = 2 * cfg.lin_k_dim + self.GDN_SLICE
        self.max_seq = (max_seq + self.KV_BLOCK - 1) // self.KV_BLOCK * self.KV_BLOCK
        if batch > 1 and batch * (self.max_seq // self.KV_BLOCK) > 512:
            raise ValueError(f"{batch} sequences of {self.max_seq} positions exceed the 512 KV pages one launch can map")
        self.grid = torch.cuda.get_device_properties(device).multi_processor_count
        self._keep = []   # every tensor whose address the kernel holds

        pack_dev = torch.device(pack_device) if pack_device is not None else None

        def keep(t):
            t = t.to(device).contiguous()
            self._keep.append(t)
            return t.data_ptr()

        def f32(t):
            return keep(t.to(device=device, dtype=torch.float32))

        q8 = quant == "int8"

        slot_bytes = _lib.query("SLOT_BYTES")

        def plain(t):
            """A weight matrix in the kernel's element format, row-major: (tensor, scales or None)."""
            t = t.to(pack_dev if pack_dev is not None else device)
            if q8:
                q, s = quantize_int8_rows(t)
                return (q.to(torch.int16) - 128).to(torch.int8), s      # signed two's complement
            return t.to(torch.bfloat16), None

        def mat(t, unit=1):
            """A GEMV weight in the kernel's tile layout: (address, scale address)."""
            m, s = plain(t)
            packed = pack_rows(as_bytes(m), unit, self.grid, slot_bytes)
            return keep(packed), (keep(s) if s is not None else 0)

        kvt = torch.float32 if kv_dtype == "fp32" else torch.bfloat16
        n_blocks = self.max_seq // self.KV_BLOCK          # pages per sequence; the pool holds `batch` times as many
        ring = _lib.query("CONV_RING")
        zeros = lambda *shape, dtype=torch.float32: torch.zeros(*shape, device=device, dtype=dtype)
        self.conv_hist, self.state, self.state_bak, self.k_cache, self.v_cache = [], [], [], [], []
        self.bconv_hist, self.bstate = [], []             # the same with a leading sequence dimension
        F = _lib.LAYER_FIELDS
        layer_vals = []
        def common(w, m):
            rec = dict.fromkeys(F, 0)
            gu = torch.stack([w[m + "mlp.gate_proj.weight"], w[m + "mlp.up_proj.weight"]], dim=1).reshape(-1, cfg.hidden)
            rec["w_gu"], rec["s_gu"] = mat(gu, unit=2)
            # the single-sequence kernels take the down-projection as column slices (the CTA that produces
            # SwiGLU outputs multiplies them itself); the batched kernel takes row slices like every other matrix
            dm, ds = plain(w[m + "mlp.down_proj.weight"])
            rec["w_down"] = keep(pack_down_cols(dm, self.grid))
            rec["s_down"] = keep(ds) if ds is not None else 0
            if q8:      # run_batch is available on every int8 engine
                rec["w_down_rows"] = keep(pack_rows(as_bytes(dm), 1, self.grid, slot_bytes))
            rec["in_norm"] = f32(w[m + "input_layernorm.weight"])
            rec["post_norm"] = f32(w[m + "post_attention_layernorm.weight"])
            return rec

        def attn_layer(w, m):
            """Pointer record of a gated full-attention decoder layer and its (paged) KV cache."""
            rec = common(w, m)
            p = m + "self_attn."
            w_in = torch.cat([w[p + "q_proj.weight"], w[p + "k_proj.weight"], w[p + "v_proj.weight"]])
            rec["w_in"], rec["s_in"] = mat(w_in)
            rec["w_out"], rec["s_out"] = mat(w[p + "o_proj.weight"])
            rec["q_norm"] = f32(w[p + "q_norm.weight"])
            rec["k_norm"] = f32(w[p + "k_norm.weight"])
            kc = zeros(batch * n_blocks, cfg.n_kv_heads, self.KV_BLOCK, cfg.head_dim, dtype=kvt)
            vc = zeros(batch * n_blocks, cfg.n_kv_heads, self.KV_BLOCK, cfg.head_dim, dtype=kvt)
            rec["k_cache"], rec["v_cache"] = keep(kc), keep(vc)
            rec["kind"] = 1
            return rec, kc, vc

        for i, kind in enumerate(cfg.layer_types):
            m = f"layers.{i}."
            if kind != "linear_attention":
                rec, kc, vc = attn_layer(w, m)
                self.k_cache.append(kc)
                self.v_cache.append(vc)
                layer_vals += [rec[f] for f in F]
                continue
            rec = common(w, m)
            if kind == "linear_attention":
                p = m + "linear_attn."
                w_in = torch.cat([w[p + "in_proj_qkv.weight"], w[p + "in_proj_z.weight"],
                                  w[p + "in_proj_b.weight"], w[p + "in_proj_a.weight"]])
                rec["w_in"], rec["s_in"] = mat(w_in)
                # a recurrence task multiplies its 16 outputs with its column slice of the out-projection
                # itself; the batched kernel takes row slices like every other matrix
                om, osc = plain(w[p + "out_proj.weight"])
                rec["w_out"] = keep(pack_out_cols(om, self.GDN_TASKS, self.GDN_SLICE))
                rec["s_out"] = keep(osc) if osc is not None else 0
                if q8:      # run_batch is available on every int8 engine
                    rec["w_out_rows"] = keep(pack_rows(as_bytes(om), 1, self.grid, slot_bytes))
                rec["conv_w"] = f32(w[p + "conv1d.weight"].reshape(-1, cfg.conv_k))
                rec["A_log"] = f32(w[p + "A_log"])
                rec["dt_bias"] = f32(w[p + "dt_bias"])
                rec["gdn_norm"] = f32(w[p + "norm.weight"])
                hist = zeros(self.GDN_TASKS, self.TASK_CHANNELS, ring)   # per recurrence task (single-sequence launches)
                st = zeros(batch, cfg.lin_heads, cfg.lin_v_dim, cfg.lin_k_dim)   # [head][v][k]: the oracle's transposed
                bak = zeros(cfg.lin_heads, cfg.lin_v_dim, cfg.lin_k_dim)
                self.conv_hist.append(hist)
                self.bstate.append(st)
                self.state.append(st[0])                  # sequence 0 is what the single-sequence launches use
                self.state_bak.append(bak)
                rec["conv_hist"], rec["state"], rec["state_bak"] = keep(hist), keep(st), keep(bak)
                # batched launches keep the history per sequence and head: [q | k | v channels of the head]
                bh = zeros(batch, cfg.lin_heads, 2 * cfg.lin_k_dim + cfg.lin_v_dim, ring)
                self.bconv_hist.append(bh)
                rec["conv_hist_b"] = keep(bh)
                rec["kind"] = 0
            layer_vals += [rec[f] for f in F]

        cos, sin = rope_tables(cfg, self.max_seq, device)
        u64 = dict(device=device, dtype=torch.int64)
        proj_max = max(cfg.gdn_in_rows, cfg.attn_in_rows)
        mix = cfg.n_heads * cfg.head_dim
        # flag-in-data activation buffers: (epoch << 32) | fp32 bits
        T = max(_lib.query("SPEC_T"), batch)   # token slots per hand-off buffer: a speculative cycle's two tokens, or one per sequence
        self.ll = [torch.zeros(n, **u64) for n in (T * cfg.hidden, T * proj_max, T * mix, T * cfg.intermediate,
                                                   (T + 1) * 2 * self.grid, T * cfg.hidden,
                                                   _lib.query("SPEC_T") * self.grid * cfg.hidden)]
        max_splits, part_stride = _lib.query("MAX_SPLITS"), _lib.query("PART_STRIDE")
        self.attn_part = zeros(T * cfg.n_kv_heads * max_splits * part_stride, dtype=torch.int64)
        self.block_table = torch.arange(batch * n_blocks, device=device, dtype=torch.int32)   # [sequence][page]
        self.status = zeros(4, dtype=torch.int32)

        self.embed = w["embed_tokens.weight"].to(device)
        self.final_norm = w["norm.weight"].to(device)
        # lookups read a plain row-major table; the LM head streams the same rows in the tile layout
        table, table_scale = plain(self.embed)
        embed_ptr, embed_scale = keep(table), (keep(table_scale) if table_scale is not None else 0)
        lm_ptr, lm_scale = mat(w["lm_head.weight"] if "lm_head.weight" in w else self.embed)
        g = dict.fromkeys(_lib.GLOBAL_FIELDS, 0)
        g.update(embed=embed_ptr, embed_scale=embed_scale, lm_head=lm_ptr, lm_scale=lm_scale,
                 final_norm=f32(self.final_norm), rope_cos=keep(cos), rope_sin=keep(sin),
                 xl=keep(self.ll[0]), projl=keep(self.ll[1]), mixl=keep(self.ll[2]), actl=keep(self.ll[3]) if quant == "int8" else 0,      # only batched launches (int8 engines) hand activations over in words
                
                 lml=keep(self.ll[4]), attn_part=keep(self.attn_part),
                 block_table=keep(self.block_table), status=keep(self.status))
        g["xml"] = keep(self.ll[5])
        g["partl"] = keep(self.ll[6])
        self.mtp = self.draft_ids = None
        self.draft_vocab = 0
        mtp_vals = None
        if mtp:
            from .mtp import MTP
            rec, mkc, mvc = attn_layer(wm, "layers.0.")
            self.mtp_k_cache, self.mtp_v_cache = mkc, mvc
            mtp_vals = [rec[f] for f in F]
            g["mtp_fc"], g["mtp_fc_scale"] = mat(wm["fc.weight"])
            g["mtp_norm_e"] = f32(wm["pre_fc_norm_embedding.weight"])
            g["mtp_norm_h"] = f32(wm["pre_fc_norm_hidden.weight"])
            g["mtp_norm"] = f32(wm["norm.weight"])
            if 0 < draft_vocab < cfg.vocab:
                if draft_ids is None:
                    raise ValueError("a reduced draft vocabulary needs `draft_ids` (token ids, most frequent first)")
                ranked = torch.as_tensor(draft_ids)[:draft_vocab]
                # ascending ids, so that an argmax tie still goes to the smallest token id
                self.draft_ids = ranked.sort().values.to(device=device, dtype=torch.int32)
                g["draft_head"], g["draft_scale"] = mat(self.embed[self.draft_ids.long()])
                g["draft_ids"] = keep(self.draft_ids)
                self.draft_vocab = len(self.draft_ids)
            else:
                g["draft_head"], g["draft_scale"] = lm_ptr, lm_scale
                self.draft_vocab = cfg.vocab
            # what the kernel's arithmetic sees, for the host-side cache fill
            seen = {k: (roundtrip_int8_rows(v.to(device)) if q8 and is_gemv_weight(k) else v.to(device).float())
                    for k, v in wm.items()}
            table = roundtrip_int8_rows(self.embed) if q8 else self.embed
            self.mtp = MTP(cfg, seen, lambda t: table[t].float(), cos, sin, self._write_mtp_kv)
        del w

        desc = _lib.ModelDesc(shape=_lib.MK_SHAPE_QWEN35_08B, n_layers=cfg.n_layers, vocab=cfg.vocab,
                              max_seq=self.max_seq, quant=_lib.MK_QUANT[quant], kv_dtype=_lib.MK_KV[kv_dtype],
                              draft_vocab=self.draft_vocab, device=device.index, grid=self.grid, max_batch=batch)
        self._h = ctypes.c_void_p()
        _lib.check(self.lib.mk_create(ctypes.byref(desc), ctypes.byref(self._h)))
        self._tables = (list(layer_vals), list(mtp_vals) if mtp_vals else None, dict(g))     # what mk_set_params was given
        lv, gv = _lib.i64_array(layer_vals), _lib.i64_array([g[f] for f in _lib.GLOBAL_FIELDS])
        mv = _lib.i64_array(mtp_vals) if mtp_vals else None
        _lib.check(self.lib.mk_set_params(self._h, lv, len(lv), mv, len(mv) if mv else 0, gv, len(gv)))
        self.weight_bytes = self._weight_bytes()
        self.last_step_ns = []
        self.launches = 0
        self.reset()

    # ------------------------------------------------------------------------------------------
    @staticmethod
    def _check_shape(c):
        want = dict(hidden=1024, intermediate=3584, n_heads=8, n_kv_heads=2, head_dim=256, rotary_dim=64,
                    lin_heads=16, lin_k_dim=128, lin_v_dim=128, conv_k=4)
        bad = {k: getattr(c, k) for k, v in want.items() if getattr(c, k) != v}
        if bad:
            raise ValueError(f"this build only has the 0.8B hybrid shape {want}; got {bad}")
        if abs(c.eps - 1e-6) > 1e-12:
            raise ValueError("rms_norm_eps must be 1e-6")

    @property
    def pos(self):
        """Position of the (first) sequence: the next token goes here."""
        return self.bpos[0]

    @pos.setter
    def pos(self, value):
        self.bpos[0] = value

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            self.lib.mk_destroy(h)
            self._h = None

    def _weight_bytes(self):
        """Bytes of weights streamed per decode step: (layers, LM head)."""
        c = self.cfg
        per = {"linear_attention": c.gdn_in_rows * c.hidden + c.hidden * c.lin_heads * c.lin_v_dim,
               "full_attention": c.attn_in_rows * c.hidden + c.hidden * c.n_heads * c.head_dim}
        mlp = 3 * c.intermediate * c.hidden
        b = 1 if self.quant == "int8" else 2
        return int(sum(per[t] + mlp for t in c.layer_types) * b), int(c.vocab * c.hidden * b)

    def state_bytes(self):
        """Recurrent-state bytes read plus written per decode step."""
        c = self.cfg
        return 2 * 4 * len(self.state) * c.lin_heads * c.lin_k_dim * c.lin_v_dim

    def kv_bytes_per_pos(self):
        c = self.cfg
        return len(self.k_cache) * 2 * c.n_kv_heads * c.head_dim * (4 if self.kv_dtype == "fp32" else 2)

    def reset(self):
        """Start a new sequence (cached K/V need no clearing: positions are rewritten)."""
        for t in self.conv_hist + self.bconv_hist + self.bstate + self.ll:
            t.zero_()
        self._mode = None              # "single" or "batch": the two kinds of launch keep separate conv histories
        self.bpos = [0] * self.batch   # position of every sequence; `pos` is that of sequence 0
        self.attn_part.zero_()
        self.status.zero_()
        self.epoch = 1   # the buffers are zero, so epoch 0 never looks ready
        self.mtp_h = None   # (position, hidden state) whose draft-cache entry still awaits its next token

    def set_block_table(self, table):
        """Map logical KV pages to physical pages (a permutation of range(max_seq / KV_BLOCK))."""
        t = torch.as_tensor(table, dtype=torch.int32, device=self.device)
        if t.shape != self.block_table.shape or sorted(t.flatten().tolist()) != list(range(t.numel())):
            raise ValueError("block table must be a permutation of all pages")
        self.block_table.copy_(t)

    # ------------------------------------------------------------------------------------------
    # One place builds the launch record, submits it and settles the host-side bookkeeping that every kind of
    # single-sequence launch shares (status, epoch); the public methods differ in what they ask for and in how
    # they read the result.
    def _submit(self, n_steps, fields, buffers, timing):
        """Launch `n_steps` steps (or cycles).  `fields`: LaunchArgs members by name; `buffers`: name -> device tensor
        or None, passed by address under the same name.  Returns the launch's info words as a list (reading them
        waits for the kernel)."""
        dev = self.device
        info = torch.zeros(8, dtype=torch.int32, device=dev)
        stamps = torch.zeros(n_steps + 1, dtype=torch.int64, device=dev) if timing else None
        args = dict(n_steps=n_steps, start_pos=self.pos, epoch_base=self.epoch, grid=self.grid,
                    spin_limit_ns=self.spin_limit_ns, out_info=info.data_ptr(), step_ts=stamps.data_ptr() if timing else 0)
        args.update(fields)
        args.update({name: (t.data_ptr() if t is not None else 0) for name, t in buffers.items()})
        record = _lib.LaunchArgs(**args)
        stream = torch.cuda.current_stream(dev).cuda_stream
        _lib.check(self.lib.mk_launch(self._h, ctypes.byref(record), ctypes.c_void_p(stream)))
        self.launches += 1
        words = info.tolist()
        if int(self.status[0]) != 0:                       # a device-side wait ran out: raises with the wait site
            where = ctypes.c_int32()
            _lib.check(self.lib.mk_status(self._h, ctypes.byref(where)))
        self.epoch = words[1] & 0xFFFFFFFF
        if self.epoch > 0xFFFF0000:
            raise RuntimeError("epoch counter exhausted; call reset()")
        if timing:
            n_run = words[5] if fields.get("spec") else words[0]
            t = stamps[: n_run + 1].cpu()
            self.last_step_ns = (t[1:] - t[:-1]).tolist()
        return words

    @staticmethod
    def _sampling(temperature, seed, stop_ids, device):
        """The LaunchArgs members that describe how a token is chosen and which ids end a launch."""
        stops = torch.tensor(list(stop_ids) or [-1], dtype=torch.int32, device=device)
        return dict(seed=seed & 0xFFFFFFFF, inv_temperature=(1.0 / temperature) if temperature > 0 else 0.0,
                    n_stop=len(stop_ids)), stops

    @torch.no_grad()
    def run(self, tokens, n_generate=1, temperature=0.0, seed=0, stop_ids=(), return_logits=False, prof=None,
            prof_step=0, timing=False, all_logits=False, track_mtp=False, return_resid=False):
        """Feed `tokens`, then continue with up to `n_generate` tokens of the model's own choosing, in one launch.

        The contract is the reference's (`qwen_mk/engine.py:198-250`): the given tokens enter one per step; from the
        last of them on, every step's choice is fed to the next step on the GPU; choosing a stop id ends the launch,
        and that id is returned without having been fed.  Result: the chosen ids; with `return_logits` also their
        logits, with `all_logits` the logits behind every fed token instead.
        """
        given = [int(t) for t in tokens]
        if not given:
            raise ValueError("need at least one input token")
        if n_generate < 1:
            raise ValueError("n_generate must be >= 1")
        self._enter_mode("single")
        n_given = len(given)
        n_steps = n_given - 1 + n_generate
        if self.pos + n_steps > self.max_seq:
            raise ValueError(f"sequence would exceed max_seq={self.max_seq}")
        dev, cfg = self.device, self.cfg
        want_hidden = track_mtp or return_resid
        how, stops = self._sampling(temperature, seed, stop_ids, dev)
        bufs = dict(forced=torch.tensor(given, dtype=torch.int32).pin_memory().to(dev, non_blocking=True),
                    stop_ids=stops, tokens_out=torch.zeros(n_steps, dtype=torch.int64, device=dev),
                    logits_out=torch.empty(n_steps, cfg.vocab, device=dev) if (return_logits or all_logits) else None,
                    resid_out=torch.empty(n_steps, cfg.hidden, device=dev) if want_hidden else None, prof=prof)
        first_choice = 0 if all_logits else n_given - 1            # the first step whose LM head runs
        words = self._submit(n_steps, dict(how, n_forced=n_given, lm_from=first_choice, prof_step=prof_step), bufs, timing)
        ran = words[0]
        # tokens_out holds keys (ordered score << 32 | ~id): the low word, complemented, is the id
        chosen = (0xFFFFFFFF - (bufs["tokens_out"][n_given - 1: ran] & 0xFFFFFFFF)).tolist()
        hidden = bufs["resid_out"][:ran] if want_hidden else None
        if ran:
            if track_mtp and self.mtp is not None:
                entered = (given + chosen)[:ran]                   # what positions pos .. pos + ran - 1 were fed
                self.mtp_fed(self.pos, mtp_mod.rmsnorm(hidden, self.final_norm, cfg.eps), entered)
            else:
                self.mtp_h = None                                  # the draft head's cache no longer follows the sequence
        self.pos += ran
        self.last_resid = hidden
        if all_logits:
            return chosen, bufs["logits_out"][:ran]
        if return_logits:
            return chosen, bufs["logits_out"][n_given - 1: ran]
        return chosen

    # ------------------------------------------------------------------------------------------
    @torch.no_grad()
    def run_batch(self, prompts, n_generate=1, temperature=0.0, seed=0, stop_ids=(), return_logits=False,
                  timing=False, prof=None, prof_step=0):
        """Advance `len(prompts)` sequences side by side: feed each its tokens, then let each continue
        for up to `n_generate` predicted tokens.  One launch; every step is one pass over the weights
        for all sequences.  Sequence j continues from `self.bpos[j]`; per sequence the contract is that
        of `run` (a predicted stop id ends that sequence and is reported but not fed; its state has
        absorbed every returned id but the last).  Returns one id list per sequence, plus one logits
        tensor per sequence with `return_logits`.  The batched counterpart in the reference is the
        gfx942 engines' `Engine.step(tok[M])` (`qwen3.8-27b-gfx942/mk/runner.py:202-213`), which takes
        one token per sequence and call; here the whole generation is one launch as in `run`."""
        B = len(prompts)
        if not 1 <= B <= self.batch:
            raise ValueError(f"this engine holds {self.batch} sequences, got {B} prompts")
        prompts = [[int(t) for t in p] for p in prompts]
        if any(not p for p in prompts):
            raise ValueError("every sequence needs at least one input token")
        if n_generate < 1:
            raise ValueError("n_generate must be >= 1")
        self._enter_mode("batch")
        NBW = _lib.MAX_BATCH
        n_forced = [len(p) for p in prompts]
        n_total = [n + n_generate - 1 for n in n_forced]
        n_steps = max(n_total)
        if any(self.bpos[j] + n_steps > self.max_seq for j in range(B)):
            raise ValueError(f"a sequence would exceed max_seq={self.max_seq}")
        dev = self.device
        forced = torch.zeros(max(n_forced), NBW, dtype=torch.int32)
        for j, p in enumerate(prompts):
            forced[: len(p), j] = torch.tensor(p, dtype=torch.int32)
        forced = forced.pin_memory().to(dev, non_blocking=True)
        stops = torch.tensor(list(stop_ids) or [-1], dtype=torch.int32, device=dev)
        out = torch.zeros(n_steps, NBW, dtype=torch.int64, device=dev)
        info = torch.zeros(8, dtype=torch.int32, device=dev)
        ts = torch.zeros(n_steps + 1, dtype=torch.int64, device=dev) if timing else None
        logits = torch.empty(n_steps, NBW, self.cfg.vocab, device=dev) if return_logits else None
        ptr = lambda t: t.data_ptr() if t is not None else 0
        pad = lambda v: (ctypes.c_int32 * NBW)(*(list(v) + [0] * (NBW - len(v))))
        a = _lib.BatchArgs(forced=forced.data_ptr(), n_forced=pad(n_forced), n_total=pad(n_total),
                           pos0=pad(self.bpos[:B]), batch=B, n_steps=n_steps, lm_from=min(n_forced) - 1,
                           epoch_base=self.epoch, seed=seed & 0xFFFFFFFF,
                           inv_temperature=1.0 / temperature if temperature > 0 else 0.0, n_stop=len(stop_ids),
                           prof_step=prof_step, stop_ids=stops.data_ptr(), tokens_out=out.data_ptr(),
                           logits_out=ptr(logits), step_ts=ptr(ts), out_info=info.data_ptr(), prof=ptr(prof),
                           spin_limit_ns=self.spin_limit_ns)
        stream = torch.cuda.current_stream(dev).cuda_stream
        _lib.check(self.lib.mk_launch_batch(self._h, ctypes.byref(a), ctypes.c_void_p(stream)))
        self.launches += 1
        done, epoch, _ = info[:3].tolist()          # synchronises with the launch
        if int(self.status[0]) != 0:
            where = ctypes.c_int32()
            _lib.check(self.lib.mk_status(self._h, ctypes.byref(where)))
        self.epoch = epoch & 0xFFFFFFFF
        if self.epoch > 0xFFFF0000:
            raise RuntimeError("epoch counter exhausted; call reset()")
        if timing:
            t = ts[: done + 1].cpu()
            self.last_step_ns = (t[1:] - t[:-1]).tolist()
        ids_all = (0xFFFFFFFF - (out[:done] & 0xFFFFFFFF)).cpu()
        stop_set = set(int(s) for s in stop_ids)
        result, result_logits = [], []
        for j in range(B):
            first, last = n_forced[j] - 1, min(done, n_total[j])
            ids = ids_all[first:last, j].tolist()
            for i, t in enumerate(ids):
                if t in stop_set:
                    ids = ids[: i + 1]
                    last = first + i + 1
                    break
            self.bpos[j] += last
            result.append(ids)
            if return_logits:
                result_logits.append(logits[first:last, j])
        self.mtp_h = None
        return (result, result_logits) if return_logits else result

    def _enter_mode(self, mode):
        """Single-sequence and batched launches keep their conv histories in different layouts, so a
        sequence cannot move between them: `reset()` in between."""
        if self._mode not in (None, mode):
            raise RuntimeError(f"this engine has {self._mode} state; call reset() before a {mode} launch")
        self._mode = mode

    def prof_buffer(self):
        """Zeroed timestamp buffer for `run(prof=...)`: [grid, PROF_MAX_OPS, PROF_FIELDS] GPU nanoseconds
        (op entered, inputs staged, work done, outputs published), as `qwen_mk/engine.py:303-305`."""
        return torch.zeros(self.grid, _lib.query("PROF_MAX_OPS"), _lib.query("PROF_FIELDS"), dtype=torch.int64,
                           device=self.device)

    def prefill(self, tokens, chunk=512):
        """Take a prompt in: everything but its last token goes through the kernel (in launches of `chunk` steps,
        keeping the draft head's cache in step); the last token is handed back for the caller to feed with the
        first generation launch, as the reference's `prefill` does (`qwen_mk/engine.py:296-301`)."""
        *body, tail = list(tokens)
        for lo in range(0, len(body), chunk):
            self.run(body[lo: lo + chunk], track_mtp=True)
        return tail

    # ---- the draft head's KV cache outside speculative cycles -------------------------------------------------
    # Entry i of that cache is computed from the model's final hidden state at position i AND the token that
    # entered position i + 1 (`qwen_mk/mtp.py:55-82`), so it trails the sequence by one token.  `mtp_h` holds
    # the one entry that is still waiting for its successor: (position, its hidden state), or None.
    def mtp_fed(self, start, hidden, tokens):
        """`tokens` entered positions start, start + 1, ... and left the final hidden states `hidden` (one row per
        token).  Completes the waiting entry with tokens[0], writes the entries that are now complete, and leaves
        the last position waiting."""
        n = len(tokens)
        if self.mtp is None or n == 0:
            return
        ids = torch.as_tensor(tokens, device=self.device)
        self._mtp_close(start, ids[0])
        if n > 1:
            self.mtp.fill_kv(hidden[: n - 1], ids[1:], start)
        self.mtp_h = (start + n - 1, hidden[n - 1: n])

    def _mtp_close(self, pos, token):
        """`token` is about to enter position `pos`.  If the waiting entry is the one just before, it is complete
        now; any other waiting entry belongs to a sequence that has moved on and is dropped."""
        waiting, self.mtp_h = self.mtp_h, None
        if waiting is not None and waiting[0] + 1 == pos:
            self.mtp.fill_kv(waiting[1], torch.as_tensor([token], device=self.device), waiting[0])

    def _write_mtp_kv(self, pos, k, v):
        bt = self.block_table.long()
        blk, off = bt[pos // self.KV_BLOCK], pos % self.KV_BLOCK
        self.mtp_k_cache[blk, :, off] = k.to(self.mtp_k_cache.dtype)
        self.mtp_v_cache[blk, :, off] = v.to(self.mtp_v_cache.dtype)

    @torch.no_grad()
    def run_spec(self, token, draft, n_generate, temperature=0.0, seed=0, stop_ids=(), timing=False,
                 return_logits=False, prof=None, prof_step=0):
        """Speculative decoding in one launch: up to `n_generate` cycles, each a single pass over the weights that
        takes the pending `token` (at `self.pos`) together with a guess `draft` for its successor.

        Returns `(ids, next_draft)`.  `ids` are exactly the ids `run([token], n_generate)` would return (at most
        `n_generate`, cut after a stop id); the state has taken in all of them but the last, which is the new pending
        token, and `next_draft` is the draft head's guess for what follows it.  A wrong `draft` is never an error: it
        costs the cycle it was offered in.  `self.last_cycles` lists (ids emitted, draft offered) per cycle.  The
        contract of the reference's `run_spec` (`qwen_mk/engine.py:252-294`).
        """
        if self.mtp is None:
            raise RuntimeError("construct the engine with mtp=True for speculative decoding")
        self._enter_mode("single")
        cycles = min(n_generate, MAX_STEPS_PER_LAUNCH)
        if self.pos + 2 * cycles + 1 > self.max_seq:
            raise ValueError(f"sequence would exceed max_seq={self.max_seq}")
        self._mtp_close(self.pos, token)
        dev = self.device
        how, stops = self._sampling(temperature, seed, stop_ids, dev)
        bufs = dict(stop_ids=stops, spec_out=torch.zeros(n_generate, dtype=torch.int32, device=dev),
                    cycle_out=torch.zeros(2 * cycles, dtype=torch.int32, device=dev),
                    logits_out=torch.empty(cycles, 2, self.cfg.vocab, device=dev) if return_logits else None, prof=prof)
        words = self._submit(cycles, dict(how, forced=0, n_forced=0, lm_from=0, tokens_out=0, spec=1, first_tok=int(token),
                                          first_draft=int(draft), limit=n_generate, prof_step=prof_step), bufs, timing)
        emitted, _, self.pos, pending, next_draft, cycles_run = words[:6]
        self.last_cycles = bufs["cycle_out"][: 2 * cycles_run].view(-1, 2).tolist()
        ids = bufs["spec_out"][:emitted].tolist()
        assert ids[-1] == pending
        if return_logits:
            self.last_logits = bufs["logits_out"][:cycles_run]
        return ids, next_draft

    def generate(self, prompt_ids, max_new_tokens=256, temperature=0.0, seed=0, stop_ids=(), chunk=16, spec=False):
        """Generator over the ids the model produces after `prompt_ids` (`qwen_mk/engine.py:307-327`).  The engine's
        state stops right behind the last token it was fed, and `self.pending` keeps the one produced id that has not
        been fed yet, so a conversation continues by passing the next prompt."""
        pending = self.prefill(prompt_ids)
        guess = pending            # the first cycle has no draft yet: whatever is offered can only cost that cycle
        left = max_new_tokens
        while left > 0:
            budget = min(chunk, left, MAX_STEPS_PER_LAUNCH)
            if spec:
                batch, guess = self.run_spec(pending, guess, budget, temperature=temperature, seed=seed, stop_ids=stop_ids)
            else:
                batch = self.run([pending], n_generate=budget, temperature=temperature, seed=seed, stop_ids=stop_ids)
            yield from batch
            left -= len(batch)
            if not batch or batch[-1] in stop_ids:
                return
            pending = batch[-1]
        self.pending = pending

    # ---- state access in the oracle's layouts (for tests, snapshots and state import) -----------
    def deltanet_state(self, i, seq=0):
        """Recurrent state of the i-th DeltaNet layer of sequence `seq` as [head][k][v] (the reference
        decoder's layout, `qwen_mk/reference.py:54`; the kernel stores [head][v][k])."""
        return self.bstate[i][seq].transpose(1, 2).contiguous()

    def conv_window(self, i, seq=0):
        """Last three conv inputs of the i-th DeltaNet layer as [conv_dim, 3], oldest first (the
        reference decoder's `conv_hist`, `qwen_mk/reference.py:53,70-71`)."""
        c, ring = self.cfg, self.conv_hist[i].shape[-1]
        slots = [(self.bpos[seq] - 3 + j) % ring for j in range(3)]
        if self._mode == "batch":
            h = self.bconv_hist[i][seq][:, :, slots]             # [head, q | k | v channel, 3]
            return torch.cat([h[:, : c.lin_k_dim].reshape(-1, 3), h[:, c.lin_k_dim: 2 * c.lin_k_dim].reshape(-1, 3),
                              h[:, 2 * c.lin_k_dim:].reshape(-1, 3)])
        h = self.conv_hist[i][:, :, slots]                       # [task, channel, 3]
        spt = c.lin_v_dim // self.GDN_SLICE                     # tasks per head
        out = torch.empty(c.conv_dim, 3, device=self.device)
        nqk = c.lin_heads * c.lin_k_dim
        first = h[::spt]                                        # the head's first task holds its q and k
        out[:nqk] = first[:, : c.lin_k_dim].reshape(nqk, 3)
        out[nqk: 2 * nqk] = first[:, c.lin_k_dim: 2 * c.lin_k_dim].reshape(nqk, 3)
        out[2 * nqk:] = h[:, 2 * c.lin_k_dim:].reshape(c.lin_heads * c.lin_v_dim, 3)
        return out

    def kv_rows(self, i, n, seq=0):
        """K, V of the i-th attention layer for positions [0, n) of sequence `seq` as [kv_head, n, head_dim] fp32."""
        bt = self.block_table.long().view(self.batch, -1)[seq]
        pos = torch.arange(n, device=self.device)
        blk, off = bt[pos // self.KV_BLOCK], pos % self.KV_BLOCK
        k = self.k_cache[i][blk, :, off].transpose(0, 1).float()
        v = self.v_cache[i][blk, :, off].transpose(0, 1).float()
        return k, v

    # ---- state import: the inverse accessors (a batched prefill computed elsewhere hands its state over) ----
    def set_conv_window(self, i, window, n_tokens):
        """`window` [conv_dim, W]: the last W conv inputs (positions n_tokens - W .. n_tokens - 1) of DeltaNet layer i,
        channels in the reference decoder's order (q | k | v).  Writes them into the single-sequence history."""
        c, ring = self.cfg, self.conv_hist[i].shape[-1]
        spt = c.lin_v_dim // self.GDN_SLICE
        nqk = c.lin_heads * c.lin_k_dim
        window = window.to(self.device, torch.float32)
        for j in range(window.shape[1]):
            p = n_tokens - window.shape[1] + j
            if p < 0:
                continue
            col = window[:, j]
            q = col[:nqk].reshape(c.lin_heads, 1, c.lin_k_dim).expand(-1, spt, -1).reshape(-1, c.lin_k_dim)
            k = col[nqk: 2 * nqk].reshape(c.lin_heads, 1, c.lin_k_dim).expand(-1, spt, -1).reshape(-1, c.lin_k_dim)
            v = col[2 * nqk:].reshape(c.lin_heads * spt, self.GDN_SLICE)
            self.conv_hist[i][:, :, p % ring] = torch.cat([q, k, v], dim=1).to(self.conv_hist[i].dtype)   # every task keeps its head's q and k

    def set_deltanet_state(self, i, state):
        """`state` [head][k][v] (the reference decoder's layout) -> the kernel's [head][v][k]."""
        self.bstate[i][0].copy_(state.to(self.device).transpose(1, 2))

    def write_kv(self, i, start, k, v, seq=0):
        """Store K, V [kv_head, n, head_dim] of attention layer i at positions start .. start + n - 1 of the paged cache."""
        bt = self.block_table.long().view(self.batch, -1)[seq]
        pos = torch.arange(start, start + k.shape[1], device=self.device)
        blk, off = bt[pos // self.KV_BLOCK], pos % self.KV_BLOCK
        self.k_cache[i][blk, :, off] = k.to(self.device).transpose(0, 1).to(self.k_cache[i].dtype)
        self.v_cache[i][blk, :, off] = v.to(self.device).transpose(0, 1).to(self.v_cache[i].dtype)

    def snapshot(self):
        """Copy of the recurrent state (conv histories + DeltaNet state of every sequence) and the positions."""
        return [t.clone() for t in self.conv_hist + self.bconv_hist + self.bstate], list(self.bpos), self._mode

    def restore(self, snap):
        tensors, pos, mode = snap
        for dst, src in zip(self.conv_hist + self.bconv_hist + self.bstate, tensors):
            dst.copy_(src)
        self.bpos = list(pos)
        self._mode = mode
