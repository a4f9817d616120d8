"""CPU oracle for the decode hot path.  TEST INFRASTRUCTURE ONLY.

Only `tests/`, `__graft_entry__.smoke()` and `bench.py`'s CPU-baseline legs may import this
module; the product package never does.  It restates, in fp32 PyTorch on the CPU, the
token-by-token decoder the reference uses as its own correctness oracle:

* `Decoder`        follows `qwen3.5-0.8b/qwen_mk/reference.py:33-127` (`ReferenceModel`)
* `rms_norm`       follows `reference.py:12-15`      (weights are offsets from 1)
* `rope_angles`    follows `reference.py:18-23`
* `rotate_partial` follows `reference.py:26-30`      (half-split rotation of the first dims)
* `MtpHead`        follows `qwen3.5-0.8b/qwen_mk/mtp.py:39-105`
* `sample_key` / `pick_token` restate the kernel-side sampling rule the reference documents at
  `csrc/megakernel.cu:101-114,1120-1129`: greedy = highest logit, ties to the lowest id;
  temperature > 0 = Gumbel-max with noise keyed on (seed, position, token id).  The hash that
  produces the noise is this library's own (`mix32` below); the reference's tests only require
  that sampling be a pure function of the seed (`tests/test_correctness.py:89-97`).

Parity pin: `tests/test_oracle_pin.py` runs this file against the reference's own
`ReferenceModel` / `MTP` classes imported from the reference checkout when it is present, and
against the fixtures under `tests/golden/` (written by `tests/golden/make_golden.py` from the
reference's classes) everywhere else.
"""

import math

import torch
import torch.nn.functional as F


def rms_norm(x, w, eps):
    x = x.float()
    inv = torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return x * inv * (w.float() + 1.0)


def rope_angles(cfg, max_seq):
    """cos, sin tables [max_seq, rotary_dim/2] in fp32."""
    idx = torch.arange(0, cfg.rotary_dim, 2, dtype=torch.int64).float()
    inv_freq = 1.0 / (cfg.rope_theta ** (idx / cfg.rotary_dim))
    ang = torch.arange(max_seq, dtype=torch.float32)[:, None] * inv_freq[None, :]
    return ang.cos(), ang.sin()


def rotate_partial(x, cos, sin, rotary_dim):
    h = rotary_dim // 2
    a, b = x[..., :h], x[..., h:rotary_dim]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., rotary_dim:]], dim=-1)


class Decoder:
    """fp32 token-by-token decoder with explicit conv / recurrent / KV state.

    `kv_dtype=torch.bfloat16` rounds cached K and V to bf16 (what the kernel's cache holds);
    the default keeps them in fp32 exactly as the reference's decoder does.
    """

    def __init__(self, cfg, weights, max_seq=4096, kv_dtype=None):
        self.cfg = cfg
        self.max_seq = max_seq
        self.kv_dtype = kv_dtype
        self.w = {k: v.detach().to("cpu", torch.float32) for k, v in weights.items()}
        self.cos, self.sin = rope_angles(cfg, max_seq)
        self.reset()

    def reset(self):
        c = self.cfg
        self.pos = 0
        self.conv_hist, self.state, self.k_cache, self.v_cache = {}, {}, {}, {}
        for i, kind in enumerate(c.layer_types):
            if kind == "linear_attention":
                self.conv_hist[i] = torch.zeros(c.conv_dim, c.conv_k - 1)
                self.state[i] = torch.zeros(c.lin_heads, c.lin_k_dim, c.lin_v_dim)  # [head][k][v]
            else:
                self.k_cache[i] = torch.zeros(c.n_kv_heads, self.max_seq, c.head_dim)
                self.v_cache[i] = torch.zeros(c.n_kv_heads, self.max_seq, c.head_dim)

    # -- mixers ------------------------------------------------------------------------------
    def _deltanet(self, i, h):
        c, w = self.cfg, self.w
        p = f"layers.{i}.linear_attn."
        nh, dk, dv = c.lin_heads, c.lin_k_dim, c.lin_v_dim
        mixed = w[p + "in_proj_qkv.weight"] @ h
        z = (w[p + "in_proj_z.weight"] @ h).view(nh, dv)
        b = w[p + "in_proj_b.weight"] @ h
        a = w[p + "in_proj_a.weight"] @ h
        window = torch.cat([self.conv_hist[i], mixed[:, None]], dim=1)          # [C, conv_k]
        self.conv_hist[i] = window[:, 1:].clone()
        taps = w[p + "conv1d.weight"][:, 0, :]
        act = F.silu((window * taps).sum(dim=1))
        q, k, v = act.split([nh * dk, nh * dk, nh * dv])
        q = F.normalize(q.view(nh, dk), dim=-1, eps=1e-6) * dk ** -0.5            # x / max(|x|, eps)
        k = F.normalize(k.view(nh, dk), dim=-1, eps=1e-6)
        v = v.view(nh, dv)
        beta = torch.sigmoid(b)
        log_decay = -torch.exp(w[p + "A_log"]) * F.softplus(a + w[p + "dt_bias"])
        S = self.state[i] * torch.exp(log_decay)[:, None, None]
        recalled = torch.einsum("hkv,hk->hv", S, k)
        delta = (v - recalled) * beta[:, None]
        S = S + k[:, :, None] * delta[:, None, :]
        self.state[i] = S
        o = torch.einsum("hkv,hk->hv", S, q)
        o = o * torch.rsqrt((o * o).mean(dim=-1, keepdim=True) + c.eps) * w[p + "norm.weight"] * F.silu(z)
        return w[p + "out_proj.weight"] @ o.reshape(-1)

    def _attention(self, i, h):
        c, w = self.cfg, self.w
        p = f"layers.{i}.self_attn."
        nq, nkv, d = c.n_heads, c.n_kv_heads, c.head_dim
        qg = (w[p + "q_proj.weight"] @ h).view(nq, 2 * d)
        q, gate = qg[:, :d], qg[:, d:]
        k = (w[p + "k_proj.weight"] @ h).view(nkv, d)
        v = (w[p + "v_proj.weight"] @ h).view(nkv, d)
        q = rms_norm(q, w[p + "q_norm.weight"], c.eps)
        k = rms_norm(k, w[p + "k_norm.weight"], c.eps)
        cs, sn = self.cos[self.pos], self.sin[self.pos]
        q = rotate_partial(q, cs, sn, c.rotary_dim)
        k = rotate_partial(k, cs, sn, c.rotary_dim)
        if self.kv_dtype is not None:
            k, v = k.to(self.kv_dtype).float(), v.to(self.kv_dtype).float()
        self.k_cache[i][:, self.pos] = k
        self.v_cache[i][:, self.pos] = v
        n = self.pos + 1
        rep = nq // nkv
        K = self.k_cache[i][:, :n].repeat_interleave(rep, dim=0)
        V = self.v_cache[i][:, :n].repeat_interleave(rep, dim=0)
        prob = (torch.einsum("hd,htd->ht", q, K) * d ** -0.5).softmax(dim=-1)
        o = torch.einsum("ht,htd->hd", prob, V) * torch.sigmoid(gate)
        return w[p + "o_proj.weight"] @ o.reshape(-1)

    # -- one token ---------------------------------------------------------------------------
    @torch.no_grad()
    def hidden_step(self, token):
        """Feed one token; return the residual stream after the last layer (before the final norm)."""
        c, w = self.cfg, self.w
        x = w["embed_tokens.weight"][token].clone()
        for i, kind in enumerate(c.layer_types):
            h = rms_norm(x, w[f"layers.{i}.input_layernorm.weight"], c.eps)
            x = x + (self._deltanet(i, h) if kind == "linear_attention" else self._attention(i, h))
            h = rms_norm(x, w[f"layers.{i}.post_attention_layernorm.weight"], c.eps)
            m = f"layers.{i}.mlp."
            x = x + w[m + "down_proj.weight"] @ (F.silu(w[m + "gate_proj.weight"] @ h) * (w[m + "up_proj.weight"] @ h))
        self.pos += 1
        return x

    @torch.no_grad()
    def step(self, token):
        """Feed one token; return fp32 logits [vocab] for the next position."""
        x = self.hidden_step(token)
        self.last_hidden = rms_norm(x, self.w["norm.weight"], self.cfg.eps)
        head = self.w.get("lm_head.weight", self.w["embed_tokens.weight"])
        return head @ self.last_hidden


# ---------------------------------------------------------------------------------------------
# sampling
def mix32(a, b, c):
    """32-bit hash of three 32-bit words (numpy-free, exact integer arithmetic on Python ints
    or int64 tensors).  Matches `mk_mix32` in `megakernels_b200/csrc/mk_device.cuh`."""
    M = 0xFFFFFFFF
    h = (a * 0x9E3779B9 + 0x7F4A7C15) & M
    h ^= (b * 0x85EBCA6B + 0x165667B1) & M
    h = (h ^ (h >> 15)) * 0x2C1B3C6D & M
    h ^= (c * 0xC2B2AE35 + 0x27D4EB2F) & M
    h = (h ^ (h >> 13)) * 0x297A2D39 & M
    h = (h ^ (h >> 16)) * 0x7FEB352D & M
    h = (h ^ (h >> 15)) * 0x846CA68B & M
    return (h ^ (h >> 16)) & M


def sample_key(logits, inv_temperature, seed, pos):
    """Per-token score whose argmax is the sampled token (fp32 tensor [vocab])."""
    if inv_temperature == 0.0:
        return logits.float()
    ids = torch.arange(logits.numel(), dtype=torch.int64)
    h = mix32(ids * 0 + (seed & 0xFFFFFFFF), ids * 0 + (pos & 0xFFFFFFFF), ids)
    u = ((h >> 8).float() + 0.5) * (1.0 / 16777216.0)
    return logits.float() * inv_temperature - torch.log(-torch.log(u))


def pick_token(logits, inv_temperature=0.0, seed=0, pos=0):
    """Highest key; ties go to the lowest id (`torch.argmax` does not promise that)."""
    key = sample_key(logits, inv_temperature, seed, pos)
    return int((key == key.max()).nonzero()[0, 0])


def greedy_run(dec, prompt, n_generate, stop_ids=()):
    """Feed `prompt`, then generate greedily.  Returns (ids, logits[len(ids), vocab]); a stop id is
    reported but not fed, like the kernel's run loop (`qwen_mk/engine.py:198-250`)."""
    lg = None
    for t in prompt:
        lg = dec.step(t)
    ids, logits = [], []
    for _ in range(n_generate):
        nxt = pick_token(lg)
        ids.append(nxt)
        logits.append(lg)
        if nxt in stop_ids or len(ids) == n_generate:
            break
        lg = dec.step(nxt)
    return ids, torch.stack(logits)


# ---------------------------------------------------------------------------------------------
class MtpHead:
    """Multi-token-prediction draft head: fuse [norm(embed(x_{i+1})), norm(h_i)] -> hidden, run one
    gated-attention decoder layer over its own KV cache (bf16, like the kernel's), final norm,
    tied LM head.  `forward` is batched over consecutive positions."""

    def __init__(self, cfg, w, embed, max_seq):
        self.cfg, self.max_seq = cfg, max_seq
        self.w = {k: v.detach().to("cpu", torch.float32) for k, v in w.items()}
        self.embed = embed.detach().to("cpu", torch.float32)
        self.cos, self.sin = rope_angles(cfg, max_seq)
        self.k_cache = torch.zeros(cfg.n_kv_heads, max_seq, cfg.head_dim, dtype=torch.bfloat16)
        self.v_cache = torch.zeros_like(self.k_cache)

    def fuse(self, h, next_tokens):
        c, w = self.cfg, self.w
        e = rms_norm(self.embed[next_tokens], w["pre_fc_norm_embedding.weight"], c.eps)
        g = rms_norm(h.float(), w["pre_fc_norm_hidden.weight"], c.eps)
        return torch.cat([e, g], dim=-1) @ w["fc.weight"].t()

    def _qkv(self, u, positions):
        c, w, p = self.cfg, self.w, "layers.0.self_attn."
        n, d = u.shape[0], c.head_dim
        x = rms_norm(u, w["layers.0.input_layernorm.weight"], c.eps)
        qg = (x @ w[p + "q_proj.weight"].t()).view(n, c.n_heads, 2 * d)
        q, gate = qg[..., :d], qg[..., d:]
        k = (x @ w[p + "k_proj.weight"].t()).view(n, c.n_kv_heads, d)
        v = (x @ w[p + "v_proj.weight"].t()).view(n, c.n_kv_heads, d)
        q = rms_norm(q, w[p + "q_norm.weight"], c.eps)
        k = rms_norm(k, w[p + "k_norm.weight"], c.eps)
        cs, sn = self.cos[positions][:, None], self.sin[positions][:, None]
        return rotate_partial(q, cs, sn, c.rotary_dim), rotate_partial(k, cs, sn, c.rotary_dim), v, gate

    @torch.no_grad()
    def fill_kv(self, h, next_tokens, start):
        pos = torch.arange(start, start + h.shape[0])
        _, k, v, _ = self._qkv(self.fuse(h, next_tokens), pos)
        self.k_cache[:, pos] = k.transpose(0, 1).to(torch.bfloat16)
        self.v_cache[:, pos] = v.transpose(0, 1).to(torch.bfloat16)

    @torch.no_grad()
    def forward(self, h, next_tokens, start):
        c, w, p = self.cfg, self.w, "layers.0.self_attn."
        n = h.shape[0]
        pos = torch.arange(start, start + n)
        u = self.fuse(h, next_tokens)
        q, k, v, gate = self._qkv(u, pos)
        self.k_cache[:, pos] = k.transpose(0, 1).to(torch.bfloat16)
        self.v_cache[:, pos] = v.transpose(0, 1).to(torch.bfloat16)
        T = start + n
        rep = c.n_heads // c.n_kv_heads
        K = self.k_cache[:, :T].float().repeat_interleave(rep, dim=0)
        V = self.v_cache[:, :T].float().repeat_interleave(rep, dim=0)
        s = torch.einsum("nhd,htd->nht", q, K) * c.head_dim ** -0.5
        future = torch.arange(T)[None, :] > pos[:, None]
        s = s.masked_fill(future[:, None, :], -math.inf)
        o = torch.einsum("nht,htd->nhd", s.softmax(dim=-1), V) * torch.sigmoid(gate)
        u = u + o.reshape(n, -1) @ w[p + "o_proj.weight"].t()
        x = rms_norm(u, w["layers.0.post_attention_layernorm.weight"], c.eps)
        m = "layers.0.mlp."
        u = u + (F.silu(x @ w[m + "gate_proj.weight"].t()) * (x @ w[m + "up_proj.weight"].t())) @ w[m + "down_proj.weight"].t()
        return rms_norm(u, w["norm.weight"], c.eps) @ self.embed.t()
