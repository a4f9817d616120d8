"""CPU oracle of one decode step of the 27B dense hybrid.  TEST INFRASTRUCTURE ONLY.

Only `tests/`, `__graft_entry__.smoke()` and `bench.py`'s CPU-baseline legs may import this module; the
product package never does.  It restates, in PyTorch, the exact-mode decoder the reference uses as its own
correctness oracle, `qwen3.8-27b-gfx942/mk/reference.py` (`step(..., emulate=False)`), with the model's
widths as parameters (the reference fixes them as module constants, `mk/dims.py:3-31`):

* `rms0`        follows `reference.py:157-160`   RMSNorm in fp32 with weights as offsets from 1
* `lin`         follows `reference.py:190-197`   GEMV input rounded to bf16, fp32 accumulation
* `rope`        follows `reference.py:226-239`   angles in fp64, half-split rotation of the first 64 dims
* `State`       follows `reference.py:242-273`   conv history (bf16 values), SSM state fp32 [v][k], bf16 KV
* `gdn`         follows `reference.py:276-311`   conv1d + SiLU, l2norm as x / sqrt(sum x^2 + 1e-6), delta rule,
                                                 gated per-head RMSNorm with a plain weight
* `attn`        follows `reference.py:314-336`   per-head q / k norm, RoPE, q in bf16, softmax(q K^T / 16) V, sigmoid gate
* `step`        follows `reference.py:339-375`   residual stream fp32, SwiGLU MLP, bf16 LM head

Parity pin: `tests/test_oracle27b_pin.py` runs this file against the reference's own `mk.reference.step`
(imported from the reference checkout when it is present) at the full 27B widths and truncated depth, and
against `tests/golden/qwen27b_*.json` (written by `tests/golden/make_golden_27b.py` from the reference)
everywhere else.
"""

import torch
import torch.nn.functional as F

DK = DV = 128
HD = 256
ROT = 64


def rms0(x, w, eps):
    r = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return x * r * (1.0 + w.float())


def lin(x, w):
    return x.to(torch.bfloat16).float() @ w.float().t()


def rope_cos_sin(theta, pos):
    inv = theta ** (-torch.arange(0, ROT, 2, dtype=torch.float64, device=pos.device) / ROT)
    ang = pos.double()[:, None] * inv[None, :]
    ang = torch.cat([ang, ang], -1)
    return ang.cos().float(), ang.sin().float()


def rope(x, cos, sin):
    xr, xp = x[..., :ROT], x[..., ROT:]
    rot = torch.cat([-xr[..., ROT // 2:], xr[..., : ROT // 2]], -1)
    return torch.cat([xr * cos[:, None, :] + rot * sin[:, None, :], xp], -1)


class State:
    """Caches of M sequences."""

    def __init__(self, shape, M, maxlen, layers=None, device="cpu"):
        s = shape
        layers = layers if layers is not None else s.layers
        n_att = sum(s.is_attn(i) for i in range(layers))
        n_gdn = layers - n_att
        z = lambda *sh, dt=torch.float32: torch.zeros(*sh, dtype=dt, device=device)
        self.conv = z(n_gdn, M, s.conv_dim, 3)
        self.ssm = z(n_gdn, M, s.nvh, DV, DK)
        self.k = z(n_att, M, s.nkv, maxlen, HD, dt=torch.bfloat16)
        self.v = z(n_att, M, s.nkv, maxlen, HD, dt=torch.bfloat16)
        self.pos = torch.zeros(M, dtype=torch.long, device=device)


def gdn(s, W, i, x, st, gi, trace=None):
    M = x.shape[0]
    p = "linear_attn."
    qkv = lin(x, W.L(i, p + "in_proj_qkv.weight"))
    z = lin(x, W.L(i, p + "in_proj_z.weight"))
    b = lin(x, W.L(i, p + "in_proj_b.weight"))
    a = lin(x, W.L(i, p + "in_proj_a.weight"))
    taps = W.L(i, p + "conv1d.weight").float()[:, 0, :]
    window = torch.cat([st.conv[gi], qkv[:, :, None]], -1)
    st.conv[gi] = window[:, :, 1:].to(torch.bfloat16).float()
    y = (window * taps[None]).sum(-1)
    y = y * torch.sigmoid(y)
    q = y[:, : s.key_dim].reshape(M, s.nkh, DK)
    k = y[:, s.key_dim: 2 * s.key_dim].reshape(M, s.nkh, DK)
    v = y[:, 2 * s.key_dim:].reshape(M, s.nvh, DV)
    q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * DK ** -0.5
    k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    rep = s.nvh // s.nkh
    q, k = q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1)
    beta = torch.sigmoid(b)
    g = -torch.exp(W.L(i, p + "A_log").float())[None] * F.softplus(a + W.L(i, p + "dt_bias").float()[None])
    S = st.ssm[gi] * torch.exp(g)[:, :, None, None]
    kv = torch.einsum("mhvk,mhk->mhv", S, k)
    S = S + ((v - kv) * beta[:, :, None])[:, :, :, None] * k[:, :, None, :]
    st.ssm[gi] = S
    o = torch.einsum("mhvk,mhk->mhv", S, q)
    o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + s.eps) * W.L(i, p + "norm.weight").float()
    zz = z.reshape(M, s.nvh, DV)
    o = o * (zz * torch.sigmoid(zz))
    if trace is not None:
        trace.update(y=torch.cat([qkv, z, b, a], -1), y2=o.reshape(M, s.val_dim))
    return lin(o.reshape(M, s.val_dim), W.L(i, p + "out_proj.weight"))


def attn(s, W, i, x, st, ai, trace=None):
    M = x.shape[0]
    p = "self_attn."
    qg = lin(x, W.L(i, p + "q_proj.weight")).reshape(M, s.nq, 2 * HD)
    q, gate = qg[..., :HD], qg[..., HD:].reshape(M, s.nq * HD)
    k = lin(x, W.L(i, p + "k_proj.weight")).reshape(M, s.nkv, HD)
    v = lin(x, W.L(i, p + "v_proj.weight")).reshape(M, s.nkv, HD)
    q, k = rms0(q, W.L(i, p + "q_norm.weight"), s.eps), rms0(k, W.L(i, p + "k_norm.weight"), s.eps)
    cos, sin = rope_cos_sin(s.theta, st.pos)
    q, k = rope(q, cos, sin), rope(k, cos, sin)
    q = q.to(torch.bfloat16).float()
    out = torch.empty(M, s.nq, HD, device=x.device)
    for m in range(M):
        n = int(st.pos[m])
        st.k[ai, m, :, n] = k[m].to(torch.bfloat16)
        st.v[ai, m, :, n] = v[m].to(torch.bfloat16)
        K, V = st.k[ai, m, :, : n + 1].float(), st.v[ai, m, :, : n + 1].float()
        qh = q[m].reshape(s.nkv, s.nq // s.nkv, HD)
        sc = torch.einsum("gqd,gld->gql", qh, K) * HD ** -0.5
        out[m] = torch.einsum("gql,gld->gqd", torch.softmax(sc, -1), V).reshape(s.nq, HD)
    if trace is not None:
        trace.update(y=torch.cat([qg.reshape(M, -1), lin(x, W.L(i, p + "k_proj.weight")), v.reshape(M, -1)], -1),
                     y2=out.reshape(M, s.nq * HD) * torch.sigmoid(gate))
    return lin(out.reshape(M, s.nq * HD) * torch.sigmoid(gate), W.L(i, p + "o_proj.weight"))


@torch.no_grad()
def step(s, W, tok, st, layers=None, dump=None, lm_head=True, trace=None):
    """One decode step for M rows: tok [M] int64 -> fp32 logits [M, vocab]; advances st.pos."""
    layers = layers if layers is not None else s.layers
    assert trace is None or isinstance(trace, list)
    h = W["model.language_model.embed_tokens.weight"][tok].float()
    gi = ai = 0
    for i in range(layers):
        tr = {} if trace is not None else None
        x = rms0(h, W.L(i, "input_layernorm.weight"), s.eps)
        if s.is_attn(i):
            h = h + attn(s, W, i, x, st, ai, tr)
            ai += 1
        else:
            h = h + gdn(s, W, i, x, st, gi, tr)
            gi += 1
        x = rms0(h, W.L(i, "post_attention_layernorm.weight"), s.eps)
        gt, up = lin(x, W.L(i, "mlp.gate_proj.weight")), lin(x, W.L(i, "mlp.up_proj.weight"))
        if trace is not None:
            tr.update(h1=h.clone(), act=gt * torch.sigmoid(gt) * up)
        h = h + lin(gt * torch.sigmoid(gt) * up, W.L(i, "mlp.down_proj.weight"))
        if trace is not None:
            tr["h0"] = h.clone()
            trace.append(tr)
        if dump is not None:
            dump[i] = h.clone()
    st.pos += 1
    if not lm_head:
        return h
    x = rms0(h, W["model.language_model.norm.weight"], s.eps)
    return x.to(torch.bfloat16).float() @ W["lm_head.weight"].float().t()
