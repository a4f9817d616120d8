"""CPU oracle of one decode step of the 35B-A3B MoE hybrid.  TEST INFRASTRUCTURE ONLY.

Only `tests/`, `__graft_entry__.smoke()` and `bench.py`'s CPU-baseline legs may import this module; the
product package never does.  It restates, in PyTorch, the exact-mode decoder the reference uses as its
correctness oracle, `qwen3.6-35b-a3b-gfx942/mk/reference.py` (`step(..., emulate=False)`: fp32 everywhere, the
FP8 weights dequantised exactly), with the model's widths as parameters (the reference fixes them as module
constants, `mk/dims.py:6-40`):

* `rms0`    follows `reference.py:188-191`   x * rsqrt(mean x^2 + eps) * (1 + w)
* `rope`    follows `reference.py:208-221`   angles in fp64, half-split rotation of the first 64 dims
* `State`   follows `reference.py:224-248`   conv history, SSM state [v][k], KV cache, all fp32
* `gdn`     follows `reference.py:251-284`   value head h uses key head h // (nvh / nkh)
* `attn`    follows `reference.py:287-314`   q head h uses kv head h // (nq / nkv), sigmoid output gate
* `route`   follows `reference.py:317-323`   top-8 by logit, ties to the lower id (stable sort), softmax over the 8
* `moe`     follows `reference.py:326-360`   per row: experts added in rank order, then the gated shared expert
* `step`    follows `reference.py:363-396`

`round_inputs=True` is this repository's kernel arithmetic instead of the reference's fp32: every GEMV input,
the conv history, the KV cache and q are rounded to bf16 (the reference has an `emulate` mode of its own for its
kernel's FP8 activations, which is not restated).  Parity tests compare the kernel with the exact mode at the
tolerance the benchmark states and use the rounded mode to show where the difference comes from.

Parity pin: `tests/test_oracle35_pin.py` runs this file against the reference's own `mk.reference.step` bitwise
(imported from the reference checkout when present) and against `tests/golden/qwen35moe_*.json`, written by
`tests/golden/make_golden_35b.py` from the reference.
"""

import torch
import torch.nn.functional as F

DK = DV = 128
HD = 256
ROT = 64
P = "model.language_model."


def _r(x, on):
    return x.to(torch.bfloat16).float() if on else x


def rms0(x, w, eps):
    r = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return x * r * (1.0 + w.float())


def rope_cos_sin(theta, pos):
    inv = theta ** (-torch.arange(0, ROT, 2, device=pos.device, dtype=torch.float64) / ROT)
    ang = pos.double()[:, None] * inv[None, :]
    ang = torch.cat([ang, ang], -1)
    return ang.cos().float(), ang.sin().float()


def rope(x, cos, sin):
    xr, xp = x[..., :ROT], x[..., ROT:]
    rot = torch.cat([-xr[..., ROT // 2:], xr[..., : ROT // 2]], -1)
    return torch.cat([xr * cos[:, None, :] + rot * sin[:, None, :], xp], -1)


class State:
    def __init__(self, s, M, maxlen, layers=None, device="cpu"):
        layers = layers if layers is not None else s.layers
        n_att = sum(s.is_attn(i) for i in range(layers))
        n_gdn = layers - n_att
        z = lambda *shp: torch.zeros(*shp, dtype=torch.float32, device=device)  # noqa: E731
        self.conv = z(n_gdn, M, s.conv_dim, 3)
        self.ssm = z(n_gdn, M, s.nvh, DV, DK)
        self.k = z(n_att, M, s.nkv, maxlen, HD)
        self.v = z(n_att, M, s.nkv, maxlen, HD)
        self.pos = torch.zeros(M, dtype=torch.long, device=device)


def gdn(s, W, i, x, st, gi, rnd, tr=None):
    M = x.shape[0]
    p = "linear_attn."
    lin = lambda n: _r(x, rnd) @ W.L(i, p + n + ".weight").float().t()  # noqa: E731
    qkv, z, b, a = lin("in_proj_qkv"), lin("in_proj_z"), lin("in_proj_b"), lin("in_proj_a")
    cw = W.L(i, p + "conv1d.weight")[:, 0, :]
    win = torch.cat([st.conv[gi], qkv[:, :, None]], -1)
    st.conv[gi] = _r(win[:, :, 1:], rnd)
    y = (win * cw[None]).sum(-1)
    y = y * torch.sigmoid(y)
    kd = s.key_dim
    q = y[:, :kd].reshape(M, s.nkh, DK)
    k = y[:, kd: 2 * kd].reshape(M, s.nkh, DK)
    v = y[:, 2 * kd:].reshape(M, s.nvh, DV)
    q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6)
    k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    q = q * DK ** -0.5
    q = q.repeat_interleave(s.nvh // s.nkh, 1)
    k = k.repeat_interleave(s.nvh // s.nkh, 1)
    beta = torch.sigmoid(b)
    g = -torch.exp(W.L(i, p + "A_log"))[None] * F.softplus(a + W.L(i, p + "dt_bias")[None])
    S = st.ssm[gi] * torch.exp(g)[:, :, None, None]
    kv = torch.einsum("mhvk,mhk->mhv", S, k)
    S = S + ((v - kv) * beta[:, :, None])[:, :, :, None] * k[:, :, None, :]
    st.ssm[gi] = S
    o = torch.einsum("mhvk,mhk->mhv", S, q)
    o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + s.eps) * W.L(i, p + "norm.weight")
    zz = z.reshape(M, s.nvh, DV)
    o = (o * (zz * torch.sigmoid(zz))).reshape(M, s.val_dim)
    if tr is not None:
        tr.update(y=torch.cat([qkv, z, b, a], -1), y2=o)
    return _r(o, rnd) @ W.L(i, p + "out_proj.weight").float().t()


def attn(s, W, i, x, st, ai, rnd, tr=None):
    M = x.shape[0]
    p = "self_attn."
    lin = lambda n: _r(x, rnd) @ W.L(i, p + n + ".weight").float().t()  # noqa: E731
    qg_flat, k_flat, v_flat = lin("q_proj"), lin("k_proj"), lin("v_proj")
    qg = qg_flat.reshape(M, s.nq, 2 * HD)
    q, gate = qg[..., :HD], qg[..., HD:].reshape(M, s.nq * HD)
    k = k_flat.reshape(M, s.nkv, HD)
    v = v_flat.reshape(M, s.nkv, HD)
    q = rms0(q, W.L(i, p + "q_norm.weight"), s.eps)
    k = rms0(k, W.L(i, p + "k_norm.weight"), s.eps)
    cos, sin = rope_cos_sin(s.theta, st.pos)
    q, k = rope(q, cos, sin), rope(k, cos, sin)
    q = _r(q, rnd)
    out = torch.empty(M, s.nq, HD, device=x.device)
    for m in range(M):
        pp = int(st.pos[m])
        st.k[ai, m, :, pp] = _r(k[m], rnd)
        st.v[ai, m, :, pp] = _r(v[m], rnd)
        K, V = st.k[ai, m, :, : pp + 1], st.v[ai, m, :, : pp + 1]
        qh = q[m].reshape(s.nkv, s.nq // s.nkv, HD)
        sc = torch.einsum("gqd,gld->gql", qh, K) * HD ** -0.5
        out[m] = torch.einsum("gql,gld->gqd", torch.softmax(sc, -1), V).reshape(s.nq, HD)
    o = out.reshape(M, s.nq * HD) * torch.sigmoid(gate)
    if tr is not None:
        tr.update(y=torch.cat([qg_flat, k_flat, v_flat], -1), y2=o)
    return _r(o, rnd) @ W.L(i, p + "o_proj.weight").float().t()


def route(logits, topk):
    idx = torch.sort(logits, dim=-1, descending=True, stable=True).indices[:, :topk]
    top = logits.gather(1, idx)
    w = torch.exp(top - top[:, :1])
    return idx, w / w.sum(-1, keepdim=True)


def moe(s, W, i, x, rnd, tr=None):
    M = x.shape[0]
    wr = torch.cat([W.L(i, "mlp.gate.weight"), W.L(i, "mlp.shared_expert_gate.weight")])
    lg = _r(x, rnd) @ wr.float().t()
    idx, w = route(lg[:, : s.experts], s.topk)
    sg = torch.sigmoid(lg[:, s.experts])

    def ffn(gate, up, down):
        g, u = _r(x, rnd) @ gate.float().t(), _r(x, rnd) @ up.float().t()
        return _r(g * torch.sigmoid(g) * u, rnd) @ down.float().t()

    ys = {e: ffn(*W.expert(i, e)) for e in torch.unique(idx).tolist()}
    se = "mlp.shared_expert."
    ysh = ffn(W.L(i, se + "gate_proj.weight"), W.L(i, se + "up_proj.weight"), W.L(i, se + "down_proj.weight"))
    out = torch.zeros_like(x)
    for m in range(M):
        acc = torch.zeros_like(x[m])
        for j in range(s.topk):
            acc = acc + w[m, j] * ys[int(idx[m, j])][m]
        out[m] = acc + sg[m] * ysh[m]
    if tr is not None:
        tr.update(router=lg, idx=idx, w=w, sg=sg)
    return out


@torch.no_grad()
def step(s, W, tok, st, layers=None, round_inputs=False, trace=None, lm_head=True):
    """One decode step for M rows: tok [M] int64 -> fp32 logits [M, vocab]; advances st.pos.  `trace`, if a
    list, receives per layer: y (in-projection), y2 (mixer output), h1 (after the mixer), router / idx / w / sg,
    h0 (after the MoE block)."""
    layers = layers if layers is not None else s.layers
    rnd = round_inputs
    h = W[P + "embed_tokens.weight"][tok].float()
    gi = ai = 0
    for i in range(layers):
        tr = {} if trace is not None else None
        x = rms0(h, W.L(i, "input_layernorm.weight"), s.eps)
        if s.is_attn(i):
            h = h + attn(s, W, i, x, st, ai, rnd, tr)
            ai += 1
        else:
            h = h + gdn(s, W, i, x, st, gi, rnd, tr)
            gi += 1
        if tr is not None:
            tr["h1"] = h.clone()
        x = rms0(h, W.L(i, "post_attention_layernorm.weight"), s.eps)
        h = h + moe(s, W, i, x, rnd, tr)
        if tr is not None:
            tr["h0"] = h.clone()
            trace.append(tr)
    st.pos += 1
    if not lm_head:
        return h
    x = rms0(h, W[P + "norm.weight"], s.eps)
    return _r(x, rnd) @ W["lm_head.weight"].float().t()
