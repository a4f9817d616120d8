"""CPU oracle of one decode step of the 26B-A4B sliding-window / full-attention MoE model.  TEST INFRASTRUCTURE ONLY.

Only `tests/`, `__graft_entry__.smoke()` and `bench.py`'s CPU-baseline legs may import this module; the
product package never does.  It restates, in PyTorch, the exact-mode decoder the reference uses as its
correctness oracle, `gemma4-26b-a4b-gfx942/mk/reference.py` (`step(..., mode="exact")`: every GEMV input rounded
to bf16, fp32 accumulation, bf16 KV cache), with the model's widths as parameters (the reference fixes them as
module constants, `mk/dims.py:8-38`):

* `rms`        follows `reference.py:127-130`   x * rsqrt(mean x^2 + eps) * w, plain weights, optional
* `lin`        follows `reference.py:150-157`   bf16-rounded input, fp32 product, times the row scale of FP8 weights
* `rope_*`     follows `reference.py:168-191`   sliding: all dims, theta 1e4; full: the first 64 of 256 pairs, theta 1e6
* `State`      follows `reference.py:194-215`   bf16 caches of the two layer types
* `attn`       follows `reference.py:218-246`   q / k norms, weightless V norm, V = k projection on full layers,
                                                scaling 1, window of 1024 on sliding layers
* `route`      follows `reference.py:249-262`   softmax, top 8 in rank order, renormalised, times per_expert_scale
* `moe`, `dense_mlp`, `ffn` follow `reference.py:265-307`   GeGLU (tanh) experts in rank order; the dense MLP as three
                                                704-column slices added in order; the sandwich norms and the layer scalar
* `embed`, `hidden_step`, `logits_of`, `step` follow `reference.py:310-345, 398-409`

Parity pin: `tests/test_oracle_gemma_pin.py` runs this file against the reference's own `mk.reference.step`
bitwise (imported from the reference checkout when present) and against `tests/golden/gemma26b_*.json`,
written by `tests/golden/make_golden_gemma.py` from the reference.
"""

import math

import torch


def bf(x):
    return x.to(torch.bfloat16).float()


def rms(x, w=None, eps=1e-6):
    r = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return x * r if w is None else x * r * w.float()


def lin(x, ws):
    w, sc = ws
    y = bf(x.float()) @ w.float().t()
    return y if sc is None else y * sc.float().reshape(1, -1)


def gelu_tanh(x):
    return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x.pow(3))))


def rope_inv_freq(s, full, device):
    if full:
        i = torch.arange(s.hd_f // 2, device=device, dtype=torch.float64)
        f = s.theta_f ** (-2 * i / s.hd_f)
        return torch.where(i < s.rot_f, f, torch.zeros_like(f))
    i = torch.arange(s.hd_s // 2, device=device, dtype=torch.float64)
    return s.theta_s ** (-2 * i / s.hd_s)


def rope_cos_sin(s, pos, full):
    ang = pos.double()[:, None] * rope_inv_freq(s, full, pos.device)[None, :]
    return ang.cos().float(), ang.sin().float()


def apply_rope(x, cos, sin):
    h = x.shape[-1] // 2
    x1, x2 = x[..., :h], x[..., h:]
    c, sn = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * sn, x2 * c + x1 * sn], -1)


class State:
    def __init__(self, s, M, maxlen, layers=None, device="cpu", dtype=torch.bfloat16):
        layers = layers if layers is not None else s.layers
        nf = sum(s.is_full(i) for i in range(layers))
        ns = layers - nf
        z = lambda *shp: torch.zeros(*shp, dtype=dtype, device=device)  # noqa: E731
        self.ks, self.vs = z(ns, M, s.nkv_s, maxlen, s.hd_s), z(ns, M, s.nkv_s, maxlen, s.hd_s)
        self.kf, self.vf = z(nf, M, s.nkv_f, maxlen, s.hd_f), z(nf, M, s.nkv_f, maxlen, s.hd_f)
        self.pos = torch.zeros(M, dtype=torch.long, device=device)


def attn(s, W, i, x, st, li, tr=None):
    M = x.shape[0]
    full = s.is_full(i)
    nkv, hd = s.attn_dims(i)
    p = "self_attn."
    q_flat, k_flat = lin(x, W.lin(i, p + "q_proj")), lin(x, W.lin(i, p + "k_proj"))
    v_flat = k_flat if full else lin(x, W.lin(i, p + "v_proj"))
    q, k, v = q_flat.reshape(M, s.nq, hd), k_flat.reshape(M, nkv, hd), v_flat.reshape(M, nkv, hd)
    q = rms(q, W.L(i, p + "q_norm.weight"), s.eps)
    k = rms(k, W.L(i, p + "k_norm.weight"), s.eps)
    v = rms(v, None, s.eps)
    cos, sin = rope_cos_sin(s, st.pos, full)
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    q = bf(q)
    kc, vc = (st.kf, st.vf) if full else (st.ks, st.vs)
    out = torch.empty(M, s.nq, hd, device=x.device)
    g = s.nq // nkv
    for m in range(M):
        pp = int(st.pos[m])
        kc[li, m, :, pp] = k[m].to(kc.dtype)
        vc[li, m, :, pp] = v[m].to(vc.dtype)
        lo = 0 if full else max(0, pp - s.window + 1)
        K, V = kc[li, m, :, lo: pp + 1].float(), vc[li, m, :, lo: pp + 1].float()
        qh = q[m].reshape(nkv, g, hd)
        sc = torch.einsum("gqd,gld->gql", qh, K)
        out[m] = torch.einsum("gql,gld->gqd", torch.softmax(sc, -1), V).reshape(s.nq, hd)
    o = out.reshape(M, s.nq * hd)
    if tr is not None:
        tr.update(y=torch.cat([q_flat, k_flat] + ([] if full else [v_flat]), -1), y2=o)
    return lin(o, W.lin(i, p + "o_proj"))


def route_logits(s, logits, pes):
    probs = torch.softmax(logits.float(), -1)
    top, ids = torch.topk(probs, s.topk, dim=-1)
    return ids, top / top.sum(-1, keepdim=True) * pes.float()[ids]


def route(s, W, i, h1):
    xr = rms(h1, None, s.eps) * (s.hidden ** -0.5) * W.L(i, "router.scale").float()
    logits = bf(xr) @ W.L(i, "router.proj.weight").float().t()
    ids, wts = route_logits(s, logits, W.L(i, "router.per_expert_scale"))
    return ids, wts, logits


def moe(s, W, i, xe, ids, wts):
    N = xe.shape[0]
    ys = torch.zeros(N, s.topk, s.hidden, device=xe.device)
    for e in ids.unique().tolist():
        r, k = (ids == e).nonzero(as_tuple=True)
        g, u, d = W.expert(i, e)
        x = xe[r]
        ys[r, k] = lin(gelu_tanh(lin(x, g)) * lin(x, u), d)
    out = torch.zeros(N, s.hidden, device=xe.device)
    for k in range(s.topk):
        out = out + wts[:, k: k + 1] * ys[:, k]
    return out


def dense_mlp(s, W, i, xd):
    (gw, gs), (uw, us), (dw, ds) = (W.lin(i, f"mlp.{n}") for n in ("gate_proj", "up_proj", "down_proj"))
    out = torch.zeros(xd.shape[0], s.hidden, device=xd.device)
    nds = s.ffn // s.eff
    assert nds * s.eff == s.ffn
    for k in range(nds):
        sl = slice(k * s.eff, (k + 1) * s.eff)
        sc = lambda t: None if t is None else t.reshape(-1)[sl]  # noqa: E731
        a = gelu_tanh(lin(xd, (gw[sl], sc(gs)))) * lin(xd, (uw[sl], sc(us)))
        out = out + lin(a, (dw[:, sl], ds))
    return out


def ffn(s, W, i, h, a, tr=None, force_ids=None):
    h1 = h + rms(a, W.L(i, "post_attention_layernorm.weight"), s.eps)
    d = dense_mlp(s, W, i, rms(h1, W.L(i, "pre_feedforward_layernorm.weight"), s.eps))
    ids, wts, logits = route(s, W, i, h1)
    own_ids = ids
    if force_ids is not None:
        # somebody else's choice of experts (a kernel's, whose router logits differ in the last bits), this decoder's weights
        ids = force_ids.long()
        top = torch.softmax(logits.float(), -1).gather(1, ids)
        wts = top / top.sum(-1, keepdim=True) * W.L(i, "router.per_expert_scale").float()[ids]
    e = moe(s, W, i, rms(h1, W.L(i, "pre_feedforward_layernorm_2.weight"), s.eps), ids, wts)
    y = rms(d, W.L(i, "post_feedforward_layernorm_1.weight"), s.eps) + rms(e, W.L(i, "post_feedforward_layernorm_2.weight"), s.eps)
    h = (h1 + rms(y, W.L(i, "post_feedforward_layernorm.weight"), s.eps)) * W.L(i, "layer_scalar").float()
    if tr is not None:
        tr.update(a=a.clone(), h1=h1.clone(), d=d.clone(), e=e.clone(), y=y.clone(), h=h.clone(), ids=own_ids.clone(), wts=wts.clone(), logits=logits.clone())
    return h


def embed(s, W, tok):
    return (W.embed[tok].float() * s.embed_scale).to(torch.bfloat16).float()


@torch.no_grad()
def hidden_step(s, W, tok, st, layers=None, trace=None, force_ids=None):
    """One decode step for M rows -> the final-normed hidden state [M, hidden] (bf16 values); advances st.pos.
    `trace`, if a list, receives per layer: attention (y, y2), a, h1, d, e, y, h, ids (this decoder's own choice), wts,
    logits.  `force_ids` [layers, M, top k] replaces the choice of experts (not the weights)."""
    layers = layers if layers is not None else s.layers
    h = embed(s, W, tok)
    si = fi = 0
    for i in range(layers):
        tr = {} if trace is not None else None
        x = rms(h, W.L(i, "input_layernorm.weight"), s.eps)
        atr = {} if trace is not None else None
        a = attn(s, W, i, x, st, fi if s.is_full(i) else si, atr)
        if s.is_full(i):
            fi += 1
        else:
            si += 1
        h = ffn(s, W, i, h, a, tr, None if force_ids is None else force_ids[i])
        if trace is not None:
            tr.update(qkv=atr["y"], mix=atr["y2"])
            trace.append(tr)
    st.pos += 1
    return bf(rms(h, W["model.language_model.norm.weight"], s.eps))


def logits_of(s, W, hidden):
    z = bf(hidden) @ W.embed.float().t()
    return s.softcap * torch.tanh(z / s.softcap)


def step(s, W, tok, st, layers=None, trace=None, force_ids=None):
    return logits_of(s, W, hidden_step(s, W, tok, st, layers, trace, force_ids))
