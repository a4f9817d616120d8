"""int8 per-channel quantiser: round-trip bound (the shape of the reference's own check,
qwen3.5-0.8b/tests/test_int8.py:39-43) and the weight dict handed to the reference decoder."""

import torch

from megakernels_b200.config import qwen35_08b
from megakernels_b200.quant import (dequantize_int8_rows, dequantized_weights, is_gemv_weight,
                                    quantize_int8_rows, roundtrip_int8_rows)
from megakernels_b200.synth import make_mtp_weights, make_prompt, make_weights


def test_roundtrip_error_is_half_a_step():
    g = torch.Generator().manual_seed(3)
    w = torch.randn(64, 1024, generator=g).to(torch.bfloat16)
    q, s = quantize_int8_rows(w)
    assert q.dtype == torch.uint8 and s.dtype == torch.float32 and s.shape == (64,)
    assert int(q.min()) >= 1 and int(q.max()) <= 255          # q in [-127, 127] stored as q + 128
    err = (dequantize_int8_rows(q, s) - w.float()).abs()
    assert (err <= s[:, None] * 0.5 * (1 + 1e-5)).all()
    assert torch.equal(s, w.float().abs().amax(1) * torch.tensor(1 / 127, dtype=torch.float32))


def test_edge_rows():
    w = torch.zeros(3, 32)
    w[1, 5] = 1.0
    w[2] = -2.5
    q, s = quantize_int8_rows(w)
    d = dequantize_int8_rows(q, s)
    assert torch.equal(d[0], torch.zeros(32))                   # all-zero row: clamped scale, q = 0
    assert torch.allclose(d[1], w[1]) and torch.allclose(d[2], w[2], rtol=1e-6)
    assert int(q[2, 0]) == 1                                    # -127 + 128


def test_nearly_idempotent():
    w = torch.randn(16, 256)
    once = roundtrip_int8_rows(w)
    twice = roundtrip_int8_rows(once)         # the scale may move by one ulp, the codes must not move
    assert torch.equal(quantize_int8_rows(once)[0], quantize_int8_rows(w)[0])
    assert torch.allclose(twice, once, rtol=1e-6, atol=0)


def test_dequantized_weight_dict():
    cfg = qwen35_08b(n_layers=4, vocab=512)
    w = make_weights(cfg, 0)
    d = dequantized_weights(w, "int8")
    assert set(d) == set(w)
    for k in w:
        if is_gemv_weight(k) or k == "embed_tokens.weight":
            assert not torch.equal(d[k].float(), w[k].float())
            assert torch.equal(d[k], roundtrip_int8_rows(w[k]))
        else:
            assert torch.equal(d[k].float(), w[k].float())
    d2 = dequantized_weights(w, "int8", embed_int8=False)      # the reference's variant: lookup stays bf16
    assert torch.equal(d2["embed_tokens.weight"].float(), w["embed_tokens.weight"].float())
    assert "lm_head.weight" in d2
    assert dequantized_weights(w, "bf16").keys() == w.keys()


def test_synthetic_weights_are_seeded():
    cfg = qwen35_08b(n_layers=4, vocab=512)
    a, b, c = make_weights(cfg, 0), make_weights(cfg, 0), make_weights(cfg, 1)
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["embed_tokens.weight"], c["embed_tokens.weight"])
    assert a["embed_tokens.weight"].dtype == torch.bfloat16
    assert abs(float(a["layers.0.mlp.gate_proj.weight"].float().std()) - 0.02) < 1e-3
    m = make_mtp_weights(cfg)
    assert m["fc.weight"].shape == (1024, 2048)
    p = make_prompt(cfg, 32)
    assert len(p) == 32 and all(0 <= t < cfg.vocab for t in p) and p == make_prompt(cfg, 32)
