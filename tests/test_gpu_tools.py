"""Bandwidth probe and per-op timeline (GPU)."""

import pytest

from megakernels_b200.config import qwen35_08b
from megakernels_b200.synth import make_prompt, make_weights

pytestmark = pytest.mark.gpu


def test_bandwidth_probe_reads_at_dram_speed(lib_built):
    from megakernels_b200 import bw
    plain, ring = bw.measure("plain", gib=1.0), bw.measure("ring", gib=1.0)
    print(f"plain {plain:.0f} GB/s, ring {ring:.0f} GB/s")
    assert 2000 < plain < 9000 and 2000 < ring < 9000      # a B200 reads 6-8 TB/s; far below means a broken probe


def test_timeline_covers_every_op(lib_built):
    from megakernels_b200 import timeline
    from megakernels_b200.engine import Megakernel
    cfg = qwen35_08b(n_layers=4, vocab=4096)
    mk = Megakernel((cfg, make_weights(cfg, 0)), max_seq=128)
    rows = timeline.profile_step(mk, make_prompt(cfg, 20), step=4, n_generate=8)
    names = [r["op"] for r in rows]
    assert "lm head" in names and "step" in names and len(rows) == 12
    step = rows[-1]
    assert 1.0 < step["busy_us"] < 5000.0
    assert all(r["busy_us"] >= 0 and r["critical_us"] > -1.0 for r in rows)
    print(timeline.format_rows(rows))
