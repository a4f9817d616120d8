"""Host-side checks of the kernel's work partition (the same functions the device code calls)."""

import pytest

from megakernels_b200 import _lib
from megakernels_b200.config import qwen35_08b


@pytest.mark.parametrize("grid", [132, 148, 160])
@pytest.mark.parametrize("rows,unit", [(8224, 1), (5120, 1), (1024, 1), (7168, 2), (151936, 1), (248320, 1), (4096, 1)])
def test_rows_cover_matrix_once(lib_built, rows, unit, grid):
    prev = 0
    sizes = []
    for cta in range(grid):
        r0, r1 = _lib.plan_rows(rows, unit, cta, grid)
        assert r0 == prev and r1 >= r0 and r0 % unit == 0 and r1 % unit == 0
        prev = r1
        sizes.append(r1 - r0)
    assert prev == rows
    assert max(sizes) - min(sizes) <= unit          # balanced to within one unit


def test_per_cta_ownership_fits_the_kernels_staging(lib_built):
    cfg = qwen35_08b()
    grid = 148
    own = lambda rows, unit: max(b - a for a, b in (_lib.plan_rows(rows, unit, c, grid) for c in range(grid)))
    assert own(cfg.gdn_in_rows, 1) <= 64 and own(2 * cfg.intermediate, 2) <= 64
    assert own(cfg.hidden, 1) <= 16
    assert own(cfg.vocab, 1) <= _lib.query("MAX_LM_ROWS") and own(262144, 1) <= _lib.query("MAX_LM_ROWS")


@pytest.mark.parametrize("max_splits", [66, 74])
def test_attention_chunks(lib_built, max_splits):
    lib = _lib.load()
    block = _lib.query("KV_BLOCK")
    last = 0
    for n in list(range(1, 300)) + [511, 512, 513, 1024, 2047, 4096, 8191, 16384, 448 * max_splits]:
        ch = lib.mk_plan_attn_chunk(n, max_splits)
        assert (n + ch - 1) // ch <= max_splits                  # never more tasks than CTAs
        assert ch % block == 0 or block % ch == 0                # a chunk never straddles a page
        assert ch >= last or n < 300                             # grows with the context
        assert ch <= 448
        last = ch
