"""`mk_launch_static`: the launch for hosts that may not allocate device memory.

A serving process that has handed its whole device to its own memory pool, or a plug-in that is
called where allocation is forbidden, cannot give the kernel a freshly allocated set of hand-off
buffers.  `mk_launch_static` keeps those words in an array that is part of the library image
instead.  This test drives it through the C ABI, two calls in a row on one sequence, and requires
the same bits as the ordinary `mk_launch` on the same inputs (both paths run the same kernel, so
the tolerance is zero).  The file is named to be collected last.
"""

import ctypes

import pytest
import torch

from megakernels_b200 import _lib
from megakernels_b200.config import qwen35_08b
from megakernels_b200.synth import make_prompt, make_weights

pytestmark = pytest.mark.gpu


def launch_static(mk, tokens, n_generate):
    """What `Megakernel.run(tokens, n_generate, return_logits=True)` does, through `mk_launch_static`."""
    dev = mk.device
    n_forced = len(tokens)
    n_steps = n_forced + n_generate - 1
    forced = torch.tensor(tokens, dtype=torch.int32, device=dev)
    stops = torch.tensor([-1], dtype=torch.int32, device=dev)
    out = torch.zeros(n_steps, dtype=torch.int64, device=dev)
    info = torch.zeros(8, dtype=torch.int32, device=dev)
    logits = torch.empty(n_steps, mk.cfg.vocab, device=dev)
    a = _lib.LaunchArgs(forced=forced.data_ptr(), n_forced=n_forced, n_steps=n_steps, lm_from=n_forced - 1,
                        start_pos=mk.pos, epoch_base=mk.epoch, seed=0, inv_temperature=0.0, n_stop=0,
                        stop_ids=stops.data_ptr(), tokens_out=out.data_ptr(), logits_out=logits.data_ptr(),
                        out_info=info.data_ptr(), grid=mk.grid, spin_limit_ns=mk.spin_limit_ns)
    stream = torch.cuda.current_stream(dev).cuda_stream
    _lib.check(mk.lib.mk_launch_static(mk._h, ctypes.byref(a), ctypes.c_void_p(stream)))
    done, epoch, _ = info[:3].tolist()
    assert int(mk.status[0]) == 0
    assert done == n_steps
    mk.pos += done
    mk.epoch = epoch & 0xFFFFFFFF
    ids = (0xFFFFFFFF - (out[n_forced - 1: done] & 0xFFFFFFFF)).tolist()
    return ids, logits[n_forced - 1: done]


@pytest.mark.parametrize("quant", ["int8", "bf16"])
def test_static_scratch_launch_matches_ordinary_launch_twice_in_a_row(quant, lib_built):
    from megakernels_b200.engine import Megakernel
    cfg = qwen35_08b(n_layers=4, vocab=4096)
    w = make_weights(cfg, 0, init="realistic")
    mk = Megakernel((cfg, w), max_seq=256, quant=quant)
    prompt = make_prompt(cfg, 70)
    # reference run with caller-allocated hand-off buffers: two launches on one sequence
    ids_a1, lg_a1 = mk.run(prompt, n_generate=12, return_logits=True)
    ids_a2, lg_a2 = mk.run([ids_a1[-1]], n_generate=12, return_logits=True)
    # the same two launches with the built-in array
    mk.reset()
    ids_b1, lg_b1 = launch_static(mk, prompt, 12)
    ids_b2, lg_b2 = launch_static(mk, [ids_b1[-1]], 12)
    assert ids_a1 == ids_b1 and ids_a2 == ids_b2
    assert torch.equal(lg_a1, lg_b1) and torch.equal(lg_a2, lg_b2)
    # and the ordinary path still works afterwards on the same engine
    mk.reset()
    assert mk.run(prompt, n_generate=12) == ids_a1


def test_an_engine_without_hand_off_buffers_runs_only_through_the_static_entry_point(lib_built):
    """The host that may not allocate passes 0 for all seven hand-off buffers; the results are those of an ordinary engine."""
    from megakernels_b200.engine import Megakernel
    cfg = qwen35_08b(n_layers=4, vocab=4096)
    w = make_weights(cfg, 0, init="realistic")
    mk = Megakernel((cfg, w), max_seq=256, quant="int8")
    prompt = make_prompt(cfg, 40)
    want = mk.run(prompt, n_generate=10)
    mk.reset()
    lv, mv, g = mk._tables
    bare = dict(g)
    for name in ("xl", "projl", "mixl", "actl", "lml", "attn_part", "partl"):
        bare[name] = 0
    gv = _lib.i64_array([bare[f] for f in _lib.GLOBAL_FIELDS])
    _lib.check(mk.lib.mk_set_params(mk._h, _lib.i64_array(lv), len(lv), None, 0, gv, len(gv)))
    got, _ = launch_static(mk, prompt, 10)
    assert got == want
    with pytest.raises(_lib.MkError, match="hand-off"):
        mk.reset()
        mk.run(prompt, n_generate=2)
    # some but not all of them is a mistake, not a static-only engine
    bare["xl"] = g["xl"]
    gv = _lib.i64_array([bare[f] for f in _lib.GLOBAL_FIELDS])
    with pytest.raises(_lib.MkError, match="all of them, or none"):
        _lib.check(mk.lib.mk_set_params(mk._h, _lib.i64_array(lv), len(lv), None, 0, gv, len(gv)))


def test_static_scratch_refuses_what_does_not_fit(lib_built):
    from megakernels_b200.engine import Megakernel
    cfg = qwen35_08b(n_layers=4, vocab=4096)
    mk = Megakernel((cfg, make_weights(cfg, 0)), max_seq=64)
    a = _lib.LaunchArgs(forced=0, n_forced=1, n_steps=1, grid=mk.grid)
    with pytest.raises(_lib.MkError, match="token list"):
        _lib.check(mk.lib.mk_launch_static(mk._h, ctypes.byref(a), None))
    a = _lib.LaunchArgs(forced=mk.status.data_ptr(), n_forced=1, n_steps=1, tokens_out=1, out_info=1, grid=mk.grid - 1,
                        epoch_base=1)
    with pytest.raises(_lib.MkError, match="packed for"):
        _lib.check(mk.lib.mk_launch_static(mk._h, ctypes.byref(a), None))
    assert _lib.load().mk_launch_static(None, None, None) == _lib.MK_ERR_BADARG
