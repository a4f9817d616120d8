"""Race detection: the library built with -DMK_CHAOS pauses for a pseudo-random time (up to 4 us) before one in eight
publishes -- flag-in-data words, partial-tile counters, barrier arrivals, ring-slot releases, mailbox stores.  A
protocol that is correct does not care when a publish lands, so every launch must produce the same bits as with the
normal library: plain, speculative and batched launches of the 0.8B kernels, and the stage machine with K splits and
routed expert groups at eight sequences.  The reference's counterpart: `qwen3.6-35b-a3b-gfx942/tests/test_chaos.py:36-46`."""

import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CHAOS_LIB = "libmk_b200_chaos.so"


def _digests(libname):
    env = dict(os.environ)
    if libname:
        env["MK_B200_LIBNAME"] = libname
    else:
        env.pop("MK_B200_LIBNAME", None)
    p = subprocess.run([sys.executable, os.path.join(HERE, "chaos_worker.py")], env=env, capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, (p.stdout + p.stderr)[-3000:]
    line = [x for x in p.stdout.splitlines() if x.startswith("CHAOS_DIGESTS ")][-1]
    return json.loads(line[len("CHAOS_DIGESTS "):])


def test_chaos_build_produces_the_same_bits():
    if not os.path.exists(os.path.join(ROOT, "megakernels_b200", CHAOS_LIB)):
        # normally prebuilt by `python -m megakernels_b200.build --chaos` (the entry point's build() does it)
        from megakernels_b200 import build
        build.build_chaos()
    plain, chaos = _digests(None), _digests(CHAOS_LIB)
    assert plain.pop("library") == "libmk_b200.so" and chaos.pop("library") == CHAOS_LIB
    assert set(plain) == set(chaos) and len(plain) >= 7
    different = [k for k in plain if plain[k] != chaos[k]]
    assert not different, f"outputs depend on the timing of publishes: {different}"
