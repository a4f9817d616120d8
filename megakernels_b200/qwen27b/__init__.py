"""27B dense Gated-DeltaNet / gated-attention hybrid (MXFP4 weights) on the stage-machine megakernel.

Counterpart of the reference's `qwen3.8-27b-gfx942/mk` package: `Packed` (weights of one tensor-parallel
rank), `Engine` (`step(tok[M]) -> logits`), `tp` (the multi-rank harness)."""

from .dims import FULL, Dims, Shape  # noqa: F401


def __getattr__(name):
    if name == "Packed":
        from .pack import Packed
        return Packed
    if name == "Engine":
        from .runner import Engine
        return Engine
    if name in ("SynthWeights", "make_prompt"):
        from . import synth
        return getattr(synth, name)
    raise AttributeError(name)
