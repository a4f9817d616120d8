"""26B-A4B sliding-window / full-attention model with a 128-expert top-8 MoE in parallel with a dense GeGLU MLP
(FP8 e4m3 weights, one scale per output row) on the stage-machine megakernel.

Counterpart of the reference's `gemma4-26b-a4b-gfx942/mk` package: `Packed` (kernel-side weights), `Engine`
(`step(tok[M]) -> logits`)."""

from .dims import FULL, Shape  # noqa: F401


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
