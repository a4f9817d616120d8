"""35B-A3B Gated-DeltaNet / gated-attention hybrid with a 256-expert top-8 MoE (FP8 e4m3 weights, 128 x 128 block
scales) on the stage-machine megakernel.

Counterpart of the reference's `qwen3.6-35b-a3b-gfx942/mk` package: `Packed` (kernel-side weights), `Engine`
(`step(tok[M]) -> logits`)."""

from .dims import FULL, Shape  # noqa: F401


def __getattr__(name):
    if name == "Packed":
        from .pack import Packed
        return Packed
    if name == "Engine":
        from .runner import Engine
        return Engine
    if name in ("SynthWeights", "make_prompt", "expert_load"):
        from . import synth
        return getattr(synth, name)
    raise AttributeError(name)
