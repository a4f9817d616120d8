"""B200 (sm_100a) persistent decode megakernel behind the reference's Python runtime API."""

from .config import Config, qwen35_08b  # noqa: F401

__all__ = ["Config", "qwen35_08b", "Megakernel"]


def __getattr__(name):
    if name == "Megakernel":
        from .engine import Megakernel
        return Megakernel
    raise AttributeError(name)
