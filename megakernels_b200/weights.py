"""Load the text-decoder weights of a Hugging Face snapshot directory.

Same contract as the reference loader (`qwen3.5-0.8b/qwen_mk/weights.py:61-90`): returns
`(Config, dict)` with the `model.language_model.` prefix dropped from the names.  Only local
directories are accepted: this library never downloads.
"""

import os

from .config import Config

PREFIX = "model.language_model."


def load(path, device="cpu", dtype=None, prefix=PREFIX):
    if not os.path.isdir(path):
        raise FileNotFoundError(f"{path!r} is not a snapshot directory (downloading is not supported)")
    from safetensors import safe_open

    cfg = Config.from_json(os.path.join(path, "config.json"))
    out = {}
    for name in sorted(os.listdir(path)):
        if not name.endswith(".safetensors"):
            continue
        with safe_open(os.path.join(path, name), "pt", device="cpu") as f:
            for k in f.keys():
                if k.startswith(prefix):
                    t = f.get_tensor(k)
                    out[k[len(prefix):]] = (t.to(dtype) if dtype is not None else t).to(device)
    return cfg, out


def load_mtp(path, device="cpu"):
    """MTP-head tensors keyed without the `mtp.` prefix (`qwen_mk/mtp.py:26-36`)."""
    return load(path, device, prefix="mtp.")[1]
