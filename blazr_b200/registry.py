"""Model registry: which loader and which model class serve a checkpoint.

    *.gguf file                    -> llama / mistral decoders over the quantized linear layer (blazr_b200/gguf_loader.py, decode.py);
                                      the GGUF `general.architecture` key picks the family (reference src/loader/gguf.rs:101-306)
    folder with config.json        -> config "architecture" picks a layer-list design (blazr_b200/layered.py) read from
                                      model.safetensors (reference src/loader/safetensors/)

`register_layered` adds a design: a name and a function config dict -> LayeredConfig.
"""
from __future__ import annotations

import os
from typing import Callable, Dict

from . import fenorax, gemosun, pafelorn, teselix
from .layered import LayeredConfig, LayeredModel

LAYERED: Dict[str, Callable[[dict], LayeredConfig]] = {}
GGUF_FAMILIES = ("llama", "mistral")


def register_layered(name: str, parse: Callable[[dict], LayeredConfig]) -> None:
    LAYERED[name] = parse


register_layered(fenorax.ARCHITECTURE, fenorax.parse_config)
register_layered(gemosun.ARCHITECTURE, gemosun.parse_config)
register_layered(pafelorn.ARCHITECTURE, pafelorn.parse_config)
register_layered(teselix.ARCHITECTURE, teselix.parse_config)


class UnknownArchitecture(ValueError):
    pass


def architecture_of(path: str) -> str:
    """name of the architecture a checkpoint declares"""
    if os.path.isdir(path):
        import json
        with open(os.path.join(path, "config.json")) as f:
            cfg = json.load(f)
        arch = cfg.get("architecture") or (cfg.get("architectures") or [None])[0]
        if not arch:
            raise UnknownArchitecture(f"{path}: config.json names no architecture")
        return arch
    from .gguf_loader import Gguf
    g = Gguf.open(path)
    try:
        return g.metadata().architecture() or ""
    finally:
        g.close()


def load_model(path: str, device="cuda:0", dtype: str = "bfloat16", **kw):
    """checkpoint -> model object.  Layer-list designs give a LayeredModel (serve it with blazr_b200.engine.Engine); GGUF files give
    the quantized Decoder (extra keywords go to gguf_loader.load_gguf)."""
    arch = architecture_of(path)
    if os.path.isdir(path):
        if arch not in LAYERED:
            raise UnknownArchitecture(f"{path}: architecture '{arch}' is not registered (known: {sorted(LAYERED)})")
        from .safetensors_loader import load_checkpoint
        cfg, st = load_checkpoint(path)
        try:
            return LayeredModel(LAYERED[arch](cfg), st.tensor, device, dtype)
        finally:
            st.close()
    if arch not in GGUF_FAMILIES:
        raise UnknownArchitecture(f"{path}: GGUF architecture '{arch}' is not supported (known: {GGUF_FAMILIES})")
    from . import ops
    from .gguf_loader import load_gguf
    import torch
    return load_gguf(ops.B200Client(torch.device(device).index or 0), path, **kw)
