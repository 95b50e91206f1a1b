"""Model registry: which model class serves a model folder.

A folder's ``config.json`` names its design either by ``"architecture"`` (language models) or by
``"model_type"`` / ``"architectures"`` (Dia checkpoints).  Families register a loader under those names;
:func:`load_model` reads the file and dispatches.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Callable

_LOADERS: dict[str, Callable] = {}


def register(name: str, loader: Callable) -> None:
    _LOADERS[name.lower()] = loader


def architectures() -> list[str]:
    _ensure_builtin()
    return sorted(_LOADERS)


def architecture_of(config: dict) -> str:
    for key in ("architecture", "model_type"):
        v = config.get(key)
        if isinstance(v, str) and v:
            return v
    v = config.get("architectures")
    if isinstance(v, list) and v:
        return str(v[0])
    raise ValueError("config.json names no architecture")


def _ensure_builtin() -> None:
    if _LOADERS:
        return

    def _load_dia(folder, dtype="float32", device=None, **kw):
        from .model import Dia
        folder = Path(folder)
        ckpt = next((folder / n for n in ("dia-v0_1.pth", "model.pth", "pytorch_model.bin") if (folder / n).exists()), None)
        if ckpt is None:
            raise FileNotFoundError(f"no Dia checkpoint (*.pth) in {folder}")
        return Dia.from_local(str(folder / "config.json"), str(ckpt), compute_dtype=dtype, device=device)

    def _load_causal_lm(folder, dtype="bfloat16", device=None, **kw):
        from .lm_model import CausalLM
        return CausalLM.from_pretrained(folder, dtype=dtype, device=device, **kw)

    register("dia", _load_dia)
    register("DiaModel", _load_dia)
    register("Pubopel", _load_causal_lm)
    register("Kupelix", _load_causal_lm)
    register("Luketar", _load_causal_lm)
    register("Fipadra", _load_causal_lm)


def load_model(folder: str | Path, dtype: str = "bfloat16", device=None, **kw):
    """Instantiate the model of ``folder`` (``config.json`` + weights) with the class its design is registered under."""
    _ensure_builtin()
    cfg = json.loads((Path(folder) / "config.json").read_text(encoding="utf-8"))
    name = architecture_of(cfg)
    loader = _LOADERS.get(name.lower())
    if loader is None:
        raise NotImplementedError(f"no model class registered for architecture {name!r} (known: {architectures()})")
    return loader(folder, dtype=dtype, device=device, **kw)
