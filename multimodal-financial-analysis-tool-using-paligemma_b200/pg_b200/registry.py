"""Model registry: `config.json` names the design, the registry maps it to the engine class that serves it.

An engine class registers under the value of the config's `architecture` key (designs that do not carry one are
recognised by a predicate on the config).  `load_engine(model_dir, ...)` reads the folder, picks the class, and
returns an engine whose `new_batcher()` gives the scheduler that serves it."""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Tuple

import torch

from .checkpoint import read_config, read_safetensors

_BY_NAME: Dict[str, Callable] = {}
_BY_PREDICATE: List[Tuple[Callable[[dict], bool], Callable]] = []


def register(name: Optional[str] = None, predicate: Optional[Callable[[dict], bool]] = None):
    """Class decorator: `@register("Name")` or `@register(predicate=lambda cfg: ...)`.  The class must offer
    `from_checkpoint(config: dict, tensors: dict, *, device, dtype, **kw)`."""
    def deco(cls):
        if name is not None:
            _BY_NAME[name] = cls
        if predicate is not None:
            _BY_PREDICATE.append((predicate, cls))
        return cls
    return deco


def architectures() -> List[str]:
    _load_builtin()
    return sorted(_BY_NAME)


def _load_builtin() -> None:
    from . import birizen  # noqa: F401  (registers itself)
    from . import gogivik  # noqa: F401
    from . import mubasun  # noqa: F401
    from . import ninisun  # noqa: F401
    from . import engine   # noqa: F401


def resolve(config: dict):
    _load_builtin()
    arch = config.get("architecture")
    if arch in _BY_NAME:
        return _BY_NAME[arch]
    for pred, cls in _BY_PREDICATE:
        if pred(config):
            return cls
    raise ValueError(f"no engine registered for architecture {arch!r} (known: {sorted(_BY_NAME)})")


def load_engine(model_dir: str, *, device="cuda", dtype=torch.bfloat16, **kw):
    """Engine for the model in `model_dir` (config.json + model.safetensors)."""
    import glob
    import os
    config = read_config(model_dir)
    cls = resolve(config)
    tensors = {}
    for path in sorted(glob.glob(os.path.join(model_dir, "*.safetensors"))):
        tensors.update(read_safetensors(path))
    return cls.from_checkpoint(config, tensors, device=device, dtype=dtype, **kw)
