"""Architecture registry: which configuration class and which model class belong to an ``"architecture"`` name
found in a checkpoint's ``config.json`` (or to a configuration object).  The GPT/LLaMA family registers itself in
``models/__init__.py``; other designs add themselves with ``register_architecture``.

Reference: the reference resolves architectures through ``AutoModelForCausalLM`` (reference
llmctl/runtime/engine.py:126-140); this is the framework's own equivalent."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional


@dataclass
class Architecture:
    name: str
    config_from_dict: Callable[[Dict[str, Any]], Any]      # parsed config.json -> configuration object
    config_type: type
    build: Callable[..., Any]                               # (cfg, dtype=, device=, **kw) -> nn.Module
    load_weights: Optional[Callable[[Any, Any], None]] = None   # (model, checkpoint directory) -> None
    # (configuration, checkpoint directory) -> None: fills in sizes that only the checkpoint's tensor shapes give
    complete_config: Optional[Callable[[Any, Any], None]] = None


_BY_NAME: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture) -> None:
    _BY_NAME[arch.name.lower()] = arch


def architecture_named(name: str) -> Optional[Architecture]:
    return _BY_NAME.get(str(name).lower())


def architecture_of(cfg: Any) -> Optional[Architecture]:
    for a in _BY_NAME.values():
        if isinstance(cfg, a.config_type):
            return a
    return None


def architecture_names():
    return sorted(a.name for a in _BY_NAME.values())
