"""Which model family a checkpoint folder holds, by its config.json.

The reference picks a model by tag and leaves loading to its engine container (app/utils/config.py:86,
docker-compose.vllm.yml:39); here the folder's config.json decides which loader and which engine constructor run:

  * Hugging Face Llama ("model_type": "llama")            -> checkpoint.load_hf_checkpoint, ModelSpec
  * layered models ("layers": [...] + "width": Gitozen, Gedelorn, Vonedra, Lotinex) -> layered.load_checkpoint, LayeredSpec

Engine(spec, weights, ...) accepts either kind of spec.
"""
from __future__ import annotations

import json
import os
from typing import Callable, Dict, Tuple

FAMILIES: Dict[str, Callable] = {}


def _llama(path, device, name):
    from .checkpoint import load_hf_checkpoint
    return load_hf_checkpoint(path, device=device, name=name)


def _layered(path, device, name):
    from .layered import load_checkpoint
    return load_checkpoint(path, device=device, name=name)


FAMILIES["llama"] = _llama
FAMILIES["layered"] = _layered
# architectures of the layered family, by the name their config.json carries
LAYERED_ARCHITECTURES = ("Gitozen", "Gedelorn", "Vonedra", "Lotinex")


def family_of(cfg: Dict) -> str:
    from .layered import is_layered_config
    if cfg.get("architecture") in LAYERED_ARCHITECTURES or is_layered_config(cfg):
        return "layered"
    if cfg.get("model_type", "llama") == "llama":
        return "llama"
    raise ValueError(f"no model family for config with model_type={cfg.get('model_type')!r}, "
                     f"architecture={cfg.get('architecture')!r}")


def load_model(path: str, device: str = "cpu", name: str = None) -> Tuple[object, Dict]:
    """(spec, weights) of the checkpoint folder `path`, whatever family it is."""
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    return FAMILIES[family_of(cfg)](path, device, name)
