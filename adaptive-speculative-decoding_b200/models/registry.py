"""Model registry: which configuration class, engine class and library components serve a checkpoint.

A checkpoint directory is recognised by its ``config.json``: ``"architecture": "Mezilix"`` / ``"Rivetar"`` / ``"Mavipel"`` / ``"Lukopel"`` or the Hugging Face keys
``architectures`` / ``model_type`` of the Qwen2 family (what the reference hands to vLLM,
src/serving/real_model_pipeline.py:98-108).  ``Stage``, the trace runner and ``bench.py`` all go through here."""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Callable, Dict, Tuple


@dataclass(frozen=True)
class Family:
    name: str
    components: Tuple[str, ...]          # build.py components the family's engine needs
    dtypes: Tuple[str, ...]              # element types its engine runs in
    config_from_dict: Callable
    engine: Callable                     # () -> engine class (imported late: engines need torch + the library)


def _qwen_cfg(d: dict, name: str = "custom"):
    from .qwen2 import Qwen2Config
    hd = d.get("head_dim") or d["hidden_size"] // d["num_attention_heads"]
    return Qwen2Config(d["hidden_size"], d["num_hidden_layers"], d["num_attention_heads"], d["num_key_value_heads"],
                       d["intermediate_size"], d["vocab_size"], head_dim=hd,
                       tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
                       rms_norm_eps=float(d.get("rms_norm_eps", 1e-6)), rope_theta=float(d.get("rope_theta", 1e6)),
                       name=name)


def _mezilix_cfg(d: dict, name: str = "mezilix"):
    from .mezilix import MezilixConfig
    return MezilixConfig.from_dict(d, name=name)


def _rivetar_cfg(d: dict, name: str = "rivetar"):
    from .rivetar import RivetarConfig
    return RivetarConfig.from_dict(d, name=name)


def _mavipel_cfg(d: dict, name: str = "mavipel"):
    from .mavipel import MavipelConfig
    return MavipelConfig.from_dict(d, name=name)


def _lukopel_cfg(d: dict, name: str = "lukopel"):
    from .lukopel import LukopelConfig
    return LukopelConfig.from_dict(d, name=name)


def _qwen_engine():
    from ..engine import QwenEngine
    return QwenEngine


def _mezilix_engine():
    from ..engine import MezilixEngine
    return MezilixEngine


def _rivetar_engine():
    from ..engine import RivetarEngine
    return RivetarEngine


def _mavipel_engine():
    from ..engine import MavipelEngine
    return MavipelEngine


def _lukopel_engine():
    from ..engine import LukopelEngine
    return LukopelEngine


FAMILIES: Dict[str, Family] = {
    "qwen2": Family("qwen2", ("linear", "qwen", "sampling"), ("bfloat16",), _qwen_cfg, _qwen_engine),
    "mezilix": Family("mezilix", ("mezilix",), ("bfloat16", "float32"), _mezilix_cfg, _mezilix_engine),
    "rivetar": Family("rivetar", ("rivetar",), ("bfloat16", "float32"), _rivetar_cfg, _rivetar_engine),
    "mavipel": Family("mavipel", ("mavipel",), ("bfloat16", "float32"), _mavipel_cfg, _mavipel_engine),
    "lukopel": Family("lukopel", ("lukopel",), ("bfloat16", "float32"), _lukopel_cfg, _lukopel_engine),
}


def family_of_dict(d: dict) -> Family:
    arch = d.get("architecture")
    if isinstance(arch, str) and arch.lower() in FAMILIES:
        return FAMILIES[arch.lower()]
    names = [str(a).lower() for a in d.get("architectures", [])] + [str(d.get("model_type", "")).lower()]
    if any(n.startswith("qwen2") for n in names):
        return FAMILIES["qwen2"]
    raise ValueError(f"config.json names no architecture this framework serves (architecture={arch!r}, "
                     f"architectures={d.get('architectures')!r}); have {sorted(FAMILIES)}")


def family_of_config(cfg) -> Family:
    arch = getattr(cfg, "architecture", None)
    return FAMILIES[arch.lower() if isinstance(arch, str) and arch.lower() in FAMILIES else "qwen2"]


def safetensors_shapes(path: str) -> Dict[str, tuple]:
    """tensor name -> shape from the headers of a checkpoint directory's ``*.safetensors`` files (no data is read)"""
    import glob
    import struct
    out: Dict[str, tuple] = {}
    for fn in sorted(glob.glob(os.path.join(path, "*.safetensors"))):
        with open(fn, "rb") as f:
            (n,) = struct.unpack("<Q", f.read(8))
            header = json.loads(f.read(n))
        out.update({k: tuple(v["shape"]) for k, v in header.items() if k != "__metadata__"})
    return out


def read_config(path: str):
    """(family, configuration) of a checkpoint directory"""
    with open(os.path.join(path, "config.json")) as f:
        d = json.load(f)
    fam = family_of_dict(d)
    cfg = fam.config_from_dict(d, name=os.path.basename(os.path.normpath(path)) or fam.name)
    if hasattr(cfg, "with_shapes"):          # sizes that only a tensor's shape gives
        cfg = cfg.with_shapes(safetensors_shapes(path))
    return fam, cfg


def has_config(path: str) -> bool:
    return os.path.isdir(path) and os.path.exists(os.path.join(path, "config.json"))
