"""Architecture registry of the token-id language models: config.json's "architecture" -> class.
`load_language_model(dir)` is what `vila_b200.load`, the CLI and the trace runner use."""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, Optional

import torch

from .ludazen import LudazenForCausalLM
from .lufatar import LufatarForCausalLM
from .moronex import MoronexForCausalLM
from .nusovik import NusovikForCausalLM

LANGUAGE_MODELS: Dict[str, type] = {"Moronex": MoronexForCausalLM, "Lufatar": LufatarForCausalLM,
                                    "Nusovik": NusovikForCausalLM, "Ludazen": LudazenForCausalLM}

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def language_model_architecture(model_dir) -> Optional[str]:
    """The registered architecture named by <model_dir>/config.json, or None (e.g. a VILA checkpoint)."""
    f = Path(model_dir) / "config.json"
    if not f.exists():
        return None
    arch = json.loads(f.read_text()).get("architecture")
    return arch if arch in LANGUAGE_MODELS else None


def load_language_model(model_dir, device="cuda", dtype="bfloat16"):
    arch = language_model_architecture(model_dir)
    if arch is None:
        raise ValueError(f"{model_dir}: config.json names no registered architecture "
                         f"(known: {sorted(LANGUAGE_MODELS)})")
    dt = _DTYPES[dtype] if isinstance(dtype, str) else dtype
    return LANGUAGE_MODELS[arch].from_pretrained(model_dir, device=device, dtype=dt)
