"""Model registry: which family serves a checkpoint directory, decided from its config.json the way
ssd/config.py + llm_engine.py:51-57 decide between Llama and Qwen3 (by `model_type`), extended with the layered
("hybrid") family, whose config.json carries an `architecture` name and a list of layers instead of HF fields.

    dense   Llama / Qwen3 decoders: PairRunner + the speculative engine of libssdk (ssdk_spec_step, ssdk_forward_tokens)
    hybrid  Pikavik, Kefurax, Lisenex, Kokatar (layered designs): HybridRunner + the ragged forward of libssdk (ssdk_hyb_forward)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable


@dataclass(frozen=True)
class Family:
    name: str
    kind: str  # "dense" | "hybrid"
    matches: Callable[[dict], bool]


FAMILIES: list[Family] = [
    Family("pikavik", "hybrid", lambda d: d.get("architecture") == "Pikavik"),
    Family("kefurax", "hybrid", lambda d: d.get("architecture") == "Kefurax"),
    Family("lisenex", "hybrid", lambda d: d.get("architecture") == "Lisenex"),
    Family("kokatar", "hybrid", lambda d: d.get("architecture") == "Kokatar"),
    Family("qwen3", "dense", lambda d: "qwen3" in str(d.get("model_type", "")).lower()),
    Family("llama", "dense", lambda d: "hidden_size" in d),
]


def family_of(config: dict) -> Family:
    for fam in FAMILIES:
        if fam.matches(config):
            return fam
    raise ValueError("config.json names no model family this framework serves "
                     f"(architecture={config.get('architecture')!r}, model_type={config.get('model_type')!r})")
