"""LoRA configuration and target matching (reference: infini_train/src/nn/lora/lora_config.cc:7-23,
include/nn/lora/lora_config.h:11-37)."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Set


@dataclass
class LoRAConfig:
    rank: int = 8
    alpha: float = 16.0
    dropout: float = 0.0            # accepted for parity; unused, as in the reference
    target_modules: Set[str] = field(default_factory=lambda: {"c_attn", "c_proj"})
    use_kaiming_a: bool = True
    kaiming_a_param: float = math.sqrt(5.0)
    # 0: A factors are drawn from the global stream in injection order (the reference's behaviour).  Otherwise every
    # adapter draws its A at its whole-model shape from a generator of its own, seeded with this value and the
    # module's whole-model path: freshly initialised adapters are then the same whatever layout (tensor / pipeline
    # split) builds the model.
    seed: int = 0

    def Scaling(self) -> float:
        return float(self.alpha) / float(self.rank)

    def ShouldApplyLoRA(self, module_name: str) -> bool:
        """A module matches when its dotted path equals a target or ends with ``.target``; dotted
        targets such as ``attn.c_proj`` therefore do not match ``mlp.c_proj``."""
        for t in self.target_modules:
            if module_name == t or module_name.endswith("." + t):
                return True
        return False


def ParseLoRATargetModules(spec: str) -> Set[str]:
    """``"c_attn, attn.c_proj ,,"`` -> {"c_attn", "attn.c_proj"} (blanks trimmed, empties dropped)."""
    return {p.strip() for p in spec.split(",") if p.strip()}
