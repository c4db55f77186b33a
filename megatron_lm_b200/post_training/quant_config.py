"""Per-layer quantisation recipes chosen by glob patterns over module names.

Reference: megatron/core/quantization/quant_config.py (``RecipeConfig`` :88 with ordered ``matchers``,
``MatchContext`` :30, ``GlobMatcher`` :49) and utils.py (``load_quantization_recipe`` :28).
"""
from __future__ import annotations

import fnmatch
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass
class MatchContext:
    module_path: str
    layer_number: Optional[int] = None


@dataclass
class GlobMatcher:
    pattern: str
    config_key: str

    def match(self, ctx: MatchContext) -> Optional[str]:
        return self.config_key if fnmatch.fnmatch(ctx.module_path, self.pattern) else None


@dataclass
class QuantizationConfig:
    config: Dict[str, Any]
    match_input: MatchContext
    config_key: str


@dataclass
class RecipeConfig:
    matchers: List[GlobMatcher] = field(default_factory=list)
    config_dict: Dict[str, Dict[str, Any]] = field(default_factory=dict)

    @staticmethod
    def from_config_dict(d: Dict) -> "RecipeConfig":
        ms = []
        for name, m in d.get("matchers", {}).items():
            if not m.get("enabled", True):
                continue
            if m.get("type", "glob") != "glob":
                raise NotImplementedError(f"matcher type {m['type']}")
            ms.append(GlobMatcher(m["pattern"], m["config"]))
        return RecipeConfig(ms, dict(d.get("configs", {})))

    @staticmethod
    def from_yaml_file(path: str) -> "RecipeConfig":
        import yaml
        with open(path) as f:
            return RecipeConfig.from_config_dict(yaml.safe_load(f))

    def match(self, ctx: MatchContext) -> Optional[QuantizationConfig]:
        for m in self.matchers:                      # first match wins
            key = m.match(ctx)
            if key is not None:
                return QuantizationConfig(self.config_dict[key], ctx, key)
        return None


def apply_recipe(model, recipe: RecipeConfig) -> Dict[str, str]:
    """Tag every linear of ``model`` with the recipe that matches its dotted path; a config with
    ``{"fp8": false}`` switches the FP8 path off for that module.  Returns {path: config key}."""
    from ..parallel.layers import ColumnParallelLinear, RowParallelLinear
    chosen = {}
    for name, mod in model.named_modules():
        if isinstance(mod, (ColumnParallelLinear, RowParallelLinear)):
            q = recipe.match(MatchContext(name))
            if q is not None:
                mod.quant_config = q
                if q.config.get("fp8") is False:
                    mod.fp8_eligible = False
                chosen[name] = q.config_key
    return chosen
