"""Explicit pipeline layer layouts (reference:
megatron/core/transformer/pipeline_parallel_layer_layout.py:14-266).

A layout string lists, stage by stage (virtual stages of rank 0, 1, ... then the next round), what
each stage holds: ``E`` embedding, ``t`` a transformer layer, ``m`` an MTP layer, ``L`` the loss;
stages are separated by ``|`` and ``x*N`` repeats, e.g. ``"Et*3|(tt|)*29,m|L"``."""
from __future__ import annotations

import re
from typing import List, Optional


def _expand(s: str) -> str:
    s = s.replace(",", "")
    pat = re.compile(r"\(([^()]*)\)\*(\d+)")
    while True:
        m = pat.search(s)
        if not m:
            break
        s = s[:m.start()] + m.group(1) * int(m.group(2)) + s[m.end():]
    pat2 = re.compile(r"([EtmL])\*(\d+)")
    while True:
        m = pat2.search(s)
        if not m:
            break
        s = s[:m.start()] + m.group(1) * int(m.group(2)) + s[m.end():]
    return s


class PipelineParallelLayerLayout:
    def __init__(self, layout, pipeline_model_parallel_size: int):
        if isinstance(layout, str):
            stages = [list(st) for st in _expand(layout).strip("|").split("|")]
        else:
            stages = [list(st) for st in layout]
        if len(stages) % pipeline_model_parallel_size != 0:
            raise ValueError("number of stages in the layout must be a multiple of the pipeline size")
        self.pp = pipeline_model_parallel_size
        self.vpp = len(stages) // pipeline_model_parallel_size
        # stage index s = v * pp + r
        self.layout = [[stages[v * self.pp + r] for v in range(self.vpp)] for r in range(self.pp)]
        flat = [x for st in stages for x in st]
        if flat.count("E") != 1 or flat.count("L") != 1:
            raise ValueError("layout needs exactly one embedding (E) and one loss (L)")
        if stages[0][0] != "E" or stages[-1][-1] != "L":
            raise ValueError("embedding must open the first stage and loss close the last")
        self.stages = stages

    @classmethod
    def from_config(cls, config):
        lay = config.pipeline_model_parallel_layout
        return lay if isinstance(lay, cls) else cls(lay, config.pipeline_model_parallel_size)

    def validate_layer_layout(self, num_layers: int, mtp_num_layers: Optional[int] = None):
        flat = [x for st in self.stages for x in st]
        if flat.count("t") != num_layers:
            raise ValueError(f"layout has {flat.count('t')} transformer layers, the model {num_layers}")
        if mtp_num_layers is not None and flat.count("m") != mtp_num_layers:
            raise ValueError("layout and model disagree on the number of MTP layers")

    def get_num_layers_to_build(self, pp_rank: int, vp_stage: Optional[int] = None, kind: str = "t") -> int:
        return self.layout[pp_rank][vp_stage or 0].count(kind)

    def get_layer_offset(self, pp_rank: int, vp_stage: Optional[int] = None, kind: str = "t") -> int:
        s = (vp_stage or 0) * self.pp + pp_rank
        return sum(st.count(kind) for st in self.stages[:s])

    def get_layer_id_list(self, pp_rank: int, vp_stage: Optional[int] = None, kind: str = "t") -> List[int]:
        o = self.get_layer_offset(pp_rank, vp_stage, kind)
        return list(range(o, o + self.get_num_layers_to_build(pp_rank, vp_stage, kind)))
