"""Explicit process-group bundles, the alternative to the global getters of ``parallel.state``
(reference: megatron/core/process_groups_config.py:14-178)."""
from __future__ import annotations

from dataclasses import dataclass, field, fields
from typing import List, Optional

from . import state


@dataclass
class ModelCommProcessGroups:
    tp: object = None
    pp: object = None
    mp: object = None
    embd: object = None
    pos_embd: object = None
    cp: object = None
    tp_cp: object = None
    hcp: Optional[List[object]] = None
    ep: object = None
    expt_tp: object = None
    tp_ep: object = None
    tp_ep_pp: object = None
    tp_dp_cp: object = None

    @classmethod
    def use_mpu_process_groups(cls, required_pgs: Optional[List[str]] = None) -> "ModelCommProcessGroups":
        getters = {
            "tp": state.get_tensor_model_parallel_group, "pp": state.get_pipeline_model_parallel_group,
            "mp": state.get_model_parallel_group, "embd": state.get_embedding_group,
            "pos_embd": state.get_position_embedding_group, "cp": state.get_context_parallel_group,
            "tp_cp": state.get_tensor_and_context_parallel_group,
            "hcp": state.get_hierarchical_context_parallel_groups, "ep": state.get_expert_model_parallel_group,
            "expt_tp": state.get_expert_tensor_parallel_group,
            "tp_ep": state.get_expert_tensor_and_model_parallel_group,
            "tp_ep_pp": state.get_expert_tensor_model_pipeline_parallel_group,
            "tp_dp_cp": lambda: state.get_tensor_and_data_parallel_group(with_context_parallel=True),
        }
        names = required_pgs if required_pgs is not None else list(getters)
        for n in names:
            if n not in getters:
                raise ValueError(f"unknown process group {n}")
        return cls(**{n: getters[n]() for n in names})


@dataclass
class GradCommProcessGroups:
    dp: object = None
    dp_cp: object = None
    expt_dp: object = None
    intra_dp_cp: object = None
    intra_expt_dp: object = None
    inter_dist_opt: object = None

    @classmethod
    def use_mpu_process_groups(cls) -> "GradCommProcessGroups":
        return cls(dp=state.get_data_parallel_group(), dp_cp=state.get_data_parallel_group(with_context_parallel=True),
                   expt_dp=state.get_expert_data_parallel_group(),
                   intra_dp_cp=state.get_data_parallel_group(with_context_parallel=True, partial_data_parallel=True))
