"""Knowledge distillation losses and the loss balancer.

Reference: megatron/post_training/algos/distillation.py (``LogitsKLLoss`` :232 with tensor-parallel
softmax statistics, ``HiddenStateCosineLoss`` :180, ``MSELoss`` :158, ``LogitsAndIntermediatesLossBalancer``
:372, projection layer :425).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F


class LogitsKLLoss(nn.Module):
    """KL(teacher || student) per token over a vocabulary that may be split over a tensor-parallel group:
    the soft-max normalisers are reduced over the group, so each rank only touches its vocabulary shard."""

    def __init__(self, temperature: float = 1.0, reverse: bool = False, tp_group=None):
        super().__init__()
        self.t, self.reverse, self.group = temperature, reverse, tp_group

    def _log_softmax(self, x):
        x = x.float() / self.t
        mx = x.max(dim=-1, keepdim=True).values
        if self.group is not None and dist.get_world_size(self.group) > 1:
            dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=self.group)
        x = x - mx
        denom = x.exp().sum(dim=-1, keepdim=True)
        if self.group is not None and dist.get_world_size(self.group) > 1:
            denom = _AllReduceSum.apply(denom, self.group)
        return x - denom.log()

    def forward(self, student_logits, teacher_logits):
        s = self._log_softmax(student_logits)
        with torch.no_grad():
            t = self._log_softmax(teacher_logits)
        if self.reverse:
            kl = (s.exp() * (s - t)).sum(dim=-1)
        else:
            kl = (t.exp() * (t - s)).sum(dim=-1)
        if self.group is not None and dist.get_world_size(self.group) > 1:
            kl = _AllReduceSum.apply(kl, self.group)
        return kl * (self.t ** 2)


class _AllReduceSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        x = x.clone()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class HiddenStateCosineLoss(nn.Module):
    def __init__(self, student_hidden: int, teacher_hidden: int):
        super().__init__()
        self.proj = nn.Linear(student_hidden, teacher_hidden) if student_hidden != teacher_hidden else nn.Identity()

    def forward(self, student, teacher):
        s = self.proj(student).float()
        return 1.0 - F.cosine_similarity(s, teacher.float().detach(), dim=-1)


class MSELoss(nn.Module):
    def forward(self, student, teacher):
        return F.mse_loss(student.float(), teacher.float().detach(), reduction="none").sum(dim=-1)


class LogitsAndIntermediatesLossBalancer(nn.Module):
    """total = original + kd_scale * (logits KD + intermediates rescaled to the logits loss' magnitude);
    ``skip_original_loss`` drops the first term."""

    def __init__(self, kd_loss_scale: float = 1.0, skip_original_loss: bool = False):
        super().__init__()
        self.scale, self.skip = kd_loss_scale, skip_original_loss

    def forward(self, losses: Dict[str, torch.Tensor]) -> torch.Tensor:
        original = losses.pop("original", None)
        logits = [v for k, v in losses.items() if "logits" in k.lower()]
        inter = [v for k, v in losses.items() if "logits" not in k.lower()]
        kd = sum(logits) if logits else torch.zeros(())
        if inter:
            isum = sum(inter)
            kd = kd + isum * (kd.detach() / isum.detach().clamp(min=1e-8) if logits else 1.0)
        if original is None or self.skip:
            return kd * self.scale
        dyn = original.detach() / kd.detach().clamp(min=1e-8)
        return original + kd * dyn * self.scale


# ---------------------------------------------------------------------------------------------- the distillation model
class ProjectionLayer(nn.Module):
    """Student hidden size -> teacher hidden size, shared by every intermediate pair (identity when they agree).
    Reference: megatron/post_training/algos/distillation.py:384-419."""

    def __init__(self, student_hidden: int, teacher_hidden: int, init_std: float = 0.02, dtype=None):
        super().__init__()
        if student_hidden == teacher_hidden:
            self.proj = nn.Identity()
        else:
            self.proj = nn.Linear(student_hidden, teacher_hidden, dtype=dtype)
            nn.init.normal_(self.proj.weight, std=init_std)
            nn.init.zeros_(self.proj.bias)

    def forward(self, x):
        return self.proj(x)


def adjust_layer_index_for_pp(name: str, layer_offset: int) -> str:
    """``decoder.layers.<global>.x`` -> ``decoder.layers.<local>.x`` on a pipeline stage that starts at
    ``layer_offset`` (reference: distillation.py:99-119); a layer before this stage is an error."""
    import re
    m = re.search(r"(?<=\.)\d+(?=\.|$)", name)
    if not m:
        return name
    local = int(m.group(0)) - layer_offset
    if local < 0:
        raise ValueError(f"layer {name} does not live on the last pipeline stage")
    return name[:m.start()] + str(local) + name[m.end():]


def load_distillation_config(path: Optional[str], student_cfg, teacher_cfg, *, tp_group=None, layer_offsets=(0, 0),
                             last_stage: bool = True) -> Dict:
    """The YAML of ``--export-kd-cfg``: ``logit_layers`` [student, teacher], ``intermediate_layer_pairs``
    [[student, teacher], ...], ``skip_lm_loss``, ``kd_loss_scale`` (+ ``logit_kl_temperature``).  Without a file:
    logits only, language-model loss skipped.  Returns the dict with ``criterion`` {(student, teacher): loss module}
    and ``loss_balancer`` added; the criteria exist on the last pipeline stage only."""
    if path:
        import yaml
        with open(path) as f:
            cfg = dict(yaml.safe_load(f))
    else:
        cfg = {}
    cfg.setdefault("logit_layers", ["output_layer", "output_layer"])
    cfg.setdefault("intermediate_layer_pairs", [])
    cfg.setdefault("skip_lm_loss", True)
    cfg.setdefault("kd_loss_scale", 1.0)
    criterion = {}
    if last_stage:
        criterion[tuple(cfg["logit_layers"])] = LogitsKLLoss(cfg.get("logit_kl_temperature", 1.0), tp_group=tp_group)
        proj = ProjectionLayer(student_cfg.hidden_size, teacher_cfg.hidden_size, student_cfg.init_method_std,
                               dtype=getattr(student_cfg, "params_dtype", None))
        for s_name, t_name in cfg["intermediate_layer_pairs"]:
            key = (adjust_layer_index_for_pp(s_name, layer_offsets[0]), adjust_layer_index_for_pp(t_name, layer_offsets[1]))
            criterion[key] = _ProjectedCosine(proj)
    cfg["criterion"] = criterion
    cfg["loss_balancer"] = LogitsAndIntermediatesLossBalancer(cfg["kd_loss_scale"], cfg["skip_lm_loss"])
    return cfg


class _ProjectedCosine(nn.Module):
    def __init__(self, proj: ProjectionLayer):
        super().__init__()
        self.proj = proj

    def forward(self, student, teacher):
        return 1.0 - F.cosine_similarity(self.proj(student).float(), teacher.float().detach(), dim=-1)


def _first(x):
    return x[0] if isinstance(x, (tuple, list)) else x


class DistillationModel(nn.Module):
    """A student with a frozen teacher riding along.

    ``forward`` runs the teacher without gradients, then the student, on the same arguments; forward hooks keep the
    outputs of the layers named in the configuration.  ``compute_kd_loss(student_loss, loss_reduction_fn)`` evaluates
    the criteria on the kept tensors and balances them against the student's own loss.  The teacher is not a
    registered sub-module: parameters, gradients buffers, optimizers and checkpoints see the student (and the
    projection layer) only.  Between pipeline stages the two hidden states travel side by side in one tensor
    (``adjust_tensor_shapes``).  Reference: megatron/post_training/algos/distillation.py:451-569."""

    def __init__(self, student: nn.Module, teacher: nn.Module, kd_cfg: Dict):
        super().__init__()
        self.student = student
        object.__setattr__(self, "_teacher", teacher)
        teacher.eval()
        for p in teacher.parameters():
            p.requires_grad_(False)
        self.criteria = nn.ModuleDict()
        self._pairs = []
        self._kept: Dict[str, torch.Tensor] = {}
        s_mods, t_mods = dict(student.named_modules()), dict(teacher.named_modules())
        for i, ((s_name, t_name), crit) in enumerate(kd_cfg["criterion"].items()):
            if s_name not in s_mods or t_name not in t_mods:
                raise KeyError(f"distillation layer pair ({s_name}, {t_name}) not found in the models")
            self.criteria[f"c{i}"] = crit
            self._pairs.append((s_name, t_name, f"c{i}"))
            s_mods[s_name].register_forward_hook(self._keep(f"s:{s_name}"))
            t_mods[t_name].register_forward_hook(self._keep(f"t:{t_name}"))
        self.loss_balancer = kd_cfg["loss_balancer"]
        self.only_student = False
        self.config = student.config
        self.pre_process = getattr(student, "pre_process", True)
        self.post_process = getattr(student, "post_process", True)
        self._t_hidden = getattr(teacher.config, "hidden_size", None)
        self._s_hidden = student.config.hidden_size

    @property
    def teacher(self):
        return self._teacher

    @property
    def module(self):
        """Checkpoint code unwraps ``.module`` chains down to the model it saves: the student."""
        return self.student

    def _keep(self, key):
        def hook(_mod, _inp, out):
            self._kept[key] = _first(out)
        return hook

    # -- pipeline plumbing: [s, b, hs + ht] between stages
    def adjust_tensor_shapes(self, shape):
        return tuple(shape[:-1]) + (self._s_hidden + self._t_hidden,)

    def set_input_tensor(self, input_tensor):
        t = _first(input_tensor)
        if t is None:
            self.student.set_input_tensor(None)
            self._teacher.set_input_tensor(None)
            return
        if self.only_student:
            self.student.set_input_tensor(t)
            return
        s, th = torch.split(t, [self._s_hidden, self._t_hidden], dim=-1)
        self.student.set_input_tensor(s.contiguous())
        self._teacher.set_input_tensor(th.detach().contiguous())

    def train(self, mode: bool = True):
        super().train(mode)
        self._teacher.eval()
        return self

    def forward(self, *args, **kwargs):
        self._kept.clear()
        # evaluation needs the student only; between pipeline stages the two hidden states still travel together,
        # so the teacher keeps running there to hold the exchanged shape
        run_teacher = not self.only_student and (self.training or not (self.pre_process and self.post_process))
        if run_teacher:
            t_kwargs = dict(kwargs)
            t_kwargs.pop("labels", None)                     # the teacher's own loss is never needed
            with torch.no_grad():
                t_out = self._teacher(*args, **t_kwargs)
        s_out = self.student(*args, **kwargs)
        if self.post_process or not run_teacher:
            return s_out
        return torch.cat([s_out, t_out.detach().to(s_out.dtype)], dim=-1)

    def compute_kd_loss(self, student_loss: Optional[torch.Tensor] = None,
                        loss_reduction_fn=None) -> torch.Tensor:
        """Balanced total of the student's loss and the distillation terms.  ``loss_reduction_fn`` maps a per-token
        tensor ([s, b]) to a scalar the way the program reduces its own loss (mask, mean)."""
        losses: Dict[str, torch.Tensor] = {}
        for s_name, t_name, key in self._pairs:
            crit = self.criteria[key]
            val = crit(self._kept[f"s:{s_name}"], self._kept[f"t:{t_name}"])
            if loss_reduction_fn is not None:
                val = loss_reduction_fn(val)
            else:
                val = val.mean()
            kind = "logits" if isinstance(crit, LogitsKLLoss) else "intermediate"
            losses[f"{kind}_{key}"] = val
        if student_loss is not None:
            losses["original"] = student_loss
        self.last_losses = {k: v.detach() for k, v in losses.items()}
        return self.loss_balancer(losses)

    # -- checkpoints hold the student only
    def state_dict(self, *args, **kwargs):
        return self.student.state_dict(*args, **kwargs)

    def load_state_dict(self, sd, strict: bool = True, **kw):
        return self.student.load_state_dict(sd, strict=strict, **kw)

    def sharded_state_dict(self, *args, **kwargs):
        return self.student.sharded_state_dict(*args, **kwargs)

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            student = self.__dict__.get("_modules", {}).get("student")
            if student is None:
                raise
            return getattr(student, name)


def unwrap_distillation_model(model) -> Optional[DistillationModel]:
    m = model
    while not isinstance(m, DistillationModel) and hasattr(m, "module"):
        m = m.module
    return m if isinstance(m, DistillationModel) else None


def masked_token_mean(loss_mask: torch.Tensor, tp_group=None):
    """Reduction for per-token distillation terms: ``[s, b]`` (or, under sequence parallelism, this rank's
    ``[s / tp, b]`` slice) -> masked mean over the whole micro-batch (reference: loss_func.py:15-44 ``_mask_loss``)."""
    mask = loss_mask.float().t().contiguous()                  # [s, b]
    denom = mask.sum().clamp(min=1.0)

    def reduce(val: torch.Tensor) -> torch.Tensor:
        if val.shape[0] != mask.shape[0]:
            world = dist.get_world_size(tp_group)
            rank = dist.get_rank(tp_group)
            per = mask.shape[0] // world
            part = (val.float() * mask[rank * per:(rank + 1) * per]).sum()
            return _AllReduceSum.apply(part.reshape(1), tp_group).squeeze(0) / denom
        return (val.float() * mask).sum() / denom
    return reduce


def distillation_loss_func(loss_mask: torch.Tensor, output_tensor: torch.Tensor, model, tp_group=None):
    """Loss function of a program that trains a ``DistillationModel``: the student's masked loss and the balanced
    distillation total, returned in the (sum, token count, report) form of the pre-training programs
    (reference: megatron/post_training/loss_func.py:64-96)."""
    dm = unwrap_distillation_model(model)
    mask = loss_mask.view(-1).float()
    tokens = mask.sum()
    lm_sum = torch.sum(output_tensor.float().view(-1) * mask)
    report = {"lm loss": torch.stack([lm_sum.detach(), tokens.detach()])}
    if dm is None or not dm.training:
        return lm_sum, tokens.to(torch.int64), report
    lm_mean = lm_sum / tokens.clamp(min=1.0)
    total = dm.compute_kd_loss(student_loss=lm_mean, loss_reduction_fn=masked_token_mean(loss_mask, tp_group))
    for k, v in dm.last_losses.items():
        if k != "original":
            name = "kd logits loss" if k.startswith("logits") else f"kd {k} loss"
            report[name] = torch.stack([v.float() * tokens.detach(), tokens.detach()])
    report["kd total loss"] = torch.stack([total.detach() * tokens.detach(), tokens.detach()])
    return total * tokens, tokens.to(torch.int64), report
