"""Command line surface and small runtime utilities: argument parsing / validation / config objects, YAML overlay,
timers, the microbatch calculator with batch-size ramp-up, FLOP and memory models, energy monitor (fake NVML),
config logger.  Mirrors the reference's tests/unit_tests/test_num_microbatches_calculator.py, test_utilities,
test_training.py and the argument checks of megatron/training/arguments.py."""
import json
import time

import pytest
import torch

from megatron_lm_b200.training import arguments as A

BASE = ["--num-layers", "4", "--hidden-size", "64", "--num-attention-heads", "4", "--seq-length", "128",
        "--micro-batch-size", "2", "--train-iters", "10", "--lr", "1e-3"]


def _args(extra=(), world=1, monkeypatch=None):
    if monkeypatch is not None:
        monkeypatch.setenv("WORLD_SIZE", str(world))
    return A.parse_args(argv=BASE + list(extra))


def test_flag_surface_matches_the_reference_count():
    from megatron_lm_b200.training.flag_table import FLAGS
    assert len(FLAGS) >= 498
    parser = A.build_parser()
    dests = {a.dest for a in parser._actions}
    for must in ("tensor_model_parallel_size", "pipeline_model_parallel_size", "use_distributed_optimizer",
                 "sequence_parallel", "num_experts", "moe_router_topk", "fp8", "recompute_granularity",
                 "rampup_batch_size", "rerun_mode", "ckpt_format", "tp_comm_overlap", "context_parallel_size"):
        assert must in dests, must


def test_defaults_are_derived(monkeypatch):
    a = A.validate_args(_args(["--swiglu", "--bf16"], world=4, monkeypatch=monkeypatch))
    assert a.data_parallel_size == 4 and a.global_batch_size == 8
    assert a.ffn_hidden_size == int((4 * 64 * 2 / 3) / 64) * 64
    assert a.kv_channels == 16 and a.num_query_groups == 4 and a.max_position_embeddings == 128
    assert a.params_dtype == torch.bfloat16 and a.accumulate_allreduce_grads_in_fp32
    assert a.virtual_pipeline_model_parallel_size is None


def test_virtual_pipeline_and_parallel_sizes(monkeypatch):
    a = A.validate_args(_args(["--tensor-model-parallel-size", "2", "--pipeline-model-parallel-size", "2",
                               "--num-layers-per-virtual-pipeline-stage", "1", "--sequence-parallel",
                               "--global-batch-size", "16"], world=8, monkeypatch=monkeypatch))
    assert a.data_parallel_size == 2 and a.virtual_pipeline_model_parallel_size == 2 and a.sequence_parallel
    a = A.validate_args(_args(["--sequence-parallel"], world=1, monkeypatch=monkeypatch))
    assert not a.sequence_parallel                          # meaningless without tensor parallelism


@pytest.mark.parametrize("extra,world,msg", [
    (["--tensor-model-parallel-size", "3"], 4, "divisible"),
    (["--fp16", "--bf16"], 1, "mutually exclusive"),
    (["--global-batch-size", "3"], 1, "multiple"),
    (["--num-layers-per-virtual-pipeline-stage", "1"], 1, "pipeline"),
    (["--tp-comm-overlap"], 1, "sequence-parallel"),
    (["--overlap-param-gather"], 1, "distributed-optimizer"),
    (["--expert-model-parallel-size", "2"], 2, "num-experts"),
    (["--num-experts", "3", "--expert-model-parallel-size", "2"], 2, "divisible"),
    (["--min-lr", "1.0"], 1, "min-lr"),
    (["--save", "/tmp/x"], 1, "save-interval"),
    (["--train-samples", "100"], 1, "either"),
    (["--context-parallel-size", "2", "--seq-length", "6"], 2, "seq-length"),
])
def test_inconsistent_arguments_are_rejected(extra, world, msg, monkeypatch):
    with pytest.raises(ValueError, match=msg):
        A.validate_args(_args(extra, world=world, monkeypatch=monkeypatch))


def test_config_objects_from_args(monkeypatch):
    a = A.validate_args(_args(["--swiglu", "--normalization", "RMSNorm", "--disable-bias-linear", "--bf16",
                               "--use-distributed-optimizer", "--overlap-grad-reduce", "--clip-grad", "0.5",
                               "--num-experts", "4", "--moe-router-topk", "2", "--group-query-attention",
                               "--num-query-groups", "2", "--position-embedding-type", "rope"],
                              monkeypatch=monkeypatch))
    cfg = A.core_transformer_config_from_args(a)
    assert cfg.num_layers == 4 and cfg.gated_linear_unit and cfg.normalization == "RMSNorm" and not cfg.add_bias_linear
    assert cfg.num_moe_experts == 4 and cfg.moe_router_topk == 2 and cfg.num_query_groups == 2 and cfg.bf16
    oc = A.optimizer_config_from_args(a)
    assert oc.lr == 1e-3 and oc.clip_grad == 0.5 and oc.use_distributed_optimizer and oc.bf16
    dc = A.ddp_config_from_args(a)
    assert dc.use_distributed_optimizer and dc.overlap_grad_reduce and dc.grad_reduce_in_fp32


def test_yaml_overlay_and_global_args(tmp_path, monkeypatch):
    p = tmp_path / "cfg.yaml"
    p.write_text("model:\n  hidden_size: 96\n  num_attention_heads: 6\ntraining:\n  micro_batch_size: 3\n")
    a = A.load_yaml_args(str(p), _args(monkeypatch=monkeypatch))
    a = A.validate_args(a)
    assert a.hidden_size == 96 and a.kv_channels == 16 and a.micro_batch_size == 3
    A.set_args(a)
    assert A.get_args() is a


# ------------------------------------------------------------------------------------------------ timers
def test_timers_levels_and_report():
    from megatron_lm_b200.utils.timers import Timers
    t = Timers(log_level=1, log_option="minmax")
    t("step", log_level=0).start()
    time.sleep(0.02)
    t("step").stop()
    t("detail", log_level=2).start()                     # above the configured level: a no-op
    t("detail", log_level=2).stop()
    with pytest.raises(RuntimeError):
        t("step").stop()
    with pytest.raises(ValueError):
        t("step", log_level=1)
    with pytest.raises(ValueError):
        t("x", log_level=5)
    s = t.get_all_timers_string(reset=False)
    assert "step" in s and "detail" not in s and "(min, max)" in s
    e = t("step").elapsed(reset=True)
    assert 0.015 < e < 0.5 and t("step").elapsed() == 0.0

    class W:
        def __init__(self): self.rows = []
        def add_scalar(self, k, v, it): self.rows.append((k, v, it))
    t("step").start(); t("step").stop()
    w = W()
    t.write(["step", "missing"], w, 7)
    assert w.rows and w.rows[0][0] == "step-time" and w.rows[0][2] == 7


# ------------------------------------------------------------------------------------------------ microbatches
def test_constant_microbatch_calculator():
    from megatron_lm_b200.utils import num_microbatches_calculator as M
    M.init_num_microbatches_calculator(0, None, 32, 2, 4)
    assert M.get_num_microbatches() == 4 and M.get_current_global_batch_size() == 32 and M.get_micro_batch_size() == 2
    M.update_num_microbatches(1000)
    assert M.get_num_microbatches() == 4
    with pytest.raises(ValueError):
        M.init_num_microbatches_calculator(0, None, 30, 4, 4)
    M.init_num_microbatches_calculator(0, None, 30, 4, 4, decrease_batch_size_if_needed=True)
    assert M.get_current_running_global_batch_size() == 16 and M.get_num_microbatches() == 1
    M.destroy_num_microbatches_calculator()


def test_rampup_microbatch_calculator():
    from megatron_lm_b200.utils import num_microbatches_calculator as M
    # 16 -> 48 in steps of 16 over 96 samples: 2 increments, 48 samples each
    M.init_num_microbatches_calculator(0, [16, 16, 96], 48, 2, 2)
    assert M.get_current_global_batch_size() == 16 and M.get_num_microbatches() == 4
    M.update_num_microbatches(47)
    assert M.get_current_global_batch_size() == 16
    M.update_num_microbatches(48)
    assert M.get_current_global_batch_size() == 32 and M.get_num_microbatches() == 8
    M.update_num_microbatches(97)
    assert M.get_current_global_batch_size() == 48 and M.get_num_microbatches() == 12
    with pytest.raises(ValueError):
        M.init_num_microbatches_calculator(0, [16, 10, 96], 48, 2, 2)
    with pytest.raises(ValueError):
        M.init_num_microbatches_calculator(0, [16, 16], 48, 2, 2)
    M.destroy_num_microbatches_calculator()


# ------------------------------------------------------------------------------------------------ models of cost
def test_flops_model_matches_hand_count():
    from megatron_lm_b200.training.flops import num_floating_point_operations
    # Llama-2-7B at 4096: 42.86 GFLOP per token (fwd+bwd), GPT-3 1.3B at 2048: 8.47
    f = num_floating_point_operations(batch_size=1, seq_length=4096, num_layers=32, hidden_size=4096,
                                      num_attention_heads=32, ffn_hidden_size=11008, padded_vocab_size=32000, swiglu=True)
    assert f / 4096 / 1e9 == pytest.approx(42.86, abs=0.02)
    g = num_floating_point_operations(batch_size=1, seq_length=2048, num_layers=24, hidden_size=2048,
                                      num_attention_heads=16, ffn_hidden_size=8192, padded_vocab_size=50304)
    assert g / 2048 / 1e9 == pytest.approx(8.47, abs=0.02)
    h, s, v, L = 64, 32, 100, 2
    hand = 3 * 2 * s * (L * (4 * h * h + 2 * s * h / 2 * 1 + 2 * h * 4 * h) + h * v)
    got = num_floating_point_operations(batch_size=1, seq_length=s, num_layers=L, hidden_size=h, num_attention_heads=4,
                                        padded_vocab_size=v)
    assert got == pytest.approx(hand, rel=1e-9)
    moe = num_floating_point_operations(batch_size=1, seq_length=s, num_layers=L, hidden_size=h, num_attention_heads=4,
                                        padded_vocab_size=v, num_experts=8, moe_router_topk=2)
    assert moe > got                                           # two experts per token cost twice the MLP


def test_theoretical_memory_scales_with_sharding(monkeypatch):
    from megatron_lm_b200.training.theoretical_memory_usage import report_theoretical_memory
    a = A.validate_args(_args(["--swiglu", "--bf16", "--vocab-size", "1000"], monkeypatch=monkeypatch))
    a.padded_vocab_size = 1024
    r1 = report_theoretical_memory(a, num_microbatches=4)
    a8 = A.validate_args(_args(["--swiglu", "--bf16", "--use-distributed-optimizer", "--vocab-size", "1000"],
                               world=8, monkeypatch=monkeypatch))
    a8.padded_vocab_size = 1024
    r8 = report_theoretical_memory(a8, num_microbatches=4)
    k = [x for x in r1 if "weight" in x][0]
    assert r8[k] < r1[k]                                       # optimizer state sharded 8 ways
    assert all(v > 0 for v in r1.values() if isinstance(v, (int, float)))


# ------------------------------------------------------------------------------------------------ energy / config log
class _FakeNvml:
    def __init__(self): self.mj, self.inited, self.down = 1_000_000, False, False
    def nvmlInit(self): self.inited = True
    def nvmlShutdown(self): self.down = True
    def nvmlDeviceGetHandleByIndex(self, i): return ("h", i)
    def nvmlDeviceGetTotalEnergyConsumption(self, h): return self.mj


def test_energy_monitor_reads_only_the_counter():
    from megatron_lm_b200.utils.energy_monitor import EnergyMonitor
    nv = _FakeNvml()
    m = EnergyMonitor(nvml=nv, device_index=0)
    m.setup()
    m.resume()
    nv.mj += 5000
    assert m.lap() == pytest.approx(5.0)
    nv.mj += 2000
    m.pause()
    nv.mj += 100000                                            # paused: not counted
    m.resume()
    nv.mj += 1000
    assert m.lap() == pytest.approx(3.0) and m.get_total() == pytest.approx(8.0)
    m.shutdown()
    assert nv.inited and nv.down
    assert not [n for n in dir(nv) if "Set" in n]              # nothing on the device is ever written


def test_config_logger_writes_json(tmp_path):
    from megatron_lm_b200.config import TransformerConfig
    from megatron_lm_b200.utils.config_logger import has_config_logger_enabled, log_config_to_disk
    cfg = TransformerConfig(num_layers=2, hidden_size=32, num_attention_heads=4, config_logger_dir=str(tmp_path))
    assert has_config_logger_enabled(cfg)
    p1 = log_config_to_disk(cfg, {"config": cfg, "dtype": torch.bfloat16, "fn": test_config_logger_writes_json}, "gpt")
    p2 = log_config_to_disk(cfg, {"x": [1, (2, 3)]}, "gpt")
    assert p1 != p2
    d = json.load(open(p1))
    assert d["config"]["hidden_size"] == 32 and d["dtype"] == "torch.bfloat16" and d["fn"] == "test_config_logger_writes_json"


def test_logging_setup_filters_quiet_loggers(capsys):
    import logging
    from megatron_lm_b200.utils.log_handler import StdoutHandler, setup_logging
    root = logging.getLogger()
    before = list(root.handlers)
    try:
        assert setup_logging(logging.WARNING) == logging.WARNING and root.level == logging.WARNING
        setup_logging(logging.INFO)
        assert sum(isinstance(h, StdoutHandler) for h in root.handlers) == 1          # installed once
        h = next(h for h in root.handlers if isinstance(h, StdoutHandler))
        mk = lambda name: logging.LogRecord(name, logging.INFO, __file__, 1, "m", None, None)
        assert h.filter(mk("megatron_lm_b200.training")) and not h.filter(mk("torch.distributed.elastic"))
    finally:
        root.handlers[:] = before


# ----------------------------------------------------------------------------- flags that nothing acts on
def _flags_nobody_reads():
    """Destinations of the flag table that appear nowhere in the package sources (the table of unused flags in
    arguments.py itself is cut out of the scan)."""
    import os
    import re
    from megatron_lm_b200.training.flag_table import FLAGS
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    texts = []
    for base, _, files in os.walk(os.path.join(root, "megatron_lm_b200")):
        for f in files:
            if not f.endswith(".py") or f == "flag_table.py":
                continue
            t = open(os.path.join(base, f)).read()
            if f == "arguments.py" and os.path.basename(base) == "training":
                a = t.index("UNUSED_FLAGS = {")
                t = t[:a] + t[t.index("\n}\n", a):]
            texts.append(t)
    for f in os.listdir(root):
        if f.startswith("pretrain_") and f.endswith(".py"):
            texts.append(open(os.path.join(root, f)).read())
    text = "\n".join(texts)
    out = set()
    for _, flags, kw in FLAGS:
        dest = kw.get("dest") or flags[0].lstrip("-").replace("-", "_")
        if not re.search(r"\b" + re.escape(dest) + r"\b", text):
            out.add(dest)
    return out


def test_every_flag_is_read_or_declared_unused():
    from megatron_lm_b200.training.arguments import UNUSED_FLAGS
    unread = _flags_nobody_reads()
    assert unread - set(UNUSED_FLAGS) == set(), f"parsed but silently ignored: {sorted(unread - set(UNUSED_FLAGS))}"
    assert set(UNUSED_FLAGS) - unread == set(), f"listed as unused but read somewhere: {sorted(set(UNUSED_FLAGS) - unread)}"
    assert all(kind in ("warn", "refuse") and why for kind, why in UNUSED_FLAGS.values())


def test_unused_flags_warn_or_refuse():
    import warnings
    from megatron_lm_b200.training.arguments import parse_args, validate_args
    base = ["--num-layers", "2", "--hidden-size", "32", "--num-attention-heads", "4", "--seq-length", "16",
            "--max-position-embeddings", "16", "--micro-batch-size", "1", "--train-iters", "1", "--lr", "1e-3"]
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        args = parse_args(argv=base + ["--use-flash-attn", "--adlr-autoresume-interval", "10"])
        args.world_size, args.rank = 1, 0
        validate_args(args)
    msgs = [str(x.message) for x in w]
    assert any("--use-flash-attn" in m for m in msgs) and any("--adlr-autoresume-interval" in m for m in msgs)
    # defaults do not warn
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        args = parse_args(argv=base)
        args.world_size, args.rank = 1, 0
        validate_args(args)
    assert not [x for x in w if "has no effect here" in str(x.message)]
    # a flag that would change the layout or the numerics stops the run
    for extra in (["--use-legacy-models"], ["--checkpoint-activations"], ["--lazy-mpu-init", "true"]):
        args = parse_args(argv=base + extra)
        args.world_size, args.rank = 1, 0
        with pytest.raises(ValueError, match="not supported"):
            validate_args(args)


def test_renaming_flags_are_plumbed():
    from megatron_lm_b200.training.arguments import (core_transformer_config_from_args, ddp_config_from_args, parse_args,
                                                      validate_args)
    base = ["--num-layers", "6", "--hidden-size", "32", "--num-attention-heads", "4", "--seq-length", "16",
            "--max-position-embeddings", "16", "--micro-batch-size", "1", "--train-iters", "1", "--lr", "1e-3",
            "--pipeline-model-parallel-size", "2", "--decoder-first-pipeline-num-layers", "2",
            "--use-rotary-position-embeddings", "--bf16", "--grad-reduce-in-bf16", "--ddp-num-buckets", "3"]
    args = parse_args(argv=base)
    args.world_size, args.rank = 2, 0
    validate_args(args)
    cfg = core_transformer_config_from_args(args)
    assert cfg.num_layers_in_first_pipeline_stage == 2 and args.position_embedding_type == "rope"
    d = ddp_config_from_args(args)
    assert d.grad_reduce_in_fp32 is False and d.num_buckets == 3


def test_unsupported_config_fields_are_refused():
    from megatron_lm_b200.config import UNSUPPORTED_FIELDS, TransformerConfig
    base = dict(num_layers=1, hidden_size=32, num_attention_heads=4)
    TransformerConfig(**base)                                           # defaults pass
    for name, value in (("init_model_with_meta_device", True),
                        ("fp8_multi_head_attention", True), ("fp8_dot_product_attention", True)):
        assert name in UNSUPPORTED_FIELDS
        with pytest.raises(ValueError, match="not supported"):
            TransformerConfig(**base, **{name: value})


def test_flags_that_used_to_do_nothing(tmp_path, monkeypatch):
    """--openai-gelu, --data-args-path / --per-split-data-args-path, --save-retain-interval, the rejected-result
    tracker file, the server's token limit."""
    import os
    import torch.nn.functional as F
    from megatron_lm_b200.activations import BY_NAME
    a = A.validate_args(_args(["--openai-gelu"], monkeypatch=monkeypatch))
    assert A.core_transformer_config_from_args(a).activation_func == "openai_gelu"
    x = torch.linspace(-3, 3, 13)
    assert torch.allclose(BY_NAME["openai_gelu"](x), F.gelu(x, approximate="tanh"))
    assert not torch.allclose(BY_NAME["openai_gelu"](x), F.gelu(x), atol=1e-6)
    (tmp_path / "paths.txt").write_text("0.3 /data/a\n0.7 /data/b\n")
    (tmp_path / "split.json").write_text(json.dumps({"train": ["/d/t"], "valid": ["0.5", "/d/v1", "0.5", "/d/v2"]}))
    a = A.validate_args(_args(["--data-args-path", str(tmp_path / "paths.txt")], monkeypatch=monkeypatch))
    assert a.data_path == ["0.3", "/data/a", "0.7", "/data/b"]
    a = A.validate_args(_args(["--per-split-data-args-path", str(tmp_path / "split.json")], monkeypatch=monkeypatch))
    assert a.train_data_path == ["/d/t"] and a.valid_data_path == ["0.5", "/d/v1", "0.5", "/d/v2"]
    # retained checkpoints: multiples of the interval and the newest
    from megatron_lm_b200.training.checkpointing import cleanup_old_checkpoints
    for it in (2, 4, 6, 8, 10):
        os.makedirs(tmp_path / "ck" / f"iter_{it:07d}")
    os.makedirs(tmp_path / "ck" / "release")
    assert cleanup_old_checkpoints(str(tmp_path / "ck"), 10, 4) == [2, 6]
    assert sorted(os.listdir(tmp_path / "ck")) == ["iter_0000004", "iter_0000008", "iter_0000010", "release"]
    assert cleanup_old_checkpoints(str(tmp_path / "ck"), 10, None) == []
    # rejected results are written down
    from megatron_lm_b200.training.resilience import RerunStateMachine
    m = RerunStateMachine("validate_results")
    m.rejected_tracker_filename = str(tmp_path / "rejected.jsonl")
    assert m.should_run_forward_backward(None)
    m.validate_result(torch.tensor(float("nan")), lambda v: bool(torch.isnan(v)), "NaN loss")
    rec = json.loads(open(tmp_path / "rejected.jsonl").read().splitlines()[0])
    assert rec["message"] == "NaN loss" and rec["rank"] == 0 and not rec["injected"]
    # the server refuses requests that would need more tokens than allowed
    from megatron_lm_b200.inference.server import MegatronServer

    class Eng:
        tokenizer = None
    srv = MegatronServer(Eng(), max_tokens_to_oom=40)
    code, resp = srv.handle(json.dumps({"prompts": ["a b c d", "e f"], "tokens_to_generate": 20}).encode())
    assert code == 400 and "Too many tokens" in resp["message"] and "48" in resp["message"]


def test_example_scripts_use_known_flags():
    """Every ``--flag`` of the launch scripts under examples/ is known to the parser of the program it starts."""
    import glob
    import os
    import re
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    from megatron_lm_b200.inference.run_server import add_server_args
    from megatron_lm_b200.inference.run_vlm_generation import add_vlm_generation_args
    from megatron_lm_b200.post_training.arguments import add_modelopt_args
    from megatron_lm_b200.tasks.quantize_gpt import add_calib_args

    def extra(parser):
        for fn in (add_server_args, add_vlm_generation_args, add_calib_args):
            try:
                fn(parser)
            except Exception:
                pass
        g = parser.add_argument_group("program-specific")
        for f in ("--dino-out-dim", "--knn-bank-size"):
            g.add_argument(f)
        return parser
    parser = A.build_parser(extra)
    known = {o for a in parser._actions for o in a.option_strings}
    launcher = {"--nnodes", "--nproc-per-node", "--master-addr", "--master-port", "--standalone", "--local-addr",
                "--node-rank", "--rdzv-backend", "--rdzv-endpoint", "--rdzv-id", "--max-restarts",
                "--loader", "--saver", "--load-dir", "--save-dir", "--tokens-to-generate"}
    scripts = glob.glob(os.path.join(root, "examples", "**", "*.sh"), recursive=True)
    assert len(scripts) >= 8
    for path in scripts:
        text = "\n".join(l for l in open(path).read().splitlines() if not l.lstrip().startswith("#"))
        for flag in set(re.findall(r"(?<![\w-])--[a-z][a-z0-9-]*", text)):
            assert flag in known or flag in launcher, (os.path.relpath(path, root), flag)


def test_replication_flags_choose_the_copying_code(monkeypatch):
    a = A.validate_args(_args(["--non-persistent-ckpt-type", "local", "--non-persistent-save-interval", "5",
                               "--replication", "--replication-factor", "3"], world=4, monkeypatch=monkeypatch))
    assert (a.ec_data_shards, a.ec_parity_shards) == (1, 2)
    with pytest.raises(ValueError, match="local"):
        A.validate_args(_args(["--replication"], monkeypatch=monkeypatch))
    # one data member + two parity members: every parity chunk equals the data chunk (GF(2^8) Vandermonde row of ones
    # or not, a [1 x 1] systematic code multiplies by a non-zero constant), and any single member restores the stripe
    from megatron_lm_b200.checkpoint import gf256
    import numpy as np
    data = np.frombuffer(bytes(range(1, 33)), dtype=np.uint8)
    G = gf256.generator_matrix(1, 2) if hasattr(gf256, "generator_matrix") else None
    if G is not None:
        for row in np.asarray(G)[1:]:
            assert int(row[0]) != 0
