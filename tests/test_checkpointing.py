"""Sharded checkpoints: block algebra, integrity validation, save under one layout / load under another."""
import argparse
import os

import pytest
import torch

from megatron_lm_b200.checkpoint import sharded as ds
from tests.dist_utils import run_distributed


def test_block_overlap_reassembly(tmp_path):
    full = torch.arange(6 * 8, dtype=torch.float32).view(6, 8)
    # saved as 2x2 blocks
    sd = {}
    for i in range(2):
        for j in range(2):
            blk = full[i * 3:(i + 1) * 3, j * 4:(j + 1) * 4].clone()
            sd[f"b{i}{j}"] = ds.ShardedTensor.from_rank_offsets("w", blk, (0, i, 2), (1, j, 2))
    ds.save(sd, str(tmp_path))
    # loaded as 3 row stripes
    for r in range(3):
        req = {"x": ds.ShardedTensor.from_rank_offsets("w", torch.zeros(2, 8), (0, r, 3))}
        out = ds.load(req, str(tmp_path))
        assert torch.equal(out["x"], full[2 * r:2 * r + 2])
    # flattened range of a block (distributed-optimizer shard)
    blk = torch.zeros(3, 8)
    st = ds.ShardedTensor.from_rank_offsets("w", blk, (0, 1, 2))
    st.flattened_range = slice(5, 17)
    st.data = torch.zeros(12)
    out = ds.load({"x": st}, str(tmp_path))
    assert torch.equal(out["x"], full[3:6].reshape(-1)[5:17])


def test_integrity_validation_catches_holes(tmp_path):
    sd = {"a": ds.ShardedTensor.from_rank_offsets("w", torch.zeros(2, 4), (0, 0, 2))}     # second half missing
    with pytest.raises(ValueError):
        ds.save(sd, str(tmp_path))


def test_objects_and_common_state(tmp_path):
    sd = {"iteration": 7, "nested": {"lr": 0.5},
          "rng": ds.ShardedObject("rng", {"seed": 3}, (1, 1), (0, 0)),
          "w": ds.ShardedTensor.from_rank_offsets("w", torch.ones(2))}
    ds.save(sd, str(tmp_path))
    req = {"rng": ds.ShardedObject("rng", None, (1, 1), (0, 0)), "w": ds.ShardedTensor.from_rank_offsets("w", torch.zeros(2)),
           "keep": ds.LocalNonpersistentObject([1, 2])}
    out = ds.load(req, str(tmp_path))
    assert out["iteration"] == 7 and out["nested"]["lr"] == 0.5 and out["rng"] == {"seed": 3}
    assert out["keep"] == [1, 2] and torch.equal(out["w"], torch.ones(2))


def _args(d, **kw):
    ns = argparse.Namespace(save=d, load=d, ckpt_format="torch_dist", async_save=False, no_save_optim=False,
                            no_save_rng=False, no_load_optim=False, no_load_rng=False, finetune=False)
    for k, v in kw.items():
        setattr(ns, k, v)
    return ns


def _build(tp, pp, dist_opt, reinit=True):
    from megatron_lm_b200.config import DistributedDataParallelConfig, OptimizerConfig, TransformerConfig
    from megatron_lm_b200.models.gpt import GPTModel
    from megatron_lm_b200.training.training import setup_model_and_optimizer
    from tests.model_utils import reinit_by_global_name
    cfg = TransformerConfig(num_layers=4, hidden_size=32, num_attention_heads=4, ffn_hidden_size=64, hidden_dropout=0.0,
                            attention_dropout=0.0, tensor_model_parallel_size=tp, pipeline_model_parallel_size=pp,
                            normalization="RMSNorm", gated_linear_unit=True, activation_func="silu",
                            add_bias_linear=False, use_cpu_initialization=True)

    def provider(pre_process=True, post_process=True, vp_stage=None):
        m = GPTModel(cfg, 96, 16, pre_process=pre_process, post_process=post_process, position_embedding_type="rope")
        if reinit:
            reinit_by_global_name(m, cfg)
        else:
            with torch.no_grad():
                for p in m.parameters():
                    p.zero_()
        return m
    model, opt, _ = setup_model_and_optimizer(
        provider, cfg, OptimizerConfig(lr=1e-2, use_distributed_optimizer=dist_opt),
        DistributedDataParallelConfig(grad_reduce_in_fp32=True, use_distributed_optimizer=dist_opt))
    return cfg, model, opt


def _save_rank(rank, world, tp, pp, d):
    from megatron_lm_b200.parallel import state
    from megatron_lm_b200.training.checkpointing import save_checkpoint
    state.initialize_model_parallel(tensor_model_parallel_size=tp, pipeline_model_parallel_size=pp)
    cfg, model, opt = _build(tp, pp, world // (tp * pp) > 1)
    # make the optimizer state recognisable: exp_avg = 2 * master, exp_avg_sq = 3 * master
    for st in opt.states:
        st.exp_avg.copy_(2 * st.master)
        st.exp_avg_sq.copy_(3 * st.master)
    opt.step_count = 5
    save_checkpoint(11, model, opt, None, _args(d))


def _load_rank(rank, world, tp, pp, d, check_optim):
    from megatron_lm_b200.parallel import state
    from megatron_lm_b200.training.checkpointing import load_checkpoint
    from tests.model_utils import reinit_by_global_name
    state.initialize_model_parallel(tensor_model_parallel_size=tp, pipeline_model_parallel_size=pp)
    cfg, model, opt = _build(tp, pp, world // (tp * pp) > 1, reinit=False)
    it, _ = load_checkpoint(model, opt, None, _args(d, no_load_optim=not check_optim))
    assert it == 11
    # the expected weights are the name-seeded ones
    from megatron_lm_b200.models.gpt import GPTModel
    for chunk in model:
        m = chunk.module
        got = {n: p.detach().clone() for n, p in m.named_parameters()}
        reinit_by_global_name(m, cfg)
        for n, p in m.named_parameters():
            assert torch.equal(got[n], p.detach()), n
    if check_optim:
        assert opt.step_count == 5
        for st in opt.states:
            st.reload_master_from_params()
            assert torch.allclose(st.exp_avg, 2 * st.master) and torch.allclose(st.exp_avg_sq, 3 * st.master)
            # every element was restored, the halves of the gated FC1 included (a rank's share may be small, but the
            # name-seeded weights are nowhere exactly zero)
            for piece in st.pieces:
                part = st.exp_avg[piece["local_start"]:piece["local_start"] + piece["numel"]]
                assert bool((part != 0).all()), [n for n, q in model[0].module.named_parameters() if q is piece["param"]]


@pytest.mark.parametrize("save_cfg,load_cfg,optim", [((2, 2, 1), (1, 1, 1), False), ((2, 1, 2), (2, 2, 1), False),
                                                     ((2, 1, 1), (2, 1, 1), True), ((1, 1, 1), (2, 1, 1), True)])
def test_save_then_load_under_another_layout(tmp_path, save_cfg, load_cfg, optim):
    d = str(tmp_path / "ckpt")
    run_distributed(_save_rank, save_cfg[0], save_cfg[1], save_cfg[2], d)
    assert os.path.isfile(os.path.join(d, "latest_checkpointed_iteration.txt"))
    run_distributed(_load_rank, load_cfg[0], load_cfg[1], load_cfg[2], d, optim)


def test_legacy_torch_format_roundtrip(tmp_path):
    from megatron_lm_b200.training.checkpointing import load_checkpoint, save_checkpoint
    d = str(tmp_path)
    cfg, model, opt = _build(1, 1, False)
    opt.step_count = 3
    save_checkpoint(4, model, opt, None, _args(d, ckpt_format="torch"))
    assert os.path.isfile(os.path.join(d, "iter_0000004", "mp_rank_00", "model_optim_rng.pt"))
    cfg2, model2, opt2 = _build(1, 1, False, reinit=False)
    it, _ = load_checkpoint(model2, opt2, None, _args(d, ckpt_format="torch"))
    assert it == 4 and opt2.step_count == 3
    for (n, a), (_, b) in zip(model[0].module.named_parameters(), model2[0].module.named_parameters()):
        assert torch.equal(a, b), n


def _torch_fmt_rank(rank, world, d, phase):
    """Legacy (torch) layout with the distributed optimizer on two data-parallel ranks: every rank writes and
    reads back *its own* shard of master weights and moments."""
    from megatron_lm_b200.parallel import state
    from megatron_lm_b200.training.checkpointing import load_checkpoint, save_checkpoint
    state.initialize_model_parallel()
    cfg, model, opt = _build(1, 1, True, reinit=(phase == "save"))
    if phase == "save":
        for st in opt.states:
            assert st.sharded
            st.exp_avg.copy_((rank + 2) * st.master)         # rank-dependent, so a mixed-up shard is noticed
            st.exp_avg_sq.copy_((rank + 5) * st.master)
        opt.step_count = 7
        save_checkpoint(3, model, opt, None, _args(d, ckpt_format="torch"))
        base = os.path.join(d, "iter_0000003", "mp_rank_00")
        assert os.path.isfile(os.path.join(base, f"distrib_optim_dp{rank:03d}.pt"))
    else:
        it, _ = load_checkpoint(model, opt, None, _args(d, ckpt_format="torch"))
        assert it == 3 and opt.step_count == 7
        for st in opt.states:
            st2_master = st.master.clone()
            st.reload_master_from_params()                    # weights came from the model file
            assert torch.allclose(st.master, st2_master)
            assert torch.allclose(st.exp_avg, (rank + 2) * st.master)
            assert torch.allclose(st.exp_avg_sq, (rank + 5) * st.master)


def test_legacy_torch_format_with_distributed_optimizer(tmp_path):
    d = str(tmp_path / "ckpt")
    run_distributed(_torch_fmt_rank, 2, d, "save")
    run_distributed(_torch_fmt_rank, 2, d, "load")


def test_torch_dist_layout_is_readable_by_torch_dcp_and_back(tmp_path):
    """The default container is the reference's ``torch_dist`` layout: what we write, torch.distributed.checkpoint
    reads with its own reader; what it writes, our loader reads (and re-blocks)."""
    import json
    import torch.distributed.checkpoint as dcp
    d = str(tmp_path / "ours")
    full = torch.arange(8 * 6, dtype=torch.float32).view(8, 6)
    sd = {"w_top": ds.ShardedTensor.from_rank_offsets("layer.w", full[:4].clone(), (0, 0, 2)),
          "w_bot": ds.ShardedTensor.from_rank_offsets("layer.w", full[4:].clone(), (0, 1, 2)),
          "b": ds.ShardedTensor.from_rank_offsets("layer.b", torch.ones(3)),
          "rng": ds.ShardedObject("rng_state", {"seed": 5}, (1,), (0,)), "iteration": 9}
    ds.save(sd, d)
    names = set(os.listdir(d))
    assert {".metadata", "__0_0.distcp", "common.pt", "metadata.json"} <= names
    assert json.load(open(os.path.join(d, "metadata.json")))["sharded_backend"] == "torch_dist"
    # torch's own reader
    target = {"layer.w": torch.zeros(8, 6), "layer.b": torch.zeros(3)}
    dcp.load(target, storage_reader=dcp.FileSystemReader(d), no_dist=True)
    assert torch.equal(target["layer.w"], full) and torch.equal(target["layer.b"], torch.ones(3))
    # a checkpoint written by torch.distributed.checkpoint, read here as three row stripes
    d2 = str(tmp_path / "theirs")
    dcp.save({"layer.w": full.clone(), "layer.b": torch.full((3,), 2.0)}, storage_writer=dcp.FileSystemWriter(d2),
             no_dist=True)
    torch.save({"iteration": 4}, os.path.join(d2, "common.pt"))
    with open(os.path.join(d2, "metadata.json"), "w") as f:
        json.dump({"sharded_backend": "torch_dist", "sharded_backend_version": 1, "common_backend": "torch",
                   "common_backend_version": 1}, f)
    for r in range(2):
        req = {"x": ds.ShardedTensor.from_rank_offsets("layer.w", torch.zeros(4, 6), (0, r, 2)),
               "b": ds.ShardedTensor.from_rank_offsets("layer.b", torch.zeros(3))}
        out = ds.load(req, d2)
        assert torch.equal(out["x"], full[4 * r:4 * r + 4]) and out["iteration"] == 4
        assert torch.equal(out["b"], torch.full((3,), 2.0))


def test_native_container_still_round_trips(tmp_path):
    d = str(tmp_path)
    sd = {"w": ds.ShardedTensor.from_rank_offsets("w", torch.arange(6.0).view(2, 3)), "it": 3}
    ds.save(sd, d, container="native")
    assert os.path.isfile(os.path.join(d, "shard_0.pt"))
    out = ds.load({"w": ds.ShardedTensor.from_rank_offsets("w", torch.zeros(2, 3))}, d)
    assert torch.equal(out["w"], torch.arange(6.0).view(2, 3)) and out["it"] == 3


# ----------------------------------------------------------------------- Mamba mixers under another tensor-parallel size
_MAMBA = dict(d_state=8, headdim=8, ngroups=2)


def _mamba_global(kind):
    """The mixer's parameters at tensor-parallel size 1 (hidden 16: inner 32, 4 heads, 2 groups of state 8), each
    value unique."""
    g = torch.Generator().manual_seed(77)
    shapes = {"in_proj.weight": (2 * 32 + 2 * 2 * 8 + 4, 16), "conv_weight": (32 + 2 * 2 * 8, 4), "conv_bias": (32 + 2 * 2 * 8,),
              "dt_bias": (4,), "A_log": (4,), "D": (4,), "norm_weight": (32,), "out_proj.weight": (16, 32)}
    return {k: torch.randn(*s, generator=g) for k, s in shapes.items()}[kind] if kind else shapes


def _mamba_local(name, full, rank, tp):
    """The rows (columns of the output projection) that rank ``rank`` of ``tp`` holds: every segment is cut on its
    own."""
    def cut(t, sizes, dim=0):
        return torch.cat([seg.chunk(tp, dim=dim)[rank] for seg in torch.split(t, sizes, dim=dim)], dim=dim)
    if name == "in_proj.weight":
        return cut(full, [32, 32, 16, 16, 4])
    if name in ("conv_weight", "conv_bias"):
        return cut(full, [32, 16, 16])
    if name == "out_proj.weight":
        return full.chunk(tp, dim=1)[rank]
    return full.chunk(tp, dim=0)[rank]


def _mamba_rank(rank, world, tp, d, phase):
    from megatron_lm_b200.checkpoint import sharded as ds
    from megatron_lm_b200.config import TransformerConfig
    from megatron_lm_b200.models.mamba import MambaMixer
    from megatron_lm_b200.parallel import state
    state.initialize_model_parallel(tensor_model_parallel_size=tp)
    cfg = TransformerConfig(num_layers=1, hidden_size=16, num_attention_heads=2, tensor_model_parallel_size=tp,
                            use_cpu_initialization=True, params_dtype=torch.float32)
    mixer = MambaMixer(cfg, 1, **_MAMBA)
    r = state.get_tensor_model_parallel_rank()
    names = list(_mamba_global(None))
    params = dict(mixer.named_parameters())
    assert sorted(params) == sorted(names)
    with torch.no_grad():
        for n in names:
            if phase == "save":
                params[n].copy_(_mamba_local(n, _mamba_global(n), r, tp))
            else:
                params[n].zero_()
    desc = ds.model_sharded_state_dict(mixer, "mixer.", tp_rank=r, tp_size=tp, dp_rank=rank // tp)
    assert {"in_proj.weight.part4", "conv_bias.part2"} <= set(desc) and desc["in_proj.weight.part0"].key == "mixer.in_proj.weight.z"
    if phase == "save":
        ds.save(desc, d)
        return
    ds.load_model_from_sharded(mixer, ds.load(desc, d))
    for n in names:
        assert torch.equal(params[n].detach(), _mamba_local(n, _mamba_global(n), r, tp)), n


@pytest.mark.parametrize("save_tp,load_tp", [(2, 1), (1, 2), (2, 2)])
def test_mamba_mixer_sharded_checkpoint_changes_tensor_parallel_size(tmp_path, save_tp, load_tp):
    d = str(tmp_path / "mamba")
    os.makedirs(d)
    run_distributed(_mamba_rank, save_tp, save_tp, d, "save")
    run_distributed(_mamba_rank, load_tp, load_tp, d, "load")
