"""Small structural components: explicit pipeline layer layouts, the N-dimensional communicator grid, module specs,
process-wide globals and writers, the half-precision module wrapper.
Mirrors the reference's tests/unit_tests/test_hyper_comm_grid.py, pipeline_parallel/test_pipeline_layout.py,
transformer/test_spec_customization.py and test_global_vars."""
import json
from types import SimpleNamespace

import pytest
import torch


def test_pipeline_layout_string_expansion_and_queries():
    from megatron_lm_b200.models.pp_layout import PipelineParallelLayerLayout as L
    one = L("Et*3|(tt|)*2,m|L", pipeline_model_parallel_size=1)
    assert ["".join(s) for s in one.stages] == ["Ettt", "tt", "tt", "m", "L"] and one.vpp == 5
    one.validate_layer_layout(7, mtp_num_layers=1)
    with pytest.raises(ValueError):
        one.validate_layer_layout(8)
    lay = L("Ett|tt|tt|ttL", pipeline_model_parallel_size=2)            # stage index = v * pp + rank
    assert lay.vpp == 2
    assert lay.get_num_layers_to_build(0, 0) == 2 and lay.get_num_layers_to_build(1, 1) == 2
    assert lay.get_layer_offset(1, 0) == 2 and lay.get_layer_offset(0, 1) == 4 and lay.get_layer_offset(1, 1) == 6
    assert lay.get_layer_id_list(0, 1) == [4, 5]
    assert lay.get_num_layers_to_build(0, 0, kind="E") == 1 and lay.get_num_layers_to_build(1, 1, kind="L") == 1
    uneven = L([["E", "t"], ["t", "t", "t", "L"]], 2)
    assert uneven.get_num_layers_to_build(0) == 1 and uneven.get_num_layers_to_build(1) == 3
    for bad in ("Ett|ttL|tt", "tt|ttL", "Ett|tt"):
        with pytest.raises(ValueError):
            L(bad, 2)


def test_hyper_comm_grid_enumerations_match_reference_order():
    from megatron_lm_b200.parallel.hyper_comm_grid import HyperCommGrid
    g = HyperCommGrid([2, 2, 2], ["tp", "dp", "pp"])                  # tp fastest
    assert g.get_rank_enum("tp") == [[0, 1], [2, 3], [4, 5], [6, 7]]
    assert g.get_rank_enum("dp") == [[0, 2], [1, 3], [4, 6], [5, 7]]
    assert g.get_rank_enum("pp") == [[0, 4], [1, 5], [2, 6], [3, 7]]
    assert g.get_rank_enum(["tp", "dp"]) == [[0, 1, 2, 3], [4, 5, 6, 7]]
    assert g.get_rank_enum("dp-tp") == g.get_rank_enum("tp-dp")      # dims are taken in grid order
    off = HyperCommGrid([2, 2], ["tp", "dp"], rank_offset=4)
    assert off.get_rank_enum("tp") == [[4, 5], [6, 7]]
    mine = g.create_pg("tp")                                          # no process group backend: the rank tuple
    assert mine == (0, 1) and g.get_pg("tp") == (0, 1)
    with pytest.raises(KeyError):
        g.create_pg("tp")
    with pytest.raises(KeyError):
        g.get_pg("dp")
    with pytest.raises(KeyError):
        g.get_rank_enum("xx")
    with pytest.raises(ValueError):
        HyperCommGrid([2, 2], ["tp"])


def test_module_spec_builds_nested_modules():
    from megatron_lm_b200.models.spec_utils import ModuleSpec, build_module, get_module, import_module
    spec = ModuleSpec(module=("torch.nn", "Linear"), params={"bias": False})
    lin = build_module(spec, 4, 3)
    assert isinstance(lin, torch.nn.Linear) and lin.bias is None and lin.weight.shape == (3, 4)
    assert get_module(spec) is torch.nn.Linear and import_module(("torch.nn", "ReLU")) is torch.nn.ReLU
    assert isinstance(build_module(torch.nn.ReLU), torch.nn.ReLU)
    fn = lambda x: x                                                  # noqa: E731
    assert build_module(fn) is fn and build_module(ModuleSpec(module=fn)) is fn

    class Block(torch.nn.Module):
        def __init__(self, width, submodules=None):
            super().__init__()
            self.inner = build_module(submodules["inner"], width, width)
    blk = build_module(ModuleSpec(module=Block, params={"width": 5}, submodules={"inner": spec}))
    assert blk.inner.weight.shape == (5, 5) and blk.inner.bias is None


def test_global_variables_and_fallback_writers(tmp_path):
    from megatron_lm_b200.training import global_vars as G
    G.unset_global_variables()
    with pytest.raises(Exception):
        G.get_args()
    args = SimpleNamespace(rank=0, world_size=1, timing_log_level=1, timing_log_option="max",
                           tensorboard_dir=str(tmp_path / "tb"), wandb_project=None, enable_one_logger=True,
                           exit_signal_handler=False, log_energy=False, tokenizer_type=None,
                           one_logger_project="proj", one_logger_run_name="run-7", app_tag_run_name="tag",
                           app_tag_run_version="1.2", one_logger_async=True)
    G.set_global_variables(args, build_tokenizer=False)
    assert G.get_args() is args and G.get_timers() is not None
    w = G.get_tensorboard_writer()
    w.add_scalar("loss", 1.5, 3)
    w.flush()
    one = G.get_one_logger()
    one.on_train_start(train_iterations_start=0)
    one.log_metrics({"a": 1})
    assert one.store_has_key("train_iterations_start")
    assert one.store_get("project") == "proj" and one.store_get("run_name") == "run-7" and one.store_get("async") is True
    assert one.store_get("app_tag_run_version") == "1.2"
    jw = G._JsonlWriter(str(tmp_path / "m" / "x.jsonl"))
    jw.add_scalar("lr", 0.1, 2)
    jw.log({"loss": 2.0}, step=3)
    jw.close()
    rows = [json.loads(l) for l in open(tmp_path / "m" / "x.jsonl")]
    assert rows[0]["tag"] == "lr" and rows[0]["value"] == 0.1 and rows[1]["tag"] == "loss" and rows[1]["value"] == 2.0 and rows[1]["step"] == 3
    G.unset_global_variables()


def test_float16_module_casts_inputs_and_outputs():
    from megatron_lm_b200.config import TransformerConfig
    from megatron_lm_b200.models.module import Float16Module, MegatronModule

    class Inner(MegatronModule):
        def __init__(self, cfg):
            super().__init__(cfg)
            self.lin = torch.nn.Linear(4, 4)
            self.seen = None

        def forward(self, x):
            self.seen = x.dtype
            return self.lin(x)
    cfg = TransformerConfig(num_layers=1, hidden_size=4, num_attention_heads=1, bf16=True, params_dtype=torch.bfloat16)
    m = Float16Module(cfg, Inner(cfg))
    assert m.module.lin.weight.dtype == torch.bfloat16
    out = m(torch.randn(2, 4))
    assert m.module.seen == torch.bfloat16 and out.dtype == torch.float32
    sd = m.state_dict()
    m.load_state_dict(sd)
    assert any(k.endswith("lin.weight") for k in sd)


def test_huggingface_adapters_wrap_transformers_modules():
    transformers = pytest.importorskip("transformers")
    from megatron_lm_b200.models.huggingface import AutoHuggingFaceModel, ClipHuggingFaceModel, QwenHuggingFaceModel
    cfg = SimpleNamespace(huggingface_model_name_or_path=None)
    clip_cfg = transformers.CLIPVisionConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=1,
                                             num_attention_heads=2, image_size=16, patch_size=8)
    clip = ClipHuggingFaceModel(cfg, clip_cfg)
    out = clip(torch.randn(2, 3, 16, 16))
    assert out.shape == (2, 5, 32)                                    # 4 patches + class token
    assert all(p.tensor_model_parallel is False for p in clip.parameters())
    q_cfg = transformers.Qwen2Config(hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=2,
                                     num_key_value_heads=2, vocab_size=50, max_position_embeddings=32)
    qwen = QwenHuggingFaceModel(cfg, q_cfg)
    ids = torch.randint(0, 50, (2, 7))
    emb = qwen.embedding(ids)
    assert emb.shape == (7, 2, 32)                                    # [s, b, h], the layout of this framework
    a = qwen(input_ids=ids)
    b = qwen(decoder_input=emb)
    assert a.shape == (2, 7, 32) and torch.allclose(a, b, atol=1e-5)
    auto = AutoHuggingFaceModel(cfg, q_cfg)
    assert auto(input_ids=ids)["last_hidden_state"].shape == (2, 7, 32)
    auto.set_input_tensor(None)


def _pg_bundles(rank, world):
    from megatron_lm_b200.parallel import state
    from megatron_lm_b200.parallel.process_groups_config import GradCommProcessGroups, ModelCommProcessGroups
    import torch.distributed as dist
    state.initialize_model_parallel(tensor_model_parallel_size=2)
    m = ModelCommProcessGroups.use_mpu_process_groups(["tp", "pp", "cp"])
    assert m.tp is state.get_tensor_model_parallel_group() and m.ep is None
    assert dist.get_world_size(m.tp) == 2 and dist.get_world_size(m.pp) == 1
    with pytest.raises(ValueError):
        ModelCommProcessGroups.use_mpu_process_groups(["nope"])
    every = ModelCommProcessGroups.use_mpu_process_groups()
    assert every.tp_cp is not None and every.mp is not None
    g = GradCommProcessGroups.use_mpu_process_groups()
    assert dist.get_world_size(g.dp) == 1 and g.expt_dp is not None
    state.destroy_model_parallel()


def test_process_group_bundles_from_global_state():
    from tests.dist_utils import run_distributed
    run_distributed(_pg_bundles, 2)


def test_packed_sequences_match_the_documents_run_one_by_one():
    """Two documents packed in one row (thd): logits equal those of each document run alone, for rotary positions
    (restart per document) and attention (no look across the boundary)."""
    import torch
    from megatron_lm_b200.config import TransformerConfig
    from megatron_lm_b200.models.gpt import GPTModel
    from megatron_lm_b200.packed_seq_params import PackedSeqParams
    torch.manual_seed(3)
    cfg = TransformerConfig(num_layers=2, hidden_size=32, num_attention_heads=4, ffn_hidden_size=64,
                            hidden_dropout=0.0, attention_dropout=0.0, normalization="RMSNorm", gated_linear_unit=True,
                            activation_func="silu", add_bias_linear=False)
    m = GPTModel(cfg, vocab_size=50, max_sequence_length=32, position_embedding_type="rope").eval()
    a, b = torch.randint(0, 50, (1, 5)), torch.randint(0, 50, (1, 7))
    packed = PackedSeqParams.from_lengths([5, 7])
    assert packed.positions(12).tolist() == [0, 1, 2, 3, 4, 0, 1, 2, 3, 4, 5, 6]
    with torch.no_grad():
        both = m(torch.cat((a, b), dim=1), packed_seq_params=packed)
        la, lb = m(a), m(b)
    assert torch.allclose(both[:, :5], la, atol=1e-5) and torch.allclose(both[:, 5:], lb, atol=1e-5)
    # without the boundary the second document sees the first: a different result
    with torch.no_grad():
        plain = m(torch.cat((a, b), dim=1))
    assert not torch.allclose(plain[:, 5:], lb, atol=1e-4)


def test_named_and_callable_activations():
    import torch
    from megatron_lm_b200 import activations as A
    from megatron_lm_b200.config import TransformerConfig
    from megatron_lm_b200.models.transformer import MLP
    x = torch.linspace(-3, 3, 25)
    assert torch.allclose(A.squared_relu(x), torch.relu(x) ** 2)
    assert torch.allclose(A.fast_gelu(x), torch.nn.functional.gelu(x, approximate="tanh"), atol=1e-6)
    assert (A.quick_gelu(x) - torch.nn.functional.gelu(x)).abs().max() < 0.03
    for act, gated in (("quick_gelu", False), ("fast_gelu", True), (A.quick_gelu, True)):
        cfg = TransformerConfig(num_layers=1, hidden_size=16, num_attention_heads=2, ffn_hidden_size=32,
                                activation_func=act, gated_linear_unit=gated, add_bias_linear=False)
        mlp = MLP(cfg)
        h = torch.randn(3, 2, 16)
        out, _ = mlp(h)
        w1, w2 = mlp.linear_fc1.weight, mlp.linear_fc2.weight
        z = h @ w1.t()
        f = act if callable(act) else A.BY_NAME[act]
        z = f(z[..., :32]) * z[..., 32:] if gated else f(z)
        assert torch.allclose(out, z @ w2.t(), atol=1e-5)


def test_sliding_window_attention_layer_on_cpu():
    """window_size=(left, 0): the layer's output for a token does not depend on tokens further back than the window."""
    import torch
    from megatron_lm_b200.config import TransformerConfig
    from megatron_lm_b200.models.transformer import SelfAttention
    torch.manual_seed(0)
    cfg = TransformerConfig(num_layers=1, hidden_size=64, num_attention_heads=4, window_size=(3, 0),
                            hidden_dropout=0.0, attention_dropout=0.0)
    attn = SelfAttention(cfg, 1)
    x = torch.randn(12, 1, 64)
    y, _ = attn(x)
    x2 = x.clone()
    x2[:5] = torch.randn(5, 1, 64)              # tokens 0..4 are outside the window of tokens 8..11
    y2, _ = attn(x2)
    assert torch.allclose(y[8:], y2[8:], atol=1e-6)
    assert not torch.allclose(y[5:8], y2[5:8], atol=1e-4)
    full = SelfAttention(TransformerConfig(num_layers=1, hidden_size=64, num_attention_heads=4, hidden_dropout=0.0,
                                           attention_dropout=0.0), 1)
    full.load_state_dict(attn.state_dict())
    assert not torch.allclose(full(x)[0][8:], y[8:], atol=1e-4)


def test_layers_without_rotary_embedding_and_post_norm_residual():
    """no_rope_freq: every n-th layer (or the layers of an explicit list) attends without rotary positions;
    apply_residual_connection_post_layernorm: the residual branch starts after the norm."""
    from megatron_lm_b200.config import TransformerConfig
    from megatron_lm_b200.models.gpt import GPTModel
    base = dict(num_layers=4, hidden_size=32, num_attention_heads=4, ffn_hidden_size=64, hidden_dropout=0.0,
                attention_dropout=0.0, use_cpu_initialization=True)
    m = GPTModel(TransformerConfig(no_rope_freq=2, **base), 32, 16, position_embedding_type="rope", parallel_output=False)
    assert [l.self_attention.no_rope for l in m.decoder.layers] == [False, True, False, True]
    m2 = GPTModel(TransformerConfig(no_rope_freq=[1, 0, 0, 1], **base), 32, 16, position_embedding_type="rope",
                  parallel_output=False)
    assert [l.self_attention.no_rope for l in m2.decoder.layers] == [True, False, False, True]
    # a layer without rotary positions is permutation-equivariant over the keys it sees: with a single layer and the
    # last query, shuffling the earlier tokens leaves the last position's output unchanged
    one = dict(base, num_layers=1)
    torch.manual_seed(0)
    nope = GPTModel(TransformerConfig(no_rope_freq=1, **one), 32, 16, position_embedding_type="rope",
                    parallel_output=False).eval()
    torch.manual_seed(0)
    rope = GPTModel(TransformerConfig(**one), 32, 16, position_embedding_type="rope", parallel_output=False).eval()
    ids = torch.randint(0, 32, (1, 9))
    perm = torch.cat([ids[:, :8].flip(1), ids[:, 8:]], dim=1)
    with torch.no_grad():
        assert torch.allclose(nope(ids)[0, -1], nope(perm)[0, -1], atol=1e-5)
        assert not torch.allclose(rope(ids)[0, -1], rope(perm)[0, -1], atol=1e-5)
    # post-norm residual: y = norm(x) + f(norm(x))
    torch.manual_seed(0)
    post = GPTModel(TransformerConfig(apply_residual_connection_post_layernorm=True, **one), 32, 16,
                    parallel_output=False).eval()
    layer = post.decoder.layers[0]
    x = torch.randn(5, 2, 32)
    with torch.no_grad():
        ln1 = layer.input_layernorm(x)
        a, ab = layer.self_attention(ln1)
        h = ln1 + a + (ab if ab is not None else 0)
        ln2 = layer.pre_mlp_layernorm(h)
        f, fb = layer.mlp(ln2)
        want = ln2 + f + (fb if fb is not None else 0)
        assert torch.allclose(layer(x), want, atol=1e-5)


def test_activation_offloading_to_the_host_keeps_the_gradients():
    """cpu_offloading: the saved tensors of the first layers pass through host memory; losses and gradients are
    those of the plain run."""
    from megatron_lm_b200.config import TransformerConfig
    from megatron_lm_b200.models.gpt import GPTModel
    base = dict(num_layers=3, hidden_size=32, num_attention_heads=4, ffn_hidden_size=64, hidden_dropout=0.0,
                attention_dropout=0.0, use_cpu_initialization=True)
    with pytest.raises(ValueError):
        TransformerConfig(cpu_offloading=True, cpu_offloading_num_layers=0, **base)
    with pytest.raises(ValueError):
        TransformerConfig(cpu_offloading=True, cpu_offloading_num_layers=2, cpu_offloading_weights=True, **base)
    ids = torch.randint(0, 32, (2, 16))
    grads, packed = [], []
    for off in (False, True):
        torch.manual_seed(0)
        cfg = TransformerConfig(cpu_offloading=off, cpu_offloading_num_layers=2 if off else 0, **base)
        m = GPTModel(cfg, 32, 16, parallel_output=False).train()
        real = torch.autograd.graph.save_on_cpu
        calls = []

        class Counting(real):
            def __init__(self, *a, **kw):
                calls.append(1)
                super().__init__(*a, **kw)
        torch.autograd.graph.save_on_cpu = Counting
        try:
            m(ids, labels=ids).mean().backward()
        finally:
            torch.autograd.graph.save_on_cpu = real
        packed.append(len(calls))
        grads.append({n: p.grad.clone() for n, p in m.named_parameters() if p.grad is not None})
    assert packed == [0, 2]                                      # one offloading context per offloaded layer
    assert grads[0].keys() == grads[1].keys() and all(torch.equal(grads[0][k], grads[1][k]) for k in grads[0])


def test_multi_storage_client_switch(tmp_path):
    """Without the package the feature reports off whatever the flag says, and file helpers use the local file
    system; msc:// dataset paths name the missing package in their error."""
    import pickle
    from types import SimpleNamespace
    from megatron_lm_b200.data import object_storage as osu
    from megatron_lm_b200.utils import msc
    have = msc._msc is not None
    assert msc.configure_from_args(SimpleNamespace(enable_msc=True)) == have
    assert msc.configure_from_args(SimpleNamespace(enable_msc=False)) is False
    assert not msc.MultiStorageClientFeature.is_enabled()
    with pytest.raises(RuntimeError):
        msc.MultiStorageClientFeature.import_package()
    flag = pickle.loads(pickle.dumps(msc.MultiStorageClientFeature))
    assert flag._enabled is False
    p = tmp_path / "d" / "x.txt"
    msc.makedirs(str(p.parent))
    with msc.open_file(str(p), "w") as f:
        f.write("hi")
    assert msc.path_exists(str(p)) and not msc.path_exists(str(p) + ".none")
    if not have:
        with pytest.raises(RuntimeError, match="multistorageclient|switched off"):
            osu.get_client("msc://profile/data.bin")


def test_graphed_module_passes_other_arguments_through_on_the_eager_path():
    """Off a GPU, and whenever a call carries a mask / context, ``GraphedModule`` is a transparent wrapper: keyword
    arguments reach the layer, attributes of the layer stay visible."""
    from megatron_lm_b200.config import TransformerConfig
    from megatron_lm_b200.models.transformer import TransformerLayer
    from megatron_lm_b200.utils.cuda_graphs import GraphedModule
    cfg = TransformerConfig(num_layers=1, hidden_size=32, num_attention_heads=4, ffn_hidden_size=64, hidden_dropout=0.0,
                            attention_dropout=0.0, use_cpu_initialization=True)
    torch.manual_seed(0)
    layer = TransformerLayer(cfg, 1)
    g = GraphedModule(layer)
    x = torch.randn(6, 2, 32)
    cos, sin = torch.randn(6, 4).cos(), torch.randn(6, 4).sin()
    assert torch.equal(g(x, rotary=(cos, sin)), layer(x, rotary=(cos, sin)))
    assert torch.equal(g(x), layer(x)) and not g._captured
    assert g.layer_number == 1 and g.self_attention is layer.self_attention
