"""The reference's import paths resolve to this library after ``install()`` (run in a child interpreter so the
aliases do not leak into the test process)."""
import subprocess
import sys
import textwrap


def test_reference_import_paths_resolve_after_install():
    code = textwrap.dedent('''
        import sys
        assert "megatron" not in sys.modules
        from megatron_lm_b200.compat import megatron_aliases
        names = megatron_aliases.install()
        from megatron.core import parallel_state, tensor_parallel
        from megatron.core.models.gpt import GPTModel
        from megatron.core.models.gpt.gpt_layer_specs import get_gpt_layer_local_spec
        from megatron.core.transformer.transformer_config import TransformerConfig
        from megatron.core.transformer.spec_utils import ModuleSpec
        from megatron.core.pipeline_parallel import get_forward_backward_func
        from megatron.core.distributed import DistributedDataParallel, DistributedDataParallelConfig, finalize_model_grads
        from megatron.core.optimizer import OptimizerConfig, get_megatron_optimizer
        from megatron.core.tensor_parallel.random import model_parallel_cuda_manual_seed
        from megatron.core.extensions.transformer_engine import TENorm
        from megatron.core.rerun_state_machine import RerunStateMachine
        from megatron.training import get_args, pretrain
        from megatron.training.arguments import parse_args
        from megatron.training.yaml_arguments import core_transformer_config_from_yaml
        from megatron.core.dist_checkpointing.tensor_aware_state_dict import TensorAwareStateDict
        from megatron.core.datasets.multimodal_dataset import MockMultimodalDataset
        from megatron.core.transformer.moe.upcycling_utils import upcycle_state_dict
        from megatron.core.models.multimodal.llava_model import LLaVAModel
        from megatron.core.export.trtllm.trtllm_helper import TRTLLMHelper
        from megatron.post_training.algos.distillation import LogitsKLLoss, load_distillation_config
        from megatron.post_training.arguments import add_modelopt_args
        import megatron_lm_b200.models.gpt as native
        assert GPTModel is native.GPTModel
        assert parallel_state.initialize_model_parallel.__module__ == "megatron_lm_b200.parallel.state"
        assert tensor_parallel.ColumnParallelLinear.__module__ == "megatron_lm_b200.parallel.layers"
        import torch
        cfg = TransformerConfig(num_layers=1, hidden_size=16, num_attention_heads=2, use_cpu_initialization=True)
        m = GPTModel(cfg, get_gpt_layer_local_spec(), 32, 8)
        assert m(torch.zeros(1, 8, dtype=torch.long), None, None).shape == (1, 8, 32)
        megatron_aliases.uninstall()
        assert "megatron.core" not in sys.modules
        print("ok", len(names))
    ''')
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and r.stdout.startswith("ok"), r.stderr[-2000:]


def test_install_refuses_to_shadow_a_real_package():
    code = textwrap.dedent('''
        import sys, types
        sys.modules["megatron"] = types.ModuleType("megatron")      # stands for the real package
        from megatron_lm_b200.compat import megatron_aliases
        try:
            megatron_aliases.install()
        except RuntimeError as e:
            print("refused")
    ''')
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120)
    assert r.stdout.strip() == "refused", r.stderr[-2000:]
