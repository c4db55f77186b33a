"""Down-stream task utilities: sample construction, the classification / multiple-choice heads, the epoch-based
fine-tuning loop with per-epoch accuracy, data-parallel evaluation counts.  Mirrors what the reference's
tasks/finetune_utils.py, eval_utils.py and data_utils.py do for GLUE / RACE style tasks."""
import numpy as np
import torch

from megatron_lm_b200.config import OptimizerConfig, TransformerConfig
from megatron_lm_b200.models.bert import BertModel, Classification, MultipleChoice
from megatron_lm_b200.tasks import data_utils, eval_utils, finetune_utils
from tests.dist_utils import run_distributed


def test_sample_construction_and_cleaning():
    assert data_utils.clean_text("a  b\nc . d") == "a b c. d"
    ids, types, pad = data_utils.build_tokens_types_paddings_from_ids([5, 6], [7, 8, 9], 10, cls_id=1, sep_id=2, pad_id=0)
    assert ids == [1, 5, 6, 2, 7, 8, 9, 2, 0, 0] and types == [0, 0, 0, 0, 1, 1, 1, 1, 0, 0] and pad == [1] * 8 + [0] * 2
    ids, types, pad = data_utils.build_tokens_types_paddings_from_ids([5, 6, 7, 8], [9, 10, 11], 8, 1, 2, 0)
    assert len(ids) == 8 and ids[-1] == 2 and ids[0] == 1 and pad == [1] * 8            # truncated, closing separator kept
    ids, types, pad = data_utils.build_tokens_types_paddings_from_ids([5, 6], None, 6, 1, 2, 0)
    assert ids == [1, 5, 6, 2, 0, 0] and types == [0] * 6 and pad == [1, 1, 1, 1, 0, 0]
    s = data_utils.build_sample(ids, types, pad, 3, 17)
    assert s["text"].dtype == np.int64 and s["label"] == 3 and s["uid"] == 17

    class Tok:
        cls, sep, pad = 1, 2, 0
        def tokenize(self, t):
            return [10 + len(w) for w in t.split()]
    ids, types, pad = data_utils.build_tokens_types_paddings_from_text("aa bbb", "c", Tok(), 8)
    assert ids == [1, 12, 13, 2, 11, 2, 0, 0]


class _Toy(torch.utils.data.Dataset):
    """Label = whether token 7 occurs in the first segment: learnable by a one-layer encoder in a few epochs."""
    dataset_name = "toy"

    def __init__(self, n, seed, seq=12):
        g = np.random.RandomState(seed)
        self.rows = []
        for i in range(n):
            label = int(g.rand() < 0.5)
            a = g.randint(10, 30, size=4).tolist()
            if label:
                a[g.randint(0, 4)] = 7
            b = g.randint(10, 30, size=3).tolist()
            ids, types, pad = data_utils.build_tokens_types_paddings_from_ids(a, b, seq, 1, 2, 0)
            self.rows.append(data_utils.build_sample(ids, types, pad, label, i))

    def __len__(self):
        return len(self.rows)

    def __getitem__(self, i):
        return self.rows[i]


def _cfg():
    return TransformerConfig(num_layers=1, hidden_size=32, num_attention_heads=4, ffn_hidden_size=64, hidden_dropout=0.0,
                             attention_dropout=0.0, use_cpu_initialization=True)


def test_heads_shapes_and_pretrained_encoder():
    torch.manual_seed(0)
    cfg = _cfg()
    bert = BertModel(cfg, 2, 40, 12)
    clf = Classification(cfg, 3, 40, 12)
    res = clf.load_pretrained_encoder(bert.state_dict())
    assert all(k.startswith("classification_head") for k in res.missing_keys)
    assert torch.equal(clf.encoder.layers[0].mlp.linear_fc1.weight, bert.encoder.layers[0].mlp.linear_fc1.weight)
    assert torch.equal(clf.pooler.dense.weight, bert.pooler.dense.weight)
    ds = _Toy(4, 0)
    batch = torch.utils.data.default_collate([ds[i] for i in range(4)])
    tokens, types, labels, mask = finetune_utils.process_batch(batch, "cpu")
    assert clf(tokens, mask, types).shape == (4, 3)
    mc = MultipleChoice(cfg, 40, 12)
    t3 = tokens.view(2, 2, 12)
    out = mc(t3, mask.view(2, 2, 12), types.view(2, 2, 12))
    assert out.shape == (2, 2)
    # a choice's score does not depend on which other choices sit beside it
    swapped = mc(t3.flip(1), mask.view(2, 2, 12).flip(1), types.view(2, 2, 12).flip(1))
    assert torch.allclose(out, swapped.flip(1), atol=1e-6)


def _finetune_rank(rank, world):
    from megatron_lm_b200.parallel import state
    state.initialize_model_parallel()
    torch.manual_seed(0)
    cfg = _cfg()
    ocfg = OptimizerConfig(optimizer="adam", lr=5e-3, min_lr=5e-4, weight_decay=0.0, clip_grad=1.0)
    logs = []
    metrics = eval_utils.accuracy_func_provider(lambda p: _Toy(64, seed=p), [101, 102], micro_batch_size=8,
                                                log=logs.append)
    saves = []
    hist = finetune_utils.finetune(
        lambda: (_Toy(256, seed=1), None), lambda pre_process=True, post_process=True: Classification(cfg, 2, 40, 12),
        config=cfg, optimizer_config=ocfg, epochs=4, micro_batch_size=8, global_batch_size=16 * world // world * world,
        end_of_epoch_callback_provider=lambda: metrics, save=lambda it, *a: saves.append(it), save_interval=5,
        log_interval=4, seq_length=12, log=logs.append)
    per_epoch = 256 // (16 * world)
    assert hist["iterations"] == 4 * per_epoch and len(hist["metrics"]) == 4
    assert saves.count(4 * per_epoch) == 1 and 5 in saves
    assert hist["metrics"][-1]["overall"] > 90.0 > 0, hist["metrics"]
    assert hist["metrics"][-1]["overall"] >= hist["metrics"][0]["overall"]
    assert any("metrics for toy" in l for l in logs) and any("lm loss" in l for l in logs)
    # evaluation counts cover both validation sets once, whatever the data-parallel size
    c, t = eval_utils.calculate_correct_answers("toy", hist["model"][0], finetune_utils.build_data_loader(
        _Toy(64, seed=101), 8, drop_last=False, shuffle=False), "cpu")
    assert t == 64 and abs(100.0 * c / t - hist["metrics"][-1]["toy"]) < 40
    # evaluate-only mode
    only = finetune_utils.finetune(lambda: (None, None), lambda pre_process=True, post_process=True:
                                   Classification(cfg, 2, 40, 12), config=cfg, optimizer_config=ocfg, epochs=0,
                                   micro_batch_size=8, end_of_epoch_callback_provider=lambda: metrics, log=logs.append)
    assert len(only["metrics"]) == 1 and 20.0 < only["metrics"][0]["overall"] < 80.0


def test_finetune_learns_single_process():
    run_distributed(_finetune_rank, 1)


def test_finetune_learns_data_parallel():
    run_distributed(_finetune_rank, 2)
