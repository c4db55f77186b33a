"""Vision encoder, projector, LLaVA splice and MIMO alignment."""
import torch

from megatron_lm_b200.config import TransformerConfig
from megatron_lm_b200.models.gpt import GPTModel
from megatron_lm_b200.models.mimo import MimoModel, ModalitySubmodules
from megatron_lm_b200.models.multimodal import IGNORE_INDEX, LLaVAModel
from megatron_lm_b200.models.vision import CLIPViTModel, RADIOViTModel, get_num_image_embeddings


def _cfg(h=32, layers=1):
    return TransformerConfig(num_layers=layers, hidden_size=h, num_attention_heads=4, ffn_hidden_size=2 * h,
                             hidden_dropout=0.0, attention_dropout=0.0)


def test_vit_shapes_and_counts():
    v = CLIPViTModel(_cfg(), patch_dim=4, img_h=16, img_w=16)
    x = torch.randn(2, 3, 16, 16)
    assert v(x).shape == (2, 17, 32)
    assert get_num_image_embeddings(16, 16, 4, "clip", False, 1) == 17
    assert get_num_image_embeddings(16, 16, 4, "clip", True, 1) == 16
    r = RADIOViTModel(_cfg(), patch_dim=4, img_h=16, img_w=16, max_img_h=32, max_img_w=32, class_token_len=2)
    assert r(x).shape == (2, 18, 32)
    assert r(torch.randn(1, 3, 8, 24)).shape == (1, 2 + 2 * 6, 32)


def test_llava_splice_and_loss():
    torch.manual_seed(0)
    m = LLaVAModel(_cfg(), 64, 64, _cfg(h=16), _cfg(), img_h=8, img_w=8, patch_dim=4, drop_vision_class_token=True,
                   image_token_index=-200)
    assert m.img_seq_len == 4
    ids = torch.tensor([[5, -200, 7, 8, 9], [1, 2, 3, -200, 4]])
    labels = torch.tensor([[6, 7, 8, 9, 10], [2, 3, 4, 5, 6]])
    mask = torch.ones(2, 5)
    images = torch.randn(2, 3, 8, 8)
    loss, new_mask = m(images, ids, labels=labels, loss_mask=mask)
    assert loss.shape == (2, 8) and new_mask.shape == (2, 8)
    # sample 0: [t, i, i, i, i, t, t, t]; only the last image slot carries a label
    assert new_mask[0].tolist() == [1, 0, 0, 0, 1, 1, 1, 1]
    (loss * new_mask).sum().backward()
    g = m.vision_model.conv1.proj.weight.grad
    assert g is not None and g.abs().sum() > 0
    logits = m(images, ids)
    assert logits.shape == (2, 8, 64)


def test_mimo_alignment():
    torch.manual_seed(0)
    lm = GPTModel(_cfg(), 64, 32)

    class Enc(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.l = torch.nn.Linear(6, 32)

        def forward(self, x):
            return self.l(x)
    sub = ModalitySubmodules(encoders={"e": Enc()}, input_projections=[torch.nn.Linear(32, 32)])
    m = MimoModel(lm, {"audio": sub}, {"audio": 63})
    ids = torch.tensor([[1, 63, 63, 4], [63, 2, 3, 4]])
    feats = torch.randn(3, 6)
    out, _ = m(ids, modality_inputs={"audio": {"e": {"x": feats}}}, labels=ids.clamp(max=62))
    assert out.shape == (2, 4)
    out.mean().backward()
    assert sub.encoders["e"].l.weight.grad.abs().sum() > 0


def test_vlm_generation_program_writes_one_record_per_image(tmp_path):
    import json
    import numpy as np
    from megatron_lm_b200.inference import run_vlm_generation as prog

    class Tok:
        eod, vocab_size = 0, 64
        def tokenize(self, s): return [1 + (ord(c) % 60) for c in s.strip()][:6]
        def detokenize(self, ids): return " ".join(str(i) for i in ids)
    img_dir = tmp_path / "imgs"
    img_dir.mkdir()
    rng = np.random.RandomState(0)
    np.save(img_dir / "a.npy", rng.randint(0, 255, (40, 30, 3)).astype(np.uint8))      # h, w, c bytes: resized
    np.save(img_dir / "b.npy", rng.rand(3, 28, 28).astype(np.float32))
    meta = tmp_path / "q.jsonl"
    meta.write_text(json.dumps({"image": "b.npy", "question": "what", "question_id": 7}) + "\n")
    flags = ["--num-layers", "1", "--hidden-size", "32", "--num-attention-heads", "4", "--seq-length", "48",
             "--max-position-embeddings", "48", "--vocab-size", "64", "--position-embedding-type", "rope",
             "--untie-embeddings-and-output-weights", "--img-h", "28", "--img-w", "28", "--patch-dim", "14",
             "--use-cpu-initialization", "--attention-dropout", "0", "--hidden-dropout", "0",
             "--input-image-path", str(img_dir), "--out-seq-length", "4"]
    recs = prog.main(flags + ["--output-path", str(tmp_path / "o.jsonl"), "--prompt", "<image>\nhi"], tokenizer=Tok())
    lines = [json.loads(l) for l in (tmp_path / "o.jsonl").read_text().splitlines()]
    assert [r["image"] for r in lines] == ["a.npy", "b.npy"] and lines == recs
    assert all(1 <= len(r["text"].split()) <= 4 for r in lines)
    recs = prog.main(flags + ["--output-path", str(tmp_path / "o2.jsonl"), "--input-metadata-path", str(meta)],
                     tokenizer=Tok())
    assert len(recs) == 1 and recs[0]["sample_id"] == 7 and recs[0]["prompt"].endswith("what")
    assert prog.tokenize_prompt("ab<image>cd", Tok(), -200)[2] == -200
    img = prog.load_image(str(img_dir / "a.npy"), 28, 28)
    assert img.shape == (3, 28, 28) and -2.5 < float(img.min()) and float(img.max()) < 2.5
