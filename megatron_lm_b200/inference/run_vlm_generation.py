"""Generate text for images with a LLaVA-style model: captions / answers for a folder of images.

    python -m megatron_lm_b200.inference.run_vlm_generation --load <ckpt> <model flags> --tokenizer-type ... \
        --input-image-path images/ --prompt "<image>\\nDescribe the picture." --output-path out.jsonl \
        [--input-metadata-path questions.jsonl] [--num-samples-per-partition 100] [--out-seq-length 64]

Every line of the output is ``{"sample_id", "image", "prompt", "text"}``.  With ``--input-metadata-path`` (JSON lines
with ``image`` and ``question`` / ``prompt``) each record brings its own prompt; otherwise ``--prompt`` goes with every
image of the folder.  Images: ``.npy`` arrays ([c, h, w] or [h, w, c]; uint8 or float) or picture files when Pillow
is importable; they are resized to ``--img-h`` x ``--img-w`` and normalised with the CLIP mean and deviation.
The token ``<image>`` in a prompt marks where the image embeddings go (default: in front).
Several ranks split the samples between them (``--num-partitions`` / ``--partition-id``).

Reference: tools/run_vlm_text_generation.py (arguments :30-80, the per-task generation loop :170-330, output
records :340-420).
"""
from __future__ import annotations

import json
import os
from copy import deepcopy
from typing import Dict, Iterator, List, Optional

import numpy as np
import torch
import torch.nn.functional as F

from ..models.multimodal import DEFAULT_IMAGE_TOKEN_INDEX, IMAGE_TOKEN, LLaVAModel
from ..training import arguments as A
from .engine import SamplingParams, VLMInferenceEngine

CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


def add_vlm_generation_args(parser):
    g = parser.add_argument_group(title="vision-language generation")
    g.add_argument("--input-image-path", required=True, help="folder of images")
    g.add_argument("--input-metadata-path", default=None, help="JSON lines: image, question / prompt")
    g.add_argument("--prompt", default=IMAGE_TOKEN + "\nDescribe the image.")
    g.add_argument("--output-path", required=True)
    g.add_argument("--num-samples-per-partition", type=int, default=0, help="0: all")
    g.add_argument("--num-partitions", type=int, default=1)
    g.add_argument("--partition-id", type=int, default=0)
    g.add_argument("--out-seq-length", type=int, default=32, help="tokens to generate")
    g.add_argument("--temperature", type=float, default=1.0)
    g.add_argument("--top-k", type=int, default=1)
    g.add_argument("--top-p", type=float, default=0.0)
    g.add_argument("--generation-batch-size", type=int, default=1)
    g.add_argument("--disable-vision-class-token", action="store_true",
                   help="drop the class token of the vision model before the projection (LLaVA)")
    return parser


def load_image(path: str, h: int, w: int) -> torch.Tensor:
    if path.endswith(".npy"):
        a = np.load(path)
    else:
        from PIL import Image
        a = np.asarray(Image.open(path).convert("RGB"))
    scale = 255.0 if a.dtype == np.uint8 else 1.0
    a = a.astype(np.float32) / scale
    if a.ndim == 3 and a.shape[0] != 3:
        a = a.transpose(2, 0, 1)
    t = torch.from_numpy(np.ascontiguousarray(a)).unsqueeze(0)
    if t.shape[-2:] != (h, w):
        t = F.interpolate(t, size=(h, w), mode="bicubic", align_corners=False).clamp(0, 1)
    mean = torch.tensor(CLIP_MEAN).view(1, 3, 1, 1)
    std = torch.tensor(CLIP_STD).view(1, 3, 1, 1)
    return ((t - mean) / std)[0]


def samples(args) -> Iterator[Dict]:
    if args.input_metadata_path:
        with open(args.input_metadata_path) as f:
            rows = [json.loads(line) for line in f if line.strip()]
        items = [{"image": r["image"], "prompt": r.get("prompt") or (IMAGE_TOKEN + "\n" + r["question"]),
                  "sample_id": r.get("sample_id", r.get("question_id", i))} for i, r in enumerate(rows)]
    else:
        names = sorted(n for n in os.listdir(args.input_image_path)
                       if n.lower().endswith((".npy", ".png", ".jpg", ".jpeg", ".bmp")))
        items = [{"image": n, "prompt": args.prompt, "sample_id": i} for i, n in enumerate(names)]
    mine = items[args.partition_id::max(args.num_partitions, 1)]
    if args.num_samples_per_partition:
        mine = mine[:args.num_samples_per_partition]
    yield from mine


def tokenize_prompt(prompt: str, tokenizer, image_token_index: int) -> List[int]:
    """Text around ``<image>`` is tokenised piecewise; the marker becomes the model's image token index."""
    if IMAGE_TOKEN not in prompt:
        prompt = IMAGE_TOKEN + "\n" + prompt
    before, _, after = prompt.partition(IMAGE_TOKEN)
    ids = tokenizer.tokenize(before) if before else []
    return list(ids) + [image_token_index] + list(tokenizer.tokenize(after) if after else [])


def build_model(args, config):
    vis = deepcopy(config)
    vis.num_layers = getattr(args, "encoder_num_layers", None) or config.num_layers
    proj = deepcopy(config)
    proj.num_layers = 2
    return LLaVAModel(config, args.padded_vocab_size, args.max_position_embeddings, vis, proj,
                      img_h=getattr(args, "img_h", 336), img_w=getattr(args, "img_w", 336),
                      patch_dim=getattr(args, "patch_dim", 14),
                      language_position_embedding_type=args.position_embedding_type,
                      drop_vision_class_token=getattr(args, "disable_vision_class_token", False),
                      share_embeddings_and_output_weights=not args.untie_embeddings_and_output_weights,
                      parallel_output=False)


def main(argv=None, tokenizer=None, model=None) -> List[Dict]:
    args = A.parse_args(add_vlm_generation_args, argv=argv)
    if args.micro_batch_size is None:
        args.micro_batch_size = 1
    args = A.validate_args(args)
    if tokenizer is None:
        from ..data.tokenizer import build_tokenizer
        tokenizer = build_tokenizer(args)
    if args.padded_vocab_size is None:
        args.padded_vocab_size = getattr(tokenizer, "vocab_size", None) or args.vocab_size
    cfg = A.core_transformer_config_from_args(args)
    dev = torch.device("cuda") if torch.cuda.is_available() else torch.device("cpu")
    if dev.type == "cpu":
        cfg.use_cpu_initialization = True
    if model is None:
        model = build_model(args, cfg).to(dev)
        if args.load is not None:
            from ..training import checkpointing
            checkpointing.load_checkpoint([model], None, None, args, strict=False)
    model.eval()
    engine = VLMInferenceEngine(model, tokenizer=tokenizer, max_batch_size=args.generation_batch_size,
                                max_sequence_length=args.max_position_embeddings)
    sp = SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                        num_tokens_to_generate=args.out_seq_length)
    dtype = next(model.parameters()).dtype
    records: List[Dict] = []
    os.makedirs(os.path.dirname(os.path.abspath(args.output_path)), exist_ok=True)
    with open(args.output_path, "w") as out:
        for item in samples(args):
            img = load_image(os.path.join(args.input_image_path, item["image"]), args.img_h, args.img_w)
            ids = tokenize_prompt(item["prompt"], tokenizer, model.image_token_index)
            req = engine.generate_with_images([ids], img.unsqueeze(0).to(dev, dtype), sp)[0]
            rec = {"sample_id": item["sample_id"], "image": item["image"], "prompt": item["prompt"],
                   "text": req.generated_text if req.generated_text is not None else req.generated_tokens}
            out.write(json.dumps(rec) + "\n")
            out.flush()
            records.append(rec)
    return records


if __name__ == "__main__":
    main()
