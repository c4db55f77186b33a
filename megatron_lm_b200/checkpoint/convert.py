"""Checkpoint format conversion: Hugging Face Llama / Mistral / Mixtral, legacy Megatron names, and this
framework's own ("core") layout; tensor- and pipeline-parallel re-partitioning.

``python -m megatron_lm_b200.checkpoint.convert --loader llama_hf --saver core --load-dir hf_dir
   --save-dir out --target-tensor-parallel-size 2 --target-pipeline-parallel-size 1``

Reference: tools/checkpoint/convert.py:107 (loader / saver plug-ins exchanging a stream of named
tensors), loader_llama_mistral.py, loader_mixtral_hf.py, loader_legacy.py, saver_core.py, schema_core.py.
Here a checkpoint in flight is simply a full (unpartitioned) core state dict.

Core layout facts used below:
* ``linear_qkv.weight`` is [ng * (np/ng + 2) * hn, h]: for each KV group, its np/ng query heads, then its key
  head, then its value head;
* ``linear_fc1.weight`` of a gated MLP is [gate ; up] stacked along the output dim; when split over tensor-
  parallel ranks each rank holds [gate_r ; up_r];
* Hugging Face Llama stores rotary halves the same way as this framework's default (non-interleaved) RoPE.
"""
from __future__ import annotations

import argparse
import json
import os
import re
from typing import Dict, List, Optional

import torch


# ----------------------------------------------------------------------------- HF Llama / Mistral <-> core
def _qkv_to_core(q, k, v, np_, ng, hn):
    qpg = np_ // ng
    h = q.shape[1]
    q = q.view(ng, qpg * hn, h)
    k = k.view(ng, hn, h)
    v = v.view(ng, hn, h)
    return torch.cat((q, k, v), dim=1).reshape(ng * (qpg + 2) * hn, h)


def _qkv_from_core(w, np_, ng, hn):
    qpg = np_ // ng
    h = w.shape[1]
    w = w.view(ng, (qpg + 2) * hn, h)
    q = w[:, : qpg * hn].reshape(np_ * hn, h)
    k = w[:, qpg * hn:(qpg + 1) * hn].reshape(ng * hn, h)
    v = w[:, (qpg + 1) * hn:].reshape(ng * hn, h)
    return q, k, v


def hf_llama_to_core(hf: Dict[str, torch.Tensor], num_layers: int, num_heads: int, num_query_groups: int,
                     head_dim: Optional[int] = None, tie_embeddings: bool = False) -> Dict[str, torch.Tensor]:
    h = hf["model.embed_tokens.weight"].shape[1]
    hn = head_dim or h // num_heads
    sd = {"embedding.word_embeddings.weight": hf["model.embed_tokens.weight"],
          "decoder.final_layernorm.weight": hf["model.norm.weight"]}
    if not tie_embeddings:
        sd["output_layer.weight"] = hf.get("lm_head.weight", hf["model.embed_tokens.weight"])
    for i in range(num_layers):
        s, d = f"model.layers.{i}.", f"decoder.layers.{i}."
        sd[d + "self_attention.linear_qkv.weight"] = _qkv_to_core(
            hf[s + "self_attn.q_proj.weight"], hf[s + "self_attn.k_proj.weight"], hf[s + "self_attn.v_proj.weight"],
            num_heads, num_query_groups, hn)
        if s + "self_attn.q_proj.bias" in hf:
            sd[d + "self_attention.linear_qkv.bias"] = _qkv_to_core(
                hf[s + "self_attn.q_proj.bias"].unsqueeze(1), hf[s + "self_attn.k_proj.bias"].unsqueeze(1),
                hf[s + "self_attn.v_proj.bias"].unsqueeze(1), num_heads, num_query_groups, hn).squeeze(1)
        sd[d + "self_attention.linear_proj.weight"] = hf[s + "self_attn.o_proj.weight"]
        sd[d + "input_layernorm.weight"] = hf[s + "input_layernorm.weight"]
        sd[d + "pre_mlp_layernorm.weight"] = hf[s + "post_attention_layernorm.weight"]
        if s + "mlp.gate_proj.weight" in hf:
            sd[d + "mlp.linear_fc1.weight"] = torch.cat((hf[s + "mlp.gate_proj.weight"], hf[s + "mlp.up_proj.weight"]), 0)
            sd[d + "mlp.linear_fc2.weight"] = hf[s + "mlp.down_proj.weight"]
        elif s + "mlp.experts.gate_up_proj" in hf:                  # Mixtral as newer library versions hold it in memory:
            sd[d + "mlp.router.weight"] = hf[s + "mlp.gate.weight"]  # experts fused, [E, 2f, h] (gate ; up) and [E, h, f]
            gu, dn = hf[s + "mlp.experts.gate_up_proj"], hf[s + "mlp.experts.down_proj"]
            for e in range(gu.shape[0]):
                sd[d + f"mlp.experts.local_experts.{e}.linear_fc1.weight"] = gu[e]
                sd[d + f"mlp.experts.local_experts.{e}.linear_fc2.weight"] = dn[e]
        else:                                                       # Mixtral checkpoint files: block_sparse_moe
            sd[d + "mlp.router.weight"] = hf[s + "block_sparse_moe.gate.weight"]
            e = 0
            while s + f"block_sparse_moe.experts.{e}.w1.weight" in hf:
                p = s + f"block_sparse_moe.experts.{e}."
                sd[d + f"mlp.experts.local_experts.{e}.linear_fc1.weight"] = torch.cat((hf[p + "w1.weight"], hf[p + "w3.weight"]), 0)
                sd[d + f"mlp.experts.local_experts.{e}.linear_fc2.weight"] = hf[p + "w2.weight"]
                e += 1
    return sd


def core_to_hf_llama(sd: Dict[str, torch.Tensor], num_layers: int, num_heads: int, num_query_groups: int,
                     head_dim: Optional[int] = None) -> Dict[str, torch.Tensor]:
    h = sd["embedding.word_embeddings.weight"].shape[1]
    hn = head_dim or h // num_heads
    hf = {"model.embed_tokens.weight": sd["embedding.word_embeddings.weight"],
          "model.norm.weight": sd["decoder.final_layernorm.weight"],
          "lm_head.weight": sd.get("output_layer.weight", sd["embedding.word_embeddings.weight"])}
    for i in range(num_layers):
        s, d = f"decoder.layers.{i}.", f"model.layers.{i}."
        q, k, v = _qkv_from_core(sd[s + "self_attention.linear_qkv.weight"], num_heads, num_query_groups, hn)
        hf[d + "self_attn.q_proj.weight"], hf[d + "self_attn.k_proj.weight"], hf[d + "self_attn.v_proj.weight"] = q, k, v
        hf[d + "self_attn.o_proj.weight"] = sd[s + "self_attention.linear_proj.weight"]
        hf[d + "input_layernorm.weight"] = sd[s + "input_layernorm.weight"]
        hf[d + "post_attention_layernorm.weight"] = sd[s + "pre_mlp_layernorm.weight"]
        fc1 = sd[s + "mlp.linear_fc1.weight"]
        hf[d + "mlp.gate_proj.weight"], hf[d + "mlp.up_proj.weight"] = fc1.chunk(2, dim=0)
        hf[d + "mlp.down_proj.weight"] = sd[s + "mlp.linear_fc2.weight"]
    return hf


def core_to_hf_mixtral(sd: Dict[str, torch.Tensor], num_layers: int, num_heads: int, num_query_groups: int,
                       head_dim: Optional[int] = None) -> Dict[str, torch.Tensor]:
    """Core MoE checkpoint (sequential experts: ``mlp.experts.local_experts.<e>.linear_fc1/2``, or grouped experts:
    ``mlp.experts.weight1/weight2`` of shape [E, ...]) -> Hugging Face Mixtral names (``block_sparse_moe.gate``,
    ``experts.<e>.w1 / w3 / w2``).  Reference: tools/checkpoint/loader_mixtral_hf.py:150-230 (the opposite way)."""
    h = sd["embedding.word_embeddings.weight"].shape[1]
    hn = head_dim or h // num_heads
    hf = {"model.embed_tokens.weight": sd["embedding.word_embeddings.weight"],
          "model.norm.weight": sd["decoder.final_layernorm.weight"],
          "lm_head.weight": sd.get("output_layer.weight", sd["embedding.word_embeddings.weight"])}
    for i in range(num_layers):
        s_, d = f"decoder.layers.{i}.", f"model.layers.{i}."
        q, k, v = _qkv_from_core(sd[s_ + "self_attention.linear_qkv.weight"], num_heads, num_query_groups, hn)
        hf[d + "self_attn.q_proj.weight"], hf[d + "self_attn.k_proj.weight"], hf[d + "self_attn.v_proj.weight"] = q, k, v
        hf[d + "self_attn.o_proj.weight"] = sd[s_ + "self_attention.linear_proj.weight"]
        hf[d + "input_layernorm.weight"] = sd[s_ + "input_layernorm.weight"]
        hf[d + "post_attention_layernorm.weight"] = sd[s_ + "pre_mlp_layernorm.weight"]
        hf[d + "block_sparse_moe.gate.weight"] = sd[s_ + "mlp.router.weight"]
        if s_ + "mlp.experts.weight1" in sd:                        # grouped experts: [E, h, 2f] and [E, f, h]
            w1, w2 = sd[s_ + "mlp.experts.weight1"], sd[s_ + "mlp.experts.weight2"]
            for e in range(w1.shape[0]):
                gate, up = w1[e].t().chunk(2, dim=0)
                hf[d + f"block_sparse_moe.experts.{e}.w1.weight"] = gate.contiguous()
                hf[d + f"block_sparse_moe.experts.{e}.w3.weight"] = up.contiguous()
                hf[d + f"block_sparse_moe.experts.{e}.w2.weight"] = w2[e].t().contiguous()
        else:
            e = 0
            while s_ + f"mlp.experts.local_experts.{e}.linear_fc1.weight" in sd:
                fc1 = sd[s_ + f"mlp.experts.local_experts.{e}.linear_fc1.weight"]
                hf[d + f"block_sparse_moe.experts.{e}.w1.weight"], hf[d + f"block_sparse_moe.experts.{e}.w3.weight"] = \
                    fc1.chunk(2, dim=0)
                hf[d + f"block_sparse_moe.experts.{e}.w2.weight"] = sd[s_ + f"mlp.experts.local_experts.{e}.linear_fc2.weight"]
                e += 1
    return hf


# ----------------------------------------------------------------------------- Mamba / hybrid: tensor-parallel size
# A Mamba mixer's input projection is a concatenation of five segments per rank, [z | x | B | C | dt], and its
# convolution of three, [x | B | C]: changing the tensor-parallel size has to re-cut every segment, not the whole
# matrix (reference: tools/checkpoint/hybrid_conversion.py:60-190).  Heads, groups and inner channels are split
# evenly; the state size is not split.
def _hf_llava_parts(hf: Dict[str, torch.Tensor]):
    """Prefixes of the three parts in either Hugging Face layout: checkpoint files of the original release
    (``vision_tower.`` / ``multi_modal_projector.`` / ``language_model.model.`` + ``language_model.lm_head``) or the
    in-memory names of newer library versions (everything under ``model.``, ``lm_head`` at the top)."""
    if any(k.startswith("model.vision_tower.") for k in hf):
        return "model.vision_tower.vision_model.", "model.multi_modal_projector.", "model.language_model.", "lm_head.weight"
    return "vision_tower.vision_model.", "multi_modal_projector.", "language_model.model.", "language_model.lm_head.weight"


def hf_llava_to_core(hf: Dict[str, torch.Tensor], *, num_layers: int, num_heads: int, num_query_groups: int,
                     vision_layers: int, vision_heads: int, head_dim: Optional[int] = None) -> Dict[str, torch.Tensor]:
    """Hugging Face LLaVA (CLIP vision tower + two-layer projector + Llama) -> ``LLaVAModel`` names.
    ``vision_layers`` is the number of encoder layers the core model keeps: LLaVA reads the features of the
    second-to-last CLIP layer, so the last one (and the tower's post-layernorm) is dropped.  The patch convolution
    becomes the linear map on unfolded patches.  Reference: tools/checkpoint/loader_llava.py,
    examples/multimodal/model_converter/clip_converter.py."""
    vp, pp, lp, head = _hf_llava_parts(hf)
    sd: Dict[str, torch.Tensor] = {}
    conv = hf[vp + "embeddings.patch_embedding.weight"]                      # [hv, 3, p, p]
    sd["vision_model.conv1.proj.weight"] = conv.reshape(conv.shape[0], -1)
    sd["vision_model.class_token"] = hf[vp + "embeddings.class_embedding"].reshape(1, 1, -1)
    sd["vision_model.position_embeddings.weight"] = hf[vp + "embeddings.position_embedding.weight"]
    pre = "pre_layrnorm." if vp + "pre_layrnorm.weight" in hf else "pre_layernorm."   # the library's spelling
    sd["vision_model.ln_pre.weight"], sd["vision_model.ln_pre.bias"] = hf[vp + pre + "weight"], hf[vp + pre + "bias"]
    hv = conv.shape[0]
    hnv = hv // vision_heads
    for i in range(vision_layers):
        s_, d = f"{vp}encoder.layers.{i}.", f"vision_model.decoder.layers.{i}."
        for kind in ("weight", "bias"):
            q, k, v = (hf[s_ + f"self_attn.{n}_proj.{kind}"] for n in "qkv")
            if kind == "bias":
                sd[d + "self_attention.linear_qkv.bias"] = _qkv_to_core(q.unsqueeze(1), k.unsqueeze(1), v.unsqueeze(1),
                                                                         vision_heads, vision_heads, hnv).squeeze(1)
            else:
                sd[d + "self_attention.linear_qkv.weight"] = _qkv_to_core(q, k, v, vision_heads, vision_heads, hnv)
            sd[d + f"self_attention.linear_proj.{kind}"] = hf[s_ + f"self_attn.out_proj.{kind}"]
            sd[d + f"input_layernorm.{kind}"] = hf[s_ + f"layer_norm1.{kind}"]
            sd[d + f"pre_mlp_layernorm.{kind}"] = hf[s_ + f"layer_norm2.{kind}"]
            sd[d + f"mlp.linear_fc1.{kind}"] = hf[s_ + f"mlp.fc1.{kind}"]
            sd[d + f"mlp.linear_fc2.{kind}"] = hf[s_ + f"mlp.fc2.{kind}"]
    for kind in ("weight", "bias"):
        sd[f"vision_projection.linear_fc1.{kind}"] = hf[pp + f"linear_1.{kind}"]
        sd[f"vision_projection.linear_fc2.{kind}"] = hf[pp + f"linear_2.{kind}"]
    llama = {"model." + k[len(lp):]: v for k, v in hf.items() if k.startswith(lp)}
    llama["lm_head.weight"] = hf.get(head, llama["model.embed_tokens.weight"])
    for k, v in hf_llama_to_core(llama, num_layers, num_heads, num_query_groups, head_dim).items():
        sd["language_model." + k] = v
    return sd


def core_to_hf_llava(sd: Dict[str, torch.Tensor], *, num_layers: int, num_heads: int, num_query_groups: int,
                     vision_layers: int, vision_heads: int, patch_dim: int, head_dim: Optional[int] = None,
                     in_memory_names: bool = True) -> Dict[str, torch.Tensor]:
    """``LLaVAModel`` names -> Hugging Face LLaVA.  The CLIP layer that LLaVA never reads and the tower's
    post-layernorm do not exist in the core model: they are written as an identity-initialised copy of the last
    kept layer and a unit layernorm, so the file loads into the library's class and computes the same features.
    Reference: tools/checkpoint/saver_hf_llava.py."""
    if in_memory_names:
        vp, pp, lp, head = "model.vision_tower.vision_model.", "model.multi_modal_projector.", "model.language_model.", "lm_head.weight"
    else:
        vp, pp, lp, head = "vision_tower.vision_model.", "multi_modal_projector.", "language_model.model.", "language_model.lm_head.weight"
    hf: Dict[str, torch.Tensor] = {}
    w = sd["vision_model.conv1.proj.weight"]
    hv = w.shape[0]
    hf[vp + "embeddings.patch_embedding.weight"] = w.reshape(hv, 3, patch_dim, patch_dim)
    hf[vp + "embeddings.class_embedding"] = sd["vision_model.class_token"].reshape(-1)
    hf[vp + "embeddings.position_embedding.weight"] = sd["vision_model.position_embeddings.weight"]
    hf[vp + "pre_layrnorm.weight"], hf[vp + "pre_layrnorm.bias"] = sd["vision_model.ln_pre.weight"], sd["vision_model.ln_pre.bias"]
    hnv = hv // vision_heads
    for i in range(vision_layers + 1):
        src = min(i, vision_layers - 1)                                       # the extra layer repeats the last one
        s_, d = f"vision_model.decoder.layers.{src}.", f"{vp}encoder.layers.{i}."
        q, k, v = _qkv_from_core(sd[s_ + "self_attention.linear_qkv.weight"], vision_heads, vision_heads, hnv)
        qb, kb, vb = (t.squeeze(1) for t in _qkv_from_core(sd[s_ + "self_attention.linear_qkv.bias"].unsqueeze(1),
                                                           vision_heads, vision_heads, hnv))
        for n, wt, bs in (("q", q, qb), ("k", k, kb), ("v", v, vb)):
            hf[d + f"self_attn.{n}_proj.weight"], hf[d + f"self_attn.{n}_proj.bias"] = wt, bs
        for kind in ("weight", "bias"):
            hf[d + f"self_attn.out_proj.{kind}"] = sd[s_ + f"self_attention.linear_proj.{kind}"]
            hf[d + f"layer_norm1.{kind}"] = sd[s_ + f"input_layernorm.{kind}"]
            hf[d + f"layer_norm2.{kind}"] = sd[s_ + f"pre_mlp_layernorm.{kind}"]
            hf[d + f"mlp.fc1.{kind}"] = sd[s_ + f"mlp.linear_fc1.{kind}"]
            hf[d + f"mlp.fc2.{kind}"] = sd[s_ + f"mlp.linear_fc2.{kind}"]
    hf[vp + "post_layernorm.weight"] = torch.ones(hv, dtype=w.dtype)
    hf[vp + "post_layernorm.bias"] = torch.zeros(hv, dtype=w.dtype)
    for kind in ("weight", "bias"):
        hf[pp + f"linear_1.{kind}"] = sd[f"vision_projection.linear_fc1.{kind}"]
        hf[pp + f"linear_2.{kind}"] = sd[f"vision_projection.linear_fc2.{kind}"]
    lm = {k[len("language_model."):]: v for k, v in sd.items() if k.startswith("language_model.")}
    for k, v in core_to_hf_llama(lm, num_layers, num_heads, num_query_groups, head_dim).items():
        if k == "lm_head.weight":
            hf[head] = v
        else:
            hf[lp + k[len("model."):]] = v
    return hf


def _mamba_dims(in_proj_rows_total: int, d_model: int, nheads: int, ngroups: int, d_state: int):
    d_inner = (in_proj_rows_total - 2 * ngroups * d_state - nheads) // 2
    if 2 * d_inner + 2 * ngroups * d_state + nheads != in_proj_rows_total or d_inner % nheads:
        raise ValueError("in_proj size does not match the given heads / groups / state size")
    return d_inner


def mamba_merge_tp(shards: List[Dict[str, torch.Tensor]], nheads: int, ngroups: int, d_state: int,
                   gated_mlp: bool = True) -> Dict[str, torch.Tensor]:
    """Per-rank state dicts of a Mamba / hybrid model -> one unpartitioned state dict."""
    tp = len(shards)
    out: Dict[str, torch.Tensor] = {}
    for name in shards[0]:
        parts = [sd[name] for sd in shards]
        if name.endswith("mixer.in_proj.weight"):
            total = sum(p.shape[0] for p in parts)
            d_inner = _mamba_dims(total, parts[0].shape[1], nheads, ngroups, d_state)
            di, gn, hl = d_inner // tp, ngroups * d_state // tp, nheads // tp
            segs = [torch.split(p, [di, di, gn, gn, hl], dim=0) for p in parts]
            out[name] = torch.cat([torch.cat([sg[j] for sg in segs], dim=0) for j in range(5)], dim=0)
        elif name.endswith(("mixer.conv_weight", "mixer.conv_bias")):
            total = sum(p.shape[0] for p in parts)
            d_inner = total - 2 * ngroups * d_state
            di, gn = d_inner // tp, ngroups * d_state // tp
            segs = [torch.split(p, [di, gn, gn], dim=0) for p in parts]
            out[name] = torch.cat([torch.cat([sg[j] for sg in segs], dim=0) for j in range(3)], dim=0)
        elif name.endswith(("mixer.dt_bias", "mixer.A_log", "mixer.D", "mixer.norm_weight")):
            out[name] = torch.cat(parts, dim=0)
        elif name.endswith("mixer.out_proj.weight"):
            out[name] = torch.cat(parts, dim=1)
    rest = [{k: v for k, v in sd.items() if k not in out} for sd in shards]
    out.update(merge_tp(rest, gated_mlp))                 # attention / MLP layers of a hybrid model, embeddings, norms
    return out


def mamba_split_for_tp(sd: Dict[str, torch.Tensor], tp: int, nheads: int, ngroups: int, d_state: int,
                       gated_mlp: bool = True) -> List[Dict[str, torch.Tensor]]:
    """Unpartitioned Mamba / hybrid state dict -> ``tp`` per-rank state dicts."""
    if nheads % tp or ngroups % tp:
        raise ValueError("heads and groups must divide by the tensor-parallel size")
    out: List[Dict[str, torch.Tensor]] = [dict() for _ in range(tp)]
    for name, w in sd.items():
        if name.endswith("mixer.in_proj.weight"):
            d_inner = _mamba_dims(w.shape[0], w.shape[1], nheads, ngroups, d_state)
            segs = torch.split(w, [d_inner, d_inner, ngroups * d_state, ngroups * d_state, nheads], dim=0)
            cut = [sg.chunk(tp, dim=0) for sg in segs]
            for r in range(tp):
                out[r][name] = torch.cat([c[r] for c in cut], dim=0).contiguous()
        elif name.endswith(("mixer.conv_weight", "mixer.conv_bias")):
            d_inner = w.shape[0] - 2 * ngroups * d_state
            segs = torch.split(w, [d_inner, ngroups * d_state, ngroups * d_state], dim=0)
            cut = [sg.chunk(tp, dim=0) for sg in segs]
            for r in range(tp):
                out[r][name] = torch.cat([c[r] for c in cut], dim=0).contiguous()
        elif name.endswith(("mixer.dt_bias", "mixer.A_log", "mixer.D", "mixer.norm_weight")):
            for r, c in enumerate(w.chunk(tp, dim=0)):
                out[r][name] = c.contiguous()
        elif name.endswith("mixer.out_proj.weight"):
            for r, c in enumerate(w.chunk(tp, dim=1)):
                out[r][name] = c.contiguous()
    rest = {k: v for k, v in sd.items() if k not in out[0]}
    for r, part in enumerate(split_for_tp(rest, tp, gated_mlp)):
        out[r].update(part)
    return out


# ----------------------------------------------------------------------------- legacy Megatron names -> core
_LEGACY = [
    (r"^language_model\.embedding\.word_embeddings\.weight$", "embedding.word_embeddings.weight"),
    (r"^language_model\.embedding\.position_embeddings\.weight$", "embedding.position_embeddings.weight"),
    (r"^language_model\.encoder\.layers\.(\d+)\.input_norm\.(weight|bias)$", r"decoder.layers.\1.input_layernorm.\2"),
    (r"^language_model\.encoder\.layers\.(\d+)\.input_layernorm\.(weight|bias)$", r"decoder.layers.\1.input_layernorm.\2"),
    (r"^language_model\.encoder\.layers\.(\d+)\.self_attention\.query_key_value\.(weight|bias)$",
     r"decoder.layers.\1.self_attention.linear_qkv.\2"),
    (r"^language_model\.encoder\.layers\.(\d+)\.self_attention\.dense\.(weight|bias)$",
     r"decoder.layers.\1.self_attention.linear_proj.\2"),
    (r"^language_model\.encoder\.layers\.(\d+)\.post_attention_(?:layer)?norm\.(weight|bias)$",
     r"decoder.layers.\1.pre_mlp_layernorm.\2"),
    (r"^language_model\.encoder\.layers\.(\d+)\.mlp\.dense_h_to_4h\.(weight|bias)$", r"decoder.layers.\1.mlp.linear_fc1.\2"),
    (r"^language_model\.encoder\.layers\.(\d+)\.mlp\.dense_4h_to_h\.(weight|bias)$", r"decoder.layers.\1.mlp.linear_fc2.\2"),
    (r"^language_model\.encoder\.final_(?:layer)?norm\.(weight|bias)$", r"decoder.final_layernorm.\1"),
    (r"^language_model\.output_layer\.weight$", "output_layer.weight"),
]


def legacy_to_core(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Flattened legacy state dict (keys joined by '.') -> core names.  Unknown keys are kept."""
    out = {}
    for k, v in sd.items():
        for pat, rep in _LEGACY:
            if re.match(pat, k):
                k = re.sub(pat, rep, k)
                break
        out[k] = v
    return out


def core_to_legacy(sd):
    inv = [
        (r"^embedding\.(word|position)_embeddings\.weight$", r"language_model.embedding.\1_embeddings.weight"),
        (r"^decoder\.layers\.(\d+)\.input_layernorm\.(weight|bias)$", r"language_model.encoder.layers.\1.input_norm.\2"),
        (r"^decoder\.layers\.(\d+)\.self_attention\.linear_qkv\.(weight|bias)$",
         r"language_model.encoder.layers.\1.self_attention.query_key_value.\2"),
        (r"^decoder\.layers\.(\d+)\.self_attention\.linear_proj\.(weight|bias)$",
         r"language_model.encoder.layers.\1.self_attention.dense.\2"),
        (r"^decoder\.layers\.(\d+)\.pre_mlp_layernorm\.(weight|bias)$", r"language_model.encoder.layers.\1.post_attention_norm.\2"),
        (r"^decoder\.layers\.(\d+)\.mlp\.linear_fc1\.(weight|bias)$", r"language_model.encoder.layers.\1.mlp.dense_h_to_4h.\2"),
        (r"^decoder\.layers\.(\d+)\.mlp\.linear_fc2\.(weight|bias)$", r"language_model.encoder.layers.\1.mlp.dense_4h_to_h.\2"),
        (r"^decoder\.final_layernorm\.(weight|bias)$", r"language_model.encoder.final_norm.\1"),
        (r"^output_layer\.weight$", "language_model.output_layer.weight"),
    ]
    out = {}
    for k, v in sd.items():
        for pat, rep in inv:
            if re.match(pat, k):
                k = re.sub(pat, rep, k)
                break
        out[k] = v
    return out


# ----------------------------------------------------------------------------- TP / PP re-partitioning
_COL = ("linear_qkv.weight", "linear_qkv.bias", "linear_fc1.weight", "linear_fc1.bias", "word_embeddings.weight",
        "output_layer.weight", "linear_q_up_proj.weight", "linear_kv_up_proj.weight", "linear_q_proj.weight")
_ROW = ("linear_proj.weight", "linear_fc2.weight")


def _kind(name: str) -> str:
    if name.endswith(_COL):
        return "col"
    if name.endswith(_ROW):
        return "row"
    return "rep"


def split_for_tp(sd: Dict[str, torch.Tensor], tp: int, gated_mlp: bool = True) -> List[Dict[str, torch.Tensor]]:
    outs = [dict() for _ in range(tp)]
    for k, v in sd.items():
        kind = _kind(k)
        if kind == "rep" or tp == 1:
            for o in outs:
                o[k] = v
        elif kind == "row":
            for r, piece in enumerate(v.chunk(tp, dim=1)):
                outs[r][k] = piece.contiguous()
        elif "linear_fc1" in k and gated_mlp:
            gate, up = v.chunk(2, dim=0)
            for r, (g_, u_) in enumerate(zip(gate.chunk(tp, 0), up.chunk(tp, 0))):
                outs[r][k] = torch.cat((g_, u_), 0)
        else:
            for r, piece in enumerate(v.chunk(tp, dim=0)):
                outs[r][k] = piece.contiguous()
    return outs


def merge_tp(shards: List[Dict[str, torch.Tensor]], gated_mlp: bool = True) -> Dict[str, torch.Tensor]:
    tp = len(shards)
    out = {}
    for k in shards[0]:
        kind = _kind(k)
        vs = [s[k] for s in shards]
        if kind == "rep" or tp == 1:
            out[k] = vs[0]
        elif kind == "row":
            out[k] = torch.cat(vs, dim=1)
        elif "linear_fc1" in k and gated_mlp:
            out[k] = torch.cat([v.chunk(2, 0)[0] for v in vs] + [v.chunk(2, 0)[1] for v in vs], 0)
        else:
            out[k] = torch.cat(vs, dim=0)
    return out


def split_for_pp(sd: Dict[str, torch.Tensor], pp: int, num_layers: int) -> List[Dict[str, torch.Tensor]]:
    """Stage s gets layers [s*L/pp, (s+1)*L/pp) renumbered from 0, the embedding on the first stage, the final norm
    and output layer on the last."""
    per = num_layers // pp
    outs = [dict() for _ in range(pp)]
    for k, v in sd.items():
        m = re.match(r"^decoder\.layers\.(\d+)\.(.*)$", k)
        if m:
            i = int(m.group(1))
            outs[i // per][f"decoder.layers.{i % per}.{m.group(2)}"] = v
        elif k.startswith("embedding."):
            outs[0][k] = v
        else:
            outs[-1][k] = v
    return outs


def merge_pp(stages: List[Dict[str, torch.Tensor]]) -> Dict[str, torch.Tensor]:
    out, base = {}, 0
    for st in stages:
        n = 0
        for k, v in st.items():
            m = re.match(r"^decoder\.layers\.(\d+)\.(.*)$", k)
            if m:
                i = int(m.group(1))
                n = max(n, i + 1)
                out[f"decoder.layers.{base + i}.{m.group(2)}"] = v
            else:
                out[k] = v
        base += n
    return out


# ----------------------------------------------------------------------------- file IO + CLI
def load_hf_dir(path: str) -> Dict[str, torch.Tensor]:
    sd = {}
    files = sorted(f for f in os.listdir(path) if f.endswith((".safetensors", ".bin", ".pt")))
    for f in files:
        fp = os.path.join(path, f)
        if f.endswith(".safetensors"):
            from safetensors.torch import load_file
            sd.update(load_file(fp))
        else:
            sd.update(torch.load(fp, map_location="cpu", weights_only=True))
    return sd


def save_core(sd_by_rank, save_dir: str, iteration: int = 0, meta: Optional[dict] = None):
    """``sd_by_rank[pp][tp]`` -> ``iter_XXXXXXX/mp_rank_TT[_PPP]/model_optim_rng.pt`` + tracker file."""
    pp, tp = len(sd_by_rank), len(sd_by_rank[0])
    it_dir = os.path.join(save_dir, "release" if iteration == 0 else f"iter_{iteration:07d}")
    for p in range(pp):
        for t in range(tp):
            name = f"mp_rank_{t:02d}" if pp == 1 else f"mp_rank_{t:02d}_{p:03d}"
            d = os.path.join(it_dir, name)
            os.makedirs(d, exist_ok=True)
            torch.save({"model": sd_by_rank[p][t], "iteration": iteration, "checkpoint_version": 3.0,
                        "args": meta or {}}, os.path.join(d, "model_optim_rng.pt"))
    with open(os.path.join(save_dir, "latest_checkpointed_iteration.txt"), "w") as f:
        f.write("release" if iteration == 0 else str(iteration))


def load_core(load_dir: str):
    with open(os.path.join(load_dir, "latest_checkpointed_iteration.txt")) as f:
        tag = f.read().strip()
    it_dir = os.path.join(load_dir, "release" if tag == "release" else f"iter_{int(tag):07d}")
    ranks = {}
    for name in sorted(os.listdir(it_dir)):
        m = re.match(r"^mp_rank_(\d+)(?:_(\d+))?$", name)
        if m:
            t, p = int(m.group(1)), int(m.group(2) or 0)
            ranks[(p, t)] = torch.load(os.path.join(it_dir, name, "model_optim_rng.pt"), map_location="cpu",
                                       weights_only=False)["model"]
    pp = max(p for p, _ in ranks) + 1
    tp = max(t for _, t in ranks) + 1
    return merge_pp([merge_tp([ranks[(p, t)] for t in range(tp)]) for p in range(pp)])


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model-type", default="GPT")
    ap.add_argument("--loader", required=True, choices=["llama_hf", "mistral_hf", "mixtral_hf", "llava_hf", "core", "legacy"])
    ap.add_argument("--saver", required=True, choices=["core", "legacy", "llama_hf", "mixtral_hf", "llava_hf"])
    ap.add_argument("--vision-layers", type=int, default=None, help="LLaVA, core -> HF: encoder layers of the vision model")
    ap.add_argument("--vision-heads", type=int, default=None)
    ap.add_argument("--patch-dim", type=int, default=14)
    ap.add_argument("--num-attention-heads", type=int, default=None, help="core -> HF: heads (not stored in the tensors)")
    ap.add_argument("--num-query-groups", type=int, default=None)
    ap.add_argument("--mamba-heads", type=int, default=0,
                    help="Mamba / hybrid checkpoints: heads, groups and state size of the mixers; the tensor-parallel split "
                         "then re-cuts every segment of in_proj and conv (z | x | B | C | dt)")
    ap.add_argument("--mamba-groups", type=int, default=8)
    ap.add_argument("--mamba-state-dim", type=int, default=128)
    ap.add_argument("--load-dir", required=True)
    ap.add_argument("--save-dir", required=True)
    ap.add_argument("--target-tensor-parallel-size", type=int, default=1)
    ap.add_argument("--target-pipeline-parallel-size", type=int, default=1)
    a = ap.parse_args(argv)
    meta = {}
    if a.loader == "llava_hf":
        with open(os.path.join(a.load_dir, "config.json")) as f:
            c = json.load(f)
        t, v = c["text_config"], c["vision_config"]
        keep = v["num_hidden_layers"] + (c.get("vision_feature_layer", -2) + 1)       # -2: all but the last layer
        meta = {"num_layers": t["num_hidden_layers"], "num_attention_heads": t["num_attention_heads"],
                "num_query_groups": t.get("num_key_value_heads", t["num_attention_heads"]),
                "hidden_size": t["hidden_size"], "ffn_hidden_size": t["intermediate_size"],
                "kv_channels": t.get("head_dim"), "padded_vocab_size": t["vocab_size"],
                "vision_layers": keep, "vision_heads": v["num_attention_heads"], "patch_dim": v["patch_size"],
                "img_h": v["image_size"], "img_w": v["image_size"], "image_token_index": c.get("image_token_index")}
        sd = hf_llava_to_core(load_hf_dir(a.load_dir), num_layers=meta["num_layers"],
                              num_heads=meta["num_attention_heads"], num_query_groups=meta["num_query_groups"],
                              vision_layers=keep, vision_heads=meta["vision_heads"], head_dim=meta["kv_channels"])
    elif a.loader.endswith("_hf"):
        with open(os.path.join(a.load_dir, "config.json")) as f:
            c = json.load(f)
        meta = {"num_layers": c["num_hidden_layers"], "num_attention_heads": c["num_attention_heads"],
                "num_query_groups": c.get("num_key_value_heads", c["num_attention_heads"]),
                "hidden_size": c["hidden_size"], "ffn_hidden_size": c["intermediate_size"],
                "kv_channels": c.get("head_dim"), "padded_vocab_size": c["vocab_size"],
                "norm_epsilon": c.get("rms_norm_eps", 1e-5), "rotary_base": c.get("rope_theta", 10000.0)}
        sd = hf_llama_to_core(load_hf_dir(a.load_dir), meta["num_layers"], meta["num_attention_heads"],
                              meta["num_query_groups"], meta["kv_channels"], c.get("tie_word_embeddings", False))
    else:
        sd = load_core(a.load_dir)
        if a.loader == "legacy":
            sd = legacy_to_core(sd)
        meta = {"num_layers": 1 + max(int(m.group(1)) for m in
                                      (re.match(r"^(?:language_model\.)?decoder\.layers\.(\d+)\.", k) for k in sd) if m)}
    if a.num_attention_heads:
        meta["num_attention_heads"] = a.num_attention_heads
        meta["num_query_groups"] = a.num_query_groups or a.num_attention_heads
    if a.saver == "llava_hf":
        vl = a.vision_layers or 1 + max(int(m.group(1)) for m in
                                        (re.match(r"^vision_model\.decoder\.layers\.(\d+)\.", k) for k in sd) if m)
        if not (a.vision_heads or meta.get("vision_heads")):
            raise SystemExit("--saver llava_hf needs --vision-heads (and --num-attention-heads / --num-query-groups)")
        hf = core_to_hf_llava(sd, num_layers=meta["num_layers"], num_heads=meta["num_attention_heads"],
                              num_query_groups=meta["num_query_groups"], vision_layers=vl,
                              vision_heads=a.vision_heads or meta["vision_heads"],
                              patch_dim=meta.get("patch_dim", a.patch_dim), head_dim=meta.get("kv_channels"),
                              in_memory_names=False)
        os.makedirs(a.save_dir, exist_ok=True)
        torch.save(hf, os.path.join(a.save_dir, "pytorch_model.bin"))
        return
    if a.saver in ("llama_hf", "mixtral_hf"):
        to_hf = core_to_hf_mixtral if a.saver == "mixtral_hf" else core_to_hf_llama
        hf = to_hf(sd, meta["num_layers"], meta["num_attention_heads"], meta["num_query_groups"],
                   meta.get("kv_channels"))
        os.makedirs(a.save_dir, exist_ok=True)
        torch.save(hf, os.path.join(a.save_dir, "pytorch_model.bin"))
        return
    if a.saver == "legacy":
        sd = core_to_legacy(sd)
        save_core([[sd]], a.save_dir, 0, meta)
        return
    if any(k.startswith("vision_model.") for k in sd):
        # vision-language model: one pipeline stage; the vision tower and the projector have plain (un-gated) MLPs
        if a.target_pipeline_parallel_size != 1:
            raise SystemExit("vision-language checkpoints are written for one pipeline stage")
        tp = a.target_tensor_parallel_size
        lang = {k: v for k, v in sd.items() if k.startswith("language_model.")}
        rest = {k: v for k, v in sd.items() if not k.startswith("language_model.")}
        shards = [dict(x, **y) for x, y in zip(split_for_tp(lang, tp, True), split_for_tp(rest, tp, False))]
        save_core([shards], a.save_dir, 0, meta)
        return
    stages = split_for_pp(sd, a.target_pipeline_parallel_size, meta["num_layers"])
    if a.mamba_heads:
        cut = lambda st: mamba_split_for_tp(st, a.target_tensor_parallel_size, a.mamba_heads, a.mamba_groups,   # noqa: E731
                                            a.mamba_state_dim)
    else:
        cut = lambda st: split_for_tp(st, a.target_tensor_parallel_size)                                        # noqa: E731
    save_core([cut(st) for st in stages], a.save_dir, 0, meta)


if __name__ == "__main__":
    main()
