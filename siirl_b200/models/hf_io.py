"""HF safetensors interchange for :class:`DecoderLM`.

Internal fused parameters <-> HF names (Llama/Qwen2/Qwen3/Qwen3-MoE):
``qkv_proj`` = cat(q_proj, k_proj, v_proj), ``gate_up_proj`` = cat(gate_proj, up_proj),
``experts_gate_up[e]`` = cat(experts.e.gate_proj, experts.e.up_proj), ``experts_down[e]`` = experts.e.down_proj.
The reference writes HF weights through FSDP full-state-dict gathering / mbridge
(siirl/utils/checkpoint/fsdp_checkpoint_manager.py:129-252); here the replicated working copy is written
directly, sharded by file size."""
from __future__ import annotations

import json
import os
from typing import Dict, Iterator, Tuple

import torch

from .config import DecoderConfig


def _moe_names(cfg: DecoderConfig) -> Dict[str, str]:
    """HF parameter names of the routed experts: Mixtral says ``block_sparse_moe.experts.N.w1 / w3 / w2`` where the
    Qwen MoE families say ``mlp.experts.N.gate_proj / up_proj / down_proj``."""
    if cfg.model_type == "mixtral":
        return {"router": "block_sparse_moe.gate.weight", "expert": "block_sparse_moe.experts.{e}.{w}.weight",
                "gate": "w1", "up": "w3", "down": "w2"}
    return {"router": "mlp.gate.weight", "expert": "mlp.experts.{e}.{w}.weight", "gate": "gate_proj",
            "up": "up_proj", "down": "down_proj"}


def _decoder_state(model) -> Iterator[Tuple[str, torch.Tensor]]:
    """Language-model parameters under transformers' causal-LM names (``model.layers.N...``, ``lm_head.weight``)."""
    cfg: DecoderConfig = model.cfg
    qw, kw = cfg.q_width, cfg.kv_width
    yield "model.embed_tokens.weight", model.embed_tokens.data
    for i, layer in enumerate(model.layers):
        p = f"model.layers.{i}."
        yield p + "input_layernorm.weight", layer.input_layernorm.data
        if cfg.is_mla:
            if cfg.q_lora_rank > 0:
                yield p + "self_attn.q_a_proj.weight", layer.q_a_proj_weight.data
                yield p + "self_attn.q_a_layernorm.weight", layer.q_a_layernorm.data
                yield p + "self_attn.q_b_proj.weight", layer.q_b_proj_weight.data
            else:
                yield p + "self_attn.q_proj.weight", layer.q_proj_weight.data
            yield p + "self_attn.kv_a_proj_with_mqa.weight", layer.kv_a_proj_weight.data
            yield p + "self_attn.kv_a_layernorm.weight", layer.kv_a_layernorm.data
            yield p + "self_attn.kv_b_proj.weight", layer.kv_b_proj_weight.data
        else:
            w = layer.qkv_proj_weight.data
            yield p + "self_attn.q_proj.weight", w[:qw]
            yield p + "self_attn.k_proj.weight", w[qw:qw + kw]
            yield p + "self_attn.v_proj.weight", w[qw + kw:]
        if layer.qkv_proj_bias is not None:
            b = layer.qkv_proj_bias.data
            yield p + "self_attn.q_proj.bias", b[:qw]
            yield p + "self_attn.k_proj.bias", b[qw:qw + kw]
            yield p + "self_attn.v_proj.bias", b[qw + kw:]
        if cfg.qk_norm:
            yield p + "self_attn.q_norm.weight", layer.q_norm.data
            yield p + "self_attn.k_norm.weight", layer.k_norm.data
        yield p + "self_attn.o_proj.weight", layer.o_proj_weight.data
        yield p + "post_attention_layernorm.weight", layer.post_attention_layernorm.data
        if getattr(layer, "is_moe", cfg.is_moe):
            I = cfg.moe_intermediate_size
            names = _moe_names(cfg)
            yield p + names["router"], layer.router_weight.data
            if hasattr(layer, "router_bias"):
                yield p + "mlp.gate.e_score_correction_bias", layer.router_bias.data
            for e in range(cfg.num_experts):
                gu = layer.experts_gate_up.data[e]
                yield p + names["expert"].format(e=e, w=names["gate"]), gu[:I]
                yield p + names["expert"].format(e=e, w=names["up"]), gu[I:]
                yield p + names["expert"].format(e=e, w=names["down"]), layer.experts_down.data[e]
            if cfg.shared_expert_intermediate_size > 0:
                Is = cfg.shared_expert_intermediate_size
                sgu = layer.shared_gate_up_weight.data
                sh = "mlp.shared_experts." if cfg.is_mla or cfg.scoring_func == "sigmoid" else "mlp.shared_expert."
                yield p + sh + "gate_proj.weight", sgu[:Is]
                yield p + sh + "up_proj.weight", sgu[Is:]
                yield p + sh + "down_proj.weight", layer.shared_down_weight.data
                if cfg.shared_expert_gate:
                    yield p + "mlp.shared_expert_gate.weight", layer.shared_expert_gate_weight.data
        else:
            I = cfg.intermediate_size
            gu = layer.gate_up_proj_weight.data
            yield p + "mlp.gate_proj.weight", gu[:I]
            yield p + "mlp.up_proj.weight", gu[I:]
            yield p + "mlp.down_proj.weight", layer.down_proj_weight.data
    yield "model.norm.weight", model.norm.data
    if getattr(model, "lm_head", None) is not None:
        yield "lm_head.weight", model.lm_head.data
    if cfg.value_head:
        yield "score.weight", model.value_head.data


# ---- family-specific names ----------------------------------------------------------------------------------------
def _llm_names(cfg: DecoderConfig) -> Tuple[str, str]:
    """(prefix replacing ``model.``, name of the vocabulary head) of the language model inside a checkpoint."""
    if cfg.prismatic is not None or cfg.moonvit is not None:
        return "language_model.model.", "language_model.lm_head.weight"
    if cfg.vit is not None and cfg.hf_naming == "internvl_chat":
        return "language_model.model.", ("language_model.output.weight" if cfg.llm_type == "internlm2"
                                         else "language_model.lm_head.weight")
    if cfg.vit is not None or cfg.vision is not None:
        return "model.language_model.", "lm_head.weight"
    return "model.", "lm_head.weight"


_INTERNLM2 = {"self_attn.o_proj": "attention.wo", "mlp.gate_proj": "feed_forward.w1", "mlp.up_proj": "feed_forward.w3",
              "mlp.down_proj": "feed_forward.w2", "input_layernorm": "attention_norm",
              "post_attention_layernorm": "ffn_norm", "embed_tokens": "tok_embeddings"}


def _fuse_wqkv(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cfg: DecoderConfig) -> torch.Tensor:
    """InternLM2's ``wqkv``: per KV head, its group of query heads, then the key head, then the value head."""
    hkv, g, d = cfg.num_kv_heads, cfg.num_heads // cfg.num_kv_heads, cfg.head_dim
    tail = q.shape[1:]
    return torch.cat([q.reshape(hkv, g, d, *tail), k.reshape(hkv, 1, d, *tail), v.reshape(hkv, 1, d, *tail)],
                     1).reshape((g + 2) * hkv * d, *tail)


def _split_wqkv(w: torch.Tensor, cfg: DecoderConfig) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    hkv, g, d = cfg.num_kv_heads, cfg.num_heads // cfg.num_kv_heads, cfg.head_dim
    tail = w.shape[1:]
    w = w.reshape(hkv, g + 2, d, *tail)
    return (w[:, :g].reshape(hkv * g * d, *tail), w[:, g].reshape(hkv * d, *tail), w[:, g + 1].reshape(hkv * d, *tail))


def _vit_state(vision, names: str) -> Iterator[Tuple[str, torch.Tensor]]:
    """InternVL tower + projector; ``names``: "hf" (transformers' classes) or "internvl_chat" (upstream layout)."""
    enc, proj = vision.encoder, vision.projector
    vc = enc.cfg
    H, P = vc.hidden_size, vc.patch_size
    conv = enc.patch_embed_weight.data[:, :enc.patch_dim].unflatten(1, (vc.in_channels, P, P))      # a view
    hf = names == "hf"
    e = "model.vision_tower.embeddings." if hf else "vision_model.embeddings."
    yield e + ("cls_token" if hf else "class_embedding"), enc.prefix_tokens.data[:1].reshape(1, 1, H)
    yield e + ("position_embeddings" if hf else "position_embedding"), enc.position_embedding.data[None]
    yield e + ("patch_embeddings.projection.weight" if hf else "patch_embedding.weight"), conv
    yield e + ("patch_embeddings.projection.bias" if hf else "patch_embedding.bias"), enc.patch_embed_bias.data
    for i, b in enumerate(enc.blocks):
        p = f"model.vision_tower.encoder.layer.{i}." if hf else f"vision_model.encoder.layers.{i}."
        if hf:
            for j, x in enumerate("qkv"):
                yield p + f"attention.{x}_proj.weight", b.qkv_weight.data[j * H:(j + 1) * H]
                if b.qkv_bias is not None:
                    yield p + f"attention.{x}_proj.bias", b.qkv_bias.data[j * H:(j + 1) * H]
        else:
            yield p + "attn.qkv.weight", b.qkv_weight.data
            if b.qkv_bias is not None:
                yield p + "attn.qkv.bias", b.qkv_bias.data
        a = "attention.projection_layer." if hf else "attn.proj."
        yield p + a + "weight", b.proj_weight.data
        yield p + a + "bias", b.proj_bias.data
        for fc in ("fc1", "fc2"):
            yield p + f"mlp.{fc}.weight", getattr(b, fc + "_weight").data
            yield p + f"mlp.{fc}.bias", getattr(b, fc + "_bias").data
        for ours, theirs in (("norm1", "layernorm_before" if hf else "norm1"), ("norm2", "layernorm_after" if hf else "norm2")):
            yield p + theirs + ".weight", getattr(b, ours + "_weight").data
            if getattr(b, ours + "_bias") is not None:
                yield p + theirs + ".bias", getattr(b, ours + "_bias").data
        if vc.layer_scale:
            yield p + ("lambda_1" if hf else "ls1"), b.ls1.data
            yield p + ("lambda_2" if hf else "ls2"), b.ls2.data
    m = ["model.multi_modal_projector.layer_norm.", "model.multi_modal_projector.linear_1.",
         "model.multi_modal_projector.linear_2."] if hf else ["mlp1.0.", "mlp1.1.", "mlp1.3."]
    yield m[0] + "weight", proj.norm_weight.data
    yield m[0] + "bias", proj.norm_bias.data
    yield m[1] + "weight", proj.fc0_weight.data
    yield m[1] + "bias", proj.fc0_bias.data
    yield m[2] + "weight", proj.fc1_weight.data
    yield m[2] + "bias", proj.fc1_bias.data


def _timm_vit_state(enc, prefix: str) -> Iterator[Tuple[str, torch.Tensor]]:
    """A :class:`ViTEncoder` under timm's ``VisionTransformer`` names (LayerScale as ``lsN.scale_factor``, the name
    OpenVLA checkpoints carry after the reference's patch, siirl/models/embodied/openvla_oft/modeling_prismatic.py:56-64)."""
    vc = enc.cfg
    P = vc.patch_size
    if vc.class_token:
        yield prefix + "cls_token", enc.prefix_tokens.data[:1][None]
    if vc.num_register_tokens:
        yield prefix + "reg_token", enc.prefix_tokens.data[(1 if vc.class_token else 0):][None]
    yield prefix + "pos_embed", enc.position_embedding.data[None]
    yield prefix + "patch_embed.proj.weight", enc.patch_embed_weight.data[:, :enc.patch_dim].unflatten(
        1, (vc.in_channels, P, P))
    yield prefix + "patch_embed.proj.bias", enc.patch_embed_bias.data
    for i, b in enumerate(enc.blocks):
        p = prefix + f"blocks.{i}."
        for ours, theirs in (("norm1", "norm1"), ("qkv", "attn.qkv"), ("proj", "attn.proj"), ("norm2", "norm2"),
                             ("fc1", "mlp.fc1"), ("fc2", "mlp.fc2")):
            yield p + theirs + ".weight", getattr(b, ours + "_weight").data
            if getattr(b, ours + "_bias", None) is not None:
                yield p + theirs + ".bias", getattr(b, ours + "_bias").data
        if vc.layer_scale:
            yield p + "ls1.scale_factor", b.ls1.data
            yield p + "ls2.scale_factor", b.ls2.data
    if vc.final_norm:
        yield prefix + "norm.weight", enc.norm_weight.data
        if enc.norm_bias is not None:
            yield prefix + "norm.bias", enc.norm_bias.data


def _prismatic_state(vision) -> Iterator[Tuple[str, torch.Tensor]]:
    yield from _timm_vit_state(vision.featurizer, "vision_backbone.featurizer.")
    if vision.fused_featurizer is not None:
        yield from _timm_vit_state(vision.fused_featurizer, "vision_backbone.fused_featurizer.")
    for i in range(vision.projector.n):
        yield f"projector.fc{i + 1}.weight", getattr(vision.projector, f"fc{i}_weight").data
        yield f"projector.fc{i + 1}.bias", getattr(vision.projector, f"fc{i}_bias").data


class _RowPermuted:
    """A parameter held with permuted rows: ``memory[i] = checkpoint[perm[i]]``."""

    def __init__(self, dst: torch.Tensor, perm: torch.Tensor):
        self.dst, self.perm = dst, perm

    def load(self, src: torch.Tensor) -> None:
        self.dst.copy_(src.to(self.dst.dtype)[self.perm.to(src.device)])

    def export(self) -> torch.Tensor:
        return self.dst[torch.argsort(self.perm).to(self.dst.device)]


def _moonvit_state(vision) -> Iterator[Tuple[str, object]]:
    """Kimi-VL's tower and projector under the checkpoint's names; ``wqkv`` rows leave the in-memory rotary layout
    (siirl_b200/models/moonvit.py) for the checkpoint's interleaved one."""
    from .moonvit import qk_row_permutation
    vc = vision.cfg
    P = vc.patch_size
    perm = qk_row_permutation(vc)
    yield "vision_tower.patch_embed.proj.weight", vision.patch_embed_weight.data[:, :vision.patch_dim].unflatten(
        1, (vc.in_channels, P, P))
    yield "vision_tower.patch_embed.proj.bias", vision.patch_embed_bias.data
    yield "vision_tower.patch_embed.pos_emb.weight", vision.pos_emb.data
    for i, b in enumerate(vision.blocks):
        p = f"vision_tower.encoder.blocks.{i}."
        for ours, theirs in (("norm0", "norm0"), ("norm1", "norm1"), ("wo", "wo"), ("fc0", "mlp.fc0"), ("fc1", "mlp.fc1")):
            yield p + theirs + ".weight", getattr(b, ours + "_weight").data
            yield p + theirs + ".bias", getattr(b, ours + "_bias").data
        yield p + "wqkv.weight", _RowPermuted(b.wqkv_weight.data, perm)
        yield p + "wqkv.bias", _RowPermuted(b.wqkv_bias.data, perm)
    yield "vision_tower.encoder.final_layernorm.weight", vision.final_norm_weight.data
    yield "vision_tower.encoder.final_layernorm.bias", vision.final_norm_bias.data
    for ours, theirs in (("pre_norm", "pre_norm"), ("linear_1", "linear_1"), ("linear_2", "linear_2")):
        yield f"multi_modal_projector.{theirs}.weight", getattr(vision, ours + "_weight").data
        yield f"multi_modal_projector.{theirs}.bias", getattr(vision, ours + "_bias").data


def _qwen_visual_state(vision, prefix: str = "model.visual.") -> Iterator[Tuple[str, torch.Tensor]]:
    """Qwen2.5-VL tower under transformers' names (``visual.patch_embed.proj``: a 3-D convolution weight)."""
    vc = vision.cfg
    H, I = vc.hidden_size, vc.intermediate_size
    yield prefix + "patch_embed.proj.weight", vision.patch_embed_weight.data[:, :vision.patch_dim].unflatten(
        1, (vc.in_channels, vc.temporal_patch_size, vc.patch_size, vc.patch_size))
    for i, b in enumerate(vision.blocks):
        p = prefix + f"blocks.{i}."
        yield p + "norm1.weight", b.norm1.data
        yield p + "norm2.weight", b.norm2.data
        yield p + "attn.qkv.weight", b.qkv_weight.data
        yield p + "attn.qkv.bias", b.qkv_bias.data
        yield p + "attn.proj.weight", b.proj_weight.data
        yield p + "attn.proj.bias", b.proj_bias.data
        Ip = b.padded_intermediate                      # rows / columns beyond I are the zero padding of the MLP width
        yield p + "mlp.gate_proj.weight", b.gate_up_weight.data[:I]
        yield p + "mlp.gate_proj.bias", b.gate_up_bias.data[:I]
        yield p + "mlp.up_proj.weight", b.gate_up_weight.data[Ip:Ip + I]
        yield p + "mlp.up_proj.bias", b.gate_up_bias.data[Ip:Ip + I]
        yield p + "mlp.down_proj.weight", b.down_weight.data[:, :I]
        yield p + "mlp.down_proj.bias", b.down_bias.data
    yield prefix + "merger.ln_q.weight", vision.merger_norm.data
    yield prefix + "merger.mlp.0.weight", vision.merger_fc1_weight.data
    yield prefix + "merger.mlp.0.bias", vision.merger_fc1_bias.data
    yield prefix + "merger.mlp.2.weight", vision.merger_fc2_weight.data
    yield prefix + "merger.mlp.2.bias", vision.merger_fc2_bias.data


def _hf_targets(model) -> Iterator[Tuple[str, object]]:
    """(checkpoint name, view into the model's parameter) for every tensor of the family's HF checkpoint; InternLM2's
    fused ``wqkv`` comes as the tuple of its three views."""
    cfg: DecoderConfig = model.cfg
    prefix, head = _llm_names(cfg)
    internlm2 = cfg.vit is not None and cfg.hf_naming == "internvl_chat" and cfg.llm_type == "internlm2"
    held: Dict[str, torch.Tensor] = {}
    for name, t in _decoder_state(model):
        if name == "lm_head.weight":
            yield head, t
            continue
        if name.startswith("model."):
            name = prefix + name[len("model."):]
        if internlm2:
            if ".self_attn." in name and name.split(".")[-2] in ("q_proj", "k_proj", "v_proj"):
                held[name.split(".")[-2][0]] = t
                if len(held) == 3:
                    yield name[: name.index("self_attn.")] + "attention.wqkv." + name.split(".")[-1], (
                        held["q"], held["k"], held["v"])
                    held = {}
                continue
            for ours, theirs in _INTERNLM2.items():
                name = name.replace(ours, theirs)
        yield name, t
    vision = getattr(model, "vision", None)
    if vision is not None and cfg.moonvit is not None:
        yield from _moonvit_state(vision)
    elif vision is not None and cfg.prismatic is not None:
        yield from _prismatic_state(vision)
    elif vision is not None and cfg.vit is not None:
        yield from _vit_state(vision, cfg.hf_naming)
    elif vision is not None:
        yield from _qwen_visual_state(vision)


def to_hf_state(model) -> Iterator[Tuple[str, torch.Tensor]]:
    """Every parameter under the names of the family's HF checkpoint (language model, then the vision tower)."""
    for name, t in _hf_targets(model):
        if isinstance(t, tuple):
            t = _fuse_wqkv(*t, model.cfg)
        elif isinstance(t, _RowPermuted):
            t = t.export()
        yield name, t


def save_hf_model(model, out_dir: str, max_shard_bytes: int = 4 << 30, tokenizer=None, tensors=None) -> None:
    """Write ``config.json`` + sharded ``model-xxxxx-of-yyyyy.safetensors`` + index.  ``tensors``: a snapshot of
    ``to_hf_state(model)`` taken earlier (asynchronous saves export the weights as they were at the snapshot)."""
    from safetensors.torch import save_file
    os.makedirs(out_dir, exist_ok=True)
    shards, cur, cur_bytes = [], {}, 0
    for name, t in (tensors if tensors is not None else to_hf_state(model)):
        t = t.detach().to("cpu").contiguous().clone()
        nbytes = t.numel() * t.element_size()
        if cur and cur_bytes + nbytes > max_shard_bytes:
            shards.append(cur)
            cur, cur_bytes = {}, 0
        cur[name] = t
        cur_bytes += nbytes
    if cur:
        shards.append(cur)
    weight_map: Dict[str, str] = {}
    total = 0
    for i, sh in enumerate(shards):
        fn = "model.safetensors" if len(shards) == 1 else f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file(sh, os.path.join(out_dir, fn), metadata={"format": "pt"})
        for k, v in sh.items():
            weight_map[k] = fn
            total += v.numel() * v.element_size()
    if len(shards) > 1:
        with open(os.path.join(out_dir, "model.safetensors.index.json"), "w") as f:
            json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=1)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(model.cfg.to_hf_config(), f, indent=1)
    with open(os.path.join(out_dir, "generation_config.json"), "w") as f:
        json.dump({"eos_token_id": model.cfg.eos_token_id, "pad_token_id": model.cfg.pad_token_id}, f)
    if tokenizer is not None and hasattr(tokenizer, "save_pretrained"):
        tokenizer.save_pretrained(out_dir)


def _open_all(path: str):
    from safetensors import safe_open
    path = os.path.expanduser(path)
    idx = os.path.join(path, "model.safetensors.index.json")
    if os.path.exists(idx):
        with open(idx) as f:
            files = sorted(set(json.load(f)["weight_map"].values()))
    else:
        files = sorted(f for f in os.listdir(path) if f.endswith(".safetensors"))
    return [safe_open(os.path.join(path, f), framework="pt", device="cpu") for f in files]


_ALIASES = (("model.language_model.", "model."), ("model.language_model.", "language_model.model."),
            ("model.visual.", "visual."), ("model.vision_tower.", "vision_tower."),
            ("model.multi_modal_projector.", "multi_modal_projector."), ("model.", "model.language_model."))


def load_hf_weights(model, path: str, strict: bool = True) -> None:
    """Fill a :class:`DecoderLM` (language model and vision tower) from an HF safetensors directory; every rank reads
    the files it needs itself -- no rank-0 broadcast as in siirl/utils/model_utils/fsdp_utils.py:437-513.  Names are
    those ``to_hf_state`` writes; checkpoints written by older transformers releases (``model.layers`` beside
    ``visual``) resolve through aliases.  A missing vocabulary head falls back to the embedding (tied checkpoints)."""
    handles = _open_all(path)
    where = {k: h for h in handles for k in h.keys()}
    cfg: DecoderConfig = model.cfg
    head = _llm_names(cfg)[1]

    def get(name: str):
        if name in where:
            return where[name].get_tensor(name)
        if name.endswith(".scale_factor") and name[: -len("scale_factor")] + "gamma" in where:
            alt = name[: -len("scale_factor")] + "gamma"             # timm's own name of the LayerScale vector
            return where[alt].get_tensor(alt)
        for a, b in _ALIASES:
            if name.startswith(a) and (b + name[len(a):]) in where:
                alt = b + name[len(a):]
                return where[alt].get_tensor(alt)
        return None

    embed = None
    with torch.no_grad():
        for name, dst in _hf_targets(model):
            src = get(name)
            if src is None and name == head and embed is not None:
                src = embed
            if src is None and name == "score.weight":
                continue                                  # a value head initialised from a causal-LM checkpoint
            if src is None:
                if strict:
                    raise KeyError(f"{name} missing in {path}")
                continue
            if name.endswith("embed_tokens.weight") or name.endswith("tok_embeddings.weight"):
                embed = src
            if isinstance(dst, _RowPermuted):
                dst.load(src)
            elif isinstance(dst, tuple):
                for d, part in zip(dst, _split_wqkv(src, cfg)):
                    d.copy_(part.to(d.dtype))
            else:
                dst.copy_(src.reshape(dst.shape).to(dst.dtype))
