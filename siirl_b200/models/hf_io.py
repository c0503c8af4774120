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


def to_hf_state(model) -> Iterator[Tuple[str, torch.Tensor]]:
    cfg: DecoderConfig = model.cfg
    qw, kw = cfg.q_width, cfg.kv_width
    yield "model.embed_tokens.weight", model.embed_tokens.data
    for i, layer in enumerate(model.layers):
        p = f"model.layers.{i}."
        yield p + "input_layernorm.weight", layer.input_layernorm.data
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
        if cfg.is_moe:
            I = cfg.moe_intermediate_size
            names = _moe_names(cfg)
            yield p + names["router"], layer.router_weight.data
            for e in range(cfg.num_experts):
                gu = layer.experts_gate_up.data[e]
                yield p + names["expert"].format(e=e, w=names["gate"]), gu[:I]
                yield p + names["expert"].format(e=e, w=names["up"]), gu[I:]
                yield p + names["expert"].format(e=e, w=names["down"]), layer.experts_down.data[e]
            if cfg.shared_expert_intermediate_size > 0:
                Is = cfg.shared_expert_intermediate_size
                sgu = layer.shared_gate_up_weight.data
                yield p + "mlp.shared_expert.gate_proj.weight", sgu[:Is]
                yield p + "mlp.shared_expert.up_proj.weight", sgu[Is:]
                yield p + "mlp.shared_expert.down_proj.weight", layer.shared_down_weight.data
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


def load_hf_weights(model, path: str, strict: bool = True) -> None:
    """Fill a :class:`DecoderLM` from an HF safetensors directory (every rank reads the files it needs itself —
    no rank-0 broadcast as in siirl/utils/model_utils/fsdp_utils.py:437-513)."""
    handles = _open_all(path)
    where = {k: h for h in handles for k in h.keys()}

    def get(name: str):
        if name not in where:
            if strict:
                raise KeyError(f"{name} missing in {path}")
            return None
        return where[name].get_tensor(name)

    cfg: DecoderConfig = model.cfg

    def put(dst: torch.Tensor, src):
        if src is not None:
            dst.copy_(src.to(dst.dtype))

    with torch.no_grad():
        put(model.embed_tokens.data, get("model.embed_tokens.weight"))
        for i, layer in enumerate(model.layers):
            p = f"model.layers.{i}."
            put(layer.input_layernorm.data, get(p + "input_layernorm.weight"))
            put(layer.qkv_proj_weight.data, torch.cat([get(p + f"self_attn.{x}_proj.weight") for x in "qkv"], 0))
            if layer.qkv_proj_bias is not None:
                put(layer.qkv_proj_bias.data, torch.cat([get(p + f"self_attn.{x}_proj.bias") for x in "qkv"], 0))
            if cfg.qk_norm:
                put(layer.q_norm.data, get(p + "self_attn.q_norm.weight"))
                put(layer.k_norm.data, get(p + "self_attn.k_norm.weight"))
            put(layer.o_proj_weight.data, get(p + "self_attn.o_proj.weight"))
            put(layer.post_attention_layernorm.data, get(p + "post_attention_layernorm.weight"))
            if cfg.is_moe:
                names = _moe_names(cfg)
                put(layer.router_weight.data, get(p + names["router"]))
                for e in range(cfg.num_experts):
                    put(layer.experts_gate_up.data[e],
                        torch.cat([get(p + names["expert"].format(e=e, w=names["gate"])),
                                   get(p + names["expert"].format(e=e, w=names["up"]))], 0))
                    put(layer.experts_down.data[e], get(p + names["expert"].format(e=e, w=names["down"])))
                if cfg.shared_expert_intermediate_size > 0:
                    put(layer.shared_gate_up_weight.data, torch.cat([get(p + "mlp.shared_expert.gate_proj.weight"),
                                                                     get(p + "mlp.shared_expert.up_proj.weight")], 0))
                    put(layer.shared_down_weight.data, get(p + "mlp.shared_expert.down_proj.weight"))
                    if cfg.shared_expert_gate:
                        put(layer.shared_expert_gate_weight.data, get(p + "mlp.shared_expert_gate.weight"))
            else:
                put(layer.gate_up_proj_weight.data, torch.cat([get(p + "mlp.gate_proj.weight"),
                                                               get(p + "mlp.up_proj.weight")], 0))
                put(layer.down_proj_weight.data, get(p + "mlp.down_proj.weight"))
        put(model.norm.data, get("model.norm.weight"))
        if getattr(model, "lm_head", None) is not None:
            src = where.get("lm_head.weight")
            put(model.lm_head.data, get("lm_head.weight") if src is not None else get("model.embed_tokens.weight"))
        if cfg.value_head and "score.weight" in where:
            put(model.value_head.data, get("score.weight"))
