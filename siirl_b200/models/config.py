"""Architecture description of the decoder families this framework trains and serves.

The reference takes architectures from HF ``config.json`` through transformers / Megatron converters
(siirl/models/loader.py, siirl/models/mcore/config_converter.py:26-284: dense Llama/Qwen2, Qwen2-MoE, Mixtral,
Qwen3-MoE, Qwen2.5-VL).  Here one dataclass covers them; ``from_hf_config`` reads the same ``config.json`` and
``PRESETS`` holds the shapes used by the benchmark configurations (random-init, no checkpoint needed).
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field
from typing import Any, Dict, List, Optional


@dataclass
class VisionConfig:
    depth: int = 32
    hidden_size: int = 1280
    num_heads: int = 16
    intermediate_size: int = 3420
    patch_size: int = 14
    temporal_patch_size: int = 2
    in_channels: int = 3
    spatial_merge_size: int = 2
    window_size: int = 112
    fullatt_block_indexes: List[int] = field(default_factory=lambda: [7, 15, 23, 31])
    out_hidden_size: int = 3584


@dataclass
class ViTConfig:
    image_size: int = 448
    patch_size: int = 14
    hidden_size: int = 1024
    num_heads: int = 16
    intermediate_size: int = 4096
    depth: int = 24
    in_channels: int = 3
    class_token: bool = True
    num_register_tokens: int = 0        # DINOv2 "reg4" models
    layer_scale: bool = True            # learnable per-channel scale on both residual branches
    norm_type: str = "layer_norm"       # or "rms_norm" (InternViT-6B)
    qkv_bias: bool = True
    norm_eps: float = 1e-6
    final_norm: bool = False            # timm ViTs end in a LayerNorm; InternVL reads the raw last layer
    select_layer: int = -1              # hidden state handed on: -1 last layer, -2 the one before (Prismatic)
    class_pos_embed: bool = True        # False: positions for the patches only (timm ``no_embed_class``, DINOv2)
    act: str = "gelu"                   # or "gelu_tanh"

    @property
    def num_patches(self) -> int:
        return (self.image_size // self.patch_size) ** 2

    @property
    def num_prefix_tokens(self) -> int:
        return (1 if self.class_token else 0) + self.num_register_tokens


@dataclass
class MoonViTConfig:
    """Kimi-VL's native-resolution vision tower: learnable 2-D position table interpolated to each image's grid,
    rotary positions over (x, y), LayerNorm / GELU blocks, 2 x 2 patch merge into the projector."""
    patch_size: int = 14
    init_pos_emb_height: int = 64
    init_pos_emb_width: int = 64
    hidden_size: int = 1152
    num_heads: int = 16
    intermediate_size: int = 4304
    depth: int = 27
    merge: int = 2
    in_channels: int = 3


@dataclass
class PrismaticConfig:
    """OpenVLA's vision side: a DINOv2 ViT and (fused backbone) a SigLIP ViT over the same image, patch features
    concatenated along the channel axis, then a GELU MLP into the language model width."""
    featurizer: ViTConfig = field(default_factory=lambda: ViTConfig(
        image_size=224, patch_size=14, hidden_size=1024, num_heads=16, intermediate_size=4096, depth=24,
        class_token=True, num_register_tokens=4, layer_scale=True, final_norm=True, select_layer=-2,
        class_pos_embed=False))
    fused_featurizer: Optional[ViTConfig] = field(default_factory=lambda: ViTConfig(
        image_size=224, patch_size=14, hidden_size=1152, num_heads=16, intermediate_size=4304, depth=27,
        class_token=False, layer_scale=False, final_norm=True, select_layer=-2))
    num_images_in_input: int = 1
    timm_model_ids: List[str] = field(default_factory=lambda: ["vit_large_patch14_reg4_dinov2.lvd142m",
                                                                "vit_so400m_patch14_siglip_224"])

    @property
    def vision_dim(self) -> int:
        return self.featurizer.hidden_size + (self.fused_featurizer.hidden_size if self.fused_featurizer else 0)

    @property
    def tokens_per_image(self) -> int:
        return self.featurizer.num_patches


@dataclass
class DecoderConfig:
    model_type: str = "qwen2"
    vocab_size: int = 1024
    hidden_size: int = 128
    intermediate_size: int = 352
    num_layers: int = 2
    num_heads: int = 4
    num_kv_heads: int = 2
    head_dim: int = 32
    rope_theta: float = 1e4
    rms_norm_eps: float = 1e-6
    max_position_embeddings: int = 32768
    qkv_bias: bool = True           # Qwen2 family
    qk_norm: bool = False           # Qwen3 family
    tie_word_embeddings: bool = False
    mrope_section: Optional[List[int]] = None   # Qwen2-VL multimodal rope (t, h, w halves)
    # checkpoint's rope_scaling of type linear / llama3 / yarn (None: plain rotary frequencies)
    rope_scaling: Optional[Dict[str, Any]] = None
    # mixture of experts (0 experts = dense)
    num_experts: int = 0
    num_experts_per_tok: int = 0
    # expert parallelism (runtime layout, not part of the HF config): this rank hosts experts
    # [ep_rank * num_experts / ep_size, (ep_rank + 1) * num_experts / ep_size)
    ep_size: int = 1
    ep_rank: int = 0
    # LoRA adapters on the four projections of every layer (0: none); runtime option, not part of the HF config
    lora_rank: int = 0
    lora_alpha: float = 16.0
    # fused projections that carry an adapter: subset of ("qkv_proj", "o_proj", "gate_up_proj", "down_proj")
    lora_targets: Optional[tuple] = None
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    # shared expert (Qwen2-MoE, DeepSeek-style): a dense SwiGLU MLP every token passes through, added to the routed
    # experts' output; ``shared_expert_gate`` multiplies it by sigmoid(x . g) (Qwen2-MoE)
    shared_expert_intermediate_size: int = 0
    shared_expert_gate: bool = False
    # multi-head latent attention (DeepSeek-V2/V3, Kimi-VL's language model): keys and values are expanded from a
    # ``kv_lora_rank``-wide latent; each head has ``qk_nope_head_dim`` position-free and ``qk_rope_head_dim`` rotary
    # query/key dimensions (the rotary key is shared by all heads) and ``v_head_dim`` value dimensions
    kv_lora_rank: int = 0
    q_lora_rank: int = 0
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0
    v_head_dim: int = 0
    rope_interleave: bool = True
    # DeepSeek-V3 routing: sigmoid scores, a per-expert selection bias, group-limited top-k, scaled weights; the first
    # ``first_k_dense_replace`` layers keep a dense MLP
    scoring_func: str = "softmax"
    topk_method: str = "greedy"
    n_group: int = 1
    topk_group: int = 1
    routed_scaling_factor: float = 1.0
    first_k_dense_replace: int = 0
    # value head (critic / reward model): one scalar per token instead of the vocabulary head
    value_head: bool = False
    vision: Optional[VisionConfig] = None
    # InternVL family: a plain ViT tower whose 2x2 pixel-shuffled patches pass an MLP projector; ``hf_naming`` picks
    # the checkpoint's parameter names ("hf": transformers' own classes, "internvl_chat": the upstream remote-code
    # layout with ``vision_model / mlp1 / language_model``, whose language model may be InternLM2 with fused ``wqkv``)
    vit: Optional[ViTConfig] = None
    downsample_ratio: float = 0.5
    hf_naming: str = "hf"
    llm_type: str = ""
    # OpenVLA / OpenVLA-OFT: Prismatic vision backbone; actions are the last ``n_action_bins`` ids below
    # ``action_vocab_size`` (the tokenizer's size: the embedding matrix is padded beyond it)
    prismatic: Optional[PrismaticConfig] = None
    moonvit: Optional[MoonViTConfig] = None
    action_vocab_size: int = 0
    n_action_bins: int = 256
    image_token_id: int = 151655
    eos_token_id: int = 2
    pad_token_id: int = 0
    bos_token_id: Optional[int] = None
    initializer_range: float = 0.02

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def is_mla(self) -> bool:
        return self.kv_lora_rank > 0

    @property
    def rope_dim(self) -> int:
        """Width the rotary embedding acts on."""
        return self.qk_rope_head_dim if self.is_mla else self.head_dim

    def layer_is_moe(self, layer_idx: int) -> bool:
        return self.is_moe and layer_idx >= self.first_k_dense_replace

    @property
    def q_width(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.num_kv_heads * self.head_dim

    @property
    def qkv_width(self) -> int:
        return self.q_width + 2 * self.kv_width

    def num_parameters(self) -> int:
        H, I, V = self.hidden_size, self.intermediate_size, self.vocab_size
        attn = H * self.qkv_width + (self.qkv_width if self.qkv_bias else 0) + self.q_width * H
        if self.qk_norm:
            attn += 2 * self.head_dim
        if self.is_moe:
            mlp = self.num_experts * 3 * H * self.moe_intermediate_size + self.num_experts * H
            mlp += 3 * H * self.shared_expert_intermediate_size + (H if self.shared_expert_gate else 0)
        else:
            mlp = 3 * H * I
        per_layer = attn + mlp + 2 * H
        head = 0 if self.tie_word_embeddings else (H if self.value_head else V * H)
        return V * H + self.num_layers * per_layer + H + head

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "DecoderConfig":
        """Inverse of ``to_dict`` (checkpoint manifests keep the model configuration in that form); unknown keys of
        a newer version are dropped."""
        import dataclasses

        def build(kind, val):
            if val is None or not isinstance(val, dict):
                return val
            names = {f.name for f in dataclasses.fields(kind)}
            return kind(**{k: v for k, v in val.items() if k in names})
        d = dict(d)
        for key, kind in (("vision", VisionConfig), ("vit", ViTConfig), ("moonvit", MoonViTConfig)):
            d[key] = build(kind, d.get(key))
        pr = d.get("prismatic")
        if isinstance(pr, dict):
            pr = dict(pr)
            pr["featurizer"] = build(ViTConfig, pr.get("featurizer"))
            pr["fused_featurizer"] = build(ViTConfig, pr.get("fused_featurizer"))
            d["prismatic"] = build(PrismaticConfig, pr)
        for key in ("lora_targets", "mrope_section"):
            if isinstance(d.get(key), list) and key == "lora_targets":
                d[key] = tuple(d[key])
        names = {f.name for f in dataclasses.fields(cls)}
        return cls(**{k: v for k, v in d.items() if k in names})

    # ---- HF interchange -----------------------------------------------------------------------
    @classmethod
    def from_hf_config(cls, cfg: Dict[str, Any]) -> "DecoderConfig":
        text = cfg.get("text_config") or cfg.get("llm_config") or cfg
        mt = cfg.get("model_type", "qwen2")
        if mt in ("llama4", "llama4_text"):
            # same answer as the reference's converter, which lists Llama4ForConditionalGeneration and raises
            # (siirl/models/mcore/config_converter.py:282-284): chunked attention, rope-free layers and the
            # interleaved dense / MoE stack of that family are not built
            raise NotImplementedError("Llama4ForConditionalGeneration is not supported")
        if mt in ("internvl", "internvl_chat"):
            return cls._from_internvl_config(cfg)
        if mt in ("openvla", "prismatic"):
            return cls._from_openvla_config(cfg)
        if mt == "kimi_vl":
            out = cls.from_hf_config(dict(cfg["text_config"], model_type="deepseek_v3"))
            out.model_type = "kimi_vl"
            out.image_token_id = int(cfg.get("media_placeholder_token_id", 163605))
            vc = cfg.get("vision_config", {})
            mk = vc.get("merge_kernel_size", [2, 2])
            out.moonvit = MoonViTConfig(
                patch_size=vc.get("patch_size", 14), init_pos_emb_height=vc.get("init_pos_emb_height", 64),
                init_pos_emb_width=vc.get("init_pos_emb_width", 64), hidden_size=vc.get("hidden_size", 1152),
                num_heads=vc.get("num_attention_heads", 16), intermediate_size=vc.get("intermediate_size", 4304),
                depth=vc.get("num_hidden_layers", 27), merge=int(mk[0] if isinstance(mk, (list, tuple)) else mk))
            return out
        nh = text["num_attention_heads"]
        hd = text.get("head_dim") or text["hidden_size"] // nh
        rope_scaling = text.get("rope_scaling") or cfg.get("rope_scaling") or {}
        out = cls(
            model_type=mt,
            vocab_size=text["vocab_size"],
            hidden_size=text["hidden_size"],
            intermediate_size=text.get("intermediate_size", 0),
            num_layers=text["num_hidden_layers"],
            num_heads=nh,
            num_kv_heads=text.get("num_key_value_heads", nh),
            head_dim=hd,
            rope_theta=float(text.get("rope_theta", 1e4)),
            rms_norm_eps=float(text.get("rms_norm_eps", 1e-6)),
            max_position_embeddings=text.get("max_position_embeddings", 32768),
            qkv_bias=mt.startswith("qwen2") or bool(text.get("attention_bias", False)),
            qk_norm=mt.startswith("qwen3"),
            tie_word_embeddings=bool(cfg.get("tie_word_embeddings", False)),
            mrope_section=rope_scaling.get("mrope_section"),
            rope_scaling=(dict(rope_scaling) if rope_scaling.get("rope_type", rope_scaling.get("type")) in
                          ("linear", "llama3", "yarn") else None),
            num_experts=text.get("num_experts", text.get("num_local_experts", 0)) or 0,
            num_experts_per_tok=text.get("num_experts_per_tok", 0) or 0,
            moe_intermediate_size=text.get("moe_intermediate_size", 0) or 0,
            norm_topk_prob=bool(text.get("norm_topk_prob", True)),
            shared_expert_intermediate_size=text.get("shared_expert_intermediate_size", 0) or 0,
            shared_expert_gate=mt == "qwen2_moe" and bool(text.get("shared_expert_intermediate_size", 0)),
            eos_token_id=(cfg.get("eos_token_id") if isinstance(cfg.get("eos_token_id"), int) else 2) or 2,
            pad_token_id=cfg.get("pad_token_id") or 0,
        )
        if mt in ("deepseek_v3", "deepseek_v2"):
            out.qkv_bias = bool(text.get("attention_bias", False))
            out.kv_lora_rank = int(text.get("kv_lora_rank") or 0)
            out.q_lora_rank = int(text.get("q_lora_rank") or 0)
            out.qk_nope_head_dim = int(text.get("qk_nope_head_dim", 128))
            out.qk_rope_head_dim = int(text.get("qk_rope_head_dim", 64))
            out.v_head_dim = int(text.get("v_head_dim", 128))
            out.rope_interleave = bool(text.get("rope_interleave", True))
            out.head_dim = out.qk_nope_head_dim + out.qk_rope_head_dim
            out.num_experts = int(text.get("n_routed_experts") or 0)
            out.scoring_func = text.get("scoring_func", "sigmoid" if mt == "deepseek_v3" else "softmax")
            out.topk_method = text.get("topk_method", "noaux_tc" if mt == "deepseek_v3" else "greedy")
            out.n_group = int(text.get("n_group") or 1)
            out.topk_group = int(text.get("topk_group") or 1)
            out.routed_scaling_factor = float(text.get("routed_scaling_factor", 1.0))
            out.first_k_dense_replace = int(text.get("first_k_dense_replace", 0))
            out.norm_topk_prob = bool(text.get("norm_topk_prob", True))
            out.shared_expert_intermediate_size = int(text.get("n_shared_experts") or 0) * out.moe_intermediate_size
            out.shared_expert_gate = False
        if mt == "mixtral":
            # Mixtral's experts use the dense intermediate size; its router renormalises the top-k weights
            out.moe_intermediate_size = text.get("intermediate_size", 0)
            out.norm_topk_prob = True
            out.qkv_bias = False
        if mt == "qwen2_moe":
            out.norm_topk_prob = bool(text.get("norm_topk_prob", False))
        if "vision_config" in cfg:
            vc = cfg["vision_config"]
            out.vision = VisionConfig(
                depth=vc.get("depth", 32), hidden_size=vc.get("hidden_size", 1280), num_heads=vc.get("num_heads", 16),
                intermediate_size=vc.get("intermediate_size", 3420), patch_size=vc.get("patch_size", 14),
                temporal_patch_size=vc.get("temporal_patch_size", 2), in_channels=vc.get("in_chans", 3),
                spatial_merge_size=vc.get("spatial_merge_size", 2), window_size=vc.get("window_size", 112),
                fullatt_block_indexes=vc.get("fullatt_block_indexes", [7, 15, 23, 31]),
                out_hidden_size=vc.get("out_hidden_size", text["hidden_size"]))
            out.image_token_id = cfg.get("image_token_id", 151655)
        return out

    @classmethod
    def _from_internvl_config(cls, cfg: Dict[str, Any]) -> "DecoderConfig":
        """``internvl`` (transformers' classes: ``text_config`` + ``vision_config`` with list-valued sizes) and
        ``internvl_chat`` (upstream remote code: ``llm_config`` + ``vision_config``; the language model is InternLM2,
        Qwen2 or Llama)."""
        native = cfg.get("model_type") == "internvl"
        text = dict(cfg.get("text_config") or cfg.get("llm_config") or {})
        llm_type = text.get("model_type", "qwen2")
        base = dict(text)
        base["model_type"] = "qwen2" if llm_type == "qwen2" else "llama"
        if llm_type == "internlm2":
            base["attention_bias"] = bool(text.get("bias", False))
        out = cls.from_hf_config(base)
        out.model_type = "internvl" if native else "internvl_chat"
        out.llm_type = llm_type
        out.hf_naming = "hf" if native else "internvl_chat"
        out.tie_word_embeddings = bool(text.get("tie_word_embeddings", False))
        vc = cfg.get("vision_config", {})

        def one(v, default):
            v = vc.get(v, default)
            return int(v[0]) if isinstance(v, (list, tuple)) else int(v)
        out.vit = ViTConfig(
            image_size=one("image_size", 448), patch_size=one("patch_size", 14), hidden_size=vc.get("hidden_size", 1024),
            num_heads=vc.get("num_attention_heads", 16), intermediate_size=vc.get("intermediate_size", 4096),
            depth=vc.get("num_hidden_layers", 24), class_token=True, layer_scale=True,
            norm_type=vc.get("norm_type", "layer_norm"),
            qkv_bias=bool(vc.get("attention_bias", False) if native else vc.get("qkv_bias", True)),
            norm_eps=float(vc.get("layer_norm_eps", 1e-6)), final_norm=False,
            select_layer=int(cfg.get("vision_feature_layer", cfg.get("select_layer", -1))))
        out.downsample_ratio = float(cfg.get("downsample_ratio", 0.5))
        out.image_token_id = int(cfg.get("image_token_id", cfg.get("img_context_token_id", 151667)))
        return out

    @classmethod
    def _from_openvla_config(cls, cfg: Dict[str, Any]) -> "DecoderConfig":
        """``openvla`` / ``prismatic`` configs (siirl/models/embodied/openvla_oft/configuration_prismatic.py): the
        vision towers are named by their timm ids, the language model is a Llama-2 ``text_config`` whose embedding
        matrix is padded to ``pad_to_multiple_of`` rows."""
        text = dict(cfg.get("text_config") or {})
        text.setdefault("model_type", "llama")
        text.setdefault("vocab_size", 32000)
        for k, v in (("hidden_size", 4096), ("intermediate_size", 11008), ("num_hidden_layers", 32),
                     ("num_attention_heads", 32), ("rms_norm_eps", 1e-6)):
            text.setdefault(k, v)
        mult = int(cfg.get("pad_to_multiple_of", 64))
        tok_vocab = int(text["vocab_size"])
        # a new pad token follows the tokenizer's entries; the matrix is then padded to a multiple of ``mult``
        text["vocab_size"] = (tok_vocab + 1 + mult - 1) // mult * mult if tok_vocab % mult == 0 else tok_vocab
        out = cls.from_hf_config(text)
        out.model_type = "openvla"
        out.llm_type = "llama"
        out.action_vocab_size = tok_vocab if tok_vocab % mult == 0 else int(cfg.get("action_vocab_size", tok_vocab))
        out.n_action_bins = int(cfg.get("n_action_bins", 256))
        out.pad_token_id = int(cfg.get("pad_token_id", 32000))
        out.image_token_id = out.pad_token_id
        out.bos_token_id = int(text.get("bos_token_id", 1))
        ids = list(cfg.get("timm_model_ids") or PrismaticConfig().timm_model_ids)
        sizes = list(cfg.get("image_sizes") or [224, 224])
        towers = [vit_from_timm_id(i, int(s)) for i, s in zip(ids, sizes)]
        if "vit_overrides" in cfg:                   # reduced towers of test checkpoints
            towers = [ViTConfig(**o) for o in cfg["vit_overrides"]]
        fused = bool(cfg.get("use_fused_vision_backbone", len(towers) > 1))
        out.prismatic = PrismaticConfig(featurizer=towers[0], fused_featurizer=towers[1] if fused else None,
                                        num_images_in_input=int(cfg.get("num_images_in_input", 1)), timm_model_ids=ids)
        return out

    @classmethod
    def from_pretrained(cls, path: str) -> "DecoderConfig":
        with open(os.path.join(os.path.expanduser(path), "config.json")) as f:
            return cls.from_hf_config(json.load(f))

    def to_hf_config(self) -> Dict[str, Any]:
        arch = {"qwen2": "Qwen2ForCausalLM", "qwen3": "Qwen3ForCausalLM", "qwen3_moe": "Qwen3MoeForCausalLM",
                "llama": "LlamaForCausalLM", "qwen2_5_vl": "Qwen2_5_VLForConditionalGeneration",
                "mixtral": "MixtralForCausalLM", "qwen2_moe": "Qwen2MoeForCausalLM",
                "deepseek_v3": "DeepseekV3ForCausalLM"}
        d = {
            "architectures": [arch.get(self.model_type, "Qwen2ForCausalLM")], "model_type": self.model_type,
            "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size, "num_hidden_layers": self.num_layers,
            "num_attention_heads": self.num_heads, "num_key_value_heads": self.num_kv_heads,
            "head_dim": self.head_dim, "rope_theta": self.rope_theta, "rms_norm_eps": self.rms_norm_eps,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings, "hidden_act": "silu", "torch_dtype": "bfloat16",
            "eos_token_id": self.eos_token_id, "pad_token_id": self.pad_token_id,
        }
        if self.is_mla:
            d.update(kv_lora_rank=self.kv_lora_rank, q_lora_rank=self.q_lora_rank or None,
                     qk_nope_head_dim=self.qk_nope_head_dim, qk_rope_head_dim=self.qk_rope_head_dim,
                     v_head_dim=self.v_head_dim, rope_interleave=self.rope_interleave, attention_bias=self.qkv_bias,
                     qk_head_dim=self.qk_nope_head_dim + self.qk_rope_head_dim, head_dim=self.qk_rope_head_dim)
        if self.is_moe and self.model_type in ("deepseek_v3", "kimi_vl"):
            d.update(n_routed_experts=self.num_experts, num_experts_per_tok=self.num_experts_per_tok,
                     moe_intermediate_size=self.moe_intermediate_size, norm_topk_prob=self.norm_topk_prob,
                     n_shared_experts=self.shared_expert_intermediate_size // max(self.moe_intermediate_size, 1),
                     n_group=self.n_group, topk_group=self.topk_group, scoring_func=self.scoring_func,
                     topk_method=self.topk_method, routed_scaling_factor=self.routed_scaling_factor,
                     first_k_dense_replace=self.first_k_dense_replace)
        elif self.is_moe and self.model_type == "mixtral":
            d.update(num_local_experts=self.num_experts, num_experts_per_tok=self.num_experts_per_tok,
                     intermediate_size=self.moe_intermediate_size)
        elif self.is_moe:
            d.update(num_experts=self.num_experts, num_experts_per_tok=self.num_experts_per_tok,
                     moe_intermediate_size=self.moe_intermediate_size, norm_topk_prob=self.norm_topk_prob)
            if self.shared_expert_intermediate_size:
                d["shared_expert_intermediate_size"] = self.shared_expert_intermediate_size
        if self.mrope_section:
            d["rope_scaling"] = {"type": "mrope", "mrope_section": self.mrope_section}
        elif self.rope_scaling:
            d["rope_scaling"] = dict(self.rope_scaling)
        if self.moonvit is not None:
            mv = self.moonvit
            text = dict(d, model_type="deepseek_v3")
            text.pop("architectures", None)
            return {"architectures": ["KimiVLForConditionalGeneration"], "model_type": "kimi_vl", "text_config": text,
                    "vision_config": {"model_type": "moonvit", "patch_size": mv.patch_size,
                                      "init_pos_emb_height": mv.init_pos_emb_height,
                                      "init_pos_emb_width": mv.init_pos_emb_width, "hidden_size": mv.hidden_size,
                                      "num_attention_heads": mv.num_heads, "intermediate_size": mv.intermediate_size,
                                      "num_hidden_layers": mv.depth, "merge_kernel_size": [mv.merge, mv.merge]},
                    "media_placeholder_token_id": self.image_token_id, "torch_dtype": "bfloat16"}
        if self.prismatic is not None:
            pc = self.prismatic
            towers = [pc.featurizer] + ([pc.fused_featurizer] if pc.fused_featurizer else [])
            text = dict(d, model_type="llama", vocab_size=self.action_vocab_size or self.vocab_size)
            text.pop("architectures", None)
            return {"architectures": ["OpenVLAForActionPrediction"], "model_type": "openvla", "text_config": text,
                    "timm_model_ids": pc.timm_model_ids[: len(towers)], "image_sizes": [t.image_size for t in towers],
                    "use_fused_vision_backbone": pc.fused_featurizer is not None,
                    "vit_overrides": [asdict(t) for t in towers], "n_action_bins": self.n_action_bins,
                    "pad_to_multiple_of": 64, "pad_token_id": self.pad_token_id,
                    "num_images_in_input": pc.num_images_in_input, "action_vocab_size": self.action_vocab_size,
                    "torch_dtype": "bfloat16"}
        if self.vit is not None:
            v = self.vit
            text = dict(d, model_type=self.llm_type or "qwen2")
            text.pop("architectures", None)
            vision = {"hidden_size": v.hidden_size, "num_hidden_layers": v.depth, "num_attention_heads": v.num_heads,
                      "intermediate_size": v.intermediate_size, "norm_type": v.norm_type, "layer_norm_eps": v.norm_eps}
            if self.hf_naming == "hf":
                vision.update(image_size=[v.image_size] * 2, patch_size=[v.patch_size] * 2, attention_bias=v.qkv_bias,
                              model_type="internvl_vision")
                return {"architectures": ["InternVLForConditionalGeneration"], "model_type": "internvl",
                        "text_config": text, "vision_config": vision, "image_token_id": self.image_token_id,
                        "downsample_ratio": self.downsample_ratio, "vision_feature_layer": v.select_layer,
                        "tie_word_embeddings": self.tie_word_embeddings, "torch_dtype": "bfloat16"}
            vision.update(image_size=v.image_size, patch_size=v.patch_size, qkv_bias=v.qkv_bias)
            if self.llm_type == "internlm2":
                text["bias"] = self.qkv_bias
            return {"architectures": ["InternVLChatModel"], "model_type": "internvl_chat", "llm_config": text,
                    "vision_config": vision, "img_context_token_id": self.image_token_id,
                    "downsample_ratio": self.downsample_ratio, "select_layer": v.select_layer,
                    "torch_dtype": "bfloat16"}
        return d


def vit_from_timm_id(model_id: str, image_size: int = 224) -> ViTConfig:
    """Shapes of the timm vision transformers the Prismatic backbones name (no timm import: the architectures are
    public and fixed)."""
    if "dinov2" in model_id:
        large = "large" in model_id
        return ViTConfig(image_size=image_size, patch_size=14, hidden_size=1024 if large else 768,
                         num_heads=16 if large else 12, intermediate_size=4096 if large else 3072,
                         depth=24 if large else 12, class_token=True, num_register_tokens=4 if "reg4" in model_id else 0,
                         layer_scale=True, final_norm=True, select_layer=-2, class_pos_embed="reg4" not in model_id)
    if "siglip" in model_id:
        so = "so400m" in model_id
        return ViTConfig(image_size=image_size, patch_size=14 if so else 16, hidden_size=1152 if so else 768,
                         num_heads=16 if so else 12, intermediate_size=4304 if so else 3072, depth=27 if so else 12,
                         class_token=False, layer_scale=False, final_norm=True, select_layer=-2)
    raise ValueError(f"unknown vision backbone {model_id}")


PRESETS: Dict[str, DecoderConfig] = {
    # 2-layer gate model used by the CPU/gloo end-to-end test
    "tiny": DecoderConfig(model_type="qwen2", vocab_size=1024, hidden_size=128, intermediate_size=352, num_layers=2,
                          num_heads=4, num_kv_heads=2, head_dim=32, rope_theta=1e4, eos_token_id=2),
    # small GPU smoke model (head_dim 64 path)
    "tiny-gpu": DecoderConfig(model_type="qwen2", vocab_size=4096, hidden_size=512, intermediate_size=1408,
                              num_layers=2, num_heads=8, num_kv_heads=2, head_dim=64, rope_theta=1e6, eos_token_id=2),
    "qwen2.5-0.5b": DecoderConfig(model_type="qwen2", vocab_size=151936, hidden_size=896, intermediate_size=4864,
                                  num_layers=24, num_heads=14, num_kv_heads=2, head_dim=64, rope_theta=1e6,
                                  tie_word_embeddings=True, eos_token_id=151645, pad_token_id=151643),
    "qwen2.5-7b": DecoderConfig(model_type="qwen2", vocab_size=152064, hidden_size=3584, intermediate_size=18944,
                                num_layers=28, num_heads=28, num_kv_heads=4, head_dim=128, rope_theta=1e6,
                                eos_token_id=151645, pad_token_id=151643),
    "qwen3-30b-a3b": DecoderConfig(model_type="qwen3_moe", vocab_size=151936, hidden_size=2048, intermediate_size=6144,
                                   num_layers=48, num_heads=32, num_kv_heads=4, head_dim=128, rope_theta=1e6,
                                   qkv_bias=False, qk_norm=True, num_experts=128, num_experts_per_tok=8,
                                   moe_intermediate_size=768, eos_token_id=151645, pad_token_id=151643),
    "mixtral-8x7b": DecoderConfig(model_type="mixtral", vocab_size=32000, hidden_size=4096, intermediate_size=14336,
                                  num_layers=32, num_heads=32, num_kv_heads=8, head_dim=128, rope_theta=1e6,
                                  qkv_bias=False, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=14336,
                                  rms_norm_eps=1e-5, eos_token_id=2, pad_token_id=0),
    "qwen1.5-moe-a2.7b": DecoderConfig(model_type="qwen2_moe", vocab_size=151936, hidden_size=2048,
                                       intermediate_size=5632, num_layers=24, num_heads=16, num_kv_heads=16,
                                       head_dim=128, rope_theta=1e6, qkv_bias=True, num_experts=60,
                                       num_experts_per_tok=4, moe_intermediate_size=1408, norm_topk_prob=False,
                                       shared_expert_intermediate_size=5632, shared_expert_gate=True,
                                       eos_token_id=151645, pad_token_id=151643),
    "tiny-mixtral": DecoderConfig(model_type="mixtral", vocab_size=1024, hidden_size=128, intermediate_size=64,
                                  num_layers=2, num_heads=4, num_kv_heads=2, head_dim=32, qkv_bias=False,
                                  num_experts=4, num_experts_per_tok=2, moe_intermediate_size=64),
    "tiny-qwen2-moe": DecoderConfig(model_type="qwen2_moe", vocab_size=1024, hidden_size=128, intermediate_size=352,
                                    num_layers=2, num_heads=4, num_kv_heads=2, head_dim=32, num_experts=8,
                                    num_experts_per_tok=2, moe_intermediate_size=64, norm_topk_prob=False,
                                    shared_expert_intermediate_size=96, shared_expert_gate=True),
    # DeepSeek-V3 (671B, 37B active): MLA + 256 routed / 1 shared experts, 3 dense layers
    "deepseek-v3": DecoderConfig(model_type="deepseek_v3", vocab_size=129280, hidden_size=7168, intermediate_size=18432,
                                 num_layers=61, num_heads=128, num_kv_heads=128, head_dim=192, rope_theta=1e4,
                                 qkv_bias=False, kv_lora_rank=512, q_lora_rank=1536, qk_nope_head_dim=128,
                                 qk_rope_head_dim=64, v_head_dim=128, num_experts=256, num_experts_per_tok=8,
                                 moe_intermediate_size=2048, shared_expert_intermediate_size=2048, n_group=8,
                                 topk_group=4, scoring_func="sigmoid", topk_method="noaux_tc",
                                 routed_scaling_factor=2.5, first_k_dense_replace=3, eos_token_id=1, pad_token_id=0),
    # Moonlight-16B-A3B, the language model of Kimi-VL-A3B
    "moonlight-16b-a3b": DecoderConfig(model_type="deepseek_v3", vocab_size=163840, hidden_size=2048,
                                       intermediate_size=11264, num_layers=27, num_heads=16, num_kv_heads=16,
                                       head_dim=192, rope_theta=5e4, qkv_bias=False, kv_lora_rank=512, q_lora_rank=0,
                                       qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, num_experts=64,
                                       num_experts_per_tok=6, moe_intermediate_size=1408,
                                       shared_expert_intermediate_size=2816, n_group=1, topk_group=1,
                                       scoring_func="sigmoid", topk_method="noaux_tc", routed_scaling_factor=2.446,
                                       first_k_dense_replace=1, eos_token_id=163585, pad_token_id=163839),
    # Kimi-VL-A3B: MoonViT-SO-400M + Moonlight-16B-A3B
    "kimi-vl-a3b": DecoderConfig(model_type="kimi_vl", vocab_size=163840, hidden_size=2048, intermediate_size=11264,
                                 num_layers=27, num_heads=16, num_kv_heads=16, head_dim=192, rope_theta=8e5,
                                 qkv_bias=False, kv_lora_rank=512, q_lora_rank=0, qk_nope_head_dim=128,
                                 qk_rope_head_dim=64, v_head_dim=128, num_experts=64, num_experts_per_tok=6,
                                 moe_intermediate_size=1408, shared_expert_intermediate_size=2816, n_group=1,
                                 topk_group=1, scoring_func="sigmoid", topk_method="noaux_tc",
                                 routed_scaling_factor=2.446, first_k_dense_replace=1, moonvit=MoonViTConfig(),
                                 image_token_id=163605, eos_token_id=163585, pad_token_id=163839),
    "tiny-kimi-vl": DecoderConfig(model_type="kimi_vl", vocab_size=1024, hidden_size=128, intermediate_size=352,
                                  num_layers=2, num_heads=4, num_kv_heads=4, head_dim=48, qkv_bias=False,
                                  kv_lora_rank=32, q_lora_rank=0, qk_nope_head_dim=32, qk_rope_head_dim=16,
                                  v_head_dim=32, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64,
                                  shared_expert_intermediate_size=128, scoring_func="sigmoid",
                                  topk_method="noaux_tc", routed_scaling_factor=2.0, first_k_dense_replace=1,
                                  moonvit=MoonViTConfig(init_pos_emb_height=8, init_pos_emb_width=8, hidden_size=64,
                                                        num_heads=2, intermediate_size=128, depth=2),
                                  image_token_id=1000),
    "tiny-deepseek-v3": DecoderConfig(model_type="deepseek_v3", vocab_size=1024, hidden_size=128, intermediate_size=352,
                                      num_layers=3, num_heads=4, num_kv_heads=4, head_dim=48, qkv_bias=False,
                                      kv_lora_rank=32, q_lora_rank=48, qk_nope_head_dim=32, qk_rope_head_dim=16,
                                      v_head_dim=32, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64,
                                      shared_expert_intermediate_size=64, n_group=2, topk_group=1,
                                      scoring_func="sigmoid", topk_method="noaux_tc", routed_scaling_factor=2.5,
                                      first_k_dense_replace=1),
    "tiny-moe": DecoderConfig(model_type="qwen3_moe", vocab_size=1024, hidden_size=128, intermediate_size=352,
                              num_layers=2, num_heads=4, num_kv_heads=2, head_dim=32, qkv_bias=False, qk_norm=True,
                              num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64),
    "qwen2.5-vl-7b": DecoderConfig(model_type="qwen2_5_vl", vocab_size=152064, hidden_size=3584,
                                   intermediate_size=18944, num_layers=28, num_heads=28, num_kv_heads=4, head_dim=128,
                                   rope_theta=1e6, mrope_section=[16, 24, 24], vision=VisionConfig(),
                                   eos_token_id=151645, pad_token_id=151643),
    "tiny-vl": DecoderConfig(model_type="qwen2_5_vl", vocab_size=1024, hidden_size=128, intermediate_size=352,
                             num_layers=2, num_heads=4, num_kv_heads=2, head_dim=32, mrope_section=[4, 6, 6],
                             vision=VisionConfig(depth=2, hidden_size=64, num_heads=4, intermediate_size=128,
                                                 patch_size=14, window_size=56, fullatt_block_indexes=[1],
                                                 out_hidden_size=128), image_token_id=1000),
    # InternVL2.5-8B: InternViT-300M-448px + InternLM2.5-7B
    "internvl2.5-8b": DecoderConfig(model_type="internvl_chat", llm_type="internlm2", hf_naming="internvl_chat",
                                    vocab_size=92553, hidden_size=4096, intermediate_size=14336, num_layers=32,
                                    num_heads=32, num_kv_heads=8, head_dim=128, rope_theta=1e6, qkv_bias=False,
                                    rms_norm_eps=1e-5, vit=ViTConfig(), image_token_id=92546, eos_token_id=92542,
                                    pad_token_id=2),
    # InternVL3-8B in transformers' layout: InternViT-300M + Qwen2.5-7B
    "internvl3-8b": DecoderConfig(model_type="internvl", llm_type="qwen2", vocab_size=151674, hidden_size=3584,
                                  intermediate_size=18944, num_layers=28, num_heads=28, num_kv_heads=4, head_dim=128,
                                  rope_theta=1e6, vit=ViTConfig(), image_token_id=151667, eos_token_id=151645,
                                  pad_token_id=151643),
    "tiny-internvl": DecoderConfig(model_type="internvl", llm_type="qwen2", vocab_size=1024, hidden_size=128,
                                   intermediate_size=352, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=32,
                                   vit=ViTConfig(image_size=56, patch_size=14, hidden_size=64, num_heads=2,
                                                 intermediate_size=128, depth=2, qkv_bias=False),
                                   image_token_id=1000),
    # OpenVLA-7B / OpenVLA-OFT: DINOv2-L/14 (4 registers) + SigLIP-so400m/14 at 224 px, Llama-2-7B
    "openvla-7b": DecoderConfig(model_type="openvla", llm_type="llama", vocab_size=32064, hidden_size=4096,
                                intermediate_size=11008, num_layers=32, num_heads=32, num_kv_heads=32, head_dim=128,
                                rope_theta=1e4, rms_norm_eps=1e-6, qkv_bias=False, prismatic=PrismaticConfig(),
                                action_vocab_size=32000, image_token_id=32000, pad_token_id=32000, eos_token_id=2,
                                bos_token_id=1, max_position_embeddings=2048),
    "tiny-openvla": DecoderConfig(model_type="openvla", llm_type="llama", vocab_size=1088, hidden_size=128,
                                  intermediate_size=352, num_layers=2, num_heads=4, num_kv_heads=4, head_dim=32,
                                  qkv_bias=False, action_vocab_size=1024, image_token_id=1024, pad_token_id=1024,
                                  bos_token_id=1, prismatic=PrismaticConfig(
                                      featurizer=ViTConfig(image_size=56, patch_size=14, hidden_size=64, num_heads=2,
                                                           intermediate_size=128, depth=3, num_register_tokens=4,
                                                           final_norm=True, select_layer=-2, class_pos_embed=False),
                                      fused_featurizer=ViTConfig(image_size=56, patch_size=14, hidden_size=72,
                                                                 num_heads=2, intermediate_size=96, depth=3,
                                                                 class_token=False, layer_scale=False, final_norm=True,
                                                                 select_layer=-2))),
    "tiny-vl-gpu": DecoderConfig(model_type="qwen2_5_vl", vocab_size=2048, hidden_size=256, intermediate_size=512,
                                 num_layers=2, num_heads=4, num_kv_heads=2, head_dim=64, mrope_section=[8, 12, 12],
                                 vision=VisionConfig(depth=2, hidden_size=128, num_heads=2, intermediate_size=256,
                                                     patch_size=14, window_size=56, fullatt_block_indexes=[1],
                                                     out_hidden_size=256), image_token_id=1500),
}


def get_config(name_or_path: str, overrides: Optional[Dict[str, Any]] = None) -> DecoderConfig:
    """Preset name (``qwen2.5-7b``) or a directory with an HF ``config.json``."""
    import copy
    if name_or_path in PRESETS:
        cfg = copy.deepcopy(PRESETS[name_or_path])
    else:
        cfg = DecoderConfig.from_pretrained(name_or_path)
    for k, v in (overrides or {}).items():
        hf_alias = {"num_hidden_layers": "num_layers", "num_attention_heads": "num_heads",
                    "num_key_value_heads": "num_kv_heads"}
        k = hf_alias.get(k, k)
        if hasattr(cfg, k):
            setattr(cfg, k, v)
    return cfg
