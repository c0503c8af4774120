"""Model families against the Hugging Face implementations: a tiny random model of each family is exported to
safetensors with HF names, loaded by ``transformers`` and both sides must give the same next-token log-probs."""
import pytest
import torch

from siirl_b200.models.config import DecoderConfig, get_config
from siirl_b200.models.decoder import build_model
from siirl_b200.models.hf_io import load_hf_weights, save_hf_model
from siirl_b200.ops.attention import SeqInfo

transformers = pytest.importorskip("transformers")


def _logprobs_ours(model, ids):
    info = SeqInfo([ids.numel()])
    logits = model.logits(ids, info.positions, info)
    return torch.log_softmax(logits.float(), -1)


@pytest.mark.parametrize("preset", ["tiny", "tiny-mixtral", "tiny-qwen2-moe", "tiny-moe"])
def test_family_matches_transformers(preset, tmp_path):
    cfg = get_config(preset)
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=4)
    save_hf_model(model, str(tmp_path))
    try:
        hf = transformers.AutoModelForCausalLM.from_pretrained(str(tmp_path), torch_dtype=torch.float32,
                                                               attn_implementation="eager")
    except Exception as e:  # noqa: BLE001  (an architecture this transformers build does not ship)
        pytest.skip(f"transformers cannot build {cfg.model_type}: {type(e).__name__}: {e}")
    hf.eval()
    ids = torch.randint(3, cfg.vocab_size, (23,), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = torch.log_softmax(hf(ids[None]).logits[0].float(), -1)
        got = _logprobs_ours(model, ids)
    assert (got - want).abs().max().item() < 2e-4, (got - want).abs().max().item()
    # and back: a model filled from the exported files reproduces the original
    cfg2 = DecoderConfig.from_pretrained(str(tmp_path))
    assert cfg2.num_experts == cfg.num_experts and cfg2.norm_topk_prob == cfg.norm_topk_prob
    assert cfg2.shared_expert_intermediate_size == cfg.shared_expert_intermediate_size
    again = build_model(cfg2, dtype=torch.float32, device="cpu", seed=99)
    load_hf_weights(again, str(tmp_path))
    with torch.no_grad():
        assert torch.allclose(_logprobs_ours(again, ids), got, atol=1e-5)


def _mm_logprobs_ours(model, ids, pixel_values, grid, positions=None):
    info = SeqInfo([ids.numel()])
    pos = info.positions if positions is None else positions
    h = model.forward_hidden(ids, pos, info, pixel_values=pixel_values, image_grid_thw=grid)
    logits = h.float() @ model.head_weight.float().t()
    return torch.log_softmax(logits, -1)


def test_internvl_matches_transformers(tmp_path):
    """InternViT tower (class token, LayerScale), pixel shuffle and projector against transformers' InternVL classes,
    through an export in transformers' parameter names."""
    cfg = get_config("tiny-internvl")
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=5)
    with torch.no_grad():                      # LayerScale and biases away from their trivial initial values
        for n, p in model.vision.named_parameters():
            if n.endswith("bias") or ".ls" in n or "prefix_tokens" in n:
                p.copy_(0.3 * torch.randn(p.shape, generator=torch.Generator().manual_seed(len(n))) + (0.5 if ".ls" in n else 0))
    save_hf_model(model, str(tmp_path))
    try:
        hf = transformers.AutoModelForImageTextToText.from_pretrained(str(tmp_path), torch_dtype=torch.float32,
                                                                      attn_implementation="eager")
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"transformers cannot build internvl: {type(e).__name__}: {e}")
    hf.eval()
    tiles = 2
    per_tile = model.vision.tokens_per_tile
    g = torch.Generator().manual_seed(2)
    text = torch.randint(3, 900, (9,), generator=g)
    ids = torch.cat([text[:3], torch.full((tiles * per_tile,), cfg.image_token_id), text[3:]])
    pixels = torch.randn(tiles, 3, cfg.vit.image_size, cfg.vit.image_size, generator=g)
    with torch.no_grad():
        want = torch.log_softmax(hf(input_ids=ids[None], pixel_values=pixels).logits[0].float(), -1)
        got = _mm_logprobs_ours(model, ids, pixels, None)
    assert (got - want).abs().max().item() < 5e-4, (got - want).abs().max().item()
    cfg2 = DecoderConfig.from_pretrained(str(tmp_path))
    assert cfg2.vit is not None and cfg2.vit.depth == cfg.vit.depth and cfg2.image_token_id == cfg.image_token_id
    again = build_model(cfg2, dtype=torch.float32, device="cpu", seed=77)
    load_hf_weights(again, str(tmp_path))
    with torch.no_grad():
        assert torch.allclose(_mm_logprobs_ours(again, ids, pixels, None), got, atol=1e-5)


def test_internvl_chat_layout_roundtrip(tmp_path):
    """The upstream remote-code layout (``vision_model`` / ``mlp1`` / ``language_model`` with InternLM2's fused
    ``wqkv``) exports and loads back to the same function."""
    import dataclasses
    from safetensors import safe_open
    cfg = dataclasses.replace(get_config("tiny-internvl"), model_type="internvl_chat", hf_naming="internvl_chat",
                              llm_type="internlm2", qkv_bias=False)
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=6)
    save_hf_model(model, str(tmp_path))
    with safe_open(str(tmp_path / "model.safetensors"), framework="pt") as f:
        names = set(f.keys())
        wqkv = f.get_tensor("language_model.model.layers.0.attention.wqkv.weight")
    assert {"vision_model.embeddings.class_embedding", "mlp1.1.weight", "language_model.output.weight",
            "language_model.model.tok_embeddings.weight", "language_model.model.layers.1.feed_forward.w3.weight",
            "vision_model.encoder.layers.0.ls1", "vision_model.encoder.layers.0.attn.qkv.weight"} <= names
    # wqkv groups: for KV head j, its query heads, then k_j, then v_j
    g, d = cfg.num_heads // cfg.num_kv_heads, cfg.head_dim
    q = model.layers[0].qkv_proj_weight.data[: cfg.q_width]
    k = model.layers[0].qkv_proj_weight.data[cfg.q_width: cfg.q_width + cfg.kv_width]
    assert torch.equal(wqkv[(g + 2) * d: (g + 2) * d + g * d], q[g * d: 2 * g * d])
    assert torch.equal(wqkv[g * d: (g + 1) * d], k[:d])
    cfg2 = DecoderConfig.from_pretrained(str(tmp_path))
    assert cfg2.hf_naming == "internvl_chat" and cfg2.llm_type == "internlm2" and not cfg2.qkv_bias
    again = build_model(cfg2, dtype=torch.float32, device="cpu", seed=3)
    load_hf_weights(again, str(tmp_path))
    ids = torch.cat([torch.tensor([5, 6]), torch.full((model.vision.tokens_per_tile,), cfg.image_token_id), torch.tensor([9])])
    pixels = torch.randn(1, 3, cfg.vit.image_size, cfg.vit.image_size, generator=torch.Generator().manual_seed(0))
    with torch.no_grad():
        assert torch.allclose(_mm_logprobs_ours(again, ids, pixels, None), _mm_logprobs_ours(model, ids, pixels, None),
                              atol=1e-5)


def test_internvl_tiling_and_processor():
    from siirl_b200.models.internvl import InternVLProcessor, closest_tile_grid, dynamic_tiles
    assert closest_tile_grid(896, 448, 1, 6, 448) == (2, 1)
    assert closest_tile_grid(448, 1344, 1, 6, 448) == (1, 3)
    assert closest_tile_grid(500, 500, 1, 6, 448) == (1, 1)
    img = torch.rand(3, 100, 200)
    t = dynamic_tiles(img, 1, 6, 56, use_thumbnail=True)
    assert t.shape == (3, 3, 56, 56)                       # 2 x 1 grid + thumbnail
    whole = torch.nn.functional.interpolate(img[None], size=(56, 112), mode="bicubic", align_corners=False).clamp(0, 1)[0]
    assert torch.allclose(t[1], whole[:, :, 56:])          # tiles cut left to right
    cfg = get_config("tiny-internvl")
    proc = InternVLProcessor(cfg, 1, 6)
    out = proc([7, cfg.image_token_id, 8], [img])
    n = 3 * proc.tokens_per_tile
    assert out["input_ids"] == [7] + [cfg.image_token_id] * n + [8]
    assert out["pixel_values"].shape == (3, 3, 56, 56) and out["image_grid_thw"].tolist() == [[3, 1, 1]]
    pos, delta = proc.rope(torch.tensor(out["input_ids"]), out["image_grid_thw"])
    assert pos.shape == (3, n + 2) and delta == 0 and pos[1, -1] == n + 1


def test_qwen2_5_vl_matches_transformers(tmp_path):
    """Vision tower (window attention, 2-D rope, merger), multimodal rope and language model against transformers'
    Qwen2.5-VL classes through an export in their parameter names."""
    from siirl_b200.models.vision import mrope_positions
    cfg = get_config("tiny-vl")
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=8)
    save_hf_model(model, str(tmp_path))
    import json
    hfc = json.load(open(tmp_path / "config.json"))
    v = cfg.vision
    hfc["vision_config"] = {"depth": v.depth, "hidden_size": v.hidden_size, "num_heads": v.num_heads,
                            "intermediate_size": v.intermediate_size, "patch_size": v.patch_size,
                            "temporal_patch_size": v.temporal_patch_size, "in_chans": v.in_channels,
                            "spatial_merge_size": v.spatial_merge_size, "window_size": v.window_size,
                            "fullatt_block_indexes": v.fullatt_block_indexes, "out_hidden_size": v.out_hidden_size,
                            "hidden_act": "silu", "model_type": "qwen2_5_vl"}
    hfc["image_token_id"] = cfg.image_token_id
    hfc["video_token_id"] = cfg.image_token_id + 1
    hfc["vision_start_token_id"] = cfg.image_token_id + 2
    json.dump(hfc, open(tmp_path / "config.json", "w"))
    try:
        hf = transformers.AutoModelForImageTextToText.from_pretrained(str(tmp_path), torch_dtype=torch.float32,
                                                                      attn_implementation="eager")
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"transformers cannot build qwen2_5_vl: {type(e).__name__}: {e}")
    hf.eval()
    g = torch.Generator().manual_seed(3)
    grid = torch.tensor([[1, 8, 12]])
    n_img = 8 * 12 // 4
    text = torch.randint(3, 900, (10,), generator=g)
    ids = torch.cat([text[:4], torch.tensor([cfg.image_token_id + 2]), torch.full((n_img,), cfg.image_token_id), text[4:]])
    pixels = torch.randn(8 * 12, model.vision.patch_dim, generator=g)
    pos = mrope_positions(ids, cfg.image_token_id, grid, v.spatial_merge_size)
    with torch.no_grad():
        # positions passed explicitly: image tokens share the temporal index of the image's first token (the
        # numbering of the model's original release, which the reference runs)
        want = torch.log_softmax(hf(input_ids=ids[None], pixel_values=pixels, image_grid_thw=grid,
                                    position_ids=pos[:, None, :]).logits[0].float(), -1)
        got = _mm_logprobs_ours(model, ids, pixels, grid, positions=pos)
    assert (got - want).abs().max().item() < 5e-4, (got - want).abs().max().item()
