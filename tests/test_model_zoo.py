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


@pytest.mark.parametrize("preset", ["tiny", "tiny-mixtral", "tiny-qwen2-moe", "tiny-moe", "tiny-deepseek-v3"])
def test_family_matches_transformers(preset, tmp_path):
    cfg = get_config(preset)
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=4)
    with torch.no_grad():                      # a non-trivial selection bias where the family has one
        for n, p in model.named_parameters():
            if n.endswith("router_bias"):
                p.copy_(0.05 * torch.randn(p.shape, generator=torch.Generator().manual_seed(7)))
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
    import dataclasses
    from siirl_b200.models.vision import mrope_positions
    cfg = get_config("tiny-vl")
    # an MLP width that is no multiple of 8, like the released 7B tower's 3420: the model pads it internally
    cfg = dataclasses.replace(cfg, vision=dataclasses.replace(cfg.vision, intermediate_size=108))
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=8)
    assert model.vision.blocks[0].padded_intermediate == 128
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


def _timm_vit_reference(sd, prefix, cfg, images):
    """Plain-PyTorch statement of timm's ``VisionTransformer.get_intermediate_layers(n={depth - 2})`` from a state
    dict with timm names: patch convolution, positions on the patches (and on the class token unless
    ``no_embed_class``), [class, registers, patches], pre-norm blocks with LayerScale, output of the second-to-last
    block without the final norm, prefix tokens dropped."""
    import torch.nn.functional as F
    g = lambda n: sd[prefix + n].float()  # noqa: E731
    x = F.conv2d(images, g("patch_embed.proj.weight"), g("patch_embed.proj.bias"), stride=cfg.patch_size)
    x = x.flatten(2).transpose(1, 2)
    N = x.shape[0]
    pre = []
    if cfg.class_token:
        pre.append(g("cls_token").expand(N, -1, -1))
    if cfg.num_register_tokens:
        pre.append(g("reg_token").expand(N, -1, -1))
    if cfg.class_token and cfg.class_pos_embed:
        x = torch.cat([pre[0], x], 1) + g("pos_embed")
        x = torch.cat([x[:, :1]] + pre[1:] + [x[:, 1:]], 1)
    else:
        x = torch.cat(pre + [x + g("pos_embed")], 1)
    nh, H = cfg.num_heads, cfg.hidden_size
    for i in range(cfg.depth - 1):
        b = f"blocks.{i}."
        y = F.layer_norm(x, (H,), g(b + "norm1.weight"), g(b + "norm1.bias"), cfg.norm_eps)
        q, k, v = F.linear(y, g(b + "attn.qkv.weight"), g(b + "attn.qkv.bias")).reshape(N, -1, 3, nh, H // nh).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(N, -1, H)
        a = F.linear(a, g(b + "attn.proj.weight"), g(b + "attn.proj.bias"))
        x = x + (a * g(b + "ls1.scale_factor") if cfg.layer_scale else a)
        y = F.layer_norm(x, (H,), g(b + "norm2.weight"), g(b + "norm2.bias"), cfg.norm_eps)
        y = F.linear(F.gelu(F.linear(y, g(b + "mlp.fc1.weight"), g(b + "mlp.fc1.bias"))), g(b + "mlp.fc2.weight"), g(b + "mlp.fc2.bias"))
        x = x + (y * g(b + "ls2.scale_factor") if cfg.layer_scale else y)
    return x[:, cfg.num_prefix_tokens:]


def test_openvla_prismatic_backbone_and_checkpoint(tmp_path):
    """DINOv2 (class + 4 register tokens, LayerScale, positions on patches only) and SigLIP (no class token, head width
    outside the attention kernel's set) towers against the timm forward stated in plain PyTorch on the exported
    weights; fused projector; OpenVLA checkpoint names round-trip."""
    import torch.nn.functional as F
    from safetensors.torch import load_file
    from siirl_b200.models.hf_io import to_hf_state
    cfg = get_config("tiny-openvla")
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=11)
    with torch.no_grad():
        for n, p in model.vision.named_parameters():
            if n.endswith("bias") or ".ls" in n:
                p.copy_(0.2 * torch.randn(p.shape, generator=torch.Generator().manual_seed(len(n))) + (0.7 if ".ls" in n else 0))
    save_hf_model(model, str(tmp_path))
    sd = load_file(str(tmp_path / "model.safetensors"))
    assert {"vision_backbone.featurizer.reg_token", "vision_backbone.fused_featurizer.pos_embed", "projector.fc3.bias",
            "language_model.lm_head.weight", "vision_backbone.featurizer.blocks.0.ls1.scale_factor"} <= set(sd)
    assert "vision_backbone.fused_featurizer.cls_token" not in sd
    assert sd["vision_backbone.featurizer.pos_embed"].shape == (1, 16, 64)         # patches only
    pc = cfg.prismatic
    x = torch.randn(3, 6, 56, 56, generator=torch.Generator().manual_seed(5))
    with torch.no_grad():
        got = model.vision(x)
        f1 = _timm_vit_reference(sd, "vision_backbone.featurizer.", pc.featurizer, x[:, :3])
        f2 = _timm_vit_reference(sd, "vision_backbone.fused_featurizer.", pc.fused_featurizer, x[:, 3:])
        f = torch.cat([f1, f2], 2)
        for i in (1, 2, 3):
            f = F.linear(f, sd[f"projector.fc{i}.weight"], sd[f"projector.fc{i}.bias"])
            if i < 3:
                f = F.gelu(f)
    assert got.shape == (3 * 16, cfg.hidden_size)
    assert torch.allclose(got, f.reshape(-1, cfg.hidden_size), atol=2e-5), (got - f.reshape(-1, cfg.hidden_size)).abs().max()
    cfg2 = DecoderConfig.from_pretrained(str(tmp_path))
    assert cfg2.prismatic is not None and cfg2.action_vocab_size == 1024 and cfg2.vocab_size == cfg.vocab_size
    again = build_model(cfg2, dtype=torch.float32, device="cpu", seed=2)
    load_hf_weights(again, str(tmp_path))
    for (n1, a), (n2, b) in zip(to_hf_state(model), to_hf_state(again)):
        assert n1 == n2 and torch.equal(a, b), n1


def test_oft_parallel_decode_matches_scoring():
    """The one-pass chunk decoding of OpenVLA-OFT: tokens come from the action bins, their log-probs are those the
    training-side statement (zero vectors at the action positions, soft-max over the bins) assigns."""
    from siirl_b200.data_coordinator.dataloader.tokenizer import SyntheticTokenizer
    from siirl_b200.models.embodied.vla import VLAProcessor, action_id_range, oft_action_logits, oft_parallel_decode
    cfg = get_config("tiny-openvla")
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=3)
    proc = VLAProcessor(cfg, SyntheticTokenizer(cfg.action_vocab_size), image_size=56)
    prompts = [proc.prompt_ids("pick up the red block"), proc.prompt_ids("open the drawer")]
    assert prompts[0][0] == cfg.bos_token_id and prompts[0][1:17] == [cfg.image_token_id] * 16
    imgs = torch.randint(0, 255, (2, 56, 56, 3), dtype=torch.uint8, generator=torch.Generator().manual_seed(1))
    A = 14
    tok, lp = oft_parallel_decode(model, proc, prompts, imgs, A, 1.0, torch.Generator().manual_seed(0))
    lo, hi = action_id_range(cfg)
    assert (lo, hi) == (768, 1024) and tok.shape == (2, A) and bool(((tok >= lo) & (tok < hi)).all())
    greedy, glp = oft_parallel_decode(model, proc, prompts, imgs, A, 0.0)
    assert bool((glp >= lp - 1e-6).all())                  # the arg-max is at least as likely as any sample
    # scoring side, one sequence at a time, sampled tokens in place (their embeddings must not matter)
    for i, p in enumerate(prompts):
        ids = torch.tensor(list(p) + tok[i].tolist())
        info = SeqInfo([ids.numel()])
        zero = torch.zeros(ids.numel(), dtype=torch.bool)
        zero[-A:] = True
        pv, grid = proc.patchify(imgs[i:i + 1], torch.float32)
        with torch.no_grad():
            h = model.forward_hidden(ids, info.positions, info, pixel_values=pv, image_grid_thw=grid,
                                     image_mask=proc.image_mask(torch.tensor([0]), ids.numel()), zero_mask=zero)
            logp = torch.log_softmax(oft_action_logits(model, h[-A:], 1.0), -1)
        assert torch.allclose(logp.gather(1, (tok[i] - lo)[:, None])[:, 0], lp[i], atol=1e-5)


def _moonvit_reference(sd, cfg, pixels, grids):
    """Plain-PyTorch statement of the tower in the checkpoint's own layout: interleaved rotary pairs (even pair: x
    position, odd pair: y position) applied as complex multiplications, full attention per image."""
    import torch.nn.functional as F
    g = lambda n: sd[n].float()  # noqa: E731
    H, nh = cfg.hidden_size, cfg.num_heads
    hd = H // nh
    x = F.linear(pixels, g("vision_tower.patch_embed.proj.weight").reshape(H, -1), g("vision_tower.patch_embed.proj.bias"))
    pe = g("vision_tower.patch_embed.pos_emb.weight")
    pos, freqs = [], []
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 4)[: hd // 4].float() / hd))
    for h, w in grids:
        if (h, w) == tuple(pe.shape[:2]):
            pos.append(pe.reshape(h * w, H))
        else:
            pos.append(F.interpolate(pe.permute(2, 0, 1)[None], size=(h, w), mode="bicubic")[0].permute(1, 2, 0).reshape(h * w, H))
        xs = torch.arange(w).repeat(h).float()
        ys = torch.arange(h).repeat_interleave(w).float()
        fx = torch.polar(torch.ones(h * w, hd // 4), torch.outer(xs, inv))
        fy = torch.polar(torch.ones(h * w, hd // 4), torch.outer(ys, inv))
        freqs.append(torch.stack([fx, fy], -1).reshape(h * w, hd // 2))
    x = x + torch.cat(pos)
    fc = torch.cat(freqs)

    def rot(t):                                   # [T, nh, hd]
        c = torch.view_as_complex(t.float().reshape(t.shape[0], nh, hd // 2, 2))
        return torch.view_as_real(c * fc[:, None, :]).reshape(t.shape[0], nh, hd)
    for i in range(cfg.depth):
        b = f"vision_tower.encoder.blocks.{i}."
        y = F.layer_norm(x, (H,), g(b + "norm0.weight"), g(b + "norm0.bias"), 1e-5)
        q, k, v = F.linear(y, g(b + "wqkv.weight"), g(b + "wqkv.bias")).reshape(-1, 3, nh, hd).unbind(1)
        q, k = rot(q), rot(k)
        outs, at = [], 0
        for h, w in grids:
            n = h * w
            o = F.scaled_dot_product_attention(q[at:at + n].transpose(0, 1), k[at:at + n].transpose(0, 1),
                                               v[at:at + n].transpose(0, 1))
            outs.append(o.transpose(0, 1).reshape(n, H))
            at += n
        x = x + F.linear(torch.cat(outs), g(b + "wo.weight"), g(b + "wo.bias"))
        y = F.layer_norm(x, (H,), g(b + "norm1.weight"), g(b + "norm1.bias"), 1e-5)
        x = x + F.linear(F.gelu(F.linear(y, g(b + "mlp.fc0.weight"), g(b + "mlp.fc0.bias")), approximate="tanh"),
                         g(b + "mlp.fc1.weight"), g(b + "mlp.fc1.bias"))
    x = F.layer_norm(x, (H,), g("vision_tower.encoder.final_layernorm.weight"), g("vision_tower.encoder.final_layernorm.bias"), 1e-5)
    x = F.layer_norm(x, (H,), g("multi_modal_projector.pre_norm.weight"), g("multi_modal_projector.pre_norm.bias"), 1e-5)
    merged, at = [], 0
    for h, w in grids:
        t = x[at:at + h * w].reshape(h // 2, 2, w // 2, 2, H).permute(0, 2, 1, 3, 4).reshape(h * w // 4, 4 * H)
        merged.append(t)
        at += h * w
    y = F.linear(torch.cat(merged), g("multi_modal_projector.linear_1.weight"), g("multi_modal_projector.linear_1.bias"))
    return F.linear(F.gelu(y), g("multi_modal_projector.linear_2.weight"), g("multi_modal_projector.linear_2.bias"))


def test_kimi_vl_tower_checkpoint_layout_and_language_model(tmp_path):
    """MoonViT (interpolated position table, (x, y) rotary pairs held permuted in memory, 2 x 2 merge, projector)
    against the tower's math stated on the exported weights in the checkpoint's interleaved layout; the checkpoint
    round-trips; image features land on the placeholders of the multi-head-latent-attention language model."""
    from safetensors.torch import load_file
    from siirl_b200.models.hf_io import to_hf_state
    from siirl_b200.models.moonvit import MoonViTProcessor
    cfg = get_config("tiny-kimi-vl")
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=13)
    with torch.no_grad():
        for n, p in model.vision.named_parameters():
            if n.endswith("bias"):
                p.copy_(0.2 * torch.randn(p.shape, generator=torch.Generator().manual_seed(len(n))))
    save_hf_model(model, str(tmp_path))
    sd = load_file(str(tmp_path / "model.safetensors"))
    assert {"vision_tower.patch_embed.pos_emb.weight", "vision_tower.encoder.blocks.1.wqkv.bias",
            "multi_modal_projector.linear_2.weight", "language_model.model.layers.0.self_attn.kv_a_proj_with_mqa.weight",
            "language_model.model.layers.1.mlp.gate.e_score_correction_bias", "language_model.lm_head.weight"} <= set(sd)
    grids = [(4, 6), (8, 8), (2, 2)]
    grid = torch.tensor([[1, h, w] for h, w in grids])
    pixels = torch.randn(sum(h * w for h, w in grids), 588, generator=torch.Generator().manual_seed(4))
    with torch.no_grad():
        got = model.vision(pixels, grid)
        want = _moonvit_reference(sd, cfg.moonvit, pixels, grids)
    assert got.shape == (sum(h * w for h, w in grids) // 4, cfg.hidden_size)
    assert torch.allclose(got, want, atol=3e-5), (got - want).abs().max()
    cfg2 = DecoderConfig.from_pretrained(str(tmp_path))
    assert cfg2.moonvit is not None and cfg2.is_mla and cfg2.moonvit.depth == 2 and cfg2.image_token_id == 1000
    again = build_model(cfg2, dtype=torch.float32, device="cpu", seed=1)
    load_hf_weights(again, str(tmp_path))
    for (n1, a), (n2, b) in zip(to_hf_state(model), to_hf_state(again)):
        assert n1 == n2 and torch.equal(a, b), n1
    proc = MoonViTProcessor(cfg, 28 * 28, 112 * 112)
    out = proc([5, cfg.image_token_id, 6], [torch.rand(3, 60, 90)])
    gh, gw = out["image_grid_thw"][0, 1:].tolist()
    assert out["input_ids"].count(cfg.image_token_id) == gh * gw // 4 and out["pixel_values"].shape == (gh * gw, 588)
    ids = torch.tensor(out["input_ids"])
    with torch.no_grad():
        lp = _mm_logprobs_ours(model, ids, out["pixel_values"], out["image_grid_thw"])
        lp2 = _mm_logprobs_ours(model, ids, out["pixel_values"] + 0.5, out["image_grid_thw"])
    assert torch.isfinite(lp).all() and torch.equal(lp[0], lp2[0]) and not torch.allclose(lp[-1], lp2[-1])


@pytest.mark.parametrize("preset,scaling", [
    ("tiny-deepseek-v3", {"rope_type": "yarn", "type": "yarn", "factor": 8.0, "original_max_position_embeddings": 16,
                          "beta_fast": 32, "beta_slow": 1, "mscale": 1.0, "mscale_all_dim": 1.0}),
    ("tiny", {"rope_type": "llama3", "type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
              "original_max_position_embeddings": 16}),
    ("tiny", {"rope_type": "linear", "type": "linear", "factor": 4.0}),
])
def test_rope_scaling_matches_transformers(preset, scaling, tmp_path):
    """Checkpoint rope scaling (YaRN with its attention-temperature factor on multi-head latent attention, Llama-3's
    wavelength-dependent scaling, linear interpolation) against transformers on a sequence longer than the original
    context of the scaling."""
    import dataclasses
    cfg = dataclasses.replace(get_config(preset), rope_scaling=scaling)
    if preset == "tiny":
        cfg = dataclasses.replace(cfg, model_type="llama", qkv_bias=False)
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=21)
    save_hf_model(model, str(tmp_path))
    try:
        hf = transformers.AutoModelForCausalLM.from_pretrained(str(tmp_path), torch_dtype=torch.float32,
                                                               attn_implementation="eager")
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"transformers cannot build {cfg.model_type} with {scaling['type']}: {type(e).__name__}: {e}")
    hf.eval()
    ids = torch.randint(3, cfg.vocab_size, (61,), generator=torch.Generator().manual_seed(2))
    with torch.no_grad():
        want = torch.log_softmax(hf(ids[None]).logits[0].float(), -1)
        got = _logprobs_ours(model, ids)
    assert (got - want).abs().max().item() < 3e-4, (got - want).abs().max().item()
    plain = build_model(dataclasses.replace(cfg, rope_scaling=None), dtype=torch.float32, device="cpu", seed=21)
    with torch.no_grad():
        assert (_logprobs_ours(plain, ids) - got).abs().max().item() > 1e-3      # the scaling is not a no-op here
    assert DecoderConfig.from_pretrained(str(tmp_path)).rope_scaling["factor"] == scaling["factor"]


@pytest.mark.parametrize("preset", ["tiny-vl", "tiny-openvla", "tiny-kimi-vl", "tiny-internvl", "tiny-deepseek-v3"])
def test_every_parameter_round_trips_through_the_checkpoint_format(tmp_path, preset):
    """Export under the family's checkpoint names and load into a differently seeded model: every parameter comes
    back bit for bit (padding added for the kernels is zero on both sides and never exported)."""
    cfg = get_config(preset)
    a = build_model(cfg, dtype=torch.float32, device="cpu", seed=3)
    save_hf_model(a, str(tmp_path))
    b = build_model(cfg, dtype=torch.float32, device="cpu", seed=9)
    load_hf_weights(b, str(tmp_path))
    bad = [n for (n, x), (_, y) in zip(a.named_parameters(), b.named_parameters()) if not torch.equal(x, y)]
    assert not bad, bad
