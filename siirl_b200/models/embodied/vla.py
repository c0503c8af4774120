"""Vision-language-action policy pieces on the native VL decoder.

The reference's embodied policies are OpenVLA / OpenVLA-OFT (siirl/models/embodied/*, used by
siirl/engine/rollout/embodied_rollout.py:312-650): a vision backbone feeds patch embeddings into a causal language
model and continuous actions are read off discrete tokens — 256 uniform bins over [-1, 1] mapped onto the LAST 256
ids of the vocabulary, ``action_token_len`` (7) tokens per action and ``action_chunks_len`` actions per model call.
Here the policy is the framework's own vision tower + decoder (``DecoderLM`` with a ``vision`` config); this module
holds what surrounds it: the action tokenizer, the device-side image preprocessing (crop + resize kernel,
normalisation, patch layout of the vision tower) and the prompt layout shared by rollout and training.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ...ops.image import center_crop_box, resize_bilinear

_MEAN = (0.48145466, 0.4578275, 0.40821073)
_STD = (0.26862954, 0.26130258, 0.27577711)


class ActionTokenizer:
    """Uniform ``n_bins`` discretisation of [lo, hi]; bin b <-> token id ``vocab_size - 1 - b`` (OpenVLA's
    convention: the least used tail of the vocabulary).  Decoding returns bin centres."""

    def __init__(self, vocab_size: int, n_bins: int = 256, lo: float = -1.0, hi: float = 1.0):
        self.vocab_size, self.n_bins, self.lo, self.hi = vocab_size, n_bins, lo, hi
        edges = np.linspace(lo, hi, n_bins)
        self.centers = torch.tensor((edges[:-1] + edges[1:]) / 2.0, dtype=torch.float32)

    @property
    def first_action_token(self) -> int:
        return self.vocab_size - self.n_bins

    def encode(self, actions: torch.Tensor) -> torch.Tensor:
        a = actions.float().clamp(self.lo, self.hi)
        b = torch.bucketize(a, torch.linspace(self.lo, self.hi, self.n_bins, device=a.device)).clamp(1, self.n_bins - 1)
        return self.vocab_size - b

    def decode(self, token_ids: torch.Tensor) -> torch.Tensor:
        """Any token id maps to an action: ids outside the action range are clamped into it (an untrained policy
        may sample them), exactly like taking ``clip(vocab - id - 1, 0, n_bins - 2)``."""
        b = (self.vocab_size - token_ids.long() - 1).clamp(0, self.n_bins - 2)
        return self.centers.to(token_ids.device)[b]


class VLAProcessor:
    """Builds model inputs for one control step of a batch of environments.

    Prompt layout per step: ``[image placeholders x tokens_per_image x num_images] [task text tokens]`` followed, in
    training, by the ``action_chunks_len * action_token_len`` action tokens.  Rope positions follow the multimodal
    convention of the VL decoder: an image of a ``g x g`` merged grid advances the position by ``g`` and the text
    continues from there, so ``rope_delta = tokens_per_image - g`` per image.

    ``num_images > 1`` (third-person + wrist camera; the reference's ``num_images_in_input``,
    siirl/engine/rollout/embodied_rollout.py:652-666): the policy images of one step are kept stacked along the
    height, ``[N, num_images * S, S, 3]``, so buffers and batches keep one image tensor per step; every image gets
    its own placeholders, in camera order."""

    def __init__(self, model_config, tokenizer, image_size: int = 224, center_crop: bool = True,
                 max_text_len: int = 48, num_images: int = 1):
        self.cfg, self.tok = model_config, tokenizer
        self.num_images = max(1, int(num_images))
        self.center_crop = center_crop
        self.max_text_len = max_text_len
        self.image_token_id = model_config.image_token_id
        self.prismatic = model_config.prismatic
        self.image_offset = 0               # tokens in front of the image placeholders
        if self.prismatic is not None:
            # OpenVLA layout: [BOS][patch features of the image][text]; plain 1-D rope positions
            pc = self.prismatic
            self.image_size = pc.featurizer.image_size
            self.patch, self.merge, self.tpatch = pc.featurizer.patch_size, 1, 1
            self.grid = self.image_size // self.patch
            self.tokens_per_image = pc.tokens_per_image
            self.image_tokens = self.tokens_per_image * self.num_images
            self.image_offset = 1
            return
        v = model_config.vision
        assert v is not None, "the VLA policy needs a decoder with a vision tower"
        self.patch, self.merge, self.tpatch = v.patch_size, v.spatial_merge_size, v.temporal_patch_size
        unit = self.patch * self.merge
        self.image_size = max(unit, image_size // unit * unit)
        self.grid = self.image_size // self.patch
        self.tokens_per_image = (self.grid // self.merge) ** 2
        self.image_tokens = self.tokens_per_image * self.num_images

    # ---- images --------------------------------------------------------------------------------------
    def resize(self, images: torch.Tensor) -> torch.Tensor:
        """``[N, H, W, 3] uint8`` camera frames -> ``[N, S, S, 3] uint8`` policy input (centre crop of 90 % area when
        enabled, then bilinear resize; reference: embodied_rollout.py:65-133).  ``[N, num_images, H, W, 3]`` gives the
        cameras stacked along the height, ``[N, num_images * S, S, 3]``."""
        stacked = images.dim() == 5
        if stacked:
            N, k = images.shape[:2]
            images = images.reshape(N * k, *images.shape[2:])
        H, W = images.shape[1:3]
        crop = center_crop_box(H, W, 0.9) if self.center_crop else None
        out = resize_bilinear(images, (self.image_size, self.image_size), crop)
        return out.reshape(N, k * self.image_size, self.image_size, 3) if stacked else out

    def patchify(self, images_u8: torch.Tensor, dtype=torch.bfloat16) -> Tuple[torch.Tensor, torch.Tensor]:
        """Resized frames ``[N, S, S, 3] uint8`` -> flattened patches ``[N * grid^2, C*T*P*P]`` in the vision tower's
        order (per image ``(h/m, w/m, m, m)`` patch order, each patch ``C x T x P x P``) and ``grid_thw [N, 3]``."""
        S = self.image_size
        if self.num_images > 1:                 # cameras stacked along the height -> one image each, camera-minor order
            images_u8 = images_u8.reshape(images_u8.shape[0] * self.num_images, S, S, 3)
        N = images_u8.shape[0]
        if self.prismatic is not None:
            from .prismatic import normalize_for_towers
            x = normalize_for_towers(images_u8, self.prismatic.fused_featurizer is not None)
            return x.to(dtype), torch.tensor([[1, self.grid, self.grid]] * N, dtype=torch.int64)
        x = images_u8.permute(0, 3, 1, 2).float() / 255.0
        mean = torch.tensor(_MEAN, device=x.device).view(1, 3, 1, 1)
        std = torch.tensor(_STD, device=x.device).view(1, 3, 1, 1)
        x = (x - mean) / std
        g, m, P = self.grid, self.merge, self.patch
        x = x.reshape(N, 3, g // m, m, P, g // m, m, P).permute(0, 2, 5, 3, 6, 1, 4, 7)   # N, gh, gw, m, m, C, P, P
        x = x.unsqueeze(6).expand(-1, -1, -1, -1, -1, -1, self.tpatch, -1, -1)            # duplicate along time
        x = x.reshape(N * g * g, 3 * self.tpatch * P * P)
        grid = torch.tensor([[1, g, g]] * N, dtype=torch.int64)
        return x.to(dtype), grid

    # ---- tokens ---------------------------------------------------------------------------------------
    def text_tokens(self, task_description: str) -> List[int]:
        q = f"What action should the robot take to {task_description.lower()}?"
        if self.prismatic is not None:          # OpenVLA's prompt template
            q = f"In: {q}\nOut:"
        ids = self.tok.encode(q)
        bos = self.cfg.bos_token_id
        if self.prismatic is not None and bos is not None and len(ids) and ids[0] == bos:
            ids = ids[1:]                       # the layout places BOS itself
        return list(ids)[: self.max_text_len]

    def prompt_ids(self, task_description: str) -> List[int]:
        img = [self.image_token_id] * self.image_tokens
        if self.prismatic is not None:
            bos = self.cfg.bos_token_id if self.cfg.bos_token_id is not None else 1
            return [bos] + img + self.text_tokens(task_description)
        return img + self.text_tokens(task_description)

    def image_mask(self, first_rows: torch.Tensor, total_rows: int) -> torch.Tensor:
        """Placeholder positions of a packed batch whose sequences start at ``first_rows``."""
        dev = first_rows.device
        mask = torch.zeros(total_rows, dtype=torch.bool, device=dev)
        at = first_rows[:, None] + self.image_offset + torch.arange(self.image_tokens, device=dev)[None, :]
        mask[at.flatten()] = True
        return mask

    def rope_layout(self, prompt_len: int, extra: int = 0) -> Tuple[torch.Tensor, int]:
        """3-row rope positions of ``[image][text][extra generated tokens]`` and the rope delta of the prompt."""
        if self.prismatic is not None:
            n = prompt_len + extra
            return torch.arange(n).expand(3, n).contiguous(), 0
        gm = self.grid // self.merge
        hh = torch.arange(gm).repeat_interleave(gm)
        ww = torch.arange(gm).repeat(gm)
        one = torch.stack([torch.zeros(gm * gm, dtype=torch.int64), hh, ww])
        img = torch.cat([one + j * gm for j in range(self.num_images)], 1)     # every image advances the position by gm
        n_text = prompt_len - self.image_tokens + extra
        txt = (torch.arange(n_text) + gm * self.num_images).expand(3, n_text)
        return torch.cat([img, txt], 1), self.image_tokens - gm * self.num_images

    def mm_inputs(self, images_u8: torch.Tensor, prompt_lens: Sequence[int], dtype=torch.bfloat16) -> List[Dict]:
        """Per-prompt multimodal inputs for ``RolloutEngine.generate``."""
        pv, grid = self.patchify(images_u8, dtype)
        k = self.num_images
        per = (1 if self.prismatic is not None else self.grid * self.grid) * k
        out = []
        for i, n in enumerate(prompt_lens):
            pos, delta = self.rope_layout(n)
            out.append({"pixel_values": pv[i * per:(i + 1) * per], "image_grid_thw": grid[i * k:(i + 1) * k],
                        "rope_positions": pos, "rope_delta": delta})
        return out


# ---- OpenVLA-OFT parallel decoding ------------------------------------------------------------------------------
def action_id_range(model_config) -> Tuple[int, int]:
    """[lo, hi) of the action token ids: the last ``n_action_bins`` ids of the tokenizer's vocabulary (the embedding
    matrix may be padded beyond it)."""
    hi = int(model_config.action_vocab_size or model_config.vocab_size)
    return hi - int(model_config.n_action_bins), hi


def uses_parallel_decode(embodied_cfg, model_config) -> bool:
    """OpenVLA-OFT reads a whole action chunk off ONE forward pass: the action positions enter as zero vectors and
    the logits at those positions, restricted to the action ids, give the tokens
    (siirl/models/embodied/openvla_oft/modeling_prismatic.py:1552-1706).  OpenVLA decodes token by token."""
    explicit = getattr(embodied_cfg, "parallel_decode", None)
    if explicit is not None:
        return bool(explicit)
    return str(getattr(embodied_cfg, "embodied_type", "")) == "openvla-oft" and model_config.prismatic is not None


def oft_action_logits(model, hidden_rows: torch.Tensor, temperature: float) -> torch.Tensor:
    """Hidden states at the action positions -> fp32 logits over the action bins ``[N, n_action_bins]``."""
    from ... import ops
    lo, hi = action_id_range(model.cfg)
    logits = ops.linear(hidden_rows, model.head_weight[lo:hi]).float()
    return logits / max(float(temperature), 1e-6)


@torch.no_grad()
def oft_parallel_decode(model, proc: "VLAProcessor", prompts: Sequence[Sequence[int]], images_u8: torch.Tensor,
                        n_action_tokens: int, temperature: float, generator: Optional[torch.Generator] = None
                        ) -> Tuple[torch.Tensor, torch.Tensor]:
    """One forward pass per control step: returns (action token ids ``[N, A]``, their log-probs ``[N, A]`` under the
    distribution over the action bins).  ``temperature`` 0 takes the arg-max."""
    from ...ops.attention import SeqInfo
    dev = images_u8.device
    A = n_action_tokens
    lo, _ = action_id_range(model.cfg)
    pad = model.cfg.pad_token_id or 0
    lens = [len(p) + A for p in prompts]
    ids = torch.tensor([t for p in prompts for t in list(p) + [pad] * A], dtype=torch.int64, device=dev)
    info = SeqInfo(lens, device=dev)
    first = torch.tensor(info.cu_seqlens_cpu[:-1], device=dev)
    ends = torch.tensor(info.cu_seqlens_cpu[1:], device=dev)
    act_rows = (ends[:, None] - A + torch.arange(A, device=dev)[None, :]).flatten()
    zero_mask = torch.zeros(ids.shape[0], dtype=torch.bool, device=dev)
    zero_mask[act_rows] = True
    pv, grid = proc.patchify(images_u8, model.embed_tokens.dtype)
    if proc.prismatic is None:
        positions = torch.cat([proc.rope_layout(len(p), A)[0] for p in prompts], 1).to(dev)
    else:
        positions = info.positions
    hidden = model.forward_hidden(ids, positions, info, pixel_values=pv, image_grid_thw=grid,
                                  image_mask=proc.image_mask(first, ids.shape[0]), zero_mask=zero_mask)
    logits = oft_action_logits(model, hidden.index_select(0, act_rows), temperature if temperature > 0 else 1.0)
    logp = torch.log_softmax(logits, -1)
    if temperature > 0:
        pick = torch.multinomial(logp.exp(), 1, generator=generator)[:, 0]
    else:
        pick = logp.argmax(-1)
    lp = logp.gather(1, pick[:, None])[:, 0]
    return (pick + lo).reshape(len(prompts), A), lp.reshape(len(prompts), A)


# ---- OpenVLA-OFT continuous actions --------------------------------------------------------------------------------
def oft_action_hidden(model, proc: "VLAProcessor", prompts: Sequence[Sequence[int]], images_u8: torch.Tensor,
                      n_action_tokens: int, proprio: Optional[torch.Tensor] = None, proprio_projector=None,
                      pseudo_tokens: Optional[Sequence[torch.Tensor]] = None,
                      action_embeds: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Final hidden states ``[N, n_action_tokens, H]`` of the action placeholder rows of one control step (one forward
    pass; gradients flow when enabled).  The action rows enter as zero vectors, or as ``action_embeds [N, A, H]`` (the
    projected noisy actions of the diffusion head).  Pseudo-tokens are placed directly behind the image patch rows,
    in this order: the projected robot state (``proprio [N, proprio_dim]`` with a projector), then every
    ``pseudo_tokens[i] [N, H]`` (the diffusion timestep embedding); the reference appends them to the projected patch
    embeddings (modeling_prismatic.py:449-459, 1425-1434)."""
    from ...ops.attention import SeqInfo
    dev = images_u8.device
    A = n_action_tokens
    N = len(prompts)
    pad = model.cfg.pad_token_id or 0
    extras = []
    if proprio is not None and proprio_projector is not None:
        extras.append(proprio_projector(proprio.reshape(N, -1)))
    extras += list(pseudo_tokens or [])
    E = len(extras)
    cut = proc.image_offset + proc.image_tokens              # first row behind the patches
    rows = []
    for p in prompts:
        p = list(p)
        rows.append(p[:cut] + [pad] * E + p[cut:] + [pad] * A)
    lens = [len(r) for r in rows]
    ids = torch.tensor([t for r in rows for t in r], dtype=torch.int64, device=dev)
    info = SeqInfo(lens, device=dev)
    first = torch.tensor(info.cu_seqlens_cpu[:-1], device=dev)
    ends = torch.tensor(info.cu_seqlens_cpu[1:], device=dev)
    act_rows = (ends[:, None] - A + torch.arange(A, device=dev)[None, :]).flatten()
    zero_mask = None
    over_rows, over_vals = [], []
    if action_embeds is None:
        zero_mask = torch.zeros(ids.shape[0], dtype=torch.bool, device=dev)
        zero_mask[act_rows] = True
    else:
        over_rows.append(act_rows)
        over_vals.append(action_embeds.reshape(N * A, -1))
    for i, e in enumerate(extras):
        over_rows.append(first + cut + i)
        over_vals.append(e)
    extra = None
    if over_rows:
        dt = model.embed_tokens.dtype
        extra = (torch.cat(over_rows), torch.cat([v.to(dev, dt) for v in over_vals]))
    pv, grid = proc.patchify(images_u8, model.embed_tokens.dtype)
    if proc.prismatic is None:
        positions = torch.cat([proc.rope_layout(len(p), A + E)[0] for p in prompts], 1).to(dev)
    else:
        positions = info.positions
    hidden = model.forward_hidden(ids, positions, info, pixel_values=pv, image_grid_thw=grid,
                                  image_mask=proc.image_mask(first, ids.shape[0]), zero_mask=zero_mask,
                                  extra_embeds=extra)
    return hidden.index_select(0, act_rows).reshape(N, A, -1)


def oft_continuous_actions(model, proc: "VLAProcessor", prompts: Sequence[Sequence[int]], images_u8: torch.Tensor,
                           action_head, chunk_len: int, proprio: Optional[torch.Tensor] = None, proprio_projector=None,
                           norm_stats: Optional[dict] = None, norm_type: str = "bounds_q99") -> torch.Tensor:
    """L1-regression prediction of one control step: ``[N, chunk_len, action_dim]`` actions, un-normalised with the
    dataset statistics when ``norm_stats`` is given (the reference: ``_regression_or_discrete_prediction`` with an
    ``action_head``, then ``_unnormalize_actions``; modeling_prismatic.py:1485-1550, 1378-1397)."""
    from .action_heads import unnormalize_actions
    with torch.no_grad():
        h = oft_action_hidden(model, proc, prompts, images_u8, chunk_len * action_head.action_dim, proprio,
                              proprio_projector)
        a = action_head.predict_action(h).float()
    return unnormalize_actions(a, norm_stats, norm_type) if norm_stats is not None else a.cpu()


def oft_diffusion_actions(model, proc: "VLAProcessor", prompts: Sequence[Sequence[int]], images_u8: torch.Tensor,
                          head, chunk_len: int, proprio: Optional[torch.Tensor] = None, proprio_projector=None,
                          norm_stats: Optional[dict] = None, norm_type: str = "bounds_q99",
                          generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """Diffusion prediction of one control step: start from Gaussian noise ``[N, chunk_len, action_dim]`` and run the
    head's reverse steps; every step is one decoder forward whose action rows carry the projected noisy actions and
    whose timestep embedding sits behind the patches (the reference: ``_run_diffusion_prediction``,
    modeling_prismatic.py:1399-1483)."""
    from .action_heads import unnormalize_actions
    N, adim = len(prompts), head.action_dim
    x = torch.randn(N, chunk_len, adim, generator=generator)
    with torch.no_grad():
        for t, t_prev in head.schedule.inference_steps(head.num_inference_steps):
            h = oft_action_hidden(model, proc, prompts, images_u8, chunk_len * adim, proprio, proprio_projector,
                                  pseudo_tokens=[head.time_embedding(torch.full((N,), t))],
                                  action_embeds=head.project_noisy_actions(x))
            x = head.schedule.step(head.predict_noise(h).float().cpu(), t, t_prev, x)
    return unnormalize_actions(x, norm_stats, norm_type) if norm_stats is not None else x
