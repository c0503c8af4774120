"""Role-level workers: actor / rollout / reference (hybrid engine), critic, reward model.

Public methods are the reference's worker API (siirl/engine/fsdp_workers.py:1152-1499, 1713-1815, 2058):
``init_model``, ``generate_sequences``, ``compute_log_prob``, ``compute_ref_log_prob``, ``update_actor``,
``compute_values``, ``update_critic``, ``compute_rm_score``, ``save_checkpoint``, ``load_checkpoint``.

What is different underneath: the model is this framework's packed decoder on sm_100a kernels; parameters live in a
:class:`FlatParamStore` (replicated bf16 working copy, sharded fp32 master + Adam state); rollout is the native
paged-KV engine that reads the actor's weights in place (weight "resync" is free when rollout TP = 1 and one
fused regather kernel otherwise); batches stay on the GPU between calls — the reference moves every batch
GPU->CPU->GPU around each worker call (fsdp_workers.py:1271-1347).
"""
from __future__ import annotations

import math
import os
import time
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

from ..dag_worker import core_algos
from ..data_coordinator.protocol import Batch
from ..models.config import DecoderConfig, get_config
from ..models.decoder import DecoderLM, build_model
from ..parallel.flat_params import FlatParamStore, lr_at_step
from ..utils.model_utils.seqlen_balancing import rearrange_micro_batches
from .packing import PackedBatch, get_response_mask, pack_batch, position_ids_from_mask
from .rollout.native_engine import RolloutEngine, SamplingParams

_DTYPES = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32, "bf16": torch.bfloat16,
           "fp32": torch.float32}


def resolve_model_config(model_args, value_head: bool = False) -> DecoderConfig:
    name = model_args.arch_preset or model_args.path
    cfg = get_config(name, dict(model_args.override_config or {}))
    if value_head:
        cfg.value_head = True
        cfg.tie_word_embeddings = False
    if int(getattr(model_args, "lora_rank", 0) or 0) > 0:
        cfg.lora_rank, cfg.lora_alpha = int(model_args.lora_rank), float(model_args.lora_alpha)
        cfg.lora_targets = lora_targets(getattr(model_args, "target_modules", "all-linear"))
    return cfg


def lora_targets(target_modules) -> Optional[tuple]:
    """peft-style ``target_modules`` ("all-linear" or names such as ``q_proj``, ``up_proj``; the reference passes them
    to peft, siirl/engine/fsdp_workers.py:516,890) -> the fused projections that get an adapter.  q / k / v share one
    fused projection here, as do gate / up: naming any member adapts the fused matrix.  ``None``: all four."""
    if target_modules is None or target_modules == "all-linear":
        return None
    names = [target_modules] if isinstance(target_modules, str) else list(target_modules)
    names = [n.strip(" []'\"") for s_ in names for n in str(s_).split(",")]     # also a list that arrived as text
    names = [n for n in names if n]
    if names == ["all-linear"]:
        return None
    fused = {"q_proj": "qkv_proj", "k_proj": "qkv_proj", "v_proj": "qkv_proj", "qkv_proj": "qkv_proj",
             "o_proj": "o_proj", "gate_proj": "gate_up_proj", "up_proj": "gate_up_proj",
             "gate_up_proj": "gate_up_proj", "down_proj": "down_proj"}
    unknown = [n for n in names if n not in fused]
    if unknown:
        raise ValueError(f"model.target_modules: unknown projection(s) {unknown} (known: {sorted(fused)} or 'all-linear')")
    out = tuple(k for k in ("qkv_proj", "o_proj", "gate_up_proj", "down_proj") if k in {fused[n] for n in names})
    return out or None


def _micro_batches(batch: Batch, micro_bs: Optional[int], use_dynamic: bool, max_tokens: int, group=None):
    """Yield ``(index list, micro batch)`` pairs."""
    if use_dynamic:
        lens = batch["attention_mask"].sum(-1).tolist()
        parts = rearrange_micro_batches(lens, max_tokens, dp_group=group)
    else:
        bs = batch.batch_size
        micro_bs = micro_bs or bs
        parts = [list(range(s, min(s + micro_bs, bs))) for s in range(0, bs, micro_bs)]
    return [(p, batch.select_idxs(p)) for p in parts]


class _GroupSum(torch.autograd.Function):
    """Sum over a process group whose backward is the same sum (all ranks evaluate the same function of the
    result)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        y = x.clone()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, dy):
        g = dy.clone()
        dist.all_reduce(g, group=ctx.group)
        return g, None


def _group_sum(x: torch.Tensor, group) -> torch.Tensor:
    return _GroupSum.apply(x, group)


class _ModelWorkerBase:
    def __init__(self, config, role: str, process_group=None, device: Optional[torch.device] = None, comm=None,
                 seed: int = 1):
        self.config = config
        self.role = role
        self.group = process_group
        self.comm = comm
        self.seed = seed
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else \
                torch.device("cpu")
        self.device = torch.device(device)
        self.world = dist.get_world_size(process_group) if (dist.is_available() and dist.is_initialized()) else 1
        self.rank = dist.get_rank(process_group) if self.world > 1 else 0
        self.model: Optional[DecoderLM] = None
        self.store: Optional[FlatParamStore] = None
        self.opt_step = 0
        self.total_training_steps = 0

    def _dtype(self, model_args) -> torch.dtype:
        if self.device.type == "cpu":
            return torch.float32
        return _DTYPES.get(model_args.fsdp_config.model_dtype, torch.bfloat16)

    def _build(self, model_args, value_head: bool, trainable: bool, seed_offset: int = 0) -> None:
        mcfg = resolve_model_config(model_args, value_head)
        ep = int(getattr(getattr(self.config, "actor", self.config).megatron, "expert_model_parallel_size", 1) or 1) \
            if mcfg.is_moe else 1
        if ep > 1:
            if ep != self.world:
                raise ValueError(f"expert_model_parallel_size={ep} must equal the worker group size {self.world}")
            mcfg.ep_size, mcfg.ep_rank = ep, self.rank
        self.model_config = mcfg
        self.model = build_model(mcfg, dtype=self._dtype(model_args), device=self.device,
                                 seed=self.seed + seed_offset,
                                 gradient_checkpointing=model_args.enable_gradient_checkpointing and trainable)
        path = model_args.path
        if path and not model_args.random_init and not model_args.arch_preset:
            from ..models.hf_io import load_hf_weights
            load_hf_weights(self.model, path)
        if ep > 1:
            self._attach_expert_parallel(model_args)
        self._attach_tensor_parallel(self.model)
        pp_filter = self._attach_pipeline_parallel(self.model, trainable)
        self._attach_sequence_parallel(self.model)
        self._attach_context_parallel(self.model)
        if trainable and getattr(model_args, "enable_activation_offload", False) and self.device.type == "cuda":
            from ..utils.model_utils.activation_offload import ActivationOffload
            self.model.activation_offload = ActivationOffload()
        if trainable and ep > 1:
            from ..parallel.flat_params import ExpertSplitStore
            self.store = ExpertSplitStore(self.model, group=self.group, comm=self.comm)
        elif trainable and mcfg.lora_rank > 0:
            # only the adapters train: base weights stay out of the gradient / optimizer buffers
            for n, p in self.model.named_parameters():
                if "_lora_" not in n:
                    p.requires_grad_(False)
            self.store = FlatParamStore(self.model, group=self.group, comm=self.comm,
                                        param_filter=lambda n: "_lora_" in n)
        elif trainable and pp_filter is not None:
            # gradients and optimizer state only for this stage's parameters; data parallelism across pipelines
            self.store = FlatParamStore(self.model, group=self._pp_dp_group, comm=None, param_filter=pp_filter)
        elif trainable and self._zero3():
            self.store = self._shard_params(self.model, model_args, trainable=True)
        elif trainable and self._hybrid_shard_groups()[0] is not None:
            sg, rg, sc = self._hybrid_shard_groups()
            self.store = FlatParamStore(self.model, group=sg, comm=sc, replica_group=rg)
        elif trainable and getattr(self, "_tp_train", None) is not None:
            # tensor-parallel trainer: every rank owns its slices; gradients and optimizer state are shared with the
            # ranks that hold the same slices (same index in their tensor-parallel group)
            self.store = FlatParamStore(self.model, group=self._tp_dp_group, comm=self._tp_dp_comm)
        elif trainable:
            self.store = FlatParamStore(self.model, group=self.group, comm=self.comm)
        else:
            for p in self.model.parameters():
                p.requires_grad_(False)

    def _zero3(self) -> bool:
        """``fsdp_config.sharding=zero3``: parameters, gradients and optimizer state sharded over the worker group
        (FSDP FULL_SHARD of the reference); ``zero2`` (default) keeps a bf16 replica of the parameters per rank."""
        cfgs = getattr(self.config, "actor", self.config)
        fc = getattr(cfgs, "fsdp_config", None)
        return str(getattr(fc, "sharding", "zero2")).lower() in ("zero3", "full_shard", "fsdp")

    def _hybrid_shard_groups(self):
        """``fsdp_config.fsdp_size`` = k with 1 < k < group size: hybrid sharding (FSDP HYBRID_SHARD,
        siirl/engine/fsdp_workers.py:151-156).  Consecutive blocks of k ranks shard the training state; the ranks with
        the same index across blocks hold the same shard and sum their gradients.  Returns (shard group, replica
        group, peer-memory communicator of the shard group), all None when the whole group shards.  Every rank
        creates all groups in the same order (``new_group`` is collective)."""
        if getattr(self, "_hsdp", None) is not None:
            return self._hsdp
        cfgs = getattr(self.config, "actor", self.config)
        fc = getattr(cfgs, "fsdp_config", None)
        k = int(getattr(fc, "fsdp_size", -1) or -1)
        self._hsdp = (None, None, None)
        if k <= 1 or k >= self.world or self.world <= 1:
            return self._hsdp
        if self.world % k:
            raise ValueError(f"fsdp_config.fsdp_size={k} must divide the worker group size {self.world}")
        if any(getattr(self, a, None) is not None for a in ("_tp_train", "_pp_ctx", "ep_ctx")):
            raise ValueError("fsdp_config.fsdp_size (hybrid sharding) cannot be combined with tensor / pipeline / "
                             "expert parallel training")
        ranks = dist.get_process_group_ranks(self.group) if self.group is not None else list(range(self.world))
        shard = rep = None
        for b in range(self.world // k):
            g = dist.new_group(ranks[b * k:(b + 1) * k])
            if b == self.rank // k:
                shard = g
        for i in range(k):
            g = dist.new_group(ranks[i::k])
            if i == self.rank % k:
                rep = g
        comm = None
        if self.device.type == "cuda":
            from ..parallel.symm import SymmComm
            comm = SymmComm.create(shard)
        self._hsdp = (shard, rep, comm)
        return self._hsdp

    def _shard_params(self, model, model_args, trainable: bool):
        from ..parallel.sharded_params import ShardedParamStore
        mc = self.model_config
        if mc.is_moe or mc.lora_rank > 0 or getattr(self, "_pp_ctx", None) is not None:
            raise ValueError("fsdp_config.sharding=zero3 supports dense models without LoRA or pipeline parallelism; "
                             "use zero2 (replicated bf16 weights, sharded optimizer state) for those")
        if trainable and not model.gradient_checkpointing:
            raise ValueError("fsdp_config.sharding=zero3 needs model.enable_gradient_checkpointing=True: a layer's "
                             "weights are regathered for its backward pass, which recomputes the layer")
        if not trainable:
            for p in model.parameters():
                p.requires_grad_(False)
        sg, rg, sc = self._hybrid_shard_groups()
        if sg is not None:
            return ShardedParamStore(model, group=sg, comm=sc, optimizer_state=trainable, trainable=trainable,
                                     replica_group=rg)
        return ShardedParamStore(model, group=self.group, comm=self.comm if self.device.type == "cuda" else None,
                                 optimizer_state=trainable, trainable=trainable)

    def _phase_sync(self) -> None:
        """Align the ranks of the worker group before a phase whose kernels wait on peers with a short bound (tensor /
        expert / sequence parallel exchanges): the previous phase may have left them seconds apart."""
        if self.world > 1 and any(getattr(self, a, None) is not None for a in ("tp_model", "ep_ctx", "_sp_ctx", "_cp_ctx", "_pp_ctx", "_tp_train")):
            if getattr(self, "_sync_word", None) is None:
                self._sync_word = torch.zeros(1, device=self.device)
            dist.all_reduce(self._sync_word, group=self.group)

    def _vl_processor(self):
        if getattr(self, "_vlp", None) is None:
            from ..models.vision_processor import make_vl_processor
            self._vlp = make_vl_processor(self.model_config, self.config.model.image_min_pixels,
                                          self.config.model.image_max_pixels)
        return self._vlp

    def _train_tp_size(self) -> int:
        cfgs = getattr(self.config, "actor", self.config)
        mg = getattr(cfgs, "megatron", None)
        if str(getattr(cfgs, "strategy", "fsdp")) != "megatron" or mg is None:
            return 1
        return max(1, int(mg.tensor_model_parallel_size or 1))

    def _attach_tensor_parallel(self, model) -> None:
        """Megatron-style tensor (and sequence) parallel training (``strategy=megatron``,
        ``megatron.tensor_model_parallel_size``, ``megatron.sequence_parallel``): consecutive blocks of ``tp`` ranks
        form a tensor-parallel group, the ranks with the same index across blocks the data-parallel group of those
        slices.  Every rank of the job creates all groups in the same order (``new_group`` is collective)."""
        n = self._train_tp_size()
        if n <= 1 or self.world <= 1:
            return
        cfgs = getattr(self.config, "actor", self.config)
        if getattr(self, "_tp_train", None) is None:
            from ..parallel.megatron_tp import TPTrainContext
            if self.world % n:
                raise ValueError(f"megatron.tensor_model_parallel_size={n} must divide the group size {self.world}")
            for name in ("ulysses_sequence_parallel_size",):
                if int(getattr(cfgs, name, 1) or 1) > 1:
                    raise ValueError("tensor-parallel training cannot be combined with Ulysses sequence parallelism")
            mg = cfgs.megatron
            if int(mg.pipeline_model_parallel_size or 1) > 1 or int(mg.context_parallel_size or 1) > 1:
                raise ValueError("tensor-parallel training cannot be combined with pipeline / context parallelism yet")
            ranks = dist.get_process_group_ranks(self.group) if self.group is not None else list(range(self.world))
            mine = dp = None
            for b in range(self.world // n):
                g = dist.new_group(ranks[b * n:(b + 1) * n])
                if b == self.rank // n:
                    mine = g
            for i in range(n):
                g = dist.new_group(ranks[i::n])
                if i == self.rank % n:
                    dp = g
            self._tp_train = TPTrainContext(mine, sequence_parallel=bool(mg.sequence_parallel))
            self._tp_train_size = n
            self._tp_dp_group = dp
            self._tp_dp_comm = None
            if self.device.type == "cuda" and self.world // n > 1:
                from ..parallel.symm import SymmComm
                self._tp_dp_comm = SymmComm.create(dp)
        from ..parallel.megatron_tp import shard_decoder
        shard_decoder(model, self._tp_train)

    def _attach_sequence_parallel(self, model) -> None:
        """Ulysses groups are consecutive blocks of ``ulysses_sequence_parallel_size`` ranks of the worker's group;
        every rank creates all of them in the same order (``new_group`` is collective)."""
        cfgs = getattr(self.config, "actor", self.config)
        n = int(getattr(cfgs, "ulysses_sequence_parallel_size", 1) or 1)
        if n <= 1 or self.world <= 1:
            return
        if getattr(self, "_sp_ctx", None) is None:
            from ..parallel.ulysses import UlyssesSP
            mc = self.model_config
            if self.world % n or mc.num_heads % n or mc.num_kv_heads % n:
                raise ValueError(f"ulysses_sequence_parallel_size={n} must divide the group size {self.world} and the "
                                 f"head counts {mc.num_heads}/{mc.num_kv_heads}")
            ranks = dist.get_process_group_ranks(self.group) if self.group is not None else list(range(self.world))
            mine = None
            for b in range(self.world // n):
                g = dist.new_group(ranks[b * n:(b + 1) * n])
                if b == self.rank // n:
                    mine = g
            comm = None
            if self.device.type == "cuda":
                from ..parallel.symm import SymmComm
                comm = SymmComm.create(mine)
            r = getattr(self.config, "rollout", None)
            seq = ((r.prompt_length or 512) + (r.response_length or 512)) if r is not None else 4096
            tokens = max(int(getattr(cfgs, "ppo_max_token_len_per_gpu", 0) or 0),
                         int(getattr(cfgs, "ppo_micro_batch_size_per_gpu", 0) or 1) * seq, seq)
            width = (mc.num_heads + 2 * mc.num_kv_heads) * mc.head_dim
            self._sp_ctx = UlyssesSP(mine, comm, max_elems=(tokens // n + n) * width)
        model.attach_sequence_parallel(self._sp_ctx)

    def _attach_pipeline_parallel(self, model, trainable: bool):
        """Pipeline groups are consecutive blocks of ``megatron.pipeline_model_parallel_size`` ranks; the ranks with
        the same stage index across blocks form the stage's data-parallel group.  Returns the parameter filter of the
        stage (or ``None`` without pipeline parallelism)."""
        cfgs = getattr(self.config, "actor", self.config)
        n = int(getattr(getattr(cfgs, "megatron", None), "pipeline_model_parallel_size", 1) or 1)
        if n <= 1 or self.world <= 1:
            return None
        if getattr(self, "_pp_ctx", None) is None:
            from ..parallel.pipeline import PipelineContext
            if self.world % n:
                raise ValueError(f"pipeline_model_parallel_size={n} must divide the group size {self.world}")
            ranks = dist.get_process_group_ranks(self.group) if self.group is not None else list(range(self.world))
            virtual = int(getattr(cfgs.megatron, "virtual_pipeline_model_parallel_size", None) or 1)
            if virtual > 1 and self.model_config.num_layers < n * virtual:
                raise ValueError(f"virtual_pipeline_model_parallel_size={virtual} x pipeline_model_parallel_size={n} "
                                 f"exceeds the {self.model_config.num_layers} layers of the model")
            mine = dp = fwd = bwd = wfwd = wbwd = None
            for b in range(self.world // n):
                g = dist.new_group(ranks[b * n:(b + 1) * n])
                gf = dist.new_group(ranks[b * n:(b + 1) * n])      # activations
                gb = dist.new_group(ranks[b * n:(b + 1) * n])      # activation gradients
                # interleaved schedule: the link that closes the ring (last stage -> first stage) in both directions
                wf = dist.new_group(ranks[b * n:(b + 1) * n]) if virtual > 1 else None
                wb = dist.new_group(ranks[b * n:(b + 1) * n]) if virtual > 1 else None
                if b == self.rank // n:
                    mine, fwd, bwd, wfwd, wbwd = g, gf, gb, wf, wb
            for s_ in range(n):
                g = dist.new_group(ranks[s_::n])
                if s_ == self.rank % n:
                    dp = g
            self._pp_ctx = PipelineContext(mine, self.model_config.num_layers, fwd, bwd, virtual=virtual,
                                           wrap_fwd_group=wfwd, wrap_bwd_group=wbwd)
            self._pp_dp_group = dp
        model.attach_pipeline_parallel(self._pp_ctx)
        pc = self._pp_ctx
        if trainable:
            for name, p in model.named_parameters():
                if not pc.owns_param(name):
                    p.requires_grad_(False)
        return pc.owns_param

    def _attach_context_parallel(self, model) -> None:
        """Ring (context-parallel) attention groups: consecutive blocks of ``megatron.context_parallel_size`` ranks."""
        cfgs = getattr(self.config, "actor", self.config)
        n = int(getattr(getattr(cfgs, "megatron", None), "context_parallel_size", 1) or 1)
        if n <= 1 or self.world <= 1:
            return
        if getattr(self, "_sp_ctx", None) is not None:
            raise ValueError("context parallelism and Ulysses sequence parallelism cannot be combined")
        if getattr(self, "_cp_ctx", None) is None:
            from ..parallel.ring_attention import RingContext
            mc = self.model_config
            if self.world % n:
                raise ValueError(f"context_parallel_size={n} must divide the group size {self.world}")
            ranks = dist.get_process_group_ranks(self.group) if self.group is not None else list(range(self.world))
            mine = None
            for b in range(self.world // n):
                g = dist.new_group(ranks[b * n:(b + 1) * n])
                if b == self.rank // n:
                    mine = g
            comm = None
            if self.device.type == "cuda":
                from ..parallel.symm import SymmComm
                comm = SymmComm.create(mine)
            r = getattr(self.config, "rollout", None)
            seq = ((r.prompt_length or 512) + (r.response_length or 512)) if r is not None else 4096
            tokens = max(int(getattr(cfgs, "ppo_max_token_len_per_gpu", 0) or 0),
                         int(getattr(cfgs, "ppo_micro_batch_size_per_gpu", 0) or 1) * seq, seq)
            rows = tokens // n + 128 * n
            layout = str(getattr(cfgs.megatron, "context_parallel_layout", "zigzag") or "zigzag")
            if layout not in ("zigzag", "contiguous"):
                raise ValueError(f"context_parallel_layout={layout!r}: expected 'zigzag' or 'contiguous'")
            self._cp_ctx = RingContext(mine, comm, max_rows=rows,
                                       qkv_width=(mc.num_heads + 2 * mc.num_kv_heads) * mc.head_dim,
                                       kv_width=2 * mc.num_kv_heads * mc.head_dim, zigzag=layout == "zigzag")
        model.attach_context_parallel(self._cp_ctx)

    def _attach_expert_parallel(self, model_args) -> None:
        """One ExpertParallel context per worker (staging buffers sized for the largest packed forward); every MoE
        layer pads its tokens to the same static bound so that ranks with different batches agree on shapes."""
        from ..ops.moe import ExpertParallel
        cfg = self.model_config
        bound = int(getattr(model_args, "ep_max_tokens", 0) or 0) or 8192
        width = max(cfg.hidden_size, 2 * cfg.moe_intermediate_size)
        slots = self.world * bound * cfg.num_experts_per_tok + (cfg.num_experts // self.world + 1) * 128
        ctx = ExpertParallel(self.group, self.comm if self.device.type == "cuda" else None, max_tokens=bound,
                             hidden=width, max_slots=slots)
        for layer in self.model.layers:
            layer.ep, layer.ep_pad_tokens = ctx, bound
        self.ep_ctx = ctx

    # ---- shared forward ---------------------------------------------------------------------------
    def _pack(self, mb: Batch) -> PackedBatch:
        R = mb["responses"].shape[1]
        return pack_batch(mb["input_ids"].to(self.device), mb["attention_mask"].to(self.device), R)

    def _forward_logprob(self, model: DecoderLM, mb: Batch, temperature: float, with_entropy: bool):
        pk = self._pack(mb)
        positions, mm = pk.positions, {}
        if "images" in mb:                  # embodied rows: one policy image per row, multimodal rope layout
            proc = self.vla_processor
            pv, grid = proc.patchify(mb["images"].to(self.device), model.embed_tokens.dtype)
            first = torch.tensor(pk.info.cu_seqlens_cpu[:-1], device=self.device)
            img_mask = proc.image_mask(first, pk.input_ids.shape[0])
            mm = {"pixel_values": pv, "image_grid_thw": grid, "image_mask": img_mask}
            positions = torch.cat([proc.rope_layout(n)[0] for n in pk.info.seqlens], 1).to(self.device)
            from ..models.embodied.vla import action_id_range, oft_action_logits, uses_parallel_decode
            if uses_parallel_decode(self.config.embodied, self.model_config):
                # OpenVLA-OFT: the action positions enter as zero vectors and are scored where they stand, over
                # the action bins only (reference: siirl/engine/actor/embodied_actor.py:137-148)
                act_rows = pk.sel + 1
                zero_mask = torch.zeros(pk.input_ids.shape[0], dtype=torch.bool, device=self.device)
                zero_mask[act_rows] = True
                hidden = model.forward_hidden(pk.input_ids, positions, pk.info, zero_mask=zero_mask, **mm)
                logits = oft_action_logits(model, hidden.index_select(0, act_rows), temperature)
                logp = torch.log_softmax(logits, -1)
                lo, hi = action_id_range(self.model_config)
                lp = logp.gather(1, (pk.labels - lo).clamp(0, hi - lo - 1)[:, None])[:, 0]
                ent = -(logp.exp() * logp).sum(-1) if with_entropy else None
                return pk.scatter(lp), (pk.scatter(ent) if ent is not None else None)
        if "multi_modal_inputs" in mb.non_tensors:
            # vision-language rows: patches of all rows in row order; placeholders are the image-token ids of the
            # PROMPT part only (a sampled response token may collide with the placeholder id); 3-row rope positions
            proc = self._vl_processor()
            mmi = mb.non_tensors["multi_modal_inputs"]
            R = mb["responses"].shape[1]
            am = mb["attention_mask"].to(self.device).bool()
            in_prompt = torch.zeros_like(am)
            in_prompt[:, : am.shape[1] - R] = True
            ids2d = mb["input_ids"].to(self.device)
            img_mask = ((ids2d == self.model_config.image_token_id) & in_prompt)[am]
            pos_rows = []
            for i in range(ids2d.shape[0]):
                pos_rows.append(proc.rope(ids2d[i][am[i]].cpu(), mmi[i]["image_grid_thw"])[0])
            positions = torch.cat(pos_rows, 1).to(self.device)
            mm = {"pixel_values": torch.cat([m["pixel_values"] for m in mmi]).to(self.device, model.embed_tokens.dtype),
                  "image_grid_thw": torch.cat([m["image_grid_thw"] for m in mmi]), "image_mask": img_mask}
        from ..ops.lm_head import lm_head_logprob_entropy
        pc = getattr(model, "pp", None)
        if pc is not None and pc.pp > 1:
            # pipeline parallel: this rank runs its stage; the last stage scores, every stage receives the values,
            # and a non-last stage ties them to the handle whose backward pulls the activation gradient
            from ..parallel import pipeline as P
            stage_local = getattr(self, "_pp_stage_local", False)
            if stage_local:
                # pipelined training: the schedule names the local model chunk of this call
                chunk = int(getattr(self, "_pp_chunk", 0))
                hidden, handle = model.forward_hidden_pp(pk.input_ids, positions, pk.info, chunk=chunk)
                scores_here = pc.chunk_is_last(chunk)
            else:
                # one micro-batch at a time: the stage runs its chunks in turn (the ring of stages once per chunk)
                assert pc.virtual == 1 or not torch.is_grad_enabled(), \
                    "virtual pipeline stages with gradients run under the interleaved schedule only"
                for chunk in range(pc.virtual):
                    hidden, handle = model.forward_hidden_pp(pk.input_ids, positions, pk.info, chunk=chunk)
                scores_here = pc.is_last
            N = pk.sel.shape[0]
            lp_l = ent_l = None
            if scores_here:
                lp_l, ent_l = lm_head_logprob_entropy(hidden.index_select(0, pk.sel), model.head_weight, pk.labels,
                                                      temperature, with_entropy)
            if stage_local:
                # nothing is broadcast per micro-batch; the last chunk of the model holds the values, every other
                # chunk only the handle whose backward receives the activation gradient
                if scores_here:
                    return pk.scatter(lp_l), (pk.scatter(ent_l) if ent_l is not None else None)
                return handle, None
            vals = P.broadcast_from_last(pc, [lp_l] + ([ent_l] if with_entropy else []), [(N,)] * (2 if with_entropy
                                         else 1), [torch.float32] * 2, self.device)
            lp = lp_l if pc.is_last else vals[0]
            ent = (ent_l if pc.is_last else vals[1]) if with_entropy else None
            if handle is not None:
                lp = lp + 0.0 * handle
            return pk.scatter(lp), (pk.scatter(ent) if ent is not None else None)
        hidden = model.forward_hidden(pk.input_ids, positions, pk.info, **mm)
        loc = model.local_row_index(pk.info, pk.input_ids.shape[0]) if hasattr(model, "local_row_index") else None
        if loc is not None:
            # sequence / context parallelism: this rank computed only the rows listed in ``loc``.  Score the selected
            # positions that fall there and let a differentiable sum over the group complete the [B, R] tensors
            # (every rank then evaluates the same loss; the backward of the sum returns each rank the gradient of
            # its own entries, once per rank of the group)
            group = (getattr(model, "sp", None) or getattr(model, "cp", None)).group
            T = pk.input_ids.shape[0]
            inv = torch.full((T,), -1, dtype=torch.int64, device=self.device)
            valid = loc >= 0
            inv[loc[valid]] = torch.arange(loc.shape[0], device=self.device)[valid]
            where = inv[pk.sel]
            idx = (where >= 0).nonzero(as_tuple=True)[0]
            lp_l, ent_l = lm_head_logprob_entropy(hidden.index_select(0, where[idx]), model.head_weight,
                                                  pk.labels[idx], temperature, with_entropy)
            N = pk.sel.shape[0]
            lp = _group_sum(torch.zeros(N, dtype=lp_l.dtype, device=lp_l.device).index_put((idx,), lp_l), group)
            ent = None
            if ent_l is not None:
                ent = _group_sum(torch.zeros(N, dtype=ent_l.dtype, device=ent_l.device).index_put((idx,), ent_l),
                                 group)
            return pk.scatter(lp), (pk.scatter(ent) if ent is not None else None)
        lp, ent = model.token_logprobs(hidden.index_select(0, pk.sel), pk.labels, temperature, with_entropy)
        return pk.scatter(lp), (pk.scatter(ent) if ent is not None else None)

    def _optimizer_step(self, optim_cfg, grad_clip: float) -> torch.Tensor:
        megatron = str(getattr(getattr(self.config, "actor", self.config), "strategy", "")) == "megatron"
        lr = lr_at_step(optim_cfg, self.opt_step, max(self.total_training_steps, optim_cfg.total_training_steps),
                        megatron=megatron)
        if megatron:
            grad_clip = float(optim_cfg.clip_grad)             # the Megatron optimizer's own key (reference:
            #                                                    siirl/utils/megatron/optimizer.py, ``clip_grad``)
        if getattr(self, "_tp_train", None) is not None:
            from ..parallel.megatron_tp import allreduce_sequence_parallel_grads
            self.store.collect_grads()
            allreduce_sequence_parallel_grads(self.model, self._tp_train)
        norm = self.store.step(lr, tuple(optim_cfg.betas), 1e-8, optim_cfg.weight_decay, grad_clip)
        if getattr(self, "_pp_ctx", None) is not None:
            from ..parallel.pipeline import sync_stage_weights
            sync_stage_weights(self.model, self._pp_ctx)     # every replica gets the stages it does not train
        self.store.zero_grad()
        self.opt_step += 1
        self.last_lr = lr
        return norm

    # ---- checkpoints --------------------------------------------------------------------------------
    def save_checkpoint(self, local_path: str, hdfs_path: Optional[str] = None, global_step: int = 0,
                        max_ckpt_to_keep: Optional[int] = None, contents=None, async_save: bool = False):
        """Write this rank's shard files under ``local_path`` (and copy them to ``hdfs_path`` when given).  Returns a
        handle whose ``wait()`` must be called before the checkpoint is declared complete (asynchronous saves write
        in a background thread; reference API: siirl/engine/fsdp_workers.py:1452-1499)."""
        from ..utils.checkpoint.checkpoint_manager import ShardedCheckpointManager
        group = self.group
        if getattr(self, "_tp_train", None) is not None:
            # one sub-directory per tensor-parallel index: inside it the shards of that slice's data-parallel group
            local_path = os.path.join(local_path, f"tp_rank_{self._tp_train.rank}")
            hdfs_path = f"{hdfs_path.rstrip('/')}/tp_rank_{self._tp_train.rank}" if hdfs_path else None
            group = self._tp_dp_group
            contents = [c for c in (contents or ["model", "optimizer", "extra"]) if c != "hf_model"]
        return ShardedCheckpointManager(self.model, self.store, self.model_config, group=group, contents=contents,
                                        tokenizer=getattr(self, "tokenizer", None)).save(
            local_path, global_step, extra={"opt_step": self.opt_step}, max_ckpt_to_keep=max_ckpt_to_keep,
            async_save=async_save, hdfs_path=hdfs_path)

    def load_checkpoint(self, local_path: str, hdfs_path: Optional[str] = None,
                        del_local_after_load: bool = False) -> None:
        """Load from ``local_path``; when it does not exist and ``hdfs_path`` is given the directory is fetched from
        there first.  ``del_local_after_load`` removes the local copy afterwards (every rank has read its shard)."""
        import os
        import shutil

        from ..utils.checkpoint.checkpoint_manager import ShardedCheckpointManager
        group = self.group
        if getattr(self, "_tp_train", None) is not None:
            local_path = os.path.join(local_path, f"tp_rank_{self._tp_train.rank}")
            hdfs_path = f"{hdfs_path.rstrip('/')}/tp_rank_{self._tp_train.rank}" if hdfs_path else None
            group = self._tp_dp_group
        if hdfs_path and not os.path.isdir(local_path):
            from ..utils.extras import fs
            if self.rank == 0:
                fs.copy(hdfs_path, local_path)
            if self.world > 1:
                dist.barrier(group=self.group)
        ck = getattr(getattr(self.config, "actor", self.config), "checkpoint", None)
        extra = ShardedCheckpointManager(self.model, self.store, self.model_config, group=group).load(
            local_path, contents=list(ck.load_contents) if ck is not None and ck.load_contents is not None else None)
        if extra:
            self.opt_step = int(extra.get("opt_step", self.opt_step))
        if del_local_after_load:
            if self.world > 1:
                dist.barrier(group=self.group)
            if self.rank == 0:
                shutil.rmtree(local_path, ignore_errors=True)


class ActorRolloutRefWorker(_ModelWorkerBase):
    """One class for the roles actor, rollout, ref and their combinations (``actor_rollout_ref`` = hybrid)."""

    def __init__(self, config, role: str = "actor_rollout_ref", process_group=None, device=None, comm=None,
                 seed: int = 1, tokenizer=None):
        super().__init__(config, role, process_group, device, comm, seed)
        assert role in ("actor", "rollout", "ref", "actor_rollout", "actor_rollout_ref")
        self._is_actor = "actor" in role
        self._is_rollout = "rollout" in role
        self._is_ref = "ref" in role
        self.tokenizer = tokenizer
        self.ref_model: Optional[DecoderLM] = None
        self.engine: Optional[RolloutEngine] = None
        self._embodied = bool(getattr(config.actor, "embodied_type", None)) or str(config.rollout.name).startswith(
            "embodied")
        self.embodied_rollout = None
        self.vla_processor = None
        self._normalize_batch_sizes()

    def _normalize_batch_sizes(self) -> None:
        """Global mini-batch -> per-rank sample count (reference: fsdp_workers.py:211-235)."""
        a = self.config.actor
        n = self.config.rollout.n
        dp = max(self.world // max(a.ulysses_sequence_parallel_size, self._train_tp_size(), 1), 1)
        self.ppo_mini_batch_size = max(1, a.ppo_mini_batch_size * n // dp)
        micro = a.ppo_micro_batch_size_per_gpu
        if micro is None and a.ppo_micro_batch_size is not None:
            micro = max(1, a.ppo_micro_batch_size // dp)
        self.ppo_micro_batch_size = micro
        if micro is not None and not a.use_dynamic_bsz:
            if self.ppo_mini_batch_size % micro != 0:
                self.ppo_micro_batch_size = math.gcd(self.ppo_mini_batch_size, micro)
        r = self.config.rollout
        self.logprob_micro = r.log_prob_micro_batch_size_per_gpu or (
            max(1, r.log_prob_micro_batch_size // dp) if r.log_prob_micro_batch_size else micro)
        rf = self.config.ref
        self.ref_logprob_micro = rf.log_prob_micro_batch_size_per_gpu or (
            max(1, rf.log_prob_micro_batch_size // dp) if rf.log_prob_micro_batch_size else self.logprob_micro)

    # ---- init ---------------------------------------------------------------------------------------
    def init_model(self) -> None:
        margs = self.config.model
        if self._is_actor or self._is_rollout:
            self._build(margs, value_head=False, trainable=self._is_actor)
        if self._is_ref and self.model is not None and self.model_config.lora_rank > 0:
            pass        # the reference policy is the actor with its adapters switched off
        elif self._is_ref:
            mcfg = resolve_model_config(margs)
            self.ref_model = build_model(mcfg, dtype=self._dtype(margs), device=self.device, seed=self.seed)
            if margs.path and not margs.random_init and not margs.arch_preset:
                from ..models.hf_io import load_hf_weights
                load_hf_weights(self.ref_model, margs.path)
            for p in self.ref_model.parameters():
                p.requires_grad_(False)
            self._attach_tensor_parallel(self.ref_model)    # a tensor-parallel trainer scores with sliced weights too
            self.ref_store = None
            if self._zero3() and self.world > 1:
                self.ref_store = self._shard_params(self.ref_model, margs, trainable=False)
            self._attach_pipeline_parallel(self.ref_model, False)
            self._attach_sequence_parallel(self.ref_model)
            self._attach_context_parallel(self.ref_model)
            if self.config.ref.fsdp_config.param_offload and self.device.type == "cuda" and self.ref_store is None:
                from ..utils.model_utils.fsdp_utils import offload_model_to_cpu
                offload_model_to_cpu(self.ref_model)
            if self.model is None:
                self.model_config = mcfg
        if self._is_rollout:
            r = self.config.rollout
            max_len = r.max_model_len or ((r.prompt_length or 512) + (r.response_length or 512))
            if self._embodied:                      # image tokens + task text + one chunk of action tokens
                e = self.config.embodied
                if self.model_config.prismatic is not None:
                    per_image = self.model_config.prismatic.tokens_per_image + 1
                else:
                    v = self.model_config.vision
                    per_image = (e.policy_image_size // (v.patch_size * v.spatial_merge_size)) ** 2
                max_len = max(max_len, per_image * e.num_images_in_input + 64 + e.action_chunks_len * e.action_token_len)
            self.tp_model = None
            tp = max(1, int(r.tensor_model_parallel_size))
            self._full_weights(True)        # the engine (and its tensor-parallel slices) reads whole weights
            if getattr(self, "_tp_train", None) is not None and tp == 1:
                raise ValueError("a tensor-parallel trainer needs rollout.tensor_model_parallel_size equal to "
                                 "megatron.tensor_model_parallel_size (the engine runs on the trainer's slices)")
            if tp > 1:
                self.tp_model = self._build_tp_model(tp, r.max_num_batched_tokens)
            if str(r.name).lower() == "hf" or self.model_config.is_mla:
                # ``rollout.name=hf``: cache-free generation through the training forward (the reference's HF
                # rollout).  Multi-head latent attention has no paged-cache kernel: it decodes against a cache of
                # the compressed latents instead.
                if tp > 1:
                    raise ValueError("this rollout engine runs on whole weights: set "
                                     "rollout.tensor_model_parallel_size=1")
                if str(r.name).lower() != "hf":
                    from .rollout.latent_engine import LatentCacheEngine
                    ep = getattr(self, "ep_ctx", None) is not None and self.world > 1
                    self.engine = LatentCacheEngine(self.model, max_num_seqs=min(r.max_num_seqs, 1024),
                                                    max_model_len=max_len,
                                                    max_num_batched_tokens=r.max_num_batched_tokens,
                                                    lockstep_group=self.group if ep else None)
                else:
                    from .rollout.recompute_engine import RecomputeEngine
                    if getattr(self, "ep_ctx", None) is not None and self.world > 1:
                        raise ValueError("rollout.name=hf cannot run under expert parallelism: its ranks would run "
                                         "different numbers of forward passes around the experts' exchanges; use "
                                         "the default engine")
                    self.engine = RecomputeEngine(self.model, max_num_seqs=min(r.max_num_seqs, 1024),
                                                  max_model_len=max_len)
            else:
                self.engine = self._paged_engine(r, max_len)
            if r.free_cache_engine and self._is_actor and getattr(self, "store", None) is not None \
                    and getattr(r, "kv_borrow_grad_buffer", True) and hasattr(self.engine, "borrowed"):
                # the fp32 gradient buffer is idle (and zeroed again) between an optimizer step and the next backward,
                # exactly while the engine is awake: lend it to the KV arena
                self.engine.borrowed = self.store.flat_grad
            if r.free_cache_engine:
                self.engine.sleep()
                self._full_weights(False)
        if self._embodied:
            self._init_embodied()

    def _paged_engine(self, r, max_len: int):
        return RolloutEngine(self.tp_model or self.model, max_num_seqs=min(r.max_num_seqs, 1024),
                                        max_model_len=max_len,
                                        gpu_memory_utilization=r.gpu_memory_utilization,
                                        use_cuda_graph=not r.enforce_eager or self.device.type == "cuda",
                                        max_num_batched_tokens=r.max_num_batched_tokens,
                                        enable_chunked_prefill=bool(r.enable_chunked_prefill),
                                        enable_prefix_caching=bool(getattr(r, "enable_prefix_caching", True)),
                                        lockstep_group=self.group if getattr(self, "ep_ctx", None) is not None
                                        and self.world > 1 else None,
                                        **dict(r.engine_kwargs.native or {}))

    def _full_weights(self, on: bool) -> None:
        """Parameter-sharded actor: regather the shards into a whole replica for the rollout engine (the train ->
        rollout weight resync of the reference's sharding managers, siirl/engine/sharding_manager/fsdp_vllm.py:
        113-159) and give the memory back afterwards.  A no-op for replicated weights."""
        st = getattr(self, "store", None)
        if st is None or not hasattr(st, "materialize_full"):
            return
        if on:
            st.materialize_full()
        else:
            st.release_full()

    def _build_tp_model(self, tp: int, max_tokens: int):
        """Tensor-parallel rollout: consecutive blocks of ``tp`` ranks of the worker's group form one engine
        replica (rank layout [DP][TP], TP fastest).  Every rank of the job creates all TP groups in the same
        order (``new_group`` is collective)."""
        import torch.distributed as dist
        from ..models.tp_decoder import TPDecoder
        from ..parallel.tensor_parallel import TPContext
        if getattr(self, "_tp_train", None) is not None:
            # the trainer is tensor parallel already: the engine runs on the very same slices
            if tp != self._tp_train_size:
                raise ValueError(f"rollout.tensor_model_parallel_size={tp} must equal the trainer's "
                                 f"megatron.tensor_model_parallel_size={self._tp_train_size}")
            comm = None
            if self.device.type == "cuda":
                from ..parallel.symm import SymmComm
                comm = SymmComm.create(self._tp_train.group)
            H = self.model_config.hidden_size
            ctx = TPContext(self._tp_train.group, comm, max_rows=max(max_tokens, 256), max_cols=H,
                            max_tiles=((max(max_tokens, 256) + 127) // 128) * ((H + 127) // 128) + 8)
            self._tp_size = tp
            return TPDecoder(self.model, ctx, presharded=True)
        if self.world % tp:
            raise ValueError(f"rollout.tensor_model_parallel_size={tp} does not divide the group size {self.world}")
        ranks = dist.get_process_group_ranks(self.group) if self.group is not None else list(range(self.world))
        mine = None
        for b in range(self.world // tp):
            g = dist.new_group(ranks[b * tp:(b + 1) * tp])
            if b == self.rank // tp:
                mine = g
        comm = None
        if self.device.type == "cuda":
            from ..parallel.symm import SymmComm
            comm = SymmComm.create(mine)
        H = self.model_config.hidden_size
        ctx = TPContext(mine, comm, max_rows=max(max_tokens, 256), max_cols=H,
                        max_tiles=((max(max_tokens, 256) + 127) // 128) * ((H + 127) // 128) + 8)
        self._tp_size = tp
        return TPDecoder(self.model, ctx)

    def _init_embodied(self) -> None:
        """VLA processor (all roles) and the closed-loop environment rollout (rollout role)."""
        from ..models.embodied.vla import VLAProcessor
        emb = self.config.embodied
        tok = self.tokenizer
        if tok is None:
            from ..data_coordinator.dataloader.tokenizer import SyntheticTokenizer
            tok = SyntheticTokenizer(self.model_config.vocab_size)
        self.vla_processor = VLAProcessor(self.model_config, tok, image_size=emb.policy_image_size,
                                          center_crop=emb.center_crop, num_images=emb.num_images_in_input)
        if self._is_rollout:
            from .rollout.embodied_rollout import EmbodiedRollout
            embedder = None
            if emb.use_video_embedding:
                from ..utils.embodied.video_emb import VideoEmbedder
                embedder = VideoEmbedder(img_size=min(emb.embedding_img_size, 224), num_frames=emb.video_num_frames,
                                         device=self.device, dtype=self._dtype(self.config.model),
                                         checkpoint=emb.video_embedding_model_path or None)
            self.embodied_rollout = EmbodiedRollout(self.engine, self.model_config, tok, emb, self.device,
                                                    seed=self.config.rollout.seed + 104729 * self.rank,
                                                    video_embedder=embedder, model_path=self.config.model.path)

    # ---- rollout -------------------------------------------------------------------------------------
    @torch.no_grad()
    def generate_sequences(self, prompts: Batch) -> Batch:
        """Roll out responses.  Input: left-padded ``input_ids/attention_mask/position_ids`` ``[B, P]`` and
        ``raw_prompt_ids``; rows with equal ``uid`` that follow each other are samples of one prompt (prefilled
        once).  Output adds ``prompts, responses, input_ids [B, P+R], attention_mask, position_ids, response_mask,
        rollout_log_probs``."""
        r = self.config.rollout
        self._phase_sync()
        if self._is_actor and getattr(self, "store", None) is not None and \
                self.config.actor.fsdp_config.optimizer_offload:
            self.store.offload_state()          # Adam moments wait in pinned host memory until the next update
        self._full_weights(True)
        if getattr(self, "tp_model", None) is not None:
            self.tp_model.sync_weights()        # column-parallel copies follow the trained replica
        if self.embodied_rollout is not None and "task_id" in prompts:
            out = self.embodied_rollout.generate_sequences(prompts)
            if r.free_cache_engine:
                self.engine.sleep()
                self._full_weights(False)
            return out
        t0 = time.time()
        self.engine.wake_up()
        meta = prompts.meta
        validate = bool(meta.get("validate", False))
        do_sample = bool(meta.get("do_sample", r.do_sample))
        temperature, top_k, top_p = r.temperature, r.top_k, r.top_p
        if validate:
            v = r.val_kwargs
            temperature, top_k, top_p, do_sample = v.temperature, v.top_k, v.top_p, v.do_sample
        if not do_sample:
            temperature = 0.0
        R = int(meta.get("response_length", r.response_length))
        ids = prompts["input_ids"]
        B, P = ids.shape
        raw = prompts["raw_prompt_ids"] if "raw_prompt_ids" in prompts else [
            ids[i][prompts["attention_mask"][i].bool()].tolist() for i in range(B)]
        uid = prompts["uid"].tolist() if "uid" in prompts else list(range(B))
        groups: List[List[int]] = []
        for i in range(B):
            if groups and uid[groups[-1][0]] == uid[i] and list(raw[groups[-1][0]]) == list(raw[i]):
                groups[-1].append(i)
            else:
                groups.append([i])
        n = len(groups[0])
        uniform = all(len(g) == n for g in groups)
        eos = meta.get("eos_token_id", self.model_config.eos_token_id)
        pad = meta.get("pad_token_id", self.model_config.pad_token_id)
        sp = SamplingParams(n=n if uniform else 1, temperature=float(temperature), top_k=int(top_k),
                            top_p=float(top_p), max_new_tokens=R, eos_token_id=eos, ignore_eos=r.ignore_eos,
                            seed=(r.seed + 7919 * int(meta.get("global_steps", 0))
                                  + 104729 * (self.rank // getattr(self, "_tp_size", 1))) & 0x7FFFFFFF)
        firsts = [g[0] for g in groups] if uniform else list(range(B))
        mm_inputs = None
        if "multi_modal_inputs" in prompts.non_tensors:
            # image prompts: patches, grid and multimodal rope numbering of every prompt (decode continues at
            # prompt length - rope delta)
            proc = self._vl_processor()
            mm_inputs = []
            for i in firsts:
                mmi = prompts.non_tensors["multi_modal_inputs"][i]
                pos, delta = proc.rope(torch.tensor(list(raw[i])), mmi["image_grid_thw"])
                mm_inputs.append({"pixel_values": mmi["pixel_values"].to(self.model.embed_tokens.dtype),
                                  "image_grid_thw": mmi["image_grid_thw"], "rope_positions": pos, "rope_delta": delta})
        outs = self.engine.generate([list(raw[i]) for i in firsts], sp, mm_inputs=mm_inputs)
        order = [i for g in groups for i in g] if uniform else list(range(B))
        responses = torch.full((B, R), pad, dtype=torch.int64)
        logps = torch.zeros(B, R, dtype=torch.float32)
        for row, o in zip(order, outs):
            L = len(o.token_ids)
            responses[row, :L] = torch.tensor(o.token_ids, dtype=torch.int64)
            logps[row, :L] = torch.tensor(o.logprobs, dtype=torch.float32)
        dev = ids.device
        responses, logps = responses.to(dev), logps.to(dev)
        resp_mask = get_response_mask(responses, eos, dtype=torch.int64)
        lens = torch.tensor([len(o.token_ids) for o in outs], dtype=torch.int64)
        len_by_row = torch.zeros(B, dtype=torch.int64)
        len_by_row[torch.tensor(order)] = lens
        resp_mask = resp_mask * (torch.arange(R)[None, :] < len_by_row[:, None]).to(dev)
        attn = torch.cat([prompts["attention_mask"], resp_mask], dim=-1)
        out = Batch(dict(prompts.tensors), dict(prompts.non_tensors), dict(prompts.meta))
        out["prompts"] = ids
        out["responses"] = responses
        out["input_ids"] = torch.cat([ids, responses], dim=-1)
        out["attention_mask"] = attn
        out["position_ids"] = position_ids_from_mask(attn)
        out["response_mask"] = resp_mask
        out["rollout_log_probs"] = logps
        out.meta["timing_generate_s"] = time.time() - t0
        out.meta["total_output_tokens"] = int(lens.sum())
        out.meta["total_input_tokens"] = int(prompts["attention_mask"].sum())
        if r.free_cache_engine:
            self.engine.sleep()
            self._full_weights(False)
        return out

    # ---- scoring ----------------------------------------------------------------------------------------
    @torch.no_grad()
    def _logprob_pass(self, model: DecoderLM, data: Batch, micro: Optional[int], dynamic: bool, max_tokens: int,
                      with_entropy: bool):
        temperature = float(data.meta.get("temperature", self.config.rollout.temperature)) or 1.0
        if data["responses"].dim() == 3:    # embodied trajectories: score the executed calls, scatter back
            from .actor.embodied_actor import flatten_trajectories, scatter_steps
            Bt, L, _A = data["responses"].shape
            rows, bi, li = flatten_trajectories(data, int(data.meta.get("actions_per_call",
                                                                        self.config.embodied.action_chunks_len)))
            lp, ent = self._logprob_pass(model, rows, micro, dynamic, max_tokens, with_entropy)
            return scatter_steps(lp, bi, li, Bt, L), (scatter_steps(ent, bi, li, Bt, L) if ent is not None else None)
        B, R = data["responses"].shape
        lp_out = torch.zeros(B, R, dtype=torch.float32, device=self.device)
        ent_out = torch.zeros(B, R, dtype=torch.float32, device=self.device) if with_entropy else None
        model.eval()
        for idx, mb in _micro_batches(data, micro, dynamic, max_tokens, self.group):
            lp, ent = self._forward_logprob(model, mb, temperature, with_entropy)
            ii = torch.tensor(idx, device=self.device)
            lp_out[ii] = lp
            if ent_out is not None:
                ent_out[ii] = ent
        return lp_out, ent_out

    def compute_log_prob(self, data: Batch) -> Batch:
        r = self.config.rollout
        self._phase_sync()
        self._full_weights(False)       # sharded parameters: scoring gathers layer by layer
        lp, ent = self._logprob_pass(self.model, data, self.logprob_micro, r.log_prob_use_dynamic_bsz,
                                     r.log_prob_max_token_len_per_gpu, with_entropy=True)
        data["old_log_probs"] = lp
        data["entropys"] = ent
        m = data["response_mask"].to(ent.device).float()
        data.meta.setdefault("metrics", {})["actor/entropy"] = float((ent * m).sum() / m.sum().clamp(min=1))
        return data

    def compute_ref_log_prob(self, data: Batch) -> Batch:
        rf = self.config.ref
        self._phase_sync()
        model = self.ref_model if self.ref_model is not None else self.model
        lora_ref = self.ref_model is None and getattr(self.model_config, "lora_rank", 0) > 0
        offload = (self.ref_model is not None and rf.fsdp_config.param_offload and self.device.type == "cuda"
                   and getattr(self, "ref_store", None) is None)
        if lora_ref:
            model.set_lora_enabled(False)
        if offload:         # the frozen policy lives in pinned host memory between its scoring passes
            from ..utils.model_utils.fsdp_utils import load_model_to_gpu
            load_model_to_gpu(model)
        try:
            lp, _ = self._logprob_pass(model, data, self.ref_logprob_micro, rf.log_prob_use_dynamic_bsz,
                                       rf.log_prob_max_token_len_per_gpu, with_entropy=False)
        finally:
            if lora_ref:
                model.set_lora_enabled(True)
            if offload:
                from ..utils.model_utils.fsdp_utils import offload_model_to_cpu
                offload_model_to_cpu(model)
        data["ref_log_prob"] = lp
        return data

    # ---- training ------------------------------------------------------------------------------------------
    def update_actor(self, data: Batch) -> Dict[str, Any]:
        """PPO / GRPO policy update over ``ppo_epochs`` x mini-batches x micro-batches
        (reference: siirl/engine/actor/dp_actor.py:349-520).  Returns the metric dict."""
        a = self.config.actor
        t0 = time.time()
        self._phase_sync()
        self._full_weights(False)
        if hasattr(self.store, "reload_state"):
            self.store.reload_state(wait=False)     # parked Adam moments stream back while the micro-batches run
        self.model.train()
        temperature = float(data.meta.get("temperature", self.config.rollout.temperature)) or 1.0
        loss_mode = a.policy_loss.loss_mode if not a.use_cpgd_loss else "cpgd"
        policy_loss_fn = core_algos.get_policy_loss_fn(loss_mode)
        entropy_coeff = a.entropy_coeff
        need_entropy = entropy_coeff != 0
        metrics: Dict[str, List[float]] = {}
        bs = data.batch_size
        mini = min(self.ppo_mini_batch_size, bs)
        n_mini = max(1, bs // mini)
        if data["responses"].dim() == 3:    # embodied: executed calls become rows; same number of optimizer steps
            from .actor.embodied_actor import flatten_trajectories
            data, _, _ = flatten_trajectories(data, int(data.meta.get("actions_per_call",
                                                                      self.config.embodied.action_chunks_len)))
            bs = data.batch_size
            mini = -(-bs // n_mini)
            n_mini = max(1, -(-bs // mini))
        on_policy = a.ppo_epochs == 1 and n_mini == 1
        pc = getattr(self.model, "pp", None)
        pipelined = pc is not None and pc.pp > 1 and pc.pipelined
        self.store.zero_grad()
        for _epoch in range(a.ppo_epochs):
            order = torch.randperm(bs).tolist() if a.shuffle else list(range(bs))
            for mi in range(n_mini):
                mini_idx = order[mi * mini:(mi + 1) * mini]
                mini_batch = data.select_idxs(mini_idx)
                mbs = _micro_batches(mini_batch, self.ppo_micro_batch_size, a.use_dynamic_bsz,
                                     a.ppo_max_token_len_per_gpu, self.group)
                def micro_forward(idx, mb, chunk=0):
                    """Forward pass and loss of one micro-batch (of one local model chunk under the interleaved
                    pipeline schedule) -> (tensor to call ``backward`` on, metrics)."""
                    scale = (len(idx) / len(mini_idx)) if a.use_dynamic_bsz else 1.0 / len(mbs)
                    mask = mb["response_mask"].to(self.device).float()
                    adv = mb["advantages"].to(self.device).float()
                    self._pp_chunk = chunk
                    logp, ent = self._forward_logprob(self.model, mb, temperature, need_entropy)
                    if pipelined and not pc.chunk_is_last(chunk):
                        return logp, {}             # the chunk's handle: its backward receives dL/dh from the next stage
                    old = logp.detach() if on_policy else mb["old_log_probs"].to(self.device).float()
                    ref = mb["ref_log_prob"].to(self.device).float() if (a.use_kl_loss and "ref_log_prob" in mb) \
                        else None
                    is_w = mb["rollout_is_weights"].to(self.device) if "rollout_is_weights" in mb else None
                    fused = (logp.is_cuda and loss_mode in ("vanilla", "gspo", "cpgd") and is_w is None
                             and a.policy_drift_coeff == 0 and not a.kl_loss_type.endswith("+"))
                    if fused:
                        from ..ops.rl import ppo_token_loss
                        lo = a.clip_ratio_low if a.clip_ratio_low is not None else a.clip_ratio
                        hi = a.clip_ratio_high if a.clip_ratio_high is not None else a.clip_ratio
                        loss, mm = ppo_token_loss(logp, old, adv, mask, entropy=ent if need_entropy else None,
                                                  ref_logp=ref, mode=loss_mode, loss_agg_mode=a.loss_agg_mode,
                                                  clip_lo=lo, clip_hi=hi, clip_c=a.clip_ratio_c,
                                                  kl_kind=a.kl_loss_type, kl_coef=a.kl_loss_coef if ref is not None
                                                  else 0.0, entropy_coef=entropy_coeff)
                        rec = {"actor/pg_loss": mm["pg_loss"], "actor/pg_clipfrac": mm["pg_clipfrac"],
                               "actor/ppo_kl": mm["ppo_kl"], "actor/pg_clipfrac_lower": mm["pg_clipfrac_lower"]}
                        if ref is not None:
                            rec["actor/kl_loss"] = mm["kl_loss"]
                            rec["actor/kl_coef"] = torch.tensor(a.kl_loss_coef)
                        if need_entropy:
                            rec["actor/entropy_loss"] = mm["entropy_loss"]
                    else:
                        pg, clipfrac, ppo_kl, clip_lower = policy_loss_fn(old, logp, adv, mask, a.loss_agg_mode, a,
                                                                          is_w)
                        loss = pg
                        rec = {"actor/pg_loss": pg.detach(), "actor/pg_clipfrac": clipfrac.detach(),
                               "actor/ppo_kl": ppo_kl.detach(), "actor/pg_clipfrac_lower": clip_lower.detach()}
                        if need_entropy:
                            el = core_algos.agg_loss(ent, mask, a.loss_agg_mode)
                            loss = loss - entropy_coeff * el
                            rec["actor/entropy_loss"] = el.detach()
                        if ref is not None:
                            kld = core_algos.kl_penalty(logp, ref, a.kl_loss_type)
                            kl = core_algos.agg_loss(kld, mask, a.loss_agg_mode)
                            loss = loss + a.kl_loss_coef * kl
                            rec["actor/kl_loss"] = kl.detach()
                            rec["actor/kl_coef"] = torch.tensor(a.kl_loss_coef)
                        if loss_mode == "cpgd" and a.policy_drift_coeff != 0:
                            drift = core_algos.cpgd_policy_drift(old, logp, mask, a.loss_agg_mode)
                            loss = loss + a.policy_drift_coeff * drift
                            rec["actor/policy_drift"] = drift.detach()
                    return loss * scale, rec

                def record(rec):
                    for k, v in rec.items():
                        metrics.setdefault(k, []).append(v)

                if pipelined:
                    # 1F1B (interleaved over the stage's model chunks when virtual stages are configured): warm-up
                    # forwards, then one forward and one backward in turn, then the remaining backwards
                    from ..parallel.pipeline import schedule_interleaved
                    inflight = {}
                    self._pp_stage_local = True
                    try:
                        for op, i, c in schedule_interleaved(pc.stage, pc.pp, len(mbs), pc.virtual):
                            if op == "F":
                                inflight[i, c] = micro_forward(*mbs[i], chunk=c)
                            else:
                                target, rec = inflight.pop((i, c))
                                target.backward()
                                record(rec)
                    finally:
                        self._pp_stage_local = False
                        self._pp_chunk = 0
                    pc.drain()
                else:
                    for idx, mb in mbs:
                        target, rec = micro_forward(idx, mb)
                        target.backward()
                        record(rec)
                norm = self._optimizer_step(a.optim, a.grad_clip)
                metrics.setdefault("actor/grad_norm", []).append(norm.detach().clone())
        out = {k: float(torch.stack([torch.as_tensor(x, dtype=torch.float32, device="cpu") if not
                                     isinstance(x, torch.Tensor) else x.float().cpu() for x in v]).mean())
               for k, v in metrics.items()}
        if pipelined:
            # the loss metrics exist on the last stage only: hand them to the other stages of the pipeline
            box = [out if pc.is_last else None]
            dist.broadcast_object_list(box, src=pc.last_global, group=pc.group)
            out = dict(box[0], **{"actor/grad_norm": out.get("actor/grad_norm", box[0].get("actor/grad_norm", 0.0))})
        out["actor/lr"] = self.last_lr
        if self.device.type == "cuda":
            out["perf/max_memory_allocated_gb"] = torch.cuda.max_memory_allocated(self.device) / 2 ** 30
            out["perf/max_memory_reserved_gb"] = torch.cuda.max_memory_reserved(self.device) / 2 ** 30
        if self.device.type == "cuda":
            torch.cuda.synchronize()
        dt = time.time() - t0
        out["timing_s/update_actor_inner"] = dt
        from ..utils.model_utils.flops_counter import FlopsCounter
        seqlens = data["attention_mask"].sum(-1).tolist()
        # forward + backward (3x) plus the recompute forward of activation checkpointing is not counted as useful
        out["perf/mfu/actor"] = FlopsCounter(self.model_config).mfu(seqlens, dt / max(a.ppo_epochs, 1))
        return out


class CriticWorker(_ModelWorkerBase):
    """Value model (decoder + scalar head) with clipped value loss
    (reference: siirl/engine/fsdp_workers.py:1506-1815, siirl/engine/critic/dp_critic.py:41-246)."""

    def __init__(self, config, process_group=None, device=None, comm=None, seed: int = 1, rollout_n: int = 1):
        super().__init__(config, "critic", process_group, device, comm, seed)
        c = config
        dp = max(self.world // max(c.ulysses_sequence_parallel_size, 1), 1)
        self.ppo_mini_batch_size = max(1, c.ppo_mini_batch_size * max(rollout_n, c.rollout_n, 1) // dp)
        micro = c.ppo_micro_batch_size_per_gpu
        if micro is None and c.ppo_micro_batch_size is not None:
            micro = max(1, c.ppo_micro_batch_size // dp)
        self.ppo_micro_batch_size = micro

    def init_model(self) -> None:
        self._build(self.config.model, value_head=True, trainable=True, seed_offset=17)

    def _forward_values(self, mb: Batch) -> torch.Tensor:
        """Values aligned with response tokens ``[B, R]``: the value at the position that predicts token k."""
        pk = self._pack(mb)
        hidden = self.model.forward_hidden(pk.input_ids, pk.positions, pk.info)
        v = (hidden.index_select(0, pk.sel).float() @ self.model.value_head.float().t()).squeeze(-1)
        return pk.scatter(v)

    @torch.no_grad()
    def compute_values(self, data: Batch) -> Batch:
        self._phase_sync()
        c = self.config
        B, R = data["responses"].shape
        out = torch.zeros(B, R, dtype=torch.float32, device=self.device)
        self.model.eval()
        for idx, mb in _micro_batches(data, self.ppo_micro_batch_size, c.use_dynamic_bsz,
                                      c.forward_max_token_len_per_gpu, self.group):
            out[torch.tensor(idx, device=self.device)] = self._forward_values(mb)
        data["values"] = out * data["response_mask"].to(self.device).float()
        return data

    def update_critic(self, data: Batch) -> Dict[str, Any]:
        self._phase_sync()
        c = self.config
        self.model.train()
        metrics: Dict[str, List[torch.Tensor]] = {}
        bs = data.batch_size
        mini = min(self.ppo_mini_batch_size, bs)
        n_mini = max(1, bs // mini)
        self.store.zero_grad()
        for _ in range(c.ppo_epochs):
            order = torch.randperm(bs).tolist() if c.shuffle else list(range(bs))
            for mi in range(n_mini):
                mini_idx = order[mi * mini:(mi + 1) * mini]
                mini_batch = data.select_idxs(mini_idx)
                mbs = _micro_batches(mini_batch, self.ppo_micro_batch_size, c.use_dynamic_bsz,
                                     c.ppo_max_token_len_per_gpu, self.group)
                for idx, mb in mbs:
                    scale = (len(idx) / len(mini_idx)) if c.use_dynamic_bsz else 1.0 / len(mbs)
                    mask = mb["response_mask"].to(self.device).float()
                    vpred = self._forward_values(mb)
                    vf_loss, vf_clipfrac = core_algos.compute_value_loss(
                        vpred, mb["returns"].to(self.device).float(), mb["values"].to(self.device).float(), mask,
                        c.cliprange_value, c.loss_agg_mode)
                    (vf_loss * scale).backward()
                    metrics.setdefault("critic/vf_loss", []).append(vf_loss.detach())
                    metrics.setdefault("critic/vf_clipfrac", []).append(vf_clipfrac.detach())
                    metrics.setdefault("critic/vpred_mean", []).append(core_algos.masked_mean(vpred.detach(), mask))
                norm = self._optimizer_step(c.optim, c.grad_clip)
                metrics.setdefault("critic/grad_norm", []).append(norm.detach().clone())
        out = {k: float(torch.stack([x.float().cpu() for x in v]).mean()) for k, v in metrics.items()}
        out["critic/lr"] = self.last_lr
        return out


class RewardModelWorker(_ModelWorkerBase):
    """Model-based reward: a decoder with a scalar head scores each response at its last valid token
    (reference: siirl/engine/fsdp_workers.py:1819-2115).

    When the reward model was trained with another tokenizer / chat template than the policy
    (``reward_model.model.input_tokenizer`` names the policy's tokenizer, ``reward_model.model.rm_tokenizer`` or the
    model directory the reward model's), every sample is re-encoded first: the response is decoded with the policy's
    tokenizer, appended to the raw chat as the assistant turn, rendered with the reward model's chat template and
    tokenised with the reward model's tokenizer (reference: ``_switch_chat_template``, fsdp_workers.py:1997-2056, and
    ``re_encode_by_rm_tokenizer``, siirl/engine/reward_model/megatron/reward_model.py:59-122)."""

    def __init__(self, config, process_group=None, device=None, comm=None, seed: int = 1, input_tokenizer=None,
                 rm_tokenizer=None):
        super().__init__(config, "reward", process_group, device, comm, seed)
        self.input_tokenizer = input_tokenizer      # the policy's tokenizer (decodes responses)
        self.rm_tokenizer = rm_tokenizer            # the reward model's own tokenizer (None: same as the policy's)

    def init_model(self) -> None:
        self._build(self.config.model, value_head=True, trainable=False, seed_offset=29)
        m = self.config.model
        if self.rm_tokenizer is None and (m.rm_tokenizer or (m.input_tokenizer and m.path and not m.arch_preset)):
            from ..data_coordinator.dataloader.tokenizer import load_tokenizer
            self.rm_tokenizer = load_tokenizer(m.rm_tokenizer or m.path, vocab_size=self.model_config.vocab_size)
        if self.input_tokenizer is None and m.input_tokenizer:
            from ..data_coordinator.dataloader.tokenizer import load_tokenizer
            self.input_tokenizer = load_tokenizer(m.input_tokenizer, vocab_size=self.model_config.vocab_size)

    @property
    def switches_template(self) -> bool:
        return self.rm_tokenizer is not None and self.input_tokenizer is not None \
            and self.rm_tokenizer is not self.input_tokenizer

    def switch_chat_template(self, data: Batch) -> Batch:
        """Re-encode every (prompt chat, response) pair for the reward model: right-padded ``input_ids`` /
        ``attention_mask`` of width ``reward_model.max_length`` (default: the policy batch's width), truncated on the
        right."""
        src, dst = self.input_tokenizer, self.rm_tokenizer
        B, R = data["responses"].shape
        width = int(self.config.max_length or data["attention_mask"].shape[-1])
        raw = data.non_tensors.get("raw_prompt")
        pad = getattr(dst, "pad_token_id", 0) or 0
        ids = torch.full((B, width), pad, dtype=torch.int64)
        mask = torch.zeros(B, width, dtype=torch.int64)
        am = data["attention_mask"].cpu()
        resp = data["responses"].cpu()
        P = am.shape[-1] - R
        eos = getattr(src, "eos_token", None)
        for i in range(B):
            n = int(am[i, -R:].sum())
            text = src.decode(resp[i, :n].tolist())
            if eos:
                text = text.replace(eos, "")
            if raw is not None:
                chat = [dict(m) for m in (raw[i].tolist() if hasattr(raw[i], "tolist") else list(raw[i]))]
            else:       # no structured chat kept: the decoded prompt is the user turn
                chat = [{"role": "user", "content": src.decode(data["input_ids"][i, :P][am[i, :P].bool()].tolist())}]
            chat.append({"role": "assistant", "content": text})
            rendered = dst.apply_chat_template(chat, add_generation_prompt=False, tokenize=False)
            enc = dst(rendered, add_special_tokens=False)["input_ids"]
            enc = list(enc[0]) if enc and isinstance(enc[0], (list, tuple)) else list(enc)
            enc = enc[:width]
            ids[i, : len(enc)] = torch.tensor(enc, dtype=torch.int64)
            mask[i, : len(enc)] = 1
        return Batch({"input_ids": ids, "attention_mask": mask}, None, {})

    @torch.no_grad()
    def compute_rm_score(self, data: Batch) -> Batch:
        self._phase_sync()
        c = self.config
        B, R = data["responses"].shape
        scores = torch.zeros(B, R, dtype=torch.float32, device=self.device)
        micro = c.micro_batch_size_per_gpu or c.micro_batch_size
        rl_all = data["response_mask"].to(self.device).sum(-1).clamp(min=1) - 1
        src = data
        if self.switches_template:
            src = self.switch_chat_template(data)
        from ..ops.attention import SeqInfo
        for idx, mb in _micro_batches(src, micro, c.use_dynamic_bsz, c.forward_max_token_len_per_gpu, self.group):
            am = mb["attention_mask"].to(self.device)
            lens = am.sum(-1).clamp(min=1)
            info = SeqInfo(lens.tolist(), device=self.device)
            keep = am.bool()
            keep[:, 0] |= am.sum(-1) == 0           # an empty row still contributes one (padding) token
            ids = mb["input_ids"].to(self.device)[keep]
            v = self.model.values(ids, info.positions, info)
            last = torch.tensor(info.cu_seqlens_cpu[1:], device=self.device) - 1
            seq_score = v.index_select(0, last)
            rows = torch.tensor(idx, device=self.device)
            scores[rows, rl_all[rows]] = seq_score
        data["rm_scores"] = scores
        return data
