"""Sharded model/optimizer checkpoints with an elastic manifest, plus the HF export.

Directory written by one role (layout names follow siirl/utils/checkpoint/fsdp_checkpoint_manager.py:129-252):

    <dir>/manifest.json                               logical layout: flat offsets, shapes, dtype, world size
    <dir>/model_world_size_{W}_rank_{r}.pt            this rank's slice of the bf16/fp32 working copy
    <dir>/optim_world_size_{W}_rank_{r}.pt            fp32 master + Adam moments of the owned shard
    <dir>/extra_state_world_size_{W}_rank_{r}.pt      step counters, RNG states (cpu, cuda, numpy, random)
    <dir>/huggingface/                                config.json (+ safetensors when "hf_model" is in contents)

Unlike the reference (file names bake in the world size and cannot be re-sharded), the manifest records the
unsharded layout, so ``load`` on a different world size reassembles the flat state from all shard files and
re-slices it.  Files are written to ``*.tmp`` and renamed, so a crash never leaves a half-written shard that looks
complete.
"""
from __future__ import annotations

import json
import os
import random
import shutil
from typing import Any, Dict, List, Optional

import numpy as np
import torch
import torch.distributed as dist


def _atomic_save(obj: Any, path: str) -> None:
    tmp = path + ".tmp"
    torch.save(obj, tmp)
    os.replace(tmp, path)


def get_rng_state() -> Dict[str, Any]:
    st = {"cpu": torch.get_rng_state(), "numpy": np.random.get_state(), "random": random.getstate()}
    if torch.cuda.is_available():
        st["cuda"] = torch.cuda.get_rng_state()
    return st


def load_rng_state(st: Dict[str, Any]) -> None:
    torch.set_rng_state(st["cpu"])
    np.random.set_state(st["numpy"])
    random.setstate(st["random"])
    if "cuda" in st and torch.cuda.is_available():
        torch.cuda.set_rng_state(st["cuda"])


def find_latest_ckpt_path(root: str) -> Optional[str]:
    """Directory of the step recorded in ``latest_checkpointed_iteration.txt`` (None if absent)."""
    tracker = os.path.join(root, "latest_checkpointed_iteration.txt")
    if not os.path.exists(tracker):
        return None
    with open(tracker) as f:
        step = int(f.read().strip())
    path = os.path.join(root, f"global_step_{step}")
    return path if os.path.isdir(path) else None


def checkpoint_problems(step_dir: str) -> List[str]:
    """Structural check of one ``global_step_N`` directory: every role directory has a readable manifest, all the
    model shards of the world size that wrote it, and no truncated ``.pt`` file (``torch.save`` writes zip archives,
    whose directory sits at the end of the file).  Returns the list of problems found (empty = complete)."""
    import glob
    import zipfile
    problems: List[str] = []
    roles = [d for d in sorted(os.listdir(step_dir)) if os.path.isdir(os.path.join(step_dir, d)) and "_agent_" in d]
    if not roles:
        problems.append("no role directory")
    for role in roles:
        d = os.path.join(step_dir, role)
        try:
            with open(os.path.join(d, "manifest.json")) as f:
                manifest = json.load(f)
        except (OSError, ValueError) as e:
            problems.append(f"{role}: manifest unreadable ({type(e).__name__})")
            continue
        world = int(manifest.get("world_size", 1))
        if "model" in manifest.get("contents", []):
            shards = glob.glob(os.path.join(d, f"model_world_size_{world}_rank_*.pt"))
            need = world if manifest.get("offsets") else 1
            if len(shards) < need:
                problems.append(f"{role}: {len(shards)} of {need} model shards")
        for f in glob.glob(os.path.join(d, "*.pt")):
            if os.path.getsize(f) == 0 or not zipfile.is_zipfile(f):
                problems.append(f"{role}: {os.path.basename(f)} is truncated or not a torch archive")
    return problems


def find_latest_complete_ckpt_path(root: str, log=print) -> Optional[str]:
    """The newest checkpoint that passes ``checkpoint_problems``: the tracked step first, then older steps."""
    first = find_latest_ckpt_path(root)
    if not os.path.isdir(root):
        return None
    steps = sorted((int(d.split("_")[-1]) for d in os.listdir(root)
                    if d.startswith("global_step_") and d.split("_")[-1].isdigit()), reverse=True)
    candidates = ([first] if first else []) + [os.path.join(root, f"global_step_{s}") for s in steps]
    seen = set()
    tracked = int(first.rstrip("/").split("_")[-1]) if first else None
    for path in candidates:
        if path in seen or not os.path.isdir(path):
            continue
        seen.add(path)
        step = int(path.rstrip("/").split("_")[-1])
        if tracked is not None and step > tracked:
            continue                    # newer than the tracker: its save never completed
        problems = checkpoint_problems(path)
        if not problems:
            return path
        log(f"[checkpoint] skipping {path}: " + "; ".join(problems))
    return None


def remove_old_checkpoints(root: str, keep: int) -> None:
    if keep is None or keep <= 0:
        return
    steps = sorted(int(d.split("_")[-1]) for d in os.listdir(root)
                   if d.startswith("global_step_") and d.split("_")[-1].isdigit())
    for s in steps[:-keep]:
        shutil.rmtree(os.path.join(root, f"global_step_{s}"), ignore_errors=True)


class ShardedCheckpointManager:
    def __init__(self, model, store, model_config, group=None, contents: Optional[List[str]] = None,
                 tokenizer=None):
        self.model, self.store, self.model_config = model, store, model_config
        self.group = group
        self.contents = list(contents or ["model", "optimizer", "extra"])
        self.tokenizer = tokenizer
        self.world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0

    def _names(self, d: str):
        w, r = self.world, self.rank
        return (os.path.join(d, f"model_world_size_{w}_rank_{r}.pt"),
                os.path.join(d, f"optim_world_size_{w}_rank_{r}.pt"),
                os.path.join(d, f"extra_state_world_size_{w}_rank_{r}.pt"))

    def save(self, directory: str, global_step: int = 0, extra: Optional[Dict[str, Any]] = None,
             max_ckpt_to_keep: Optional[int] = None) -> None:
        os.makedirs(directory, exist_ok=True)
        mpath, opath, epath = self._names(directory)
        st = self.store
        if st is not None:
            if "model" in self.contents:
                _atomic_save({"flat": st.flat_param[st.lo:st.hi].detach().cpu(), "lo": st.lo, "hi": st.hi}, mpath)
            if "optimizer" in self.contents and st.master is not None:
                _atomic_save(st.shard_state_dict(), opath)
            ex = getattr(st, "expert", None)
            if ex is not None:      # this rank's experts (expert parallelism): parameters + full local state
                _atomic_save({"flat": ex.flat_param.detach().cpu(), "state": ex.shard_state_dict()},
                             os.path.join(directory, f"experts_world_size_{self.world}_rank_{self.rank}.pt"))
        elif "model" in self.contents and self.rank == 0:
            _atomic_save({"state_dict": {k: v.detach().cpu() for k, v in self.model.state_dict().items()}}, mpath)
        if "extra" in self.contents:
            _atomic_save({"global_step": global_step, "rng": get_rng_state(), "extra": extra or {}}, epath)
        if self.rank == 0:
            manifest = {"world_size": self.world, "global_step": global_step,
                        "dtype": str(st.dtype) if st is not None else None,
                        "total": st.total if st is not None else None,
                        "offsets": {n: [o, k, list(s)] for n, (o, k, s) in st.offsets.items()} if st else None,
                        "model_config": self.model_config.to_dict() if self.model_config is not None else None,
                        "contents": self.contents}
            tmp = os.path.join(directory, "manifest.json.tmp")
            with open(tmp, "w") as f:
                json.dump(manifest, f)
            os.replace(tmp, os.path.join(directory, "manifest.json"))
            hf_dir = os.path.join(directory, "huggingface")
            os.makedirs(hf_dir, exist_ok=True)
            if "hf_model" in self.contents:
                from ...models.hf_io import save_hf_model
                save_hf_model(self.model, hf_dir, tokenizer=self.tokenizer)
            elif self.model_config is not None:
                with open(os.path.join(hf_dir, "config.json"), "w") as f:
                    json.dump(self.model_config.to_hf_config(), f, indent=1)

    def load(self, directory: str) -> Optional[Dict[str, Any]]:
        with open(os.path.join(directory, "manifest.json")) as f:
            manifest = json.load(f)
        saved_world = manifest["world_size"]
        st = self.store
        mpath, opath, epath = self._names(directory)
        ex = getattr(st, "expert", None)
        if ex is not None:
            if saved_world != self.world:
                raise ValueError("an expert-parallel checkpoint resumes only on the expert-parallel width that wrote it")
            e = torch.load(os.path.join(directory, f"experts_world_size_{self.world}_rank_{self.rank}.pt"),
                           map_location="cpu", weights_only=False)
            ex.flat_param.copy_(e["flat"].to(ex.device))
            ex.load_shard_state_dict(e["state"])
        if st is not None:
            if saved_world == self.world and os.path.exists(mpath):
                m = torch.load(mpath, map_location="cpu", weights_only=False)
                st.flat_param[st.lo:st.hi].copy_(m["flat"].to(st.device))
                if self.world > 1:
                    st._all_gather_params()
                if os.path.exists(opath) and st.master is not None:
                    st.load_shard_state_dict(torch.load(opath, map_location="cpu", weights_only=False))
                elif st.master is not None:
                    st.sync_master_from_params()
            else:
                self._load_resharded(directory, saved_world, manifest)
        elif os.path.exists(os.path.join(directory, f"model_world_size_{saved_world}_rank_0.pt")):
            m = torch.load(os.path.join(directory, f"model_world_size_{saved_world}_rank_0.pt"), map_location="cpu",
                           weights_only=False)
            if "state_dict" in m:
                self.model.load_state_dict(m["state_dict"])
        extra = None
        if not os.path.exists(epath):
            epath = os.path.join(directory, f"extra_state_world_size_{saved_world}_rank_0.pt")
        if os.path.exists(epath):
            e = torch.load(epath, map_location="cpu", weights_only=False)
            if saved_world == self.world:
                try:
                    load_rng_state(e["rng"])
                except Exception:  # noqa: BLE001  (a CUDA state cannot be restored on a CPU-only machine)
                    pass
            extra = dict(e.get("extra", {}))
            extra["global_step"] = e.get("global_step", 0)
        return extra

    def _load_resharded(self, directory: str, saved_world: int, manifest: Dict[str, Any]) -> None:
        """Reassemble the flat state written by ``saved_world`` ranks and keep this rank's new shard."""
        st = self.store
        if manifest["offsets"] is None or {n: tuple(v[:2]) for n, v in manifest["offsets"].items()} != {
                n: (o, k) for n, (o, k, _) in st.offsets.items()}:
            raise ValueError("checkpoint layout does not match this model")
        total_saved = manifest["total"]
        flat = torch.zeros(max(total_saved, st.total), dtype=torch.float32)
        master = torch.zeros_like(flat)
        m1 = torch.zeros_like(flat)
        m2 = torch.zeros_like(flat)
        step, have_opt = 0, True
        for r in range(saved_world):
            m = torch.load(os.path.join(directory, f"model_world_size_{saved_world}_rank_{r}.pt"), map_location="cpu",
                           weights_only=False)
            flat[m["lo"]:m["hi"]] = m["flat"].float()
            op = os.path.join(directory, f"optim_world_size_{saved_world}_rank_{r}.pt")
            if os.path.exists(op):
                o = torch.load(op, map_location="cpu", weights_only=False)
                master[m["lo"]:m["hi"]] = o["master"]
                m1[m["lo"]:m["hi"]] = o["exp_avg"]
                m2[m["lo"]:m["hi"]] = o["exp_avg_sq"]
                step = int(o["step"])
            else:
                have_opt = False
        n = st.total
        if have_opt and st.master is not None:
            st.load_full_state(master[:n], m1[:n], m2[:n], step)
        else:
            st.flat_param.copy_(flat[:n].to(st.device, st.dtype))
            st.sync_master_from_params()
