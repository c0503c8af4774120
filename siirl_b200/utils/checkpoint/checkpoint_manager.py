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
    expanded = []
    for role in roles:
        subs = sorted(x for x in os.listdir(os.path.join(step_dir, role)) if x.startswith("tp_rank_"))
        expanded += [os.path.join(role, x) for x in subs] if subs else [role]
    for role in expanded:
        d = os.path.join(step_dir, role)
        try:
            with open(os.path.join(d, "manifest.json")) as f:
                manifest = json.load(f)
        except (OSError, ValueError) as e:
            problems.append(f"{role}: manifest unreadable ({type(e).__name__})")
            continue
        world = int(manifest.get("world_size", 1))
        contents = manifest.get("contents", [])
        sharded = bool(manifest.get("offsets"))
        wanted = []
        if "model" in contents:
            wanted.append(("model", world if sharded else 1))
        if "optimizer" in contents and sharded and manifest.get("has_optimizer_state", True):
            wanted.append(("optim", world))
        if "extra" in contents:
            wanted.append(("extra_state", world))
        if manifest.get("expert_parallel"):
            wanted.append(("experts", world))
        for kind, need in wanted:
            have = {os.path.basename(f) for f in glob.glob(os.path.join(d, f"{kind}_world_size_{world}_rank_*.pt"))}
            missing = [r for r in range(need) if f"{kind}_world_size_{world}_rank_{r}.pt" not in have]
            if missing:
                problems.append(f"{role}: {kind} shards of ranks {missing[:8]} missing ({need - len(missing)} of {need})")
        for f in glob.glob(os.path.join(d, "*.pt")):
            if os.path.getsize(f) == 0 or not zipfile.is_zipfile(f):
                problems.append(f"{role}: {os.path.basename(f)} is truncated or not a torch archive")
    data_files = glob.glob(os.path.join(step_dir, "data_dp_rank_*.pt"))
    if not data_files:
        problems.append("no dataloader state (data_dp_rank_*.pt)")
    for f in data_files:
        if os.path.getsize(f) == 0 or not zipfile.is_zipfile(f):
            problems.append(f"{os.path.basename(f)} is truncated or not a torch archive")
    return problems


def find_latest_complete_ckpt_path(root: str, log=print) -> Optional[str]:
    """The newest checkpoint that passes ``checkpoint_problems``: the tracked step first, then older steps.  The
    tracker file is written last, after every rank has finished its files: without one no save has ever completed
    (a crash during the first save leaves step directories that may look whole), so nothing is resumed."""
    first = find_latest_ckpt_path(root)
    if not os.path.isdir(root):
        return None
    if not os.path.exists(os.path.join(root, "latest_checkpointed_iteration.txt")):
        if any(d.startswith("global_step_") for d in os.listdir(root)):
            log(f"[checkpoint] {root} has step directories but no latest_checkpointed_iteration.txt: no save ever "
                f"completed, starting fresh")
        return None
    steps = sorted((int(d.split("_")[-1]) for d in os.listdir(root)
                    if d.startswith("global_step_") and d.split("_")[-1].isdigit()), reverse=True)
    candidates = ([first] if first else []) + [os.path.join(root, f"global_step_{s}") for s in steps]
    seen = set()
    with open(os.path.join(root, "latest_checkpointed_iteration.txt")) as f:
        txt = f.read().strip()
    tracked = int(txt) if txt.isdigit() else None
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


class PendingSave:
    """Handle of one rank's checkpoint write: done already (synchronous save) or running in a thread.  ``wait()``
    joins the thread and re-raises what it raised."""

    def __init__(self, fn, run_async: bool):
        self._error: Optional[BaseException] = None
        self._thread = None
        if not run_async:
            fn()
            return
        import threading

        def guarded():
            try:
                fn()
            except BaseException as e:  # noqa: BLE001  (re-raised on the caller's thread by wait())
                self._error = e

        self._thread = threading.Thread(target=guarded, name="siirl-ckpt-writer", daemon=False)
        self._thread.start()

    def done(self) -> bool:
        return self._thread is None or not self._thread.is_alive()

    def wait(self) -> None:
        if self._thread is not None:
            self._thread.join()
            self._thread = None
        if self._error is not None:
            err, self._error = self._error, None
            raise err


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
             max_ckpt_to_keep: Optional[int] = None, async_save: bool = False,
             hdfs_path: Optional[str] = None) -> "PendingSave":
        """Write this rank's files.  The state is snapshotted to host memory before the call returns; with
        ``async_save`` the files are written by a background thread (reference: the Megatron manager's async save,
        siirl/utils/checkpoint/megatron_checkpoint_manager.py:356-543) and the caller must ``wait()`` on the returned
        handle before it declares the checkpoint complete.  ``hdfs_path``: after the local files are in place this
        rank's files are also copied there (``hdfs dfs -put``; any path ``utils.extras.fs.copy`` accepts)."""
        os.makedirs(directory, exist_ok=True)
        mpath, opath, epath = self._names(directory)
        st = self.store
        jobs: List[Any] = []            # (object, path) pairs, all tensors already on the host
        if st is not None:
            if "model" in self.contents:
                jobs.append(({"flat": st.flat_param[st.lo:st.hi].detach().cpu(), "lo": st.lo, "hi": st.hi}, mpath))
            if "optimizer" in self.contents and st.master is not None:
                jobs.append((st.shard_state_dict(), opath))
            ex = getattr(st, "expert", None)
            if ex is not None:      # this rank's experts (expert parallelism): parameters + full local state
                jobs.append(({"flat": ex.flat_param.detach().cpu(), "state": ex.shard_state_dict()},
                             os.path.join(directory, f"experts_world_size_{self.world}_rank_{self.rank}.pt")))
        elif "model" in self.contents and self.rank == 0:
            jobs.append(({"state_dict": {k: v.detach().cpu() for k, v in self.model.state_dict().items()}}, mpath))
        if "extra" in self.contents:
            jobs.append(({"global_step": global_step, "rng": get_rng_state(), "extra": extra or {}}, epath))
        manifest = None
        if self.rank == 0:
            manifest = {"world_size": self.world, "global_step": global_step,
                        "dtype": str(st.dtype) if st is not None else None,
                        "total": st.total if st is not None else None,
                        "offsets": {n: [o, k, list(s)] for n, (o, k, s) in st.offsets.items()} if st else None,
                        "model_config": self.model_config.to_dict() if self.model_config is not None else None,
                        "has_optimizer_state": bool(st is not None and st.master is not None),
                        "expert_parallel": bool(st is not None and getattr(st, "expert", None) is not None),
                        "contents": self.contents}
        hf_state = None
        if "hf_model" in self.contents and hasattr(st, "materialize_full"):
            st.materialize_full()       # parameter-sharded store: the exporter needs whole weights (a collective)
        if self.rank == 0 and "hf_model" in self.contents and (async_save or hasattr(st, "materialize_full")):
            # the exporter reads the live parameters: snapshot them now, the next optimizer step may run meanwhile
            from ...models.hf_io import to_hf_state
            hf_state = [(n, t.detach().to("cpu").clone()) for n, t in to_hf_state(self.model)]

        def write() -> None:
            written = []
            for obj, path in jobs:
                _atomic_save(obj, path)
                written.append(path)
            if manifest is not None:
                tmp = os.path.join(directory, "manifest.json.tmp")
                with open(tmp, "w") as f:
                    json.dump(manifest, f)
                os.replace(tmp, os.path.join(directory, "manifest.json"))
                written.append(os.path.join(directory, "manifest.json"))
                hf_dir = os.path.join(directory, "huggingface")
                os.makedirs(hf_dir, exist_ok=True)
                if "hf_model" in self.contents:
                    from ...models.hf_io import save_hf_model
                    save_hf_model(self.model, hf_dir, tokenizer=self.tokenizer, tensors=hf_state)
                elif self.model_config is not None:
                    with open(os.path.join(hf_dir, "config.json"), "w") as f:
                        json.dump(self.model_config.to_hf_config(), f, indent=1)
                written.append(hf_dir)
            if hdfs_path:
                from ..extras import fs
                fs.makedirs(hdfs_path)
                for path in written:
                    fs.copy(path, hdfs_path.rstrip("/") + "/" + os.path.basename(path))

        if "hf_model" in self.contents and hasattr(st, "release_full"):
            st.release_full()
        return PendingSave(write, async_save)

    def load(self, directory: str, contents: Optional[List[str]] = None) -> Optional[Dict[str, Any]]:
        """``contents`` (the reference's ``checkpoint.load_contents``): which parts of the checkpoint to take.
        Without ``"optimizer"`` the weights are loaded and the optimizer starts fresh from them; without ``"extra"``
        neither the random streams nor the scheduler / dataloader fields are restored (the step counter still is);
        without ``"model"`` nothing of the training state is read."""
        take = set(contents) if contents is not None else {"model", "optimizer", "extra"}
        with open(os.path.join(directory, "manifest.json")) as f:
            manifest = json.load(f)
        saved_world = manifest["world_size"]
        st = self.store if "model" in take else None
        mpath, opath, epath = self._names(directory)
        ex = getattr(st, "expert", None)
        if ex is not None:
            if saved_world != self.world:
                raise ValueError("an expert-parallel checkpoint resumes only on the expert-parallel width that wrote it")
            e = torch.load(os.path.join(directory, f"experts_world_size_{self.world}_rank_{self.rank}.pt"),
                           map_location="cpu", weights_only=False)
            ex.flat_param.copy_(e["flat"].to(ex.device))
            ex.load_shard_state_dict(e["state"])
            if hasattr(st, "invalidate"):
                st.invalidate()
        if st is not None:
            if saved_world == self.world and os.path.exists(mpath):
                m = torch.load(mpath, map_location="cpu", weights_only=False)
                st.flat_param[st.lo:st.hi].copy_(m["flat"].to(st.device))
                if self.world > 1:
                    st._all_gather_params()
                if "optimizer" not in take:
                    if st.master is not None:
                        st.sync_master_from_params()
                elif os.path.exists(opath) and st.master is not None:
                    st.load_shard_state_dict(torch.load(opath, map_location="cpu", weights_only=False))
                elif st.master is not None:
                    if "optimizer" in manifest.get("contents", []) and manifest.get("has_optimizer_state", True):
                        # the other ranks load their Adam moments and step count: starting this shard from zero
                        # would give the shards different bias corrections
                        raise FileNotFoundError(f"{opath}: the checkpoint lists optimizer state but this rank's "
                                                f"shard is missing")
                    st.sync_master_from_params()
            else:
                self._load_resharded(directory, saved_world, manifest)
                if "optimizer" not in take and st.master is not None:
                    st.sync_master_from_params()
        elif "model" in take and os.path.exists(os.path.join(directory, f"model_world_size_{saved_world}_rank_0.pt")):
            m = torch.load(os.path.join(directory, f"model_world_size_{saved_world}_rank_0.pt"), map_location="cpu",
                           weights_only=False)
            if "state_dict" in m:
                self.model.load_state_dict(m["state_dict"])
        extra = None
        if not os.path.exists(epath):
            epath = os.path.join(directory, f"extra_state_world_size_{saved_world}_rank_0.pt")
        if os.path.exists(epath):
            e = torch.load(epath, map_location="cpu", weights_only=False)
            if saved_world == self.world and "extra" in take:
                try:
                    load_rng_state(e["rng"])
                except Exception:  # noqa: BLE001  (a CUDA state cannot be restored on a CPU-only machine)
                    pass
            extra = dict(e.get("extra", {})) if "extra" in take else {}
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
