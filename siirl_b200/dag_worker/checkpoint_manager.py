"""Step-level checkpoint orchestration.

Layout (reference: siirl/dag_worker/checkpoint_manager.py:53-197):

    {default_local_dir}/global_step_{N}/{role}_agent_{g}/...     one directory per model role (actor, critic)
    {default_local_dir}/global_step_{N}/data_dp_rank_{r}.pt      dataloader state, written by tp0/pp0 ranks
    {default_local_dir}/latest_checkpointed_iteration.txt         written LAST by rank 0 (atomic rename) after a barrier

``resume_mode``: ``disable`` | ``auto`` (latest tracker entry if any) | ``resume_path`` (``trainer.resume_from_path``
names a ``global_step_N`` directory).  Rank 0 resolves the path and broadcasts it.

``actor.checkpoint.async_save``: the ranks snapshot their state to host memory, return to training and write their
files from a background thread; the checkpoint is *finalised* (writers joined, barrier, tracker file) at the start of
the next save, at the end of training or when ``finalize()`` is called -- until then the tracker still names the
previous checkpoint, so a crash in between resumes from that one.  ``trainer.default_hdfs_dir``: every rank copies
the files it wrote to ``{default_hdfs_dir}/global_step_{N}/{role}`` and rank 0 the tracker file (reference:
siirl/utils/checkpoint/megatron_checkpoint_manager.py:356-543, siirl/utils/extras/fs.py)."""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist

from ..utils.checkpoint.checkpoint_manager import find_latest_complete_ckpt_path, remove_old_checkpoints


class CheckpointManager:
    def __init__(self, worker):
        self.w = worker
        self.root = os.path.expanduser(worker.config.trainer.default_local_dir)
        self.hdfs_root = worker.config.trainer.default_hdfs_dir or None
        self._pending = None        # (global_step, [PendingSave, ...]) of a save whose tracker is not written yet

    @staticmethod
    def _save_contents(ck):
        """``checkpoint.save_contents`` (the reference's key) when the user set it, else ``checkpoint.contents``."""
        default = ["model", "optimizer", "extra"]
        sc = list(getattr(ck, "save_contents", None) or default)
        return sc if sorted(sc) != sorted(default) else list(ck.contents)

    def _roles(self):
        out = []
        seen = set()
        for key, wk in self.w.workers.items():
            if id(wk) in seen:
                continue            # an agent group that shares another group's instance
            seen.add(id(wk))
            if key.startswith("actor_rollout_ref_") and getattr(wk, "store", None) is not None:
                out.append((f"actor_agent_{key.rsplit('_', 1)[-1]}", wk,
                            self._save_contents(self.w.config.actor_rollout_ref.actor.checkpoint),
                            self.w.config.trainer.max_actor_ckpt_to_keep))
            elif key.startswith("critic_"):
                out.append((f"critic_agent_{key.rsplit('_', 1)[-1]}", wk, self._save_contents(self.w.config.critic.checkpoint),
                            self.w.config.trainer.max_critic_ckpt_to_keep))
        return out

    def save_checkpoint(self, global_step: int) -> str:
        self.finalize()                 # an earlier asynchronous save becomes visible before its successor starts
        step_dir = os.path.join(self.root, f"global_step_{global_step}")
        os.makedirs(step_dir, exist_ok=True)
        run_async = bool(self.w.config.actor_rollout_ref.actor.checkpoint.async_save)
        handles = []
        for name, wk, contents, keep in self._roles():
            hdfs = f"{self.hdfs_root.rstrip('/')}/global_step_{global_step}/{name}" if self.hdfs_root else None
            h = wk.save_checkpoint(os.path.join(step_dir, name), hdfs, global_step, keep, contents=contents,
                                   async_save=run_async)
            if h is not None:
                handles.append(h)
        dl = self.w.dataloader
        tp = self.w.config.actor_rollout_ref.rollout.tensor_model_parallel_size
        if self.w._rank % max(tp, 1) == 0:
            tmp = os.path.join(step_dir, f"data_dp_rank_{dl.ddp_rank}.pt.tmp")
            torch.save({"dataloader": dl.state_dict(), "global_step": global_step}, tmp)
            os.replace(tmp, tmp[:-4])
            if self.hdfs_root:
                from ..utils.extras import fs
                fs.makedirs(f"{self.hdfs_root.rstrip('/')}/global_step_{global_step}")
                fs.copy(tmp[:-4], f"{self.hdfs_root.rstrip('/')}/global_step_{global_step}/{os.path.basename(tmp[:-4])}")
        self._pending = (global_step, handles)
        if not run_async:
            self.finalize()
        return step_dir

    def finalize(self) -> None:
        """Join this rank's checkpoint writers, wait for the other ranks, then publish the step in the tracker file.
        A collective: every rank calls it at the same point of its control flow (next save, end of the loop)."""
        if self._pending is None:
            return
        global_step, handles = self._pending
        self._pending = None
        for h in handles:
            h.wait()
        if self.w._dist:
            dist.barrier()
        if self.w._rank == 0:
            tracker = os.path.join(self.root, "latest_checkpointed_iteration.txt")
            with open(tracker + ".tmp", "w") as f:
                f.write(str(global_step))
            os.replace(tracker + ".tmp", tracker)
            if self.hdfs_root:
                from ..utils.extras import fs
                fs.copy(tracker, f"{self.hdfs_root.rstrip('/')}/latest_checkpointed_iteration.txt")
            keep = self.w.config.trainer.max_actor_ckpt_to_keep
            if self.w.config.trainer.remove_previous_ckpt_in_save:
                keep = 1
            remove_old_checkpoints(self.root, keep)
        if self.w._dist:
            dist.barrier()

    def _resolve(self) -> Optional[str]:
        t = self.w.config.trainer
        if t.resume_mode == "disable":
            return None
        if t.resume_mode == "auto":
            # a damaged latest checkpoint (a shard cut short by a crash or a full disk) falls back to the one before
            found = find_latest_complete_ckpt_path(self.root)
            if found is None and self.hdfs_root:
                # nothing usable on the local disk (a fresh node): fetch the tracked step from the remote copy
                from ..utils.extras import fs
                remote_tracker = f"{self.hdfs_root.rstrip('/')}/latest_checkpointed_iteration.txt"
                if fs.exists(remote_tracker):
                    os.makedirs(self.root, exist_ok=True)
                    fs.copy(remote_tracker, os.path.join(self.root, "latest_checkpointed_iteration.txt"))
                    with open(os.path.join(self.root, "latest_checkpointed_iteration.txt")) as f:
                        step = f.read().strip()
                    fs.copy(f"{self.hdfs_root.rstrip('/')}/global_step_{step}",
                            os.path.join(self.root, f"global_step_{step}"))
                    found = find_latest_complete_ckpt_path(self.root)
            return found
        if t.resume_mode == "resume_path":
            p = t.resume_from_path
            if not isinstance(p, str) or "global_step_" not in p:
                raise ValueError("trainer.resume_from_path must name a global_step_N directory")
            return os.path.expanduser(p)
        raise ValueError(f"unknown resume_mode '{t.resume_mode}'")

    def load_checkpoint(self) -> int:
        """Returns the global step to continue from (0 when starting fresh)."""
        path = self._resolve() if self.w._rank == 0 else None
        if self.w._dist:
            box = [path]
            dist.broadcast_object_list(box, src=0)
            path = box[0]
        if not path or not os.path.isdir(path):
            return 0
        step = int(path.rstrip("/").split("global_step_")[-1])
        for name, wk, _, _ in self._roles():
            d = os.path.join(path, name)
            if os.path.isdir(d):
                wk.load_checkpoint(d, None, self.w.config.trainer.del_local_ckpt_after_load)
        dl = self.w.dataloader
        f = os.path.join(path, f"data_dp_rank_{dl.ddp_rank}.pt")
        if os.path.exists(f):
            dl.load_state_dict(torch.load(f, map_location="cpu", weights_only=False)["dataloader"])
        return step
