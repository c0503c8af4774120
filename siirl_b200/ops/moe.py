"""Mixture-of-experts primitives: routing layout, peer-memory dispatch / combine, grouped tcgen05 GEMM.

Layout.  The routed (token, k) pairs of ALL ranks are sorted by expert; every expert's segment is padded to a
multiple of 128 rows so that a 128-row GEMM tile never mixes experts.  A rank that hosts experts
``[e0, e1)`` owns the slice of that global layout covering its experts (its "slots").  Everything is computed
with device ops from the all-gathered routing table, identically on every rank, without a host synchronisation:
buffer sizes are static upper bounds and unused 128-row blocks are marked ``-1`` (the GEMM skips them).

CPU tensors take a plain PyTorch path with the same semantics (oracle of the GPU tests, gloo tests).

Reference counterpart: Megatron-core's MoE layer configured in siirl/models/mcore/config_converter.py (qwen3moe /
qwen2moe / mixtral branches: ``moe_token_dispatcher_type="alltoall"``, ``moe_grouped_gemm=True``)."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import torch

from . import lib as _lib

BLOCK_ROWS = 128


@dataclass
class MoeLayout:
    world: int
    rank: int
    num_experts: int
    top_k: int
    tokens_per_rank: int            # T (same on every rank)
    capacity: int                   # rows of a rank's slot buffer (multiple of 128, static)
    # global pair p = (src_rank * T + t) * k + j
    pair_rank: torch.Tensor         # [world*T*k] int32: rank hosting the pair's expert
    pair_slot: torch.Tensor         # [world*T*k] int32: slot inside that rank's buffer
    slot_src_rank: torch.Tensor     # [capacity] int32: rank of the token occupying my slot (0 when unused)
    slot_src_row: torch.Tensor      # [capacity] int32: token row on that rank (-1 when unused)
    slot_pair: torch.Tensor         # [capacity] int64: global pair id of my slot (-1 when unused)
    tile_group: torch.Tensor        # [capacity/128] int32: LOCAL expert id of each 128-row block (-1 unused)
    group_rows: torch.Tensor        # [E_local+1] int32: row range of every local expert (multiples of 128)

    @property
    def experts_per_rank(self) -> int:
        return self.num_experts // self.world

    def my_pairs(self):
        T, k = self.tokens_per_rank, self.top_k
        lo = self.rank * T * k
        return self.pair_rank[lo:lo + T * k], self.pair_slot[lo:lo + T * k]


_LAYOUT_MAX_EXPERTS = 256
_FUSED_LAYOUT = True        # tests flip this to compare the kernels with the device-op construction below


def _build_layout_fused(all_idx: torch.Tensor, num_experts: int, world: int, rank: int,
                        capacity: Optional[int]) -> "MoeLayout":
    """The same layout from three launches (histogram per 1024-pair chunk, scan, stable placement) instead of the
    ~70 small device ops and the sort of the construction in ``build_layout``."""
    W, T, k = all_idx.shape
    dev = all_idx.device
    El = num_experts // world
    P = W * T * k
    if capacity is None:
        capacity = (P + El * BLOCK_ROWS + BLOCK_ROWS - 1) // BLOCK_ROWS * BLOCK_ROWS
    idx = all_idx.reshape(-1)
    idx = idx if idx.dtype == torch.int32 else idx.to(torch.int32)
    idx = idx.contiguous()
    n_chunks = (P + 1023) // 1024
    i32 = dict(dtype=torch.int32, device=dev)
    scratch = torch.empty(n_chunks * (num_experts + 1) + (num_experts + 2) + (world + 1), **i32)
    chunk_counts = scratch[:n_chunks * (num_experts + 1)]
    starts = scratch[n_chunks * (num_experts + 1):n_chunks * (num_experts + 1) + num_experts + 2]
    rank_base = scratch[n_chunks * (num_experts + 1) + num_experts + 2:]
    pair = torch.empty(2, P, **i32)
    slot_src = torch.empty(2, capacity, **i32)
    slot_pair = torch.empty(capacity, dtype=torch.int64, device=dev)
    tile_group = torch.empty(capacity // BLOCK_ROWS, **i32)
    group_rows = torch.empty(El + 1, **i32)
    L = _lib.get_lib()
    _lib.check(L.sb_moe_build_layout(_lib.ptr(idx), P, num_experts, world, rank, T, k, capacity, _lib.ptr(chunk_counts),
                                     _lib.ptr(starts), _lib.ptr(rank_base), _lib.ptr(pair[0]), _lib.ptr(pair[1]),
                                     _lib.ptr(slot_pair), _lib.ptr(slot_src[0]), _lib.ptr(slot_src[1]),
                                     _lib.ptr(tile_group), _lib.ptr(group_rows), _lib.stream()), "sb_moe_build_layout")
    return MoeLayout(world, rank, num_experts, k, T, capacity, pair[0], pair[1], slot_src[0], slot_src[1], slot_pair,
                     tile_group, group_rows)


def build_layout(all_idx: torch.Tensor, num_experts: int, world: int, rank: int,
                 capacity: Optional[int] = None) -> MoeLayout:
    """``all_idx [world, T, k]`` expert ids of every rank's tokens (all-gathered routing table).  Negative ids mark
    padding tokens (ranks pad their token count to a common static bound): they get no slot."""
    W, T, k = all_idx.shape
    assert W == world and num_experts % world == 0
    dev = all_idx.device
    El = num_experts // world
    P = W * T * k
    if all_idx.is_cuda and num_experts <= _LAYOUT_MAX_EXPERTS and _FUSED_LAYOUT:
        return _build_layout_fused(all_idx, num_experts, world, rank, capacity)
    flat = all_idx.reshape(-1).long()
    real_experts = num_experts
    flat = torch.where(flat < 0, torch.full_like(flat, real_experts), flat)     # padding -> a dummy last expert
    num_experts = real_experts + 1
    counts = torch.bincount(flat, minlength=num_experts)
    padded = (counts + BLOCK_ROWS - 1) // BLOCK_ROWS * BLOCK_ROWS
    ends = torch.cumsum(padded, 0)
    starts = ends - padded                                        # global padded start of every expert
    order = torch.argsort(flat, stable=True)
    sorted_e = flat[order]
    first_of_e = torch.cumsum(counts, 0) - counts
    rank_in_e = torch.arange(P, device=dev) - first_of_e[sorted_e]
    gslot_sorted = starts[sorted_e] + rank_in_e                   # global padded slot of each sorted pair
    host = sorted_e // El                                         # hosting rank (== world for padding pairs)
    rank_base = starts[torch.arange(world + 1, device=dev) * El]  # first global slot of every rank
    lslot_sorted = gslot_sorted - rank_base[host]
    pair_rank = torch.empty(P, dtype=torch.int32, device=dev)
    pair_slot = torch.empty(P, dtype=torch.int32, device=dev)
    pair_rank[order] = host.clamp(max=world - 1).to(torch.int32)
    pair_slot[order] = torch.where(host < world, lslot_sorted, torch.full_like(lslot_sorted, -1)).to(torch.int32)
    if capacity is None:
        capacity = (P + El * BLOCK_ROWS + BLOCK_ROWS - 1) // BLOCK_ROWS * BLOCK_ROWS   # worst case: all pairs here
    mine = host == rank
    slot_pair = torch.full((capacity + 1,), -1, dtype=torch.int64, device=dev)
    # pairs hosted elsewhere (or beyond a user-set capacity: dropped) are routed to the spare last element
    tgt = torch.where(mine & (lslot_sorted < capacity), lslot_sorted, torch.full_like(lslot_sorted, capacity))
    slot_pair[tgt] = order
    slot_pair = slot_pair[:capacity]
    used = slot_pair >= 0
    pr = slot_pair.clamp(min=0)
    slot_src_rank = torch.where(used, pr // (T * k), torch.zeros_like(pr)).to(torch.int32)
    slot_src_row = torch.where(used, (pr // k) % T, torch.full_like(pr, -1)).to(torch.int32)
    pair_slot = torch.where(pair_slot >= capacity, torch.full_like(pair_slot, -1), pair_slot)
    # per-block expert of my buffer
    e0 = rank * El
    local_ends = ends[e0:e0 + El] - rank_base[rank]               # padded end of my experts, local coordinates
    blk = torch.arange(capacity // BLOCK_ROWS, device=dev) * BLOCK_ROWS
    g = torch.searchsorted(local_ends, blk, right=True)
    tile_group = torch.where(g < El, g, torch.full_like(g, -1)).to(torch.int32)
    group_rows = torch.cat([torch.zeros(1, dtype=local_ends.dtype, device=dev), local_ends]).clamp(max=capacity)
    num_experts = real_experts
    return MoeLayout(world, rank, num_experts, k, T, capacity, pair_rank, pair_slot, slot_src_rank, slot_src_row,
                     slot_pair, tile_group.contiguous(), group_rows.to(torch.int32).contiguous())


# ---------------------------------------------------------------------------------------------
# expert-parallel context: symmetric staging buffers + barrier
# ---------------------------------------------------------------------------------------------
class ExpertParallel:
    """Group of ranks that share the experts of every MoE layer.  ``comm`` is the peer-memory communicator of the
    group (CUDA); without one (CPU / gloo, or a single rank) rows move through ``all_gather`` or stay local."""

    def __init__(self, group=None, comm=None, max_tokens: int = 0, hidden: int = 0, max_slots: int = 0):
        import torch.distributed as dist
        self.group, self.comm = group, comm
        self.world = dist.get_world_size(group) if (group is not None and dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.stage_x = self.stage_slots = None
        if comm is not None and self.world > 1:
            self.stage_x = comm.alloc(max_tokens * hidden, torch.bfloat16)
            self.stage_slots = comm.alloc(max_slots * hidden, torch.bfloat16)
            comm.barrier()

    @property
    def peer_memory(self) -> bool:
        return self.stage_x is not None

    def barrier(self) -> None:
        if self.peer_memory:
            self.comm.barrier()

    def all_gather(self, t: torch.Tensor) -> torch.Tensor:
        """``[...]`` -> ``[world, ...]``."""
        if self.world == 1:
            return t.unsqueeze(0)
        import torch.distributed as dist
        out = torch.empty(self.world * t.numel(), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, t.contiguous().reshape(-1), group=self.group)
        return out.reshape(self.world, *t.shape)

    def _ptrs(self, staged: Optional[torch.Tensor], local: torch.Tensor):
        if staged is not None:
            return self.comm.peers_of(staged).ptr_array, self.world
        return (ctypes.c_void_p * 1)(local.data_ptr()), 1

    def _stage(self, buf: torch.Tensor, t: torch.Tensor) -> torch.Tensor:
        n = t.numel()
        assert n <= buf.numel(), "expert-parallel staging buffer too small"
        buf[:n].copy_(t.reshape(-1))
        return buf

    # ---- the three row movers ----------------------------------------------------------------------
    def gather_rows(self, src: torch.Tensor, src_rank: torch.Tensor, src_row: torch.Tensor,
                    scale: Optional[torch.Tensor], use_slots_stage: bool = False) -> torch.Tensor:
        """``out[i] = scale[i] * src@rank[src_rank[i]][src_row[i]]`` (zero rows where ``src_row < 0``)."""
        M, H = src_row.shape[0], src.shape[1]
        if not src.is_cuda:
            full = self.all_gather(src) if self.world > 1 else src.unsqueeze(0)
            rows = full[src_rank.long().clamp(min=0), src_row.long().clamp(min=0)]
            rows = rows * (src_row >= 0).to(rows.dtype)[:, None]
            return rows * scale.to(rows.dtype)[:, None] if scale is not None else rows
        staged = None
        if self.peer_memory:
            staged = self._stage(self.stage_slots if use_slots_stage else self.stage_x, src)
            self.barrier()
        ptrs, world = self._ptrs(staged, src.contiguous())
        out = torch.empty(M, H, dtype=src.dtype, device=src.device)
        L = _lib.get_lib()
        _lib.check(L.sb_moe_gather_rows(ptrs, world, _lib.ptr(src_rank if world > 1 else None), _lib.ptr(src_row),
                                        _lib.ptr(scale), _lib.ptr(out), M, H, _lib.stream()), "sb_moe_gather_rows")
        self.barrier()          # peers have finished reading my staging buffer
        return out

    def combine(self, y: torch.Tensor, pair_rank: torch.Tensor, pair_slot: torch.Tensor, w: Optional[torch.Tensor],
                T: int, k: int, use_slots_stage: bool = True) -> torch.Tensor:
        """``out[t] = sum_j w[t,j] * y@rank[pair_rank[t,j]][pair_slot[t,j]]``."""
        H = y.shape[1]
        if not y.is_cuda:
            full = self.all_gather(y) if self.world > 1 else y.unsqueeze(0)
            rows = full[pair_rank.long().clamp(min=0), pair_slot.long().clamp(min=0)].float()
            rows = rows * (pair_slot >= 0).float()[:, None]
            if w is not None:
                rows = rows * w.reshape(-1).float()[:, None]
            return rows.reshape(T, k, H).sum(1).to(y.dtype)
        staged = None
        if self.peer_memory:
            staged = self._stage(self.stage_slots if use_slots_stage else self.stage_x, y)
            self.barrier()
        ptrs, world = self._ptrs(staged, y.contiguous())
        out = torch.empty(T, H, dtype=y.dtype, device=y.device)
        L = _lib.get_lib()
        _lib.check(L.sb_moe_combine(ptrs, world, _lib.ptr(pair_rank if world > 1 else None), _lib.ptr(pair_slot),
                                    _lib.ptr(w.reshape(-1).float().contiguous() if w is not None else None),
                                    _lib.ptr(out), T, k, H, _lib.stream()), "sb_moe_combine")
        self.barrier()
        return out

    def pair_dot(self, y: torch.Tensor, pair_rank: torch.Tensor, pair_slot: torch.Tensor, dout: torch.Tensor,
                 T: int, k: int) -> torch.Tensor:
        """``dots[t,j] = <dout[t], y@rank[...][slot]>`` fp32 ``[T, k]``."""
        H = y.shape[1]
        if not y.is_cuda:
            full = self.all_gather(y) if self.world > 1 else y.unsqueeze(0)
            rows = full[pair_rank.long().clamp(min=0), pair_slot.long().clamp(min=0)].float()
            rows = rows * (pair_slot >= 0).float()[:, None]
            return (rows.reshape(T, k, H) * dout.float()[:, None, :]).sum(-1)
        staged = None
        if self.peer_memory:
            staged = self._stage(self.stage_slots, y)
            self.barrier()
        ptrs, world = self._ptrs(staged, y.contiguous())
        dots = torch.empty(T, k, dtype=torch.float32, device=y.device)
        L = _lib.get_lib()
        _lib.check(L.sb_moe_pair_dot(ptrs, world, _lib.ptr(pair_rank if world > 1 else None), _lib.ptr(pair_slot),
                                     _lib.ptr(dout.contiguous()), _lib.ptr(dots), T, k, H, _lib.stream()),
                   "sb_moe_pair_dot")
        self.barrier()
        return dots


# ---------------------------------------------------------------------------------------------
# grouped GEMM (all local experts in one launch)
# ---------------------------------------------------------------------------------------------
_EPI_BF16, _EPI_F32_ACC, _EPI_F32 = 0, 1, 2


def _grouped(A, B2d, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, epi, tile_group, b_group_rows, group_rows, groups,
             c_stride) -> None:
    L = _lib.get_lib()
    ll = ctypes.c_longlong
    _lib.check(L.sb_gemm_grouped_bf16(_lib.ptr(A), _lib.ptr(B2d), _lib.ptr(C), M, N, K, ll(lda), ll(ldb), ll(ldc),
                                      a_mn, b_mn, epi, 0, _lib.ptr(tile_group), ll(b_group_rows),
                                      _lib.ptr(group_rows), groups, ll(c_stride),
                                      _lib.ptr(_lib.status_word(A.device)), _lib.stream()), "sb_gemm_grouped_bf16")


class _GroupedLinear(torch.autograd.Function):
    """``ys[rows of expert e] = xs[rows of expert e] @ W[e]^T`` for expert-sorted, 128-padded rows."""

    @staticmethod
    def forward(ctx, xs, W, tile_group, group_rows):
        E, N, K = W.shape
        M = xs.shape[0]
        out = torch.empty(M, N, dtype=xs.dtype, device=xs.device)
        _grouped(xs, W, out, M, N, K, K, K, N, 0, 0, _EPI_BF16, tile_group, N, None, E, 0)
        ctx.save_for_backward(xs, W, tile_group, group_rows)
        ctx.w_ref = W
        return out

    @staticmethod
    def backward(ctx, dy):
        xs, W, tile_group, group_rows = ctx.saved_tensors
        E, N, K = W.shape
        M = xs.shape[0]
        dy = dy.contiguous()
        dxs = dW = None
        if ctx.needs_input_grad[0]:
            dxs = torch.empty(M, K, dtype=xs.dtype, device=xs.device)
            # contraction over N: B = W[e] seen as [N (contraction rows), K] MN-major, groups stacked along rows
            _grouped(dy, W, dxs, M, K, N, N, K, K, 0, 1, _EPI_BF16, tile_group, N, None, E, 0)
        if ctx.needs_input_grad[1]:
            mg = getattr(ctx.w_ref, "main_grad", None)
            if mg is not None:
                _grouped(dy, xs, mg, N, K, M, N, K, K, 1, 1, _EPI_F32_ACC, None, 0, group_rows, E, N * K)
            else:
                acc = torch.zeros(E, N, K, dtype=torch.float32, device=xs.device)
                _grouped(dy, xs, acc, N, K, M, N, K, K, 1, 1, _EPI_F32_ACC, None, 0, group_rows, E, N * K)
                dW = acc.to(W.dtype)
        return dxs, dW, None, None


def grouped_linear(xs: torch.Tensor, W: torch.Tensor, layout: MoeLayout) -> torch.Tensor:
    """``xs [capacity, K]`` expert-sorted rows, ``W [E_local, N, K]`` -> ``[capacity, N]``.  Rows of unused
    128-row blocks are left unwritten."""
    if not xs.is_cuda:
        out = torch.zeros(xs.shape[0], W.shape[1], dtype=xs.dtype, device=xs.device)
        rows = layout.group_rows.tolist()
        for e in range(W.shape[0]):
            if rows[e + 1] > rows[e]:
                out[rows[e]:rows[e + 1]] = xs[rows[e]:rows[e + 1]] @ W[e].t()
        return out
    return _GroupedLinear.apply(xs.contiguous(), W, layout.tile_group, layout.group_rows)


# ---------------------------------------------------------------------------------------------
# differentiable dispatch / combine
# ---------------------------------------------------------------------------------------------
class _Dispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, ep, layout):
        ctx.ep, ctx.layout = ep, layout
        return ep.gather_rows(x, layout.slot_src_rank, layout.slot_src_row, None)

    @staticmethod
    def backward(ctx, dxs):
        ep, lay = ctx.ep, ctx.layout
        pr, ps = lay.my_pairs()
        return ep.combine(dxs.contiguous(), pr, ps, None, lay.tokens_per_rank, lay.top_k), None, None


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ys, w, w_all, ep, layout):
        ctx.ep, ctx.layout = ep, layout
        pr, ps = layout.my_pairs()
        ctx.save_for_backward(ys, w_all)
        return ep.combine(ys, pr, ps, w, layout.tokens_per_rank, layout.top_k)

    @staticmethod
    def backward(ctx, dout):
        ep, lay = ctx.ep, ctx.layout
        ys, w_all = ctx.saved_tensors
        pr, ps = lay.my_pairs()
        dout = dout.contiguous()
        # d ys[slot] = w[pair of slot] * dout[token of slot]  (pulled from the rank that owns the token)
        scale = torch.where(lay.slot_pair >= 0, w_all.reshape(-1)[lay.slot_pair.clamp(min=0)],
                            torch.zeros((), dtype=w_all.dtype, device=w_all.device)).float().contiguous()
        dys = ep.gather_rows(dout, lay.slot_src_rank, lay.slot_src_row, scale)
        dw = ep.pair_dot(ys, pr, ps, dout, lay.tokens_per_rank, lay.top_k)
        return dys, dw, None, None, None


def dispatch(x: torch.Tensor, ep: ExpertParallel, layout: MoeLayout) -> torch.Tensor:
    return _Dispatch.apply(x.contiguous(), ep, layout)


def combine(ys: torch.Tensor, w: torch.Tensor, w_all: torch.Tensor, ep: ExpertParallel, layout: MoeLayout):
    """``w [T, k]`` routing weights of the local tokens (differentiable), ``w_all [world, T, k]`` their all-gathered
    values (used for the backward of remote rows)."""
    return _Combine.apply(ys, w.float(), w_all, ep, layout)



# ---------------------------------------------------------------------------------------------
# router: softmax + top-k (+ renormalisation) and its backward in one kernel each
# ---------------------------------------------------------------------------------------------
_ROUTE_MAX_EXPERTS = 256


def route_topk_reference(logits: torch.Tensor, top_k: int, norm_topk_prob: bool):
    """fp32 softmax over experts, top-k probabilities (renormalised to sum 1 if asked) and expert ids."""
    probs = torch.softmax(logits.float(), dim=-1)
    w, idx = torch.topk(probs, top_k, dim=-1)
    if norm_topk_prob:
        w = w / w.sum(-1, keepdim=True)
    return w, idx


class _RouteTopk(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits: torch.Tensor, top_k: int, norm: bool):
        T, E = logits.shape
        lg = logits if logits.stride(-1) == 1 else logits.contiguous()
        w = torch.empty(T, top_k, dtype=torch.float32, device=logits.device)
        idx = torch.empty(T, top_k, dtype=torch.int32, device=logits.device)
        L = _lib.get_lib()
        _lib.check(L.sb_moe_route_topk(_lib.ptr(lg), int(lg.dtype == torch.bfloat16), lg.stride(0), _lib.ptr(w),
                                       _lib.ptr(idx), T, E, top_k, int(norm), _lib.stream()), "sb_moe_route_topk")
        ctx.save_for_backward(lg, idx)
        ctx.norm, ctx.top_k = bool(norm), top_k
        ctx.mark_non_differentiable(idx)
        return w, idx

    @staticmethod
    def backward(ctx, dw, _didx):
        lg, idx = ctx.saved_tensors
        T, E = lg.shape
        dlog = torch.empty(T, E, dtype=torch.float32, device=lg.device)
        L = _lib.get_lib()
        _lib.check(L.sb_moe_route_topk_bwd(_lib.ptr(lg), int(lg.dtype == torch.bfloat16), lg.stride(0), _lib.ptr(idx),
                                           _lib.ptr(dw.float().contiguous()), _lib.ptr(dlog), T, E, ctx.top_k,
                                           int(ctx.norm), _lib.stream()), "sb_moe_route_topk_bwd")
        return dlog.to(lg.dtype), None, None


def route_topk(logits: torch.Tensor, top_k: int, norm_topk_prob: bool = True):
    """``logits [T, E]`` (bf16 or fp32) -> ``(weights [T, k] fp32, expert ids [T, k] int64)``.  On a GPU one warp per
    token does the softmax, the k arg-max rounds (ties to the lower expert id) and the renormalisation; the backward
    recomputes the softmax from the logits.  Replaces softmax + topk + sum + div (4 launches and two ``[T, E]`` fp32
    temporaries) of the library path."""
    if logits.is_cuda and logits.shape[1] <= _ROUTE_MAX_EXPERTS and top_k <= 32 \
            and logits.dtype in (torch.bfloat16, torch.float32):
        w, idx = _RouteTopk.apply(logits, top_k, norm_topk_prob)
        return w, idx.long()
    return route_topk_reference(logits, top_k, norm_topk_prob)
