"""Expert-parallel wrapper around the grouped operators: shards the experts of one MoE layer
evenly over the ranks of a process group (one process per GPU) and moves routed rows to the GPU
that owns their expert and back with one variable-size all-to-all each way (NCCL over NVLink /
NVSwitch on GPUs; the same code runs on CPU tensors over gloo, which is how its bookkeeping is
tested without GPUs).

The reference has no multi-GPU path; its contract for one GPU is "rows pre-sorted by expert +
int64 expert ids + int32 cumulative end offsets" (reference: csrc/mmq_hip.cu:325-406), and this
module produces exactly that on every rank for the experts it owns.

Layout.  Expert ``e`` lives on rank ``e // (E / world)``.  A routed row is one (token, slot) pair.
``dispatch`` sorts the local routed rows by global expert id (which is also rank-major), exchanges
the per-expert counts, then the rows; the receiver re-orders what it got (source-rank-major) into
expert-major order with a permutation computed from the count matrix.  ``combine`` runs the same
plan backwards.  The plan (permutations, split sizes, offsets) is built once per routing and
reused by the forward and backward exchanges of a step.

The split sizes of an all-to-all must be known on the host, so building a plan reads one small
integer matrix (world x world) back from the device; nothing else synchronises.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass
class DispatchPlan:
    """Everything needed to move rows to their experts and back for one routing decision."""

    top_k: int
    send_perm: torch.Tensor          # [R_local] routed-row index (token * top_k + slot), sorted by expert
    send_splits: list                # rows sent to each rank
    recv_splits: list                # rows received from each rank
    recv_perm: torch.Tensor          # [R_recv] position in the received buffer of each expert-major row
    expert_indices: torch.Tensor     # int64 [E_local] local expert ids 0..E_local-1
    expert_offsets: torch.Tensor     # int32 [E_local] cumulative end rows in expert-major order
    rows_local: int                  # R_local
    rows_recv: int                   # R_recv
    pair_to_sorted: torch.Tensor = None   # [R_local] inverse of send_perm
    recv_inv: torch.Tensor = None         # [R_recv] inverse of recv_perm


def _native_rows(t: torch.Tensor) -> bool:
    """True when the hand-written gather / combine kernels apply (CUDA, bf16, 16-byte rows)."""
    return t.is_cuda and t.dtype == torch.bfloat16 and t.dim() == 2 and t.shape[1] % 8 == 0 and t.is_contiguous()


class ExpertParallel:
    """Row exchange for expert-parallel grouped matmuls over ``group`` (None = default group)."""

    def __init__(self, num_experts: int, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if num_experts % self.world:
            raise ValueError(f"{num_experts} experts do not divide over {self.world} ranks")
        self.num_experts = num_experts
        self.experts_per_rank = num_experts // self.world

    # ------------------------------------------------------------------ plan
    def plan(self, topk_ids: torch.Tensor) -> DispatchPlan:
        """``topk_ids``: integer [tokens, top_k] global expert ids (each in [0, num_experts)) of
        this rank's tokens."""
        if topk_ids.dim() != 2:
            raise ValueError("topk_ids must have shape [tokens, top_k]")
        device = topk_ids.device
        W, EL = self.world, self.experts_per_rank
        if topk_ids.is_cuda and self.num_experts <= 4096:
            # device counting sort (routing.cu): permutation, its inverse and the per-expert ends
            from . import native

            flat = topk_ids.reshape(-1).to(torch.int32)
            # ids outside [0, E) are left out of the sort: their entries must not stay uninitialised
            pre = {"s2p": torch.full((flat.numel(),), -1, dtype=torch.int32, device=device)}
            send_perm, pair_to_sorted, _, ends = native.route_sort(flat, self.num_experts, out=pre)
            ends = ends.to(torch.int64)
            send_counts = (ends - torch.cat([ends.new_zeros(1), ends[:-1]])).reshape(W, EL)
        else:
            flat = topk_ids.reshape(-1).to(torch.int64)
            send_perm = torch.argsort(flat, stable=True)
            pair_to_sorted = torch.empty_like(send_perm)
            pair_to_sorted[send_perm] = torch.arange(flat.numel(), device=device)
            send_counts = torch.bincount(flat, minlength=self.num_experts).reshape(W, EL)
        if W > 1:
            recv_counts = torch.empty_like(send_counts)
            dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        else:
            recv_counts = send_counts
        # the one device-to-host read: per-rank totals in both directions
        totals = torch.stack([send_counts.sum(1), recv_counts.sum(1)]).cpu()
        send_splits = [int(v) for v in totals[0]]
        recv_splits = [int(v) for v in totals[1]]
        if sum(send_splits) != flat.numel():
            raise ValueError(f"topk_ids holds {flat.numel() - sum(send_splits)} expert ids outside [0, {self.num_experts})")
        rows_recv = sum(recv_splits)
        # received buffer order: (source rank, local expert, arrival); wanted: (local expert, source rank, arrival)
        cnt = recv_counts.reshape(-1)                          # index s * EL + e
        seg_start = torch.cumsum(cnt, 0) - cnt                 # start of segment (s, e) in the received buffer
        cnt_em = recv_counts.t().contiguous().reshape(-1)      # index e * W + s
        seg_start_em = seg_start.reshape(W, EL).t().contiguous().reshape(-1)
        out_start = torch.cumsum(cnt_em, 0) - cnt_em           # start of segment (e, s) in expert-major order
        seg_of_row = torch.repeat_interleave(torch.arange(W * EL, device=device), cnt_em, output_size=rows_recv)
        within = torch.arange(rows_recv, device=device) - out_start[seg_of_row]
        recv_perm = seg_start_em[seg_of_row] + within
        recv_inv = torch.empty_like(recv_perm)
        recv_inv[recv_perm] = torch.arange(rows_recv, device=device)
        if topk_ids.is_cuda:
            recv_perm, recv_inv = recv_perm.to(torch.int32), recv_inv.to(torch.int32)
        expert_offsets = torch.cumsum(recv_counts.sum(0), 0).to(torch.int32)
        expert_indices = torch.arange(EL, device=device, dtype=torch.int64)
        return DispatchPlan(topk_ids.shape[1], send_perm, send_splits, recv_splits, recv_perm, expert_indices,
                            expert_offsets, int(flat.numel()), rows_recv, pair_to_sorted, recv_inv)

    # ------------------------------------------------------------------ exchanges
    def _all_to_all(self, send: torch.Tensor, out_rows: int, out_splits, in_splits) -> torch.Tensor:
        recv = send.new_empty((out_rows, send.shape[1]))
        if self.world > 1:
            dist.all_to_all_single(recv, send, output_split_sizes=out_splits, input_split_sizes=in_splits,
                                   group=self.group)
        else:
            recv.copy_(send)
        return recv

    @staticmethod
    def _gather(src: torch.Tensor, index: torch.Tensor, divisor: int = 1) -> torch.Tensor:
        """out[r] = src[index[r] // divisor]; the CUDA kernel for bf16 rows, torch otherwise."""
        if _native_rows(src) and index.dtype == torch.int32:
            from . import native

            return native.gather_rows(src, index, divisor)
        idx = index.long()
        if divisor != 1:
            idx = torch.div(idx, divisor, rounding_mode="floor")
        return src.index_select(0, idx)

    def dispatch_tokens(self, plan: DispatchPlan, x: torch.Tensor) -> torch.Tensor:
        """[tokens, width] -> [R_recv, width]: each token row replicated to its top_k experts,
        delivered to the owning ranks, expert-major."""
        return self.dispatch_rows_sorted(plan, self._gather(x, plan.send_perm, plan.top_k))

    def dispatch_rows(self, plan: DispatchPlan, rows: torch.Tensor) -> torch.Tensor:
        """[R_local, width] per routed row (token-major, slot-minor) -> [R_recv, width] expert-major."""
        return self.dispatch_rows_sorted(plan, self._gather(rows, plan.send_perm))

    def dispatch_rows_sorted(self, plan: DispatchPlan, rows_sorted: torch.Tensor) -> torch.Tensor:
        recv = self._all_to_all(rows_sorted.contiguous(), plan.rows_recv, plan.recv_splits, plan.send_splits)
        if self.world == 1:
            return recv  # one rank: the sorted order already is expert-major
        return self._gather(recv, plan.recv_perm)

    def _return_sorted(self, plan: DispatchPlan, rows: torch.Tensor) -> torch.Tensor:
        """[R_recv, width] expert-major -> [R_local, width] in this rank's send (sorted) order."""
        if self.world == 1:
            return rows
        buf = self._gather(rows.contiguous(), plan.recv_inv)
        return self._all_to_all(buf, plan.rows_local, plan.send_splits, plan.recv_splits)

    def combine_rows(self, plan: DispatchPlan, rows: torch.Tensor) -> torch.Tensor:
        """Inverse of ``dispatch_rows``: [R_recv, width] expert-major -> [R_local, width] per routed row."""
        return self._gather(self._return_sorted(plan, rows), plan.pair_to_sorted)

    def combine_tokens(self, plan: DispatchPlan, rows: torch.Tensor, weights: torch.Tensor | None = None):
        """``combine_rows`` followed by the sum over the top_k slots of every token (optionally
        weighted by [tokens, top_k] routing weights), accumulated in fp32 and rounded once."""
        back = self._return_sorted(plan, rows)
        if _native_rows(back) and plan.pair_to_sorted.dtype == torch.int32:
            from . import native

            w = None if weights is None else weights.reshape(-1).float().contiguous()
            return native.combine_rows(back, plan.pair_to_sorted, plan.top_k, w)
        per_row = back.index_select(0, plan.pair_to_sorted.long()).reshape(-1, plan.top_k, rows.shape[1]).float()
        if weights is not None:
            per_row = per_row * weights.reshape(-1, plan.top_k, 1).float()
        return per_row.sum(1).to(rows.dtype)

    # ------------------------------------------------------------------ sharding helper
    def local_experts(self, packed: torch.Tensor) -> torch.Tensor:
        """The slice [E_local, N, row_bytes] of a full grouped weight that this rank owns."""
        lo = self.rank * self.experts_per_rank
        return packed[lo:lo + self.experts_per_rank].contiguous()


__all__ = ["DispatchPlan", "ExpertParallel"]
