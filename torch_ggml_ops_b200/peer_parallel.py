"""Expert-parallel grouped matmul with the row exchange done by this library's own kernels over
peer memory (NVLink / NVSwitch) instead of NCCL all-to-alls.

One process per GPU.  Every rank owns four receive / result buffers that its peers can address
(torch symmetric memory; plain tensors on one rank).  A step is

    route_sort -> all_gather(counts) -> tgo_ep_plan             (where does every routed pair go)
    tgo_ep_dispatch(x)   | fence | grouped forward  | fence | tgo_ep_pull(y)
    tgo_ep_dispatch(dy)  | fence | grouped dX       | fence | tgo_ep_pull(dx, summed over top-k)

Rows cross NVLink exactly once per exchange, written (dispatch) or read (pull) by plain 16-byte
peer stores / loads straight into / out of the expert-major layout the grouped kernels consume, so
there is no permutation pass on either side and no host read of the routing: the grouped kernels
are launched over the whole receive buffer (`capacity` rows) and the device-side group offsets say
which rows exist.

Token-level exchange (when ``tokens_per_rank`` and ``top_k`` are given): the two wide exchanges
move one row per (token, destination GPU) instead of one per routed pair - a token's row goes once
to every GPU that owns one of its experts and is replicated into the expert-major buffer there
(tgo_ep_dispatch_tokens + tgo_ep_expand), and the input gradient comes back as one partial sum per
GPU (tgo_ep_reduce + tgo_ep_pull_tokens).  With 8 experts per token this cuts the NVLink bytes of
those exchanges by 4x on 2 GPUs and 2.2x on 4.  "fence" orders the ranks' phases: by default a one-block
barrier kernel over peer memory with a bounded wait (tgo_ep_barrier), optionally a stream-ordered
one-element all-reduce (fences="nccl"); the exchange kernels themselves never wait.  Multicast is never used (the symmetric-memory
allocator is told not to bind a multicast object).

The reference has no multi-GPU path; the per-rank contract it defines (rows sorted by expert +
int64 expert ids + int32 cumulative end offsets, csrc/mmq_hip.cu:325-406) is what each rank's
buffers satisfy.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from . import native


class PeerExpertParallel:
    """Fused dispatch / grouped matmul / combine for one MoE projection [E, N, K] of quant type
    ``quant_type``; ``local_weight`` is this rank's shard [E / world, N, row_bytes] (uint8, CUDA)."""

    def __init__(self, local_weight: torch.Tensor, quant_type: int, num_experts: int, out_features: int,
                 in_features: int, capacity_rows: int, group=None, tokens_per_rank: int | None = None,
                 top_k: int | None = None, fences: str = "peer", push_forward: bool = True):
        """``fences``: how the ranks' phases are ordered - "peer": this library's barrier kernel over
        peer memory (bounded wait, no collective library in the step); "nccl": one-element all-reduces
        and an all-gather of the counts.  ``push_forward`` (token-level exchange only): the forward
        matmul's epilogue stores every routed pair's row straight into the memory of the GPU that owns
        the token (tgo_grouped_fwd_rows), instead of a local result buffer that the owners pull from
        afterwards; ``forward`` then returns a view of this rank's result buffer."""
        if fences not in ("peer", "nccl"):
            raise ValueError("fences must be 'peer' or 'nccl'")
        self.fences = fences
        self._epoch = 0
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if num_experts % self.world:
            raise ValueError(f"{num_experts} experts do not divide over {self.world} ranks")
        if local_weight.shape[0] != num_experts // self.world:
            raise ValueError("local_weight must hold this rank's num_experts / world experts")
        self.weight, self.qt = local_weight, int(quant_type)
        self.E, self.EL = num_experts, num_experts // self.world
        self.N, self.K, self.cap = int(out_features), int(in_features), int(capacity_rows)
        dev = local_weight.device
        self.device = dev
        # (rows, columns, dtype) of every buffer the peers address
        shapes = {"x_in": (self.cap, self.K, torch.bfloat16), "y_out": (self.cap, self.N, torch.bfloat16),
                  "dy_in": (self.cap, self.N, torch.bfloat16), "dx_out": (self.cap, self.K, torch.bfloat16)}
        self.token_level = tokens_per_rank is not None and top_k is not None
        shapes.update({"flags": (1, max(self.world, 2), torch.int32), "counts_tab": (self.world, self.E, torch.int32)})
        if self.token_level:
            self.tpr, self.top_k = int(tokens_per_rank), int(top_k)
            slots = self.world * self.tpr
            shapes.update({"tok_in": (slots, self.K, torch.bfloat16), "dx_part": (slots, self.K, torch.bfloat16),
                           "row_slot": (self.cap, 1, torch.int32), "slot_rows": (slots, self.top_k, torch.int32)})
            if push_forward and self.N % 8 == 0:
                shapes["y_tok"] = (self.tpr * self.top_k, self.N, torch.bfloat16)
        self.buf, self.peers = {}, {}
        if self.world > 1:
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm_mem

            for name, (rows, cols, dtype) in shapes.items():
                t = symm_mem.empty(rows, cols, dtype=dtype, device=dev)
                hdl = symm_mem.rendezvous(t, dist.group.WORLD if group is None else group)
                self.buf[name] = t
                self.peers[name] = [int(p) for p in hdl.buffer_ptrs]
                self.buf[name + "_hdl"] = hdl  # keeps the mapping alive
        else:
            for name, (rows, cols, dtype) in shapes.items():
                t = torch.empty(rows, cols, dtype=dtype, device=dev)
                self.buf[name] = t
                self.peers[name] = [t.data_ptr()]
        self.buf["flags"].zero_()
        if self.token_level:
            # a slot nobody has written yet must not name a row, and a row nobody has announced must
            # not name a slot outside the token buffer
            self.buf["slot_rows"].fill_(-1)
            self.buf["row_slot"].fill_(-1)
        if self.world > 1:
            # peers write into these buffers from their first plan on, so everybody finishes the
            # fills before anybody goes on
            torch.cuda.synchronize()
            dist.barrier(group=group)
        self.push = "y_tok" in self.buf
        if self.push:
            self.row_ptrs = torch.zeros(self.cap, dtype=torch.int64, device=dev)
        self.ws = torch.empty(native.grouped_workspace_bytes(self.cap, self.EL), dtype=torch.uint8, device=dev)
        self._token = torch.zeros(1, dtype=torch.int32, device=dev)
        self.overflow = None
        self._plan_bufs = None   # routing outputs are reused from step to step (stream-ordered)
        self.marks = None        # set to a list to collect (phase name, CUDA event) pairs, see `phase_times`

    # ------------------------------------------------------------------ phase timing (diagnostics)
    def _mark(self, name: str) -> None:
        if self.marks is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.marks.append((name, ev))

    def phase_times(self, step) -> dict:
        """Runs ``step()`` (a callable that calls plan / forward / grad_input of this object) once with a
        CUDA event after every phase and returns {phase: milliseconds} on this rank.  Not for timed
        regions: the events add launches."""
        step()            # keeps the GPU busy while the marked step is enqueued (the host stays ahead, as in a loop)
        self.marks = []
        self._mark("start")
        step()
        torch.cuda.synchronize()
        marks, self.marks = self.marks, None
        out = {}
        for (_, e0), (name, e1) in zip(marks[:-1], marks[1:]):
            out[name] = out.get(name, 0.0) + e0.elapsed_time(e1)
        return out

    # ------------------------------------------------------------------ ordering between ranks
    def _fence(self) -> None:
        """All ranks have finished everything they enqueued before this point (stream-ordered)."""
        if self.world == 1:
            return
        if self.fences == "peer":
            self._epoch += 1
            native.ep_barrier(self.peers["flags"], self.rank, self._epoch)
        else:
            dist.all_reduce(self._token, group=self.group)

    # ------------------------------------------------------------------ routing
    def plan(self, topk_ids: torch.Tensor):
        """``topk_ids``: integer [tokens, top_k] global expert ids on this rank's GPU (int32 avoids a
        conversion).  The returned plan refers to buffers that the next call of ``plan`` overwrites."""
        flat = topk_ids.reshape(-1)
        if flat.dtype != torch.int32:
            flat = flat.to(torch.int32)
        n = flat.numel()
        if self._plan_bufs is None or self._plan_bufs["n"] != n:
            dev, i32 = self.device, torch.int32
            self._plan_bufs = {
                "n": n,
                "s2p": torch.empty(n, dtype=i32, device=dev), "p2s": torch.empty(n, dtype=i32, device=dev),
                "ei": torch.empty(self.E, dtype=torch.int64, device=dev), "eo": torch.empty(self.E, dtype=i32, device=dev),
                "counts": torch.empty(self.E, dtype=i32, device=dev),
                "ws": torch.empty(native.lib().tgo_route_workspace_bytes(n, self.E), dtype=torch.uint8, device=dev),
                "counts_all": torch.empty(self.world, self.E, dtype=i32, device=dev),
                "dst_rank": torch.empty(n, dtype=i32, device=dev), "dst_row": torch.empty(n, dtype=i32, device=dev),
                "li": torch.empty(self.EL, dtype=torch.int64, device=dev), "lo": torch.empty(self.EL, dtype=i32, device=dev),
                "scratch": torch.empty(2 * self.E, dtype=i32, device=dev),
                "overflow": torch.zeros(1, dtype=i32, device=dev),
            }
        if self.token_level and (topk_ids.shape[1] != self.top_k or topk_ids.shape[0] > self.tpr):
            # every rank must take the same kind of exchange: a rank that fell back to one row per
            # pair on its own would leave the owners' row -> slot maps unwritten
            raise ValueError(f"this exchange was set up for top_k = {self.top_k} and at most {self.tpr} tokens per rank; "
                             f"got top_k = {topk_ids.shape[1]}, {topk_ids.shape[0]} tokens")
        b = self._plan_bufs
        b["overflow"].zero_()   # the flag describes this plan only
        _, p2s, _, _ = native.route_sort(flat, self.E, out=b)
        if self.world > 1 and self.fences == "peer":
            # every rank writes its counts into every rank's table; the barrier also tells this rank
            # that the peers' previous step is over before their maps are rewritten below
            native.ep_share_counts(b["counts"], self.rank, self.peers["counts_tab"])
            self._fence()
            counts_all = self.buf["counts_tab"]
        elif self.world > 1:
            counts_all = b["counts_all"]
            dist.all_gather_into_tensor(counts_all, b["counts"], group=self.group)
        else:
            counts_all = b["counts"].reshape(1, self.E)
        dst_rank, dst_row, li, lo, overflow = native.ep_plan(counts_all, self.rank, flat, p2s, self.cap, out=b)
        self._mark("plan")
        self.overflow = overflow  # device flag: a row did not fit in `capacity_rows` (read it when convenient)
        plan = {"top_k": topk_ids.shape[1], "tokens": topk_ids.shape[0], "dst_rank": dst_rank, "dst_row": dst_row,
                "indices": li, "offsets": lo, "token_level": False}
        if self.token_level:
            # the peers' maps are rewritten here; the exchanges that read them come after a fence
            if self.push:
                # nobody writes the result rows of dropped pairs: the same launch zeroes them
                native.ep_token_maps_rows(dst_rank, dst_row, plan["tokens"], self.top_k, self.rank, self.tpr,
                                          self.peers["row_slot"], self.peers["slot_rows"],
                                          self.buf["y_tok"][: plan["tokens"] * self.top_k])
            else:
                native.ep_token_maps(dst_rank, dst_row, plan["tokens"], self.top_k, self.rank, self.tpr,
                                     self.peers["row_slot"], self.peers["slot_rows"])
            plan["token_level"] = True
            plan["n_rows"] = lo[self.EL - 1:]   # device int32: rows that exist in this rank's buffers
        self._mark("plan")
        return plan

    def check_overflow(self) -> None:
        """Raises if the last plan dropped routed pairs because a receive buffer (``capacity_rows``)
        was too small: those pairs got zero outputs and contributed no gradient.  Reads one device
        integer, so it waits for the stream; call it where the host synchronises anyway."""
        if self.overflow is not None and int(self.overflow.item()) != 0:
            raise RuntimeError(f"expert-parallel receive buffer overflow: capacity_rows = {self.cap} is too small for "
                               "this routing; dropped pairs were computed as zeros")

    # ------------------------------------------------------------------ forward
    def forward(self, plan, x_tokens: torch.Tensor, out: torch.Tensor | None = None, fence: bool = True) -> torch.Tensor:
        """[tokens, K] bf16 -> [tokens * top_k, N]: every routed pair's expert projection
        (written to ``out`` when given).  ``fence=False`` (only with the forward that returns its own
        rows, and without ``out``): the call ends without the rank barrier, so the rows that peers store
        into the returned buffer are complete only after this object's next barrier - the one inside
        ``grad_input`` when that follows, as in a training step."""
        k = plan["top_k"]
        if plan["token_level"] and self.push:
            native.ep_dispatch_tokens(x_tokens, plan["dst_rank"], k, self.rank, self.tpr, self.peers["tok_in"])
            self._mark("dispatch_tokens")
            self._fence()
            self._mark("barriers")
            native.ep_expand(self.buf["tok_in"], self.buf["row_slot"], plan["n_rows"], self.buf["x_in"])
            native.ep_row_pointers(self.buf["row_slot"], self.buf["slot_rows"], plan["n_rows"], k, self.tpr,
                                   self.peers["y_tok"], self.N, self.row_ptrs)
            self._mark("expand")
            # the matmul's epilogue returns every row to the token's owner (plain 16-byte peer stores)
            native.grouped_fwd_rows(self.buf["x_in"], self.weight, self.row_ptrs, plan["indices"], plan["offsets"],
                                    self.EL, self.cap, self.N, self.K, self.qt, self.ws)
            self._mark("forward_matmul_and_return")
            if fence or out is not None:
                self._fence()
                self._mark("barriers")
            y = self.buf["y_tok"][: x_tokens.shape[0] * k]
            if out is not None:
                out.copy_(y)
                return out
            return y
        if plan["token_level"]:
            native.ep_dispatch_tokens(x_tokens, plan["dst_rank"], k, self.rank, self.tpr, self.peers["tok_in"])
            self._fence()
            native.ep_expand(self.buf["tok_in"], self.buf["row_slot"], plan["n_rows"], self.buf["x_in"])
        else:
            native.ep_dispatch(x_tokens, k, plan["dst_rank"], plan["dst_row"], self.peers["x_in"])
            self._fence()
        native.grouped_fwd(self.buf["x_in"], self.weight, None, self.buf["y_out"], None, plan["indices"],
                           plan["offsets"], self.EL, self.cap, self.N, self.K, self.qt, self.ws)
        self._fence()
        y = out if out is not None else torch.empty(x_tokens.shape[0] * k, self.N, dtype=torch.bfloat16,
                                                     device=self.device)
        native.ep_pull(self.peers["y_out"], plan["dst_rank"], plan["dst_row"], y, 1)
        return y

    # ------------------------------------------------------------------ input gradient
    def grad_input(self, plan, dy_pairs: torch.Tensor, weights: torch.Tensor | None = None,
                   out: torch.Tensor | None = None) -> torch.Tensor:
        """[tokens * top_k, N] cotangents per routed pair -> [tokens, K]: dX summed over the top-k
        slots of each token (optionally weighted), fp32 accumulation, one bf16 rounding."""
        k = plan["top_k"]
        native.ep_dispatch(dy_pairs, 1, plan["dst_rank"], plan["dst_row"], self.peers["dy_in"])
        self._mark("dispatch_dy")
        self._fence()
        self._mark("barriers")
        native.grouped_dx(self.buf["dy_in"], None, self.weight, None, self.buf["dx_out"], plan["indices"],
                          plan["offsets"], self.EL, self.cap, self.N, self.K, self.qt, self.ws)
        dx = out if out is not None else torch.empty(dy_pairs.shape[0] // k, self.K, dtype=torch.bfloat16,
                                                      device=self.device)
        if plan["token_level"] and weights is None:
            self._mark("dx_matmul")
            native.ep_reduce(self.buf["dx_out"], self.buf["slot_rows"], k, self.buf["dx_part"])
            self._mark("reduce")
            self._fence()
            self._mark("barriers")
            native.ep_pull_tokens(self.peers["dx_part"], plan["dst_rank"], k, self.rank, self.tpr, dx)
            self._mark("pull_partial_sums")
            return dx
        self._fence()
        w = None if weights is None else weights.reshape(-1).float().contiguous()
        native.ep_pull(self.peers["dx_out"], plan["dst_rank"], plan["dst_row"], dx, k, w)
        return dx


__all__ = ["PeerExpertParallel"]
