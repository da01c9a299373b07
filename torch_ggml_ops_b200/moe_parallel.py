"""Expert-parallel MoE feed-forward step built on the grouped operators: gate/up pair
(``grouped_mmq_pair``), ``silu(gate) * up``, down projection (``grouped_mmq``), weighted top-k
combine; forward and input gradient.  Experts are sharded evenly over the ranks (expert ``e`` lives
on rank ``e // (E / world)``); tokens stay with the rank that produced them.

Every exchange is at token level: a token's row goes once to every GPU that owns one of its top-k
experts and is replicated into the expert-major buffer there, and one partial sum per GPU comes
back (forward: the weighted sum of the token's down-projection rows on that GPU; backward: the sum
of its input-gradient rows).  The routing weight of a pair travels with the plan to the pair's
owner and is applied inside the activation kernels, so nothing per routed pair ever crosses NVLink.
Rows move by this library's peer-memory kernels (plain 16-byte peer stores and loads, no multicast,
no wait inside any of those kernels); the phases of different ranks are ordered by a one-block
barrier kernel over peer memory whose wait is bounded (``tgo_ep_barrier``), or by one-element
all-reduces (``fences="nccl"``).

The reference has no such block: it stops at the matmul pair and leaves activation, down
projection and combine to its caller (README.md:3, csrc/mmq_hip.cu:1054-1193); each rank's buffers
here satisfy the per-GPU contract those operators define (rows sorted by expert, int64 expert ids,
int32 cumulative end offsets: csrc/mmq_hip.cu:325-406).

``MoEMLPRank`` holds one rank's state and runs one phase at a time without any collective, so a
test can step several virtual ranks on one GPU in lockstep; ``PeerMoEMLP`` is the real thing, one
per process, with the barriers between the phases.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from . import native

PEER_BUFFERS = ("tok_in", "y_part", "dy_in", "dx_part", "row_slot", "slot_rows", "row_weight", "flags", "counts_tab")


class MoEMLPRank:
    """One rank of the expert-parallel MLP.  ``w_gate`` / ``w_up``: [E / world, ffn, row bytes] of
    quant type ``qt_gate_up`` (in_features = hidden); ``w_down``: [E / world, hidden, row bytes] of
    ``qt_down`` (in_features = ffn).  ``alloc(name, rows, cols, dtype)`` supplies the buffers the
    peers address (names in ``PEER_BUFFERS``); ``connect`` then receives every rank's pointers."""

    def __init__(self, rank, world, w_gate, w_up, w_down, qt_gate_up, qt_down, num_experts, hidden, ffn,
                 capacity_rows, tokens_per_rank, top_k, alloc=None):
        if num_experts % world:
            raise ValueError(f"{num_experts} experts do not divide over {world} ranks")
        self.rank, self.world, self.E, self.EL = int(rank), int(world), int(num_experts), num_experts // world
        for w, rows in ((w_gate, ffn), (w_up, ffn), (w_down, hidden)):
            if w.shape[0] != self.EL or w.shape[1] != rows:
                raise ValueError("expert weights must be [num_experts / world, out_features, row bytes]")
        self.wg, self.wu, self.wd = w_gate, w_up, w_down
        self.qt_gu, self.qt_d = int(qt_gate_up), int(qt_down)
        self.H, self.F, self.cap = int(hidden), int(ffn), int(capacity_rows)
        self.tpr, self.top_k = int(tokens_per_rank), int(top_k)
        self.slots = self.world * self.tpr
        dev = w_gate.device
        self.device = dev
        bf, i32 = torch.bfloat16, torch.int32
        if alloc is None:
            alloc = lambda name, rows, cols, dtype: torch.empty(rows, cols, dtype=dtype, device=dev)  # noqa: E731
        shapes = {"tok_in": (self.slots, self.H, bf), "y_part": (self.slots, self.H, bf),
                  "dy_in": (self.slots, self.H, bf), "dx_part": (self.slots, self.H, bf),
                  "row_slot": (self.cap, 1, i32), "slot_rows": (self.slots, self.top_k, i32),
                  "row_weight": (self.cap, 1, torch.float32),
                  "flags": (1, max(self.world, 2), i32), "counts_tab": (self.world, self.E, i32)}
        self.buf = {name: alloc(name, *shapes[name]) for name in PEER_BUFFERS}
        self.buf["slot_rows"].fill_(-1)   # a slot nobody has announced names no row
        self.buf["row_slot"].fill_(-1)    # a row nobody has announced names no slot
        self.buf["row_weight"].fill_(1.0)
        self.buf["flags"].zero_()         # rank barrier epochs start from zero
        # expert-major rows of this rank only; the wide buffers serve forward and backward in turn
        self.rows_a = torch.empty(self.cap, self.H, dtype=bf, device=dev)   # x rows, then dy rows
        self.rows_b = torch.empty(self.cap, self.H, dtype=bf, device=dev)   # y rows, then dx rows
        self.gate = torch.empty(self.cap, self.F, dtype=bf, device=dev)     # kept for the backward pass
        self.up = torch.empty(self.cap, self.F, dtype=bf, device=dev)
        self.h = torch.empty(self.cap, self.F, dtype=bf, device=dev)        # activation, then its gradient
        self.dgate = torch.empty(self.cap, self.F, dtype=bf, device=dev)
        self.dup = torch.empty(self.cap, self.F, dtype=bf, device=dev)
        self.ws = torch.empty(native.grouped_workspace_bytes(self.cap, self.EL), dtype=torch.uint8, device=dev)
        self.peers = None
        self._route = None
        self.plan = None

    def connect(self, peers: dict) -> None:
        """``peers[name][r]`` = device address of rank r's buffer ``name``."""
        self.peers = {k: [int(p) for p in v] for k, v in peers.items()}

    # ------------------------------------------------------------------ routing
    def route(self, topk_ids: torch.Tensor) -> torch.Tensor:
        """Sorts this rank's routed pairs by expert; returns the per-expert pair counts (int32 [E],
        on the device) that every rank needs from every other rank."""
        if topk_ids.shape[1] != self.top_k or topk_ids.shape[0] > self.tpr:
            raise ValueError(f"set up for top_k = {self.top_k} and at most {self.tpr} tokens per rank; "
                             f"got top_k = {topk_ids.shape[1]}, {topk_ids.shape[0]} tokens")
        flat = topk_ids.reshape(-1)
        if flat.dtype != torch.int32:
            flat = flat.to(torch.int32)
        n, dev, i32 = flat.numel(), self.device, torch.int32
        if self._route is None or self._route["n"] != n:
            self._route = {
                "n": n, "s2p": torch.empty(n, dtype=i32, device=dev), "p2s": torch.empty(n, dtype=i32, device=dev),
                "ei": torch.empty(self.E, dtype=torch.int64, device=dev), "eo": torch.empty(self.E, dtype=i32, device=dev),
                "counts": torch.empty(self.E, dtype=i32, device=dev),
                "ws": torch.empty(native.lib().tgo_route_workspace_bytes(n, self.E), dtype=torch.uint8, device=dev),
                "dst_rank": torch.empty(n, dtype=i32, device=dev), "dst_row": torch.empty(n, dtype=i32, device=dev),
                "li": torch.empty(self.EL, dtype=torch.int64, device=dev), "lo": torch.empty(self.EL, dtype=i32, device=dev),
                "scratch": torch.empty(2 * self.E, dtype=i32, device=dev), "overflow": torch.zeros(1, dtype=i32, device=dev)}
        b = self._route
        b["flat"], b["tokens"] = flat, topk_ids.shape[0]
        native.route_sort(flat, self.E, out=b)
        return b["counts"]

    def make_plan(self, counts_all: torch.Tensor, weights: torch.Tensor | None = None) -> None:
        """``counts_all``: int32 [world, E], row r = what ``route`` returned on rank r.  ``weights``:
        [tokens, top_k] routing weights (None = 1).  Writes the slot / row maps into the owners'
        memory: peers must have finished every phase that reads theirs."""
        b = self._route
        b["overflow"].zero_()
        dst_rank, dst_row, li, lo, overflow = native.ep_plan(counts_all, self.rank, b["flat"], b["p2s"], self.cap, out=b)
        w = None if weights is None else weights.reshape(-1).to(torch.float32).contiguous()
        native.ep_token_maps(dst_rank, dst_row, b["tokens"], self.top_k, self.rank, self.tpr, self.peers["row_slot"],
                             self.peers["slot_rows"], pair_weights=w,
                             row_weight_ptrs=None if w is None else self.peers["row_weight"])
        self.plan = {"tokens": b["tokens"], "dst_rank": dst_rank, "indices": li, "offsets": lo,
                     "n_rows": lo[self.EL - 1:], "overflow": overflow, "weighted": w is not None}

    def check_overflow(self) -> None:
        """Raises if the last plan dropped pairs because ``capacity_rows`` was too small (one device
        read: it waits for the stream)."""
        if self.plan is not None and int(self.plan["overflow"].item()) != 0:
            raise RuntimeError(f"expert-parallel receive buffer overflow: capacity_rows = {self.cap} is too small")

    # ------------------------------------------------------------------ forward
    def fwd_send(self, x_tokens: torch.Tensor) -> None:
        native.ep_dispatch_tokens(x_tokens, self.plan["dst_rank"], self.top_k, self.rank, self.tpr, self.peers["tok_in"])

    def fwd_compute(self) -> None:
        """After every rank's ``fwd_send``: this rank's experts, from token rows to partial sums."""
        p = self.plan
        scale = self.buf["row_weight"].reshape(-1) if p["weighted"] else None
        native.ep_expand(self.buf["tok_in"], self.buf["row_slot"], p["n_rows"], self.rows_a)
        native.grouped_fwd(self.rows_a, self.wg, self.wu, self.gate, self.up, p["indices"], p["offsets"], self.EL,
                           self.cap, self.F, self.H, self.qt_gu, self.ws)
        native.swiglu_fwd(self.gate, self.up, self.h, row_scale=scale, n_rows_device=p["n_rows"])
        native.grouped_fwd(self.h, self.wd, None, self.rows_b, None, p["indices"], p["offsets"], self.EL, self.cap,
                           self.H, self.F, self.qt_d, self.ws)
        native.ep_reduce(self.rows_b, self.buf["slot_rows"], self.top_k, self.buf["y_part"])

    def fwd_recv(self, out: torch.Tensor | None = None) -> torch.Tensor:
        """After every rank's ``fwd_compute``: [tokens, hidden] = sum of the owners' partial sums."""
        y = out if out is not None else torch.empty(self.plan["tokens"], self.H, dtype=torch.bfloat16, device=self.device)
        native.ep_pull_tokens(self.peers["y_part"], self.plan["dst_rank"], self.top_k, self.rank, self.tpr, y)
        return y

    # ------------------------------------------------------------------ input gradient
    def bwd_send(self, dy_tokens: torch.Tensor) -> None:
        native.ep_dispatch_tokens(dy_tokens, self.plan["dst_rank"], self.top_k, self.rank, self.tpr, self.peers["dy_in"])

    def bwd_compute(self) -> None:
        p = self.plan
        scale = self.buf["row_weight"].reshape(-1) if p["weighted"] else None
        native.ep_expand(self.buf["dy_in"], self.buf["row_slot"], p["n_rows"], self.rows_a)
        native.grouped_dx(self.rows_a, None, self.wd, None, self.h, p["indices"], p["offsets"], self.EL, self.cap,
                          self.H, self.F, self.qt_d, self.ws)                       # dh = dy * Wd
        native.swiglu_bwd(self.h, self.gate, self.up, self.dgate, self.dup, row_scale=scale, n_rows_device=p["n_rows"])
        native.grouped_dx(self.dgate, self.dup, self.wg, self.wu, self.rows_b, p["indices"], p["offsets"], self.EL,
                          self.cap, self.F, self.H, self.qt_gu, self.ws)            # dx = dgate * Wg + dup * Wu
        native.ep_reduce(self.rows_b, self.buf["slot_rows"], self.top_k, self.buf["dx_part"])

    def bwd_recv(self, out: torch.Tensor | None = None) -> torch.Tensor:
        dx = out if out is not None else torch.empty(self.plan["tokens"], self.H, dtype=torch.bfloat16, device=self.device)
        native.ep_pull_tokens(self.peers["dx_part"], self.plan["dst_rank"], self.top_k, self.rank, self.tpr, dx)
        return dx


class PeerMoEMLP:
    """The expert-parallel MLP of this process (one process per GPU, ``torch.distributed`` already
    initialised for more than one rank).  ``step`` order: ``plan`` -> ``forward`` -> ``grad_input``."""

    def __init__(self, w_gate, w_up, w_down, qt_gate_up, qt_down, num_experts, hidden, ffn, capacity_rows,
                 tokens_per_rank, top_k, group=None, fences: str = "peer"):
        """``fences``: "peer" orders the ranks' phases with this library's barrier kernel over peer
        memory (bounded wait; no collective library inside a step), "nccl" with one-element
        all-reduces and an all-gather of the counts."""
        if fences not in ("peer", "nccl"):
            raise ValueError("fences must be 'peer' or 'nccl'")
        self.fences, self._epoch = fences, 0
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        self._handles = []
        dev = w_gate.device
        if self.world > 1:
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm_mem

            ptrs = {}

            def alloc(name, rows, cols, dtype):
                t = symm_mem.empty(rows, cols, dtype=dtype, device=dev)
                hdl = symm_mem.rendezvous(t, dist.group.WORLD if group is None else group)
                self._handles.append(hdl)   # keeps the mapping alive
                ptrs[name] = [int(p) for p in hdl.buffer_ptrs]
                return t
        else:
            alloc, ptrs = None, None
        self.r = MoEMLPRank(rank, self.world, w_gate, w_up, w_down, qt_gate_up, qt_down, num_experts, hidden, ffn,
                            capacity_rows, tokens_per_rank, top_k, alloc=alloc)
        self.r.connect(ptrs if ptrs is not None else {k: [self.r.buf[k].data_ptr()] for k in PEER_BUFFERS})
        self._token = torch.zeros(1, dtype=torch.int32, device=dev)
        self._counts_all = torch.empty(self.world, num_experts, dtype=torch.int32, device=dev)
        if self.world > 1:
            torch.cuda.synchronize()
            dist.barrier(group=group)   # everybody has filled its maps before anybody writes into them

    def _fence(self) -> None:
        """All ranks have finished everything they enqueued before this point (stream-ordered)."""
        if self.world == 1:
            return
        if self.fences == "peer":
            self._epoch += 1
            native.ep_barrier(self.r.peers["flags"], self.r.rank, self._epoch)
        else:
            dist.all_reduce(self._token, group=self.group)

    def plan(self, topk_ids: torch.Tensor, weights: torch.Tensor | None = None) -> None:
        counts = self.r.route(topk_ids)
        # either form also orders the ranks: the peers' previous step is over before their maps are rewritten
        if self.world > 1 and self.fences == "peer":
            native.ep_share_counts(counts, self.r.rank, self.r.peers["counts_tab"])
            self._fence()
            counts_all = self.r.buf["counts_tab"]
        elif self.world > 1:
            dist.all_gather_into_tensor(self._counts_all, counts, group=self.group)
            counts_all = self._counts_all
        else:
            counts_all = counts.reshape(1, -1)
        self.r.make_plan(counts_all, weights)

    def forward(self, x_tokens: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """[tokens, hidden] bf16 -> [tokens, hidden]: sum over the token's top-k experts of
        weight * down(silu(gate(x)) * up(x))."""
        self.r.fwd_send(x_tokens)
        self._fence()
        self.r.fwd_compute()
        self._fence()
        return self.r.fwd_recv(out)

    def grad_input(self, dy_tokens: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """Cotangent of ``forward``'s result -> gradient of its input, [tokens, hidden]."""
        self.r.bwd_send(dy_tokens)
        self._fence()
        self.r.bwd_compute()
        self._fence()
        return self.r.bwd_recv(out)

    def check_overflow(self) -> None:
        self.r.check_overflow()


__all__ = ["MoEMLPRank", "PeerMoEMLP"]
