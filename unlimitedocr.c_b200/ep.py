"""Expert-parallel MoE layer over the GPUs of one node.

The reference engine runs on a single device; this module is the host side of the new multi-GPU path.
Rank g of G owns the contiguous expert ids [g*E/G, (g+1)*E/G) and a share of the tokens; router and shared
MLP are computed where a token lives.  One layer call is

    dispatch (router, plan, rows sorted by expert)           library, local
    all-to-all of the pair counts, then of the fp16 rows     torch.distributed (NCCL over NVLink)
    routed experts on the received rows                      library, local
    all-to-all of the results back to the token owners       torch.distributed
    weighted combine with the shared MLP's output (+ residual)   library, local
(the shared MLP of the local tokens runs on the context's second stream beside the exchange and the routed experts)

With G = 1 the two exchanges are skipped and the same three library calls run back to back.
The exchange plan (who sends how many rows to whom, in which order) is plain integer arithmetic kept in
`ExchangePlan`, so it can be tested without a GPU.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


@dataclass
class ExchangePlan:
    """Row counts of one layer call seen from one rank.

    send_counts[d, e]   rows this rank sends to rank d for d's e-th local expert
    recv_counts[s, e]   rows this rank receives from rank s for its own e-th local expert
    """

    send_counts: np.ndarray
    recv_counts: np.ndarray

    @property
    def send_splits(self) -> list[int]:
        return [int(v) for v in self.send_counts.sum(axis=1)]

    @property
    def recv_splits(self) -> list[int]:
        return [int(v) for v in self.recv_counts.sum(axis=1)]

    @property
    def rows_received(self) -> int:
        return int(self.recv_counts.sum())


def owner_ranges(n_experts: int, world: int) -> list[tuple[int, int]]:
    """Contiguous expert range of every rank; n_experts must divide evenly."""
    if n_experts % world != 0:
        raise ValueError(f"{n_experts} experts do not divide over {world} ranks")
    per = n_experts // world
    return [(g * per, (g + 1) * per) for g in range(world)]


def counts_from_offsets(all_offsets: np.ndarray) -> np.ndarray:
    """[G, E+1] exclusive prefix sums (one row per rank) -> [G, E] pairs per rank and expert."""
    return np.diff(np.asarray(all_offsets, np.int64), axis=1)


def plan_from_counts(counts: np.ndarray, rank: int) -> ExchangePlan:
    """counts[g, e]: pairs rank g has for expert e.  Rows are sorted by expert id on every rank, so what a rank
    sends to destination d is one contiguous block: the experts d owns."""
    world, n_experts = counts.shape
    per = n_experts // world
    send = counts[rank].reshape(world, per)
    recv = counts[:, rank * per:(rank + 1) * per]
    return ExchangePlan(np.ascontiguousarray(send), np.ascontiguousarray(recv))


def dst_rows_from_counts(counts: np.ndarray, rank: int) -> np.ndarray:
    """counts[g, e]: pairs rank g has for expert e.  For this rank and every expert e: the row of the OWNER's receive
    buffer where this rank's rows for e start.  An owner's buffer holds, for source rank 0, 1, ... in turn, the rows
    of each of its experts in turn (the order uocr_cuda_moe_ep_experts expects)."""
    counts = np.asarray(counts, np.int64)
    world, n_experts = counts.shape
    per = n_experts // world
    out = np.zeros(n_experts, np.int64)
    for owner in range(world):
        block = counts[:, owner * per:(owner + 1) * per]            # [source][local expert]
        before = int(block[:rank].sum())                             # everything the lower ranks send to this owner
        out[owner * per:(owner + 1) * per] = before + np.concatenate(([0], np.cumsum(block[rank])[:-1]))
    return out.astype(np.uint32)


def balanced_placement(pairs_per_expert: np.ndarray, world: int) -> np.ndarray:
    """Which expert sits in which slot so that the ranks' loads are even.  The library shards contiguous SLOT ranges
    (rank g owns slots [g*E/G, (g+1)*E/G)); relabelling the experts of a layer (oracle.quant.permute_experts, or the
    same permutation applied when the model is converted) therefore places them freely.  Longest-processing-time
    rule: experts in descending order of their observed pair count, each to the rank with the least load that still
    has a free slot.  Returns order[slot] = expert id; deterministic (ties: lower id first)."""
    counts = np.asarray(pairs_per_expert, np.int64).reshape(-1)
    n_experts = counts.shape[0]
    if n_experts % world != 0:
        raise ValueError(f"{n_experts} experts do not divide over {world} ranks")
    per = n_experts // world
    load = np.zeros(world, np.int64)
    members: list[list[int]] = [[] for _ in range(world)]
    for e in sorted(range(n_experts), key=lambda i: (-int(counts[i]), i)):
        g = min((r for r in range(world) if len(members[r]) < per), key=lambda r: (int(load[r]), r))
        members[g].append(e)
        load[g] += counts[e]
    return np.array([e for g in range(world) for e in sorted(members[g])], np.int64)


def rank_loads(pairs_per_expert: np.ndarray, order: np.ndarray, world: int) -> np.ndarray:
    """Pairs every rank receives when slot s holds expert order[s]."""
    counts = np.asarray(pairs_per_expert, np.int64).reshape(-1)
    return counts[np.asarray(order)].reshape(world, -1).sum(axis=1)


class ExpertParallelLayer:
    """One mapped MoE layer whose routed experts are sharded over the ranks of a process group.
    The context must run on the stream the collectives use (ctx.set_stream(torch.cuda.current_stream().cuda_stream))."""

    def __init__(self, ctx, layer: int, n_experts: int, top_k: int, hidden_size: int, *, rank: int = 0, world: int = 1,
                 dist_module=None, group=None, device: str = "cuda"):
        import torch
        self.device = device
        self.ctx, self.layer = ctx, layer
        self.E, self.K, self.H = n_experts, top_k, hidden_size
        self.rank, self.world, self.dist, self.group = rank, world, dist_module, group
        self.first, self.last = owner_ranges(n_experts, world)[rank]
        self.torch = torch
        self._bufs: dict[str, object] = {}
        self._offsets = None
        self._all_offsets = None
        self.last_plan: ExchangePlan | None = None

    def gathered_counts(self) -> np.ndarray:
        """[world, E] pairs per rank and expert of the last forward call (read back from the device)."""
        return counts_from_offsets(self._all_offsets.cpu().numpy())

    def _buffer(self, name: str, rows: int):
        t = self._bufs.get(name)
        if t is None or t.shape[0] < rows:
            t = self.torch.empty((max(rows, 1), self.H), dtype=self.torch.float16, device=self.device)
            self._bufs[name] = t
        return t

    def reserve(self, n_tokens: int, max_rows_received: int) -> None:
        """Allocate the exchange buffers up front (so a timed step allocates nothing)."""
        self._buffer("send", n_tokens * self.K)
        self._buffer("back", n_tokens * self.K)
        self._buffer("recv", max_rows_received)
        self._buffer("done", max_rows_received)

    def forward(self, hidden, out, *, residual=None) -> ExchangePlan:
        n = hidden.shape[0]
        torch = self.torch
        send = self._buffer("send", n * self.K)
        if self._offsets is None:
            self._offsets = torch.zeros(self.E + 1, dtype=torch.int32, device=self.device)
            self._all_offsets = torch.zeros((self.world, self.E + 1), dtype=torch.int32, device=self.device)
        self.ctx.ep_dispatch(self.layer, hidden, n, send, self._offsets)
        self.ctx.ep_shared(self.layer, hidden, n)       # on the context's second stream, beside all that follows
        if self.world == 1:
            all_offsets = self._offsets.reshape(1, -1)
        else:      # one small collective on the device, then ONE host read gives every rank the whole count matrix
            self.dist.all_gather(list(self._all_offsets.unbind(0)), self._offsets, group=self.group)
            all_offsets = self._all_offsets
        plan = plan_from_counts(counts_from_offsets(all_offsets.cpu().numpy()), self.rank)
        recv_counts = plan.recv_counts
        self.last_plan = plan
        if self.world == 1:
            rows_done = self._buffer("back", n * self.K)
            self.ctx.ep_experts(self.layer, self.first, self.last - self.first, recv_counts, send, rows_done)
            back = rows_done
        else:
            r = plan.rows_received
            rows_in, rows_done = self._buffer("recv", r), self._buffer("done", r)
            self.dist.all_to_all_single(rows_in[:r], send[: n * self.K], plan.recv_splits, plan.send_splits, group=self.group)
            self.ctx.ep_experts(self.layer, self.first, self.last - self.first, recv_counts, rows_in, rows_done)
            back = self._buffer("back", n * self.K)
            self.dist.all_to_all_single(back[: n * self.K], rows_done[:r], plan.send_splits, plan.recv_splits, group=self.group)
        self.ctx.ep_combine(self.layer, back, n, out, residual=residual)
        return plan


class PeerExpertParallelLayer:
    """The same layer with the exchange fused into the library's kernels: each rank's gather writes its rows straight
    into the owners' buffers and its combine reads the outputs straight from them over NVLink (CUDA IPC mappings, one
    process per GPU of one node), so no all-to-all runs.  torch.distributed carries only the IPC handles (once), the
    per-rank counts and two barriers per call."""

    def __init__(self, ctx, layer: int, n_experts: int, top_k: int, hidden_size: int, *, row_capacity: int, rank: int = 0,
                 world: int = 1, dist_module=None, group=None, device: str = "cuda"):
        import torch
        self.torch, self.device = torch, device
        self.ctx, self.layer = ctx, layer
        self.E, self.K, self.H = n_experts, top_k, hidden_size
        self.rank, self.world, self.dist, self.group = rank, world, dist_module, group
        owner_ranges(n_experts, world)                       # raises when the experts do not divide
        mine = ctx.ep_peer_create(hidden_size, row_capacity)
        if world > 1:
            t = torch.frombuffer(bytearray(mine), dtype=torch.uint8).to(device)
            every = torch.empty((world, 128), dtype=torch.uint8, device=device)
            self.dist.all_gather(list(every.unbind(0)), t, group=group)
            blob = every.cpu().numpy().tobytes()
        else:
            blob = mine
        ctx.ep_peer_open(world, rank, blob)
        self._offsets = torch.zeros(n_experts + 1, dtype=torch.int32, device=device)
        self._all_offsets = torch.zeros((world, n_experts + 1), dtype=torch.int32, device=device)
        self._token = torch.zeros(1, dtype=torch.int32, device=device)

    def _barrier(self) -> None:
        """Everything every rank has queued so far is done (a tiny all-reduce on the compute stream)."""
        if self.world > 1:
            self.dist.all_reduce(self._token, group=self.group)

    def forward(self, hidden, out, *, residual=None) -> None:
        """One layer call, queued in one go: the ranks exchange their counts and signal "rows landed" / "outputs written"
        to one another through flags in peer memory, inside the library's own kernels; no collective of
        torch.distributed runs and the host reads nothing."""
        self.ctx.ep_peer_forward(self.layer, hidden, hidden.shape[0], out, residual=residual)
        self._device_synced = True

    def forward_collectives(self, hidden, out, *, residual=None) -> None:
        """The same call with torch.distributed between the phases: one all_gather of the per-rank counts into device
        memory and two 4-byte all-reduces as barriers (the form the device-side flags replaced; kept for comparison)."""
        n = hidden.shape[0]
        self.ctx.ep_peer_dispatch(self.layer, hidden, n, self._offsets)
        self.ctx.ep_shared(self.layer, hidden, n)            # on the context's second stream, beside all that follows
        if self.world == 1:
            self._all_offsets.copy_(self._offsets.reshape(1, -1))
        else:
            self.dist.all_gather(list(self._all_offsets.unbind(0)), self._offsets, group=self.group)
        self.ctx.ep_peer_scatter_dev(self.layer, hidden, n, self._all_offsets)
        self._barrier()                                      # every rank's rows are in the owners' buffers
        self.ctx.ep_peer_experts_dev(self.layer)
        self._barrier()                                      # every owner's outputs are written
        self.ctx.ep_peer_combine(self.layer, n, out, residual=residual)
        self._device_synced = False

    def forward_host_counts(self, hidden, out, *, residual=None) -> ExchangePlan:
        """The same call with the counts read back and the row offsets computed on the host (the earlier form, kept for
        comparison and as the reference of the device-side arithmetic)."""
        n = hidden.shape[0]
        self.ctx.ep_peer_dispatch(self.layer, hidden, n, self._offsets)
        self.ctx.ep_shared(self.layer, hidden, n)
        if self.world == 1:
            all_offsets = self._offsets.reshape(1, -1)
        else:
            self.dist.all_gather(list(self._all_offsets.unbind(0)), self._offsets, group=self.group)
            all_offsets = self._all_offsets
        counts = counts_from_offsets(all_offsets.cpu().numpy())
        plan = plan_from_counts(counts, self.rank)
        self.ctx.ep_peer_scatter(self.layer, hidden, n, dst_rows_from_counts(counts, self.rank))
        self._barrier()
        self.ctx.ep_peer_experts(self.layer, plan.recv_counts)
        self._barrier()
        self.ctx.ep_peer_combine(self.layer, n, out, residual=residual)
        return plan

    def gathered_counts(self) -> np.ndarray:
        """[world, E] pairs per rank and expert of the last forward call (read back from the device)."""
        if getattr(self, "_device_synced", False):
            return counts_from_offsets(self.ctx.ep_peer_last_offsets(self.world, self.E).astype(np.int64))
        return counts_from_offsets(self._all_offsets.cpu().numpy())

    @property
    def last_plan(self) -> ExchangePlan:
        """Row counts of the last forward call (reads the gathered offsets from the device)."""
        if getattr(self, "_device_synced", False):
            offsets = self.ctx.ep_peer_last_offsets(self.world, self.E).astype(np.int64)
        else:
            offsets = self._all_offsets.cpu().numpy()
        return plan_from_counts(counts_from_offsets(offsets), self.rank)

    def close(self, *, group_barrier: bool = True) -> None:
        """Unmap the peers' buffers and free this rank's.  A peer's scatter or combine kernel may still be reading or
        writing this rank's buffers, so first this rank's own work is awaited, then every rank's (group barrier on
        the compute stream, then a host wait), and only then is anything freed.  Every rank of the group must call
        this together; group_barrier=False is for a rank that knows that no forward call has run yet."""
        try:
            self.ctx.synchronize()
        finally:
            if group_barrier:
                self._barrier()
            self.torch.cuda.synchronize()
            self.ctx.ep_peer_destroy()

