"""Host logic of the expert-parallel layer, on CPU: the exchange plan arithmetic, and the real
ExpertParallelLayer.forward driven over a 2-rank gloo group with a NumPy stand-in for the three library
phases (dispatch / experts / combine).  The stand-in follows the library's contracts (rows sorted by expert,
per-expert counts, results returned in dispatch order), so what is tested is everything the host adds:
owner ranges, count matrices, split sizes, both all-to-alls and the order of the returned rows."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

E, K, H = 8, 2, 16


def load_ep():
    import __graft_entry__ as entry
    return entry.load_package().ep


class FakeContext:
    """CPU stand-in: expert e maps a row x to x * (e + 1) + e; the shared MLP is x * 0.5."""

    def __init__(self, ids, weights):
        self.ids, self.weights = ids, weights            # [n, K]

    def ep_dispatch(self, layer, hidden, n, sorted_rows, expert_offsets):
        flat = self.ids.reshape(-1)
        order = np.argsort(flat, kind="stable")
        self.order = order
        sorted_rows[: n * K] = hidden[torch.from_numpy(order // K)]
        counts = np.bincount(flat, minlength=E)
        expert_offsets[:] = torch.from_numpy(np.concatenate([[0], np.cumsum(counts)]).astype(np.int32))

    def ep_experts(self, layer, first, n_local, seg_counts, rows_in, rows_out):
        pos = 0
        for s in range(seg_counts.shape[0]):
            for e in range(n_local):
                c = int(seg_counts[s, e])
                ex = first + e
                rows_out[pos:pos + c] = rows_in[pos:pos + c] * (ex + 1) + ex
                pos += c

    def ep_shared(self, layer, hidden, n):
        self.shared = hidden.float() * 0.5

    def ep_combine(self, layer, rows_back, n, out, residual=None):
        inv = np.empty_like(self.order)
        inv[self.order] = np.arange(self.order.size)
        acc = self.shared.clone()
        for t in range(n):
            for s in range(K):
                acc[t] += self.weights[t, s] * rows_back[inv[t * K + s]].float()
        if residual is not None:
            acc += residual.float()
        out[:] = acc.half()


def reference(hidden, ids, weights, residual=None):
    acc = hidden.float() * 0.5
    for t in range(hidden.shape[0]):
        for s in range(K):
            e = int(ids[t, s])
            acc[t] += weights[t, s] * (hidden[t] * (e + 1) + e).float()
    if residual is not None:
        acc += residual.float()
    return acc.half()


def make_inputs(rank, n):
    rng = np.random.default_rng(100 + rank)
    ids = np.stack([rng.permutation(E)[:K] for _ in range(n)]).astype(np.int64)
    if rank == 1:
        ids[:, 0] = 0                                   # skew: everything from rank 1 also hits expert 0 (rank 0's)
    weights = rng.random((n, K)).astype(np.float32)
    hidden = torch.from_numpy(rng.integers(-4, 5, (n, H)).astype(np.float16))
    return hidden, ids, weights


def worker(rank, world, port, n_by_rank, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ep = load_ep()
        hidden, ids, weights = make_inputs(rank, n_by_rank[rank])
        layer = ep.ExpertParallelLayer(FakeContext(ids, weights), 0, E, K, H, rank=rank, world=world, dist_module=dist,
                                       device="cpu")
        out = torch.zeros_like(hidden)
        plan = layer.forward(hidden, out)
        ok = torch.equal(out, reference(hidden, ids, weights))
        # every row this rank received is for one of its own experts, and nothing was lost
        total_sent = torch.tensor([int(plan.send_counts.sum())])
        total_recv = torch.tensor([plan.rows_received])
        dist.all_reduce(total_sent); dist.all_reduce(total_recv)
        results[rank] = (ok, int(total_sent) == int(total_recv) == sum(n_by_rank) * K, plan.recv_counts.tolist())
    finally:
        dist.destroy_process_group()


def test_owner_ranges_and_count_matrices():
    ep = load_ep()
    assert ep.owner_ranges(64, 8) == [(8 * g, 8 * g + 8) for g in range(8)]
    with pytest.raises(ValueError):
        ep.owner_ranges(64, 3)
    offsets = np.array([[0, 1, 3, 6, 10, 15, 21, 28, 36], [0, 8, 15, 21, 26, 30, 33, 35, 36]])     # two ranks, E = 8
    counts = ep.counts_from_offsets(offsets)
    assert counts.tolist() == [[1, 2, 3, 4, 5, 6, 7, 8], [8, 7, 6, 5, 4, 3, 2, 1]]
    p0, p1 = ep.plan_from_counts(counts, 0), ep.plan_from_counts(counts, 1)
    assert p0.send_counts.tolist() == [[1, 2, 3, 4], [5, 6, 7, 8]] and p0.recv_counts.tolist() == [[1, 2, 3, 4], [8, 7, 6, 5]]
    assert p0.send_splits == [10, 26] and p0.recv_splits == [10, 26] and p0.rows_received == 36
    assert p1.recv_counts.tolist() == [[5, 6, 7, 8], [4, 3, 2, 1]] and p1.send_splits == [26, 10]
    # what rank a sends to b is what b receives from a
    assert p0.send_splits[1] == p1.recv_splits[0] and p1.send_splits[0] == p0.recv_splits[1]


def test_single_rank_forward_matches_reference():
    ep = load_ep()
    hidden, ids, weights = make_inputs(0, 13)
    layer = ep.ExpertParallelLayer(FakeContext(ids, weights), 0, E, K, H, device="cpu")
    out = torch.zeros_like(hidden)
    resid = torch.ones_like(hidden)
    layer.forward(hidden, out, residual=resid)
    assert torch.equal(out, reference(hidden, ids, weights, resid))


def test_two_rank_gloo_forward_matches_reference():
    world, n_by_rank = 2, [11, 7]                        # ragged token counts
    port = 29500 + os.getpid() % 2000
    manager = mp.get_context("spawn").Manager()
    results = manager.dict()
    mp.spawn(worker, args=(world, port, n_by_rank, results), nprocs=world, join=True)
    assert all(results[r][0] for r in range(world)), "outputs differ from the single-process computation"
    assert all(results[r][1] for r in range(world)), "rows were lost or duplicated in the exchange"
    # rank 0 owns expert 0 and must have received one row per rank-1 token for it
    assert results[0][2][1][0] == n_by_rank[1]


def test_peer_scatter_offsets_match_the_owner_side_row_order():
    """dst_rows_from_counts: where a rank's rows for an expert start in the owner's buffer.  Simulated exchange: every
    rank writes row labels at its offsets; each owner must then hold, source by source and expert by expert, exactly
    the segments plan_from_counts announces, with no gap and no overlap."""
    ep = load_ep()
    rng = np.random.default_rng(5)
    world, n_experts = 4, 64
    per = n_experts // world
    counts = rng.integers(0, 40, size=(world, n_experts))
    counts[2, 5] = 0
    buffers = [dict() for _ in range(world)]
    for r in range(world):
        dst = ep.dst_rows_from_counts(counts, r)
        for e in range(n_experts):
            for i in range(counts[r, e]):
                row = int(dst[e]) + i
                assert row not in buffers[e // per]
                buffers[e // per][row] = (r, e)
    for owner in range(world):
        plan = ep.plan_from_counts(counts, owner)
        assert sorted(buffers[owner]) == list(range(plan.rows_received))
        want = [(s, owner * per + e) for s in range(world) for e in range(per) for _ in range(plan.recv_counts[s, e])]
        assert [buffers[owner][i] for i in range(plan.rows_received)] == want



def test_balanced_placement_evens_out_skewed_loads():
    """Longest-processing-time placement: under a Zipf(1.1) popularity the contiguous ranges leave one rank with almost
    twice the mean load at 8 ranks; the placement brings every rank within a few percent, is a permutation with
    E / world experts per rank, and is deterministic."""
    ep = load_ep()
    rng = np.random.default_rng(9)
    ranks = rng.permutation(64).astype(np.float64) + 1.0
    counts = np.round(98304 * ranks ** -1.1 / np.sum(ranks ** -1.1)).astype(np.int64)
    for world in (2, 4, 8):
        contiguous = ep.rank_loads(counts, np.arange(64), world)
        order = ep.balanced_placement(counts, world)
        assert sorted(order.tolist()) == list(range(64))
        assert np.array_equal(order, ep.balanced_placement(counts, world))
        balanced = ep.rank_loads(counts, order, world)
        assert balanced.sum() == counts.sum()
        per = 64 // world
        # a rank holds E / world experts: the one with the hottest expert cannot get below that expert plus the coldest others
        floor = counts.max() + np.sort(counts)[: per - 1].sum()
        assert balanced.max() <= max(1.05 * balanced.mean(), floor)
        assert balanced.max() <= contiguous.max()
        for g in range(world):                      # slots of a rank are listed in ascending expert id
            assert list(order[g * per:(g + 1) * per]) == sorted(order[g * per:(g + 1) * per])
    with pytest.raises(ValueError):
        ep.balanced_placement(counts, 3)


def test_permuted_experts_give_the_same_layer_output():
    """Relabelling the experts (how a placement is applied) changes ids, not results: the CPU oracle on the permuted
    layer selects the same experts (its ids are the slots of the original ids) and returns the same outputs up to the
    order in which the softmax denominator is summed (expert order, which the relabelling changes)."""
    from oracle import oracle as orc
    from oracle import quant
    port = orc.Port()
    rng = np.random.default_rng(3)
    L = quant.synth_layer(rng, H=128, E=8, K=2, F=64, S=64, expert_qtype=quant.QTYPE_Q4_0,
                          logit_bias=rng.standard_normal(8).astype(np.float32))
    hidden = quant.synth_activations(rng, 12, 128)
    order = np.array([5, 2, 7, 0, 3, 6, 1, 4])
    a, b = port.layer(L, hidden), port.layer(quant.permute_experts(L, order), hidden)
    slot_of = np.argsort(order)
    assert np.array_equal(slot_of[a.ids], b.ids)
    assert np.max(np.abs(a.weights - b.weights)) <= 1e-6 and np.max(np.abs(a.out - b.out)) <= 1e-5


def test_device_side_offset_arithmetic_restated():
    """The row offsets the library computes on the device (ep_offsets_kernel) follow two formulas; restated here in
    NumPy they must agree with the host helpers the earlier form of the exchange uses."""
    ep = load_ep()
    rng = np.random.default_rng(6)
    world, n_experts = 4, 64
    per = n_experts // world
    counts = rng.integers(0, 50, size=(world, n_experts))
    offsets = np.concatenate([np.zeros((world, 1), np.int64), np.cumsum(counts, axis=1)], axis=1)
    for rank in range(world):
        dst = np.empty(n_experts, np.int64)
        for e in range(n_experts):
            first = (e // per) * per
            dst[e] = sum(offsets[g, first + per] - offsets[g, first] for g in range(rank)) + offsets[rank, e] - offsets[rank, first]
        assert np.array_equal(dst, ep.dst_rows_from_counts(counts, rank))
        seg = [0]
        for src in range(world):
            for le in range(per):
                seg.append(seg[-1] + offsets[src, rank * per + le + 1] - offsets[src, rank * per + le])
        plan = ep.plan_from_counts(counts, rank)
        assert seg[-1] == plan.rows_received
        assert np.array_equal(np.diff(seg), plan.recv_counts.reshape(-1))
