"""CPU, world_size 2 and 4, gloo: the host-side bookkeeping of tensor-parallel sharding and of the expert-parallel exchange
(counts, variable all-to-all, regrouping by local expert, return to the sender in the original order)."""
import importlib
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _ep_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        P = importlib.import_module("mxfp4-int8-m5_b200.parallel")
        import scmx_oracle as O
        E, k, L, D = 8, 2, 37 + 5 * rank, 16
        El = E // world
        rng = np.random.default_rng(100 + rank)
        inds = np.stack([rng.permutation(E)[:k] for _ in range(L)]).astype(np.int32)
        inds[inds == 5] = 4                                   # expert 5 receives nothing from anyone
        R = L * k
        pos, tok, es, off, ts, _ = O.route_sort(inds, E, 128)
        # payload row i of the sorted buffer = (source rank, sorted row index, global expert)
        rows = torch.tensor(np.stack([np.full(R, rank), np.arange(R), es], 1), dtype=torch.int32)
        cnt = torch.tensor(np.diff(off).astype(np.int64))
        recv_cnt = P.exchange_counts(cnt, world)
        send_splits = P.expert_owner_splits(cnt, world).tolist()
        recv_splits = recv_cnt.sum(1).tolist()
        rx = P.exchange_rows(rows, send_splits, recv_splits)
        le = P.local_expert_ids(recv_cnt)
        ok = rx.shape[0] == sum(recv_splits)
        ok &= bool(((rx[:, 2] // El) == rank).all())          # every received row belongs to an expert owned here
        ok &= bool((rx[:, 2] - rank * El == le).all())        # and the reconstructed local expert id is right
        # rows from one source arrive contiguously and in that source's sorted order
        for s in range(world):
            part = rx[rx[:, 0] == s]
            ok &= bool((part[1:, 1] > part[:-1, 1]).all()) if len(part) > 1 else True
        # regroup by local expert, "compute" (tag rows), un-sort, send back
        pos2, tok2, es2, off2, ts2, _ = O.route_sort(le.numpy().reshape(-1, 1), El, 128)
        sorted_rows = rx[torch.tensor(tok2[:rx.shape[0]].astype(np.int64))]
        ok &= bool((np.diff(sorted_rows[:, 2].numpy()) >= 0).all())          # grouped by expert
        y_sorted = sorted_rows.clone()
        y_sorted[:, 0] += 1000                                              # the expert "output"
        y_rx = y_sorted[torch.tensor(pos2.astype(np.int64))]
        back = P.exchange_rows(y_rx, recv_splits, send_splits)
        ok &= bool((back[:, 0] == rank + 1000).all()) and bool((back[:, 1] == torch.arange(R)).all())
        ok &= bool((back[:, 2] == torch.tensor(es)).all())
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def _run_ranks(worker, world, port):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=180) for _ in procs)
    for p in procs:
        p.join(60)
    assert res == {r: True for r in range(world)}


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_exchange_gloo(world):
    _run_ranks(_ep_worker, world, 29613 + 10 * world)


def test_shard_rows_and_packed(scmx, oracle, golden):
    P = scmx.parallel
    assert P.shard_rows(12288, 3, 8, 4) == (4608, 6144)
    with pytest.raises(AssertionError):
        P.shard_rows(100, 0, 8)
    codes, bc, ws = (torch.from_numpy(np.ascontiguousarray(golden[f"quantize_a_{n}"].view(np.int32) if n == "codes" else golden[f"quantize_a_{n}"]))
                     for n in ("codes", "bcodes", "wscale"))
    qw = golden["quantize_a_qw"]
    N, K = qw.shape
    parts = [P.shard_packed(codes, bc, ws, N, K, r, 4) for r in range(4)]
    dec = np.concatenate([oracle.decode(c.numpy().view(np.uint32), b.numpy(), n, K) for c, b, _, n, _ in parts])
    assert np.array_equal(dec, qw)                          # row shards decode to the rows of the full operand
    assert np.array_equal(np.concatenate([p[2].numpy() for p in parts]), golden["quantize_a_wscale"])


def _seg_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, w = 6, 4
        full = torch.arange(M * w * world, dtype=torch.float32).view(M, world * w)
        local = full[:, rank * w:(rank + 1) * w].contiguous()
        seg = torch.empty((world, M, w))
        dist.all_gather_into_tensor(seg.view(-1, w), local)
        # segment layout: element (m, s*w + j) of the full matrix is seg[s, m, j]
        q.put((rank, bool(torch.equal(seg.permute(1, 0, 2).reshape(M, world * w), full))))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_segment_layout_of_column_gather_gloo(world):
    _run_ranks(_seg_worker, world, 29614 + 10 * world)


def test_peer_exchange_slot_algebra():
    """The index arithmetic of the kernel-side expert-parallel exchange, restated in NumPy for 3 ranks: dispatch slots
    (source rank * cap + position among the rows that source sends there), the receiver's regrouping list, the scatter of
    the expert outputs back to slot order, and the addresses the pull-form combine reads.  Every token must get, for each
    of its top-k slots, the output of exactly its own (token, expert) assignment."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import scmx_oracle as O
    G, E, k, tm = 3, 12, 2, 128
    El = E // G
    L = [19, 7, 30]
    cap = max(L) * k
    rng = np.random.default_rng(5)
    sent = []
    rx = [[None] * (G * cap) for _ in range(G)]           # rx[d][slot] = payload (source rank, token, expert)
    meta = [np.zeros((G, El + 1), np.int64) for _ in range(G)]
    for r in range(G):
        inds = np.stack([rng.permutation(E)[:k] for _ in range(L[r])]).astype(np.int32)
        inds[inds == 7] = 6                                # an expert nobody routes to
        pos, tok, es, off, _, _ = O.route_sort(inds, E, tm)
        sent.append((inds, pos, es, off))
        for p in range(L[r] * k):                          # ep_dispatch
            d = es[p] // El
            rx[d][r * cap + (p - off[d * El])] = (r, int(tok[p]), int(es[p]))
        for d in range(G):
            meta[d][r, :El] = np.diff(off[d * El:(d + 1) * El + 1])
            meta[d][r, El] = off[d * El]
    y_slot = []
    for d in range(G):                                     # ep_plan + grouped GEMM with the slot scatter
        cnt = meta[d][:, :El]
        tok2 = []
        for le in range(El):
            for s in range(G):
                a = s * cap + int(cnt[s, :le].sum())
                tok2 += list(range(a, a + int(cnt[s, le])))
        ys = [None] * (G * cap)
        seen_experts = []
        for p2, slot in enumerate(tok2):
            src, t, e = rx[d][slot]
            assert e // El == d
            seen_experts.append(e)
            ys[slot] = ("out", src, t, e)                  # what the expert GEMM computes for regrouped row p2
        assert seen_experts == sorted(seen_experts)        # regrouped rows are expert-major
        y_slot.append(ys)
    for r in range(G):                                     # the pull-form combine of rank r
        inds, pos, es, off = sent[r]
        for t in range(L[r]):
            for j in range(k):
                p = pos[t * k + j]
                d = es[p] // El
                got = y_slot[d][r * cap + (p - off[d * El])]
                assert got == ("out", r, t, int(inds[t, j]))
