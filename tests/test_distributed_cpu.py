"""World-size-2 gloo tests of the data-parallel gradient reduction bookkeeping (no GPU involved)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

C_, T_, D_ = 11, 4, 8


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _local_entries(rank):
    """Two memory layers sharing one bank on each rank: chapter 0 (shared) plus rank-specific picks."""
    g = torch.Generator().manual_seed(100 + rank)
    picks = [[0, 3, 7], [0, 5, 3 + rank]] if rank == 0 else [[0, 2, 7], [0, 9, 4]]
    out = []
    for ids in picks:
        ids_sorted = sorted(set(ids))
        n_pairs = 6                                  # buffers are padded to the pair count, like the kernels' outputs
        uniq = torch.full((n_pairs,), -1, dtype=torch.int32)
        uniq[:len(ids_sorted)] = torch.tensor(ids_sorted, dtype=torch.int32)
        rows = torch.zeros(n_pairs * T_, D_)
        rows[:len(ids_sorted) * T_] = torch.randn(len(ids_sorted) * T_, D_, generator=g)
        out.append((uniq, torch.tensor([len(ids_sorted)], dtype=torch.int32), rows, T_))
    return out


def _dense_of(entries):
    dense = torch.zeros(C_ * T_, D_)
    for uniq, n, rows, t in entries:
        for u in range(int(n)):
            c = int(uniq[u])
            dense[c * t:(c + 1) * t] += rows[u * t:(u + 1) * t]
    return dense


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from memory_b200.distributed import GradReducer
        from memory_b200.functional import SparseBankGrad
        sink = SparseBankGrad()
        for e in _local_entries(rank):
            sink.add(*e)
        g = torch.Generator().manual_seed(7 + rank)
        dense = [torch.randn(5, 3, generator=g), None, torch.randn(4, generator=g)]
        want_dense = [d.clone() if d is not None else None for d in dense]
        red = GradReducer(C_, T_, D_, "cpu")
        pending = red.reduce_async([d.clone() if d is not None else None for d in dense], sink)
        dense_async, bank_async = pending.result()
        snap = red.snapshot([d.clone() if d is not None else None for d in dense], sink)
        dense_snap, bank_snap = red.reduce_snapshot_async(snap).result()
        for a, b in zip(dense_snap, dense_async):
            torch.testing.assert_close(a, b)
        torch.testing.assert_close(_dense_of(bank_snap.entries), _dense_of(bank_async.entries))
        # zero-copy staging: same result once the consumer applies the returned scale
        refs = [d.clone() if d is not None else None for d in dense]
        snap0 = red.snapshot(refs, sink, copy=False)
        dense_zc, bank_zc = red.reduce_snapshot_async(snap0).result()
        for a, b in zip(dense_zc, dense_async):
            torch.testing.assert_close(a, b)
        assert bank_zc.scale == 0.5
        torch.testing.assert_close(_dense_of(bank_zc.entries) * bank_zc.scale, _dense_of(bank_async.entries))
        reduced = red.reduce(dense, sink)
        assert len(sink.entries) == 2, "the local entries must be left in place"
        for a, b in zip(dense_async, [d for d in dense if d is not None]):
            torch.testing.assert_close(a, b)
        torch.testing.assert_close(_dense_of(bank_async.entries), _dense_of(reduced.entries))
        uniq, n, rows, t = reduced.entries[0]
        got = _dense_of(reduced.entries)
        # numpy arrays travel by value; a tensor would travel as a file descriptor that dies with this process
        q.put((rank, got.numpy(), [d.numpy() for d in dense if d is not None], uniq[:int(n)].tolist(),
               red.last_union_size, [d.numpy() for d in want_dense if d is not None]))
    finally:
        dist.destroy_process_group()


def test_sparse_bank_gradient_reduction_world2():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    results = [(r, torch.from_numpy(got), [torch.from_numpy(d) for d in dense], uniq, usize,
                [torch.from_numpy(d) for d in want]) for r, got, dense, uniq, usize, want in results]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    expect = sum(_dense_of(_local_entries(r)) for r in range(world)) / world
    union = sorted({0, 3, 7, 5, 2, 9, 4})
    local_dense = {r: res for r, *res in [(x[0], x[5]) for x in results]}
    for rank, got, dense, uniq, usize, _ in results:
        assert uniq == union and usize == len(union)
        torch.testing.assert_close(got, expect)
        mask = torch.ones(C_, dtype=torch.bool)
        mask[union] = False
        assert not got.view(C_, T_, D_)[mask].any()
    # dense gradients: mean over ranks, identical on both
    mean0 = [(a + b) / 2 for a, b in zip(local_dense[0][0], local_dense[1][0])]
    for rank, got, dense, *_ in results:
        for d, m in zip(dense, mean0):
            torch.testing.assert_close(d, m)


def test_union_helpers_single_process():
    from memory_b200.distributed import compact_to_union, union_of_touched
    counts = torch.tensor([1, 0, 2, 0, 0, 1], dtype=torch.int32)
    u = union_of_touched(counts)
    assert u.tolist() == [0, 2, 5]
    rows = torch.arange(2 * 3 * 2, dtype=torch.float32).view(6, 2)       # chapters [2, 5], T = 3
    out = compact_to_union(torch.tensor([2, 5], dtype=torch.int32), rows, u, 6, 3)
    assert out.shape == (9, 2) and not out[:3].any()
    assert torch.equal(out[3:], rows)
    with pytest.raises(IndexError):
        compact_to_union(torch.tensor([9], dtype=torch.int32), rows[:3], u, 6, 3)


def test_reducer_rejects_unknown_options():
    from memory_b200.distributed import GradReducer
    for bad in (dict(exchange="rdma"), dict(wire_dtype=torch.float16), dict(merge_dtype=torch.float16),
                dict(sync="spin")):
        with pytest.raises(ValueError):
            GradReducer(8, 4, 16, "cpu", **bad)
    r = GradReducer(8, 4, 16, "cpu", parities=1)
    assert r.parities == 2 and r.sync == "collective" and r.merge_dtype == torch.float32
