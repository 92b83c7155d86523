"""Symmetric-memory heap protocol (allocate, export, pass descriptors over unix sockets, import, map) between real
processes, with the stand-in driver that backs "device memory" by memfd host memory.  No GPU, no CUDA driver."""
import multiprocessing as mp
import os
import time

import pytest
import torch


def _rank(rank, world, key, barrier, q, stagger):
    try:
        from tinyinfinitrain_b200._lib import C

        heap = C.SymmHeap(rank, world, 0, key, "host", True)   # the stand-in has no multicast: mc_ptr stays 0
        heap.set_timeout(20.0)
        heap.listen()
        barrier.wait()
        if stagger and rank == 1:
            time.sleep(0.3)            # rank 0 runs ahead: its second allocation's descriptors arrive early
        ids, infos = [], []
        for nbytes in (100_000, 4096):
            i = heap.exchange(nbytes)
            assert heap.multicast_ready(i) is False
            infos.append(heap.finish(i, False))
            ids.append(i)
        ok = True
        for i, info, n in zip(ids, infos, (25_000, 1024)):
            ok &= info["bytes"] % 65536 == 0 and info["bytes"] >= 4 * n and len(info["ptrs"]) == world and info["mc_ptr"] == 0
            heap.tensor(i, rank, torch.float32, n).fill_(float(10 * i + rank + 1))
        barrier.wait()
        for i, n in zip(ids, (25_000, 1024)):
            for r in range(world):
                t = heap.tensor(i, r, torch.float32, n)       # rank r's memory, mapped in this process
                ok &= bool((t == float(10 * i + r + 1)).all())
        barrier.wait()
        # a store through the peer mapping is seen by the owner
        heap.tensor(ids[0], (rank + 1) % world, torch.float32, 4)[rank % 4] = -7.0
        barrier.wait()
        ok &= float(heap.tensor(ids[0], rank, torch.float32, 4)[(rank - 1) % world % 4]) == -7.0
        try:
            heap.tensor(ids[1], 0, torch.float32, 1 << 20)
            ok = False
        except RuntimeError:
            pass
        heap.release(ids[0])
        q.put((rank, ok))
    except Exception as e:  # noqa: BLE001
        q.put((rank, repr(e)))


@pytest.mark.parametrize("world,stagger", [(2, False), (3, True)])
def test_heap_maps_every_ranks_memory_in_every_process(world, stagger):
    ctx = mp.get_context("spawn")
    q, barrier = ctx.Queue(), ctx.Barrier(world)
    key = f"t{os.getpid()}w{world}"
    procs = [ctx.Process(target=_rank, args=(r, world, key, barrier, q, stagger)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=30)
    assert res == [(r, True) for r in range(world)], res


def test_exchange_with_absent_peer_times_out_instead_of_hanging():
    from tinyinfinitrain_b200._lib import C

    heap = C.SymmHeap(0, 2, 0, f"lonely{os.getpid()}", "host", False)
    heap.set_timeout(0.5)
    heap.listen()
    t0 = time.time()
    with pytest.raises(RuntimeError, match="connect to rank 1"):
        heap.exchange(4096)
    assert time.time() - t0 < 10


def test_single_rank_heap_needs_no_sockets():
    from tinyinfinitrain_b200._lib import C

    heap = C.SymmHeap(0, 1, 0, f"solo{os.getpid()}", "host", False)
    i = heap.exchange(1000)
    info = heap.finish(i)
    assert len(info["ptrs"]) == 1 and info["bytes"] == 65536
    t = heap.tensor(i, 0, torch.int32, 250)
    t.copy_(torch.arange(250, dtype=torch.int32))
    assert int(heap.tensor(i, 0, torch.int32, 250).sum()) == 250 * 249 // 2


def test_multicast_is_opt_in(monkeypatch):
    """NVLink kernels use peer loads / stores unless TITB200_MULTIMEM=1 asks for the NVSwitch multicast address; the older
    TITB200_NO_MULTIMEM=1 still forces it off."""
    from tinyinfinitrain_b200.parallel.symm import use_multimem

    monkeypatch.delenv("TITB200_MULTIMEM", raising=False)
    monkeypatch.delenv("TITB200_NO_MULTIMEM", raising=False)
    assert use_multimem() is False
    monkeypatch.setenv("TITB200_MULTIMEM", "1")
    assert use_multimem() is True
    monkeypatch.setenv("TITB200_NO_MULTIMEM", "1")
    assert use_multimem() is False
