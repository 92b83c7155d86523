"""Failure detection without any GPU fault: host-made failures among CPU (gloo) ranks."""
import datetime
import os
import sys
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _hb_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    from tinyinfinitrain_b200.parallel.health import HealthMonitor, PeerFailure

    hm = HealthMonitor()
    out = "finished"
    try:
        for step in range(1, 6):
            with hm.guard():
                if rank == 1 and step == 3:
                    raise ValueError("injected host failure")     # a rank dies between steps
            hm.beat(step)                                         # "about to run step"
            hm.check(step, timeout_s=10.0)                        # learn about peers before the next launch
            t = torch.ones(4) * step
            dist.all_reduce(t)
            assert t[0].item() == step * world
    except PeerFailure as e:
        out = f"peer_failure:{e.rank}:{e.reason}"
    except ValueError:
        out = "raised"
    q.put((rank, out))
    # no destroy_process_group: the failed rank would not take part in it


def test_peer_failure_is_seen_before_next_step():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + os.getpid() % 90
    procs = [ctx.Process(target=_hb_worker, args=(r, 2, port, q)) for r in range(2)]
    t0 = time.time()
    for p in procs:
        p.start()
    res = dict(q.get(timeout=60) for _ in procs)
    for p in procs:
        p.join(timeout=20)
    assert res[1] == "raised"
    assert res[0].startswith("peer_failure:1:ValueError: injected host failure"), res
    assert time.time() - t0 < 50


def _timeout_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    out = "ok"
    if rank == 0:
        try:
            t = torch.ones(2)
            dist.all_reduce(t)            # rank 1 never joins
        except RuntimeError as e:
            out = "collective_error"
    else:
        time.sleep(6)
    q.put((rank, out))


def test_short_group_timeout_turns_a_missing_peer_into_an_error():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29790 + os.getpid() % 90
    procs = [ctx.Process(target=_timeout_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=60) for _ in procs)
    for p in procs:
        p.join(timeout=20)
    assert res[0] == "collective_error", res


def test_truncated_or_foreign_checkpoint_is_rejected(tmp_path):
    from tinyinfinitrain_b200.models import GPT2, GPT2Config

    cfg = GPT2Config(block_size=16, vocab_size=100, n_layer=1, n_head=2, n_embd=32)
    p = str(tmp_path / "m.bin")
    GPT2(cfg).SaveLLMC(p)
    raw = open(p, "rb").read()
    open(p, "wb").write(raw[: len(raw) // 2])
    with pytest.raises(RuntimeError, match="unexpected end of file"):
        GPT2.FromLLMC(p)
    open(p, "wb").write(b"\x01\x02\x03\x04" + raw[4:])
    with pytest.raises(RuntimeError, match="not an llm.c GPT-2 checkpoint"):
        GPT2.FromLLMC(p)
