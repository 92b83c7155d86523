"""Bucket planning and the gradient-ready state machine of the ZeRO-1 optimizer, on one CPU process: which bucket is
handed to the communication kernel when, with the launch itself replaced by a recorder."""
import os

import torch
import torch.distributed as dist

from tinyinfinitrain_b200.parallel.zero import DistributedOptimizer


def _make(num_buckets):
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", str(29400 + os.getpid() % 500))
        dist.init_process_group("gloo", rank=0, world_size=1)
    torch.manual_seed(0)
    # parameter order as in a model: embedding (tied: reported twice), four "layers", final norm
    params = [torch.nn.Parameter(torch.randn(n)) for n in (4096, 1000, 1024, 1000, 1024, 1000, 1024, 1000, 1024, 64)]
    opt = DistributedOptimizer(params, lr=1e-3)
    # drive the fused-path bookkeeping by hand (the CPU build has no NVLink kernels to launch)
    opt.comm, opt.overlap = "fused", True
    opt._plan_buckets(num_buckets)
    launched = []
    opt._launch_bucket = lambda b, side: (launched.append((opt.buckets.index(b), side)), b.__setitem__("launched", True))
    return opt, params, launched


def test_buckets_cover_the_flat_space_on_parameter_boundaries():
    opt, params, _ = _make(4)
    f = opt.flat
    assert opt.buckets[0]["start"] == 0 and opt.buckets[-1]["end"] == f.total
    offs = set(f.offsets) | {f.total}
    for a, b in zip(opt.buckets, opt.buckets[1:]):
        assert a["end"] == b["start"] and a["end"] in offs          # no parameter straddles two buckets
    assert sum(len(b["params"]) for b in opt.buckets) == len(params)
    for b in opt.buckets:
        assert (b["end"] - b["start"]) % (8 * opt.world) == 0 and b["shard"] * opt.world == b["end"] - b["start"]
    assert sum(b["shard"] for b in opt.buckets) == opt.shard_n        # local state = one slice per bucket
    assert 2 <= len(opt.buckets) <= 4


def test_first_step_learns_report_counts_then_buckets_fire_in_backward_order():
    opt, params, launched = _make(4)
    backward_order = list(reversed(params))       # deep layers report first; the embedding reports last, and twice

    def one_step(skip=()):
        opt._reset_pending()
        for p in backward_order:
            if p in skip:
                continue
            opt._grad_ready(p)
            if p is params[0]:
                opt._grad_ready(p)                 # tied tensor: lm-head wgrad + embedding backward
    one_step()
    assert launched == []                          # learning step: nothing fires from backward
    opt._finish_learning()
    assert params[0]._expected == 2 and all(p._expected == 1 for p in params[1:])
    assert not any(b["late"] for b in opt.buckets)

    one_step()
    order = [i for i, _ in launched]
    assert order == sorted(order, reverse=True) and len(order) == len(opt.buckets)   # last bucket first
    assert all(side for _, side in launched)
    # the bucket holding the tied embedding fired only after its second report
    assert order[-1] == 0

    # a parameter that does not report leaves its bucket for step()
    launched.clear()
    one_step(skip={params[3]})
    missing = opt.buckets.index(params[3]._bucket)
    assert missing not in [i for i, _ in launched] and len(launched) == len(opt.buckets) - 1
    assert opt.buckets[missing]["launched"] is False


def test_parameter_without_reports_marks_its_bucket_late():
    opt, params, launched = _make(3)
    opt._reset_pending()
    for p in params[1:]:
        opt._grad_ready(p)                         # params[0] never reports (gradient through plain autograd)
    opt._finish_learning()
    late = [b["late"] for b in opt.buckets]
    assert late[0] is True and not any(late[1:])
    opt._reset_pending()
    for p in reversed(params[1:]):
        opt._grad_ready(p)
    assert 0 not in [i for i, _ in launched] and len(launched) == len(opt.buckets) - 1
