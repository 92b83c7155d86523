"""Partition arithmetic as pure functions ("virtual ranks", no process group): mesh coordinates and groups,
tensor-parallel head ranges and fused-QKV row sets, pipeline layer partition and 1F1B order, ZeRO bucket shards."""
import itertools

import torch

from tinyinfinitrain_b200.models.tp_models import _qkv_rows, head_range
from tinyinfinitrain_b200.parallel.mesh import group_ranks, rank_coords
from tinyinfinitrain_b200.parallel.pp import one_f_one_b_order, partition_layers


def test_mesh_groups_partition_the_world():
    for tp, pp, dp in itertools.product((1, 2, 4), (1, 2), (1, 2, 4)):
        world = tp * pp * dp
        tpg, ppg, dpg = group_ranks(tp, pp, dp)
        for groups, size in ((tpg, tp), (ppg, pp), (dpg, dp)):
            assert all(len(g) == size for g in groups)
            assert sorted(r for g in groups for r in g) == list(range(world))       # every rank in exactly one group
        for r in range(world):
            d, p, t = rank_coords(r, tp, pp, dp)
            assert r == d * pp * tp + p * tp + t and 0 <= d < dp and 0 <= p < pp and 0 <= t < tp
            assert r in tpg[d * pp + p] and r in ppg[d * tp + t] and r in dpg[p * tp + t]
        # tensor-parallel ranks are adjacent, data-parallel replicas are the outermost stride
        assert all(g == list(range(g[0], g[0] + tp)) for g in tpg)


def test_head_ranges_cover_all_heads_even_when_uneven():
    for n, tp in ((12, 4), (25, 2), (25, 4), (32, 8), (8, 8), (7, 3)):
        spans = [head_range(n, tp, r) for r in range(tp)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [b - a for a, b in spans]
        assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)   # the first ranks take the extra head


def test_qkv_rows_pick_each_row_exactly_once_over_the_ranks():
    for n_head, n_kv, hd, tp in ((12, 12, 64, 4), (25, 25, 64, 2), (32, 8, 64, 8), (8, 2, 16, 2)):
        total = (n_head + 2 * n_kv) * hd
        seen = torch.zeros(total, dtype=torch.int32)
        for r in range(tp):
            rows = _qkv_rows(n_head, n_kv, hd, tp, r)
            q0, q1 = head_range(n_head, tp, r)
            k0, k1 = head_range(n_kv, tp, r)
            assert rows.numel() == ((q1 - q0) + 2 * (k1 - k0)) * hd
            assert torch.equal(rows[:(q1 - q0) * hd], torch.arange(q0 * hd, q1 * hd))            # q | k | v order is kept
            seen[rows] += 1
        assert bool((seen == 1).all())


def test_pipeline_partition_and_1f1b_properties():
    for layers, stages in ((12, 2), (48, 4), (5, 2), (7, 3), (4, 4)):
        parts = partition_layers(layers, stages)
        assert [x for p in parts for x in p] == list(range(layers))
        sizes = [len(p) for p in parts]
        assert max(sizes) - min(sizes) <= 1
    for stages, micro in ((2, 4), (4, 8), (4, 4), (3, 7), (1, 3)):
        for s in range(stages):
            order = one_f_one_b_order(s, stages, micro)
            fs = [m for k, m in order if k == "F"]
            bs = [m for k, m in order if k == "B"]
            assert fs == list(range(micro)) and bs == list(range(micro))
            in_flight, peak = 0, 0
            done_f = set()
            for k, m in order:
                if k == "F":
                    in_flight += 1
                    done_f.add(m)
                else:
                    assert m in done_f                      # backward of a micro-batch never precedes its forward
                    in_flight -= 1
                peak = max(peak, in_flight)
            assert peak <= min(micro, stages - s)           # activation stash bounded by the remaining depth
