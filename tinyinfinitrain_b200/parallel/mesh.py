"""Process-group layout for DP x PP x TP on one node.

Global rank = dp_rank * (pp * tp) + pp_rank * tp + tp_rank: tensor-parallel ranks are adjacent
GPUs, pipeline stages the next stride, data-parallel replicas the outermost.  On a B200 NVSwitch
box every pair of GPUs has the same bandwidth, so the order only matters for readability.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch.distributed as dist


@dataclass
class ParallelMesh:
    tp: int
    pp: int
    dp: int
    rank: int
    tp_rank: int
    pp_rank: int
    dp_rank: int
    tp_group: Optional[dist.ProcessGroup]
    pp_group: Optional[dist.ProcessGroup]
    dp_group: Optional[dist.ProcessGroup]
    pp_ranks: List[int]   # global ranks of this rank's pipeline, by stage
    mp_group: Optional[dist.ProcessGroup] = None   # the tp * pp ranks that hold one model replica (None when that is 1 rank)
    # first and last pipeline stage of this rank's pipeline (same tp rank): the two holders of a tied embedding /
    # output projection.  None when pp == 1 or on middle stages.
    embed_group: Optional[dist.ProcessGroup] = None

    @property
    def is_first_stage(self) -> bool:
        return self.pp_rank == 0

    @property
    def is_last_stage(self) -> bool:
        return self.pp_rank == self.pp - 1

    def prev_stage_rank(self) -> int:
        return self.pp_ranks[self.pp_rank - 1]

    def next_stage_rank(self) -> int:
        return self.pp_ranks[self.pp_rank + 1]


def rank_coords(rank: int, tp: int, pp: int, dp: int):
    """(dp_rank, pp_rank, tp_rank) of a global rank."""
    return rank // (pp * tp), (rank // tp) % pp, rank % tp


def group_ranks(tp: int, pp: int, dp: int):
    """All tensor-, pipeline- and data-parallel rank lists of a tp*pp*dp world (pure function)."""
    tp_groups = [[d * pp * tp + p * tp + t for t in range(tp)] for d in range(dp) for p in range(pp)]
    pp_groups = [[d * pp * tp + p * tp + t for p in range(pp)] for d in range(dp) for t in range(tp)]
    dp_groups = [[d * pp * tp + p * tp + t for d in range(dp)] for p in range(pp) for t in range(tp)]
    return tp_groups, pp_groups, dp_groups


def init_mesh(tp: int = 1, pp: int = 1, dp: Optional[int] = None) -> ParallelMesh:
    """Creates the tp / pp / dp process groups (collective: every rank must call it)."""
    world, rank = dist.get_world_size(), dist.get_rank()
    if dp is None:
        assert world % (tp * pp) == 0, f"world {world} not divisible by tp*pp = {tp * pp}"
        dp = world // (tp * pp)
    assert tp * pp * dp == world, f"tp*pp*dp = {tp * pp * dp} != world {world}"
    tpg, ppg, dpg = group_ranks(tp, pp, dp)
    mine = {"tp": None, "pp": None, "dp": None}
    my_pp_ranks: List[int] = [rank]
    for kind, groups in (("tp", tpg), ("pp", ppg), ("dp", dpg)):
        for ranks in groups:
            g = dist.new_group(ranks) if len(ranks) > 1 else None  # every rank creates every group, in the same order
            if rank in ranks:
                mine[kind] = g
                if kind == "pp":
                    my_pp_ranks = ranks
    d, p, t = rank_coords(rank, tp, pp, dp)
    mp_group = None
    for dd in range(dp):                                   # one model-parallel group per data-parallel replica
        ranks = list(range(dd * pp * tp, (dd + 1) * pp * tp))
        g = dist.new_group(ranks) if len(ranks) > 1 else None
        if rank in ranks:
            mp_group = g
    embed_group = None
    if pp > 1:
        for ranks in ppg:                                  # one group per pipeline: its first and last stage
            pair = [ranks[0], ranks[-1]]
            g = dist.new_group(pair)
            if rank in pair:
                embed_group = g
    return ParallelMesh(tp, pp, dp, rank, t, p, d, mine["tp"], mine["pp"], mine["dp"], my_pp_ranks, mp_group, embed_group)
