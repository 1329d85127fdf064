"""5-D process topology: DP x PP x CP x EP x TP.

Ranks are laid out so that tensor-parallel peers are adjacent (fastest-varying) and
data-parallel replicas are furthest apart: ``rank = (((dp*PP + pp)*CP + cp)*EP + ep)*TP + tp``.
The attribute names and the set of groups follow picotron/process_group_manager.py:7-159, so
code written against the reference's ``process_group_manager`` global finds the same fields.

Unlike the reference, the coordinates and every group's member list are computed with plain
integer arithmetic (``GridTopology``) that needs no process group, so schedules, tests and
tools can reason about any rank's neighbours offline; ``ProcessGroupManager`` then creates
the ``torch.distributed`` groups from those lists.

Two extra groups exist for expert parallelism run as data parallelism for the dense weights
(``ep_as_dp``): ``dense_dp_group`` = all ranks sharing (pp, tp), used to reduce non-expert
gradients when every EP rank sees different tokens.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

AXES = ("dp", "pp", "cp", "ep", "tp")


@dataclass(frozen=True)
class GridTopology:
    """Pure arithmetic over the rank grid; no communication."""

    tp: int = 1
    cp: int = 1
    pp: int = 1
    dp: int = 1
    ep: int = 1

    @property
    def world_size(self) -> int:
        return self.tp * self.cp * self.pp * self.dp * self.ep

    @property
    def shape(self) -> Tuple[int, int, int, int, int]:
        return (self.dp, self.pp, self.cp, self.ep, self.tp)

    def coords(self, rank: int) -> Dict[str, int]:
        assert 0 <= rank < self.world_size
        out = {}
        for name, size in zip(reversed(AXES), reversed(self.shape)):
            out[name] = rank % size
            rank //= size
        return out

    def rank_of(self, **coords: int) -> int:
        r = 0
        for name, size in zip(AXES, self.shape):
            c = coords[name]
            assert 0 <= c < size, f"{name}={c} out of range {size}"
            r = r * size + c
        return r

    def group_ranks(self, rank: int, vary: Tuple[str, ...]) -> List[int]:
        """Ranks that share every coordinate of ``rank`` except those named in ``vary``."""
        base = self.coords(rank)
        ranks = [base]
        for name in vary:
            size = dict(zip(AXES, self.shape))[name]
            ranks = [dict(r, **{name: i}) for r in ranks for i in range(size)]
        return sorted(self.rank_of(**r) for r in ranks)

    def all_groups(self, vary: Tuple[str, ...]) -> List[List[int]]:
        seen, out = set(), []
        for r in range(self.world_size):
            g = tuple(self.group_ranks(r, vary))
            if g not in seen:
                seen.add(g)
                out.append(list(g))
        return out


class ProcessGroupManager:
    def __init__(self, tp_size: int, cp_size: int, pp_size: int, dp_size: int, ep_size: int = 1,
                 create_groups: bool = True):
        self.global_rank = dist.get_rank() if dist.is_initialized() else 0
        self.world_size = dist.get_world_size() if dist.is_initialized() else 1
        self.local_rank = self.global_rank  # single node; launchers may overwrite from LOCAL_RANK
        topo = GridTopology(tp=tp_size, cp=cp_size, pp=pp_size, dp=dp_size, ep=ep_size)
        assert self.world_size == topo.world_size, (
            f"world size ({self.world_size}) != tp({tp_size}) x cp({cp_size}) x ep({ep_size}) x "
            f"pp({pp_size}) x dp({dp_size})")
        self.topology = topo
        #: ranks as a [dp, pp, cp, ep, tp] tensor, the reference's view of the grid (process_group_manager.py:24-26)
        self.grid = torch.arange(self.world_size).view(dp_size, pp_size, cp_size, ep_size, tp_size)
        c = topo.coords(self.global_rank)
        self.dp_rank, self.pp_rank, self.cp_rank, self.ep_rank, self.tp_rank = (
            c["dp"], c["pp"], c["cp"], c["ep"], c["tp"])

        families = {
            "tp": ("tp",), "cp": ("cp",), "ep": ("ep",), "pp": ("pp",), "dp": ("dp",),
            "cp_dp": ("cp", "dp"), "pp_dp": ("pp", "dp"),
            "dense_dp": ("cp", "ep", "dp"),
        }
        self._group_ids: Dict[str, List[int]] = {}
        self._groups: Dict[str, Optional[dist.ProcessGroup]] = {}
        for name, vary in families.items():
            self._group_ids[name] = topo.group_ranks(self.global_rank, vary)
            self._groups[name] = None
            if create_groups and dist.is_initialized():
                # every rank must take part in the creation of every group of the family
                for members in topo.all_groups(vary):
                    g = dist.new_group(ranks=members)
                    if self.global_rank in members:
                        self._groups[name] = g
        self.world_group = dist.group.WORLD if dist.is_initialized() else None

        self.tp_group, self.cp_group, self.ep_group = self._groups["tp"], self._groups["cp"], self._groups["ep"]
        self.pp_group, self.dp_group = self._groups["pp"], self._groups["dp"]
        self.cp_dp_group, self.pp_dp_group = self._groups["cp_dp"], self._groups["pp_dp"]
        self.dense_dp_group = self._groups["dense_dp"]

        self.tp_group_ids, self.cp_group_ids = self._group_ids["tp"], self._group_ids["cp"]
        self.ep_group_ids, self.pp_group_ids = self._group_ids["ep"], self._group_ids["pp"]
        self.dp_group_ids, self.cp_dp_group_ids = self._group_ids["dp"], self._group_ids["cp_dp"]
        self.pp_dp_group_ids = self._group_ids["pp_dp"]
        self.dense_dp_group_ids = self._group_ids["dense_dp"]

        # tensor parallel
        self.tp_world_size = tp_size
        self.tp_first_rank, self.tp_last_rank = self.tp_group_ids[0], self.tp_group_ids[-1]
        # context parallel (ring neighbours)
        self.cp_world_size = cp_size
        self.cp_first_rank, self.cp_last_rank = self.cp_group_ids[0], self.cp_group_ids[-1]
        self.cp_send_rank = self.cp_group_ids[(self.cp_rank + 1) % cp_size]
        self.cp_recv_rank = self.cp_group_ids[(self.cp_rank - 1) % cp_size]
        # expert parallel
        self.ep_world_size = ep_size
        self.ep_first_rank, self.ep_last_rank = self.ep_group_ids[0], self.ep_group_ids[-1]
        # pipeline parallel
        self.pp_world_size = pp_size
        self.pp_first_rank, self.pp_last_rank = self.pp_group_ids[0], self.pp_group_ids[-1]
        self.pp_is_first_stage = self.pp_rank == 0
        self.pp_is_last_stage = self.pp_rank == pp_size - 1
        self.pp_next_rank = None if self.pp_is_last_stage else self.pp_group_ids[self.pp_rank + 1]
        self.pp_prev_rank = None if self.pp_is_first_stage else self.pp_group_ids[self.pp_rank - 1]
        # data parallel
        self.dp_world_size = dp_size
        self.dp_first_rank, self.dp_last_rank = self.dp_group_ids[0], self.dp_group_ids[-1]
        self.cp_dp_world_size = cp_size * dp_size
        self.pp_dp_world_size = pp_size * dp_size
        self.dense_dp_world_size = cp_size * ep_size * dp_size

    def get_info(self) -> str:
        return str(self)

    def __str__(self) -> str:
        return (f"TP({self.tp_world_size})-CP({self.cp_world_size})-EP({self.ep_world_size})-"
                f"PP({self.pp_world_size})-DP({self.dp_world_size})-Rank({self.global_rank})")


#: module-level singleton, set by ``setup_process_group_manager`` (same contract as the reference)
process_group_manager: Optional[ProcessGroupManager] = None


def setup_process_group_manager(tp_size: int, cp_size: int, pp_size: int, dp_size: int, ep_size: int = 1,
                                create_groups: bool = True) -> ProcessGroupManager:
    global process_group_manager
    process_group_manager = ProcessGroupManager(tp_size, cp_size, pp_size, dp_size, ep_size,
                                                create_groups=create_groups)
    return process_group_manager


def get_pgm() -> ProcessGroupManager:
    """The current manager; a trivial single-process one is created on first use if none was set."""
    global process_group_manager
    if process_group_manager is None:
        assert not dist.is_initialized() or dist.get_world_size() == 1, \
            "call setup_process_group_manager() after init_process_group()"
        process_group_manager = ProcessGroupManager(1, 1, 1, 1, 1, create_groups=False)
    return process_group_manager
