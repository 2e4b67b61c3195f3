"""Rank <-> (dp, pp, ep, tp) mapping and process-group construction.

Same public surface as the reference mappers (optimus/mapper.py:5-42 ``ShapeND``,
:44 ``ParallelDpTpMapper``, :143 ``ParallelDpEpMapper``, :243 ``ParallelDpEpTpMapper``,
:385-554 ``ParallelDpPpEpTpMapper``): the same constructor keywords, the same attribute
names (``dp_ind``, ``mp_ind``, ``dpep_group`` ...) and the same rank numbering (TP is the
fastest-varying axis, ``use_pp_first`` swaps the DP and PP axes).

The design differs: one generic ``RankGrid`` does the index arithmetic for any number of
named axes, and one ``_GridMapper`` base builds every process group from a list of "which
axes vary inside the group".  All ranks of the job build all groups in the same order,
as ``torch.distributed.new_group`` requires.
"""
from __future__ import annotations

import itertools
import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


class RankGrid:
    """Row-major N-D grid of ranks with an optional axis permutation.

    ``sizes`` are given in logical axis order; ``permute_order[i]`` names the logical
    axis stored at physical position ``i`` (position 0 varies slowest).
    """

    def __init__(self, sizes: Sequence[int], permute_order: Optional[Sequence[int]] = None):
        self.dim = len(sizes)
        self.permute_order = list(permute_order) if permute_order is not None else list(range(self.dim))
        if sorted(self.permute_order) != list(range(self.dim)):
            raise ValueError(f"permute_order {self.permute_order} is not a permutation of {self.dim} axes")
        self.logical_sizes = list(sizes)
        self.sizes = [sizes[p] for p in self.permute_order]
        # stride of each physical position
        self._strides = [1] * self.dim
        for i in range(self.dim - 2, -1, -1):
            self._strides[i] = self._strides[i + 1] * self.sizes[i + 1]
        self.numel = self._strides[0] * self.sizes[0] if self.dim else 1

    def get_flat_index(self, *index: int) -> int:
        if len(index) != self.dim:
            raise ValueError(f"expected {self.dim} coordinates, got {len(index)}")
        return sum(index[p] * s for p, s in zip(self.permute_order, self._strides))

    def get_index(self, flat_index: int) -> Tuple[int, ...]:
        physical = [(flat_index // s) % n for s, n in zip(self._strides, self.sizes)]
        # The reference applies the same permutation on the way back; for the two
        # permutations in use (identity and the DP/PP swap) that is its own inverse.
        return tuple(physical[p] for p in self.permute_order)

    def __str__(self) -> str:
        return "Shape : [" + " ".join(str(s) for s in self.logical_sizes) + "]"


# The reference name for the grid class.
ShapeND = RankGrid


def _read_hostfile_nodes() -> List[str]:
    """Node list of the current job, one entry per node, or [] when there is none.

    The directory is ``$OPTIMUS_LAUNCH_INFO_DIR/<job id>/hostfile`` (default
    ``launch_info/<job id>/hostfile`` under the working directory); the job id comes
    from ``$PBS_JOBID``/``$SLURM_JOB_ID``/"0".
    """
    job_id = os.getenv("PBS_JOBID", os.getenv("SLURM_JOB_ID", "0")).split(".")[0]
    root = os.getenv("OPTIMUS_LAUNCH_INFO_DIR", "launch_info")
    path = os.path.join(root, job_id, "hostfile")
    if not os.path.exists(path):
        return []
    with open(path) as fh:
        return [ln.strip() for ln in fh if ln.strip()]


class _GridMapper:
    """Shared machinery: coordinates, node map, group construction."""

    AXES: Tuple[str, ...] = ()

    def _init_grid(self, sizes: Sequence[int], rank: int, permute_order=None):
        self.rank = rank
        self.permute_order = list(permute_order) if permute_order is not None else list(range(len(sizes)))
        self.shape = RankGrid(sizes, self.permute_order)
        self._coord = dict(zip(self.AXES, self.shape.get_index(rank)))
        self.node = None
        self.rank_to_node_list: List[str] = []
        if dist.is_available() and dist.is_initialized():
            nodes = _read_hostfile_nodes()
            if nodes:
                world = dist.get_world_size()
                per_node = max(1, world // len(nodes))
                self.rank_to_node_list = [nodes[min(r // per_node, len(nodes) - 1)] for r in range(world)]
                self.node = self.rank_to_node_list[self.rank]

    def group_ranks(self, varying: Sequence[str], coord: Optional[Dict[str, int]] = None) -> List[int]:
        """Ranks of the group that contains ``coord`` and spans the ``varying`` axes."""
        coord = dict(self._coord if coord is None else coord)
        out = []
        ranges = [range(self.shape.logical_sizes[self.AXES.index(a)]) for a in varying]
        for combo in itertools.product(*ranges):
            c = dict(coord)
            c.update(zip(varying, combo))
            out.append(self.shape.get_flat_index(*[c[a] for a in self.AXES]))
        return out

    def _build_group(self, varying: Sequence[str]):
        """Create every group spanning ``varying`` (all ranks take part) and return mine."""
        fixed = [a for a in self.AXES if a not in varying]
        mine = -1
        ranges = [range(self.shape.logical_sizes[self.AXES.index(a)]) for a in fixed]
        for combo in itertools.product(*ranges):
            coord = dict(self._coord)
            coord.update(zip(fixed, combo))
            ranks = self.group_ranks(varying, coord)
            group = dist.new_group(ranks)
            if self.rank in ranks:
                mine = group
        return mine

    @staticmethod
    def _describe(group, name: str) -> str:
        ranks = dist.get_process_group_ranks(group) if group != -1 else [-1]
        return f"{name} group ranks : {ranks}\n"


class ParallelDpTpMapper(_GridMapper):
    """DP x TP mapper (reference optimus/mapper.py:44-141)."""

    AXES = ("dp", "tp")

    def __init__(self, data_parallelism=1, tensor_parallelism=1, rank=0, create_groups=False):
        self.data_parallelism = self.DP = data_parallelism
        self.tensor_parallelism = self.TP = tensor_parallelism
        self._init_grid([self.DP, self.TP], rank)
        self.dp_ind, self.tp_ind = self._coord["dp"], self._coord["tp"]
        self.mp_ind = self.tp_ind
        self.dp_group = self.tp_group = -1
        if create_groups:
            self.create_groups()

    def create_groups(self):
        self.dp_group = self.create_and_get_dp_group()
        self.tp_group = self.create_and_get_tp_group()

    def create_and_get_dp_group(self):
        return self._build_group(["dp"])

    def create_and_get_tp_group(self):
        return self._build_group(["tp"])

    def get_index(self):
        return f"(DP: {self.dp_ind}, TP : {self.tp_ind})"

    def get_rank_with_index(self):
        return f"Rank : {self.rank} ({self.get_index()})"

    def __str__(self):
        s = f"******* Process map information for rank {self.rank} *******\n"
        s += f"Node : {self.node}\nRank : {self.rank}, (dp_ind : {self.dp_ind}, tp_ind : {self.tp_ind})\n"
        s += self._describe(self.tp_group, "TP") + self._describe(self.dp_group, "DP")
        return s + "*" * 50


class ParallelDpEpMapper(_GridMapper):
    """DP x EP mapper (reference optimus/mapper.py:143-241)."""

    AXES = ("dp", "ep")

    def __init__(self, data_parallelism=1, expert_parallelism=1, rank=0, create_groups=False):
        self.data_parallelism = self.DP = data_parallelism
        self.expert_parallelism = self.EP = expert_parallelism
        self._init_grid([self.DP, self.EP], rank)
        self.dp_ind, self.ep_ind = self._coord["dp"], self._coord["ep"]
        self.mp_ind = self.ep_ind
        self.dpep_ind = self.dp_ind * self.EP + self.ep_ind
        self.dp_group = self.ep_group = self.dpep_group = -1
        if create_groups:
            self.create_groups()

    def create_groups(self):
        self.dp_group = self._build_group(["dp"])
        self.ep_group = self._build_group(["ep"])
        self.dpep_group = self._build_group(["dp", "ep"])

    def get_index(self):
        return f"(DP: {self.dp_ind}, EP : {self.ep_ind})"

    def get_rank_with_index(self):
        return f"Rank : {self.rank} ({self.get_index()})"

    def __str__(self):
        s = f"******* Process map information for rank {self.rank} *******\n"
        s += f"Node : {self.node}\nRank : {self.rank}, (dp_ind : {self.dp_ind}, ep_ind : {self.ep_ind})\n"
        s += self._describe(self.ep_group, "EP") + self._describe(self.dp_group, "DP")
        return s + "*" * 50


class ParallelDpEpTpMapper(_GridMapper):
    """DP x EP x TP mapper (reference optimus/mapper.py:243-383)."""

    AXES = ("dp", "ep", "tp")

    def __init__(self, data_parallelism=1, expert_parallelism=1, tensor_parallelism=1, rank=0,
                 create_groups=False):
        self.data_parallelism = self.DP = data_parallelism
        self.expert_parallelism = self.EP = expert_parallelism
        self.tensor_parallelism = self.TP = tensor_parallelism
        self._init_grid([self.DP, self.EP, self.TP], rank)
        self.dp_ind, self.ep_ind, self.tp_ind = (self._coord[a] for a in self.AXES)
        self.mp_ind = self.ep_ind * self.TP + self.tp_ind
        self.dpep_ind = self.dp_ind * self.EP + self.ep_ind
        self.dp_group = self.tp_group = self.ep_group = self.dpep_group = -1
        if create_groups:
            self.create_groups()

    def create_groups(self):
        self.dp_group = self._build_group(["dp"])
        self.tp_group = self._build_group(["tp"])
        self.ep_group = self._build_group(["ep"])
        self.dpep_group = self._build_group(["dp", "ep"])

    def get_index(self):
        return f"(DP: {self.dp_ind}, EP : {self.ep_ind}, TP : {self.tp_ind})"

    def get_rank_with_index(self):
        return f"Rank : {self.rank} ({self.get_index()})"

    def __str__(self):
        s = f"******* Process map information for rank {self.rank} *******\n"
        s += f"Node : {self.node}\n"
        s += f"Rank : {self.rank}, (dp_ind : {self.dp_ind}, ep_ind : {self.ep_ind}, tp_ind : {self.tp_ind})\n"
        s += self._describe(self.tp_group, "TP") + self._describe(self.ep_group, "EP")
        s += self._describe(self.dp_group, "DP") + self._describe(self.dpep_group, "DPEP")
        return s + "*" * 50


class ParallelDpPpEpTpMapper(_GridMapper):
    """The 4-axis mapper used by the trainer (reference optimus/mapper.py:385-554).

    Axis order is [DP, PP, EP, TP] with TP fastest; ``use_pp_first`` stores PP ahead of DP.
    ``mp_ind = pp*EP*TP + ep*TP + tp`` names the model shard, ``mp_rank`` is the rank
    inside one data-parallel replica, ``dpep_ind = dp*EP + ep`` is the data-parallel index
    of non-expert parameters (EP ranks are data parallel for everything that is not an
    expert).
    """

    AXES = ("dp", "pp", "ep", "tp")

    def __init__(self, data_parallelism=1, pipeline_parallelism=1, expert_parallelism=1,
                 tensor_parallelism=1, rank=0, create_groups=False, use_pp_first=False):
        self.data_parallelism = self.DP = data_parallelism
        self.pipeline_parallelism = self.PP = pipeline_parallelism
        self.expert_parallelism = self.EP = expert_parallelism
        self.tensor_parallelism = self.TP = tensor_parallelism
        self.use_pp_first = use_pp_first
        self._init_grid([self.DP, self.PP, self.EP, self.TP], rank,
                        [1, 0, 2, 3] if use_pp_first else [0, 1, 2, 3])
        self.dp_ind, self.pp_ind, self.ep_ind, self.tp_ind = (self._coord[a] for a in self.AXES)
        self.dpep_ind = self.dp_ind * self.EP + self.ep_ind

        self.is_model_parallel = self.PP > 1 or self.EP > 1 or self.TP > 1
        self.mp_ind = self.pp_ind * (self.EP * self.TP) + self.ep_ind * self.TP + self.tp_ind
        self.mp_rank = self.rank - self.dp_ind * (self.PP * self.EP * self.TP)

        self.is_first_stage_rank = self.pp_ind == 0
        self.is_last_stage_rank = self.pp_ind == self.PP - 1
        self.pp_ind_reverse = (self.PP - 1) - self.pp_ind

        flat = self.shape.get_flat_index
        self.prev_stage_rank = flat(self.dp_ind, (self.pp_ind - 1) % self.PP, self.ep_ind, self.tp_ind)
        self.next_stage_rank = flat(self.dp_ind, (self.pp_ind + 1) % self.PP, self.ep_ind, self.tp_ind)
        self.all_stage_ranks = [
            [flat(self.dp_ind, p, e, t) for e in range(self.EP) for t in range(self.TP)]
            for p in range(self.PP)
        ]
        self.first_stage_ranks = self.all_stage_ranks[0]
        self.last_stage_ranks = self.all_stage_ranks[-1]

        self.dp_group = self.tp_group = self.ep_group = self.dpep_group = -1
        if create_groups:
            self.create_groups()

    @property
    def world_size(self) -> int:
        return self.DP * self.PP * self.EP * self.TP

    def create_groups(self):
        self.dp_group = self.create_and_get_dp_group()
        self.tp_group = self.create_and_get_tp_group()
        self.ep_group = self.create_and_get_ep_group()
        self.dpep_group = self.create_and_get_dpep_group()

    def create_and_get_dp_group(self):
        return self._build_group(["dp"])

    def create_and_get_tp_group(self):
        return self._build_group(["tp"])

    def create_and_get_ep_group(self):
        return self._build_group(["ep"])

    def create_and_get_dpep_group(self):
        return self._build_group(["dp", "ep"])

    def get_index(self):
        return f"(DP: {self.dp_ind}, EP : {self.ep_ind}, TP : {self.tp_ind})"

    def get_rank_with_index(self):
        return f"Rank : {self.rank} ({self.get_index()})"

    def __str__(self):
        s = f"******* Process map information for rank {self.rank} *******\n"
        s += f"Node : {self.node}\n"
        s += (f"Rank : {self.rank}, (dp_ind : {self.dp_ind}, pp_ind : {self.pp_ind}, "
              f"ep_ind : {self.ep_ind}, tp_ind : {self.tp_ind})\n")
        s += self._describe(self.tp_group, "TP") + self._describe(self.ep_group, "EP")
        s += self._describe(self.dp_group, "DP") + self._describe(self.dpep_group, "DPEP")
        s += f"First/Last stage ranks : {self.first_stage_ranks, self.last_stage_ranks}\n"
        s += f"All stage ranks : {self.all_stage_ranks}\n"
        return s + "*" * 50
