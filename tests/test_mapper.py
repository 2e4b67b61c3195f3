import itertools

import pytest

from optimus_lm_b200.mapper import ParallelDpPpEpTpMapper, RankGrid, ShapeND


def test_rank_grid_roundtrip():
    for sizes in ([2, 3, 4], [1, 5, 2, 2]):
        g = RankGrid(sizes)
        seen = set()
        for idx in itertools.product(*[range(s) for s in sizes]):
            f = g.get_flat_index(*idx)
            assert g.get_index(f) == idx
            seen.add(f)
        assert seen == set(range(g.numel))
    assert ShapeND is RankGrid


def test_rank_grid_permuted_matches_reference_numbering():
    # [DP, PP, EP, TP] = [2, 2, 2, 1]; with pp-first the PP axis varies slowest
    g = RankGrid([2, 2, 2, 1], [1, 0, 2, 3])
    assert g.get_flat_index(1, 0, 0, 0) == 2   # dp=1 -> stride EP*TP
    assert g.get_flat_index(0, 1, 0, 0) == 4   # pp=1 -> stride DP*EP*TP
    for r in range(8):
        assert g.get_flat_index(*g.get_index(r)) == r


@pytest.mark.parametrize("dp,pp,ep,tp,pp_first", [(2, 1, 4, 1, False), (1, 4, 2, 1, False), (2, 2, 2, 1, True),
                                                  (2, 2, 1, 2, False)])
def test_mapper_indices(dp, pp, ep, tp, pp_first):
    world = dp * pp * ep * tp
    coords = set()
    for r in range(world):
        m = ParallelDpPpEpTpMapper(dp, pp, ep, tp, rank=r, use_pp_first=pp_first)
        coords.add((m.dp_ind, m.pp_ind, m.ep_ind, m.tp_ind))
        assert m.mp_ind == m.pp_ind * ep * tp + m.ep_ind * tp + m.tp_ind
        assert m.dpep_ind == m.dp_ind * ep + m.ep_ind
        assert m.is_first_stage_rank == (m.pp_ind == 0) and m.is_last_stage_rank == (m.pp_ind == pp - 1)
        assert m.pp_ind_reverse == pp - 1 - m.pp_ind
        nxt = ParallelDpPpEpTpMapper(dp, pp, ep, tp, rank=m.next_stage_rank, use_pp_first=pp_first)
        assert (nxt.dp_ind, nxt.ep_ind, nxt.tp_ind) == (m.dp_ind, m.ep_ind, m.tp_ind)
        assert nxt.pp_ind == (m.pp_ind + 1) % pp
        assert r in m.all_stage_ranks[m.pp_ind]
        assert m.first_stage_ranks == m.all_stage_ranks[0] and m.last_stage_ranks == m.all_stage_ranks[-1]
        if not pp_first:
            assert m.mp_rank == r - m.dp_ind * pp * ep * tp
        # TP is the fastest axis
        if tp > 1 and m.tp_ind + 1 < tp:
            assert ParallelDpPpEpTpMapper(dp, pp, ep, tp, rank=r + 1, use_pp_first=pp_first).tp_ind == m.tp_ind + 1
        assert sorted(m.group_ranks(["ep"])) == sorted(
            q for q in range(world)
            if (lambda o: (o.dp_ind, o.pp_ind, o.tp_ind) == (m.dp_ind, m.pp_ind, m.tp_ind))(
                ParallelDpPpEpTpMapper(dp, pp, ep, tp, rank=q, use_pp_first=pp_first)))
    assert len(coords) == world


def _groups_worker(rank, world):
    import torch
    import torch.distributed as dist
    m = ParallelDpPpEpTpMapper(2, 1, 2, 1, rank=rank, create_groups=True)
    assert dist.get_process_group_ranks(m.ep_group) == m.group_ranks(["ep"])
    assert dist.get_process_group_ranks(m.dp_group) == m.group_ranks(["dp"])
    assert dist.get_process_group_ranks(m.dpep_group) == [0, 1, 2, 3]
    t = torch.tensor([float(rank)])
    dist.all_reduce(t, group=m.ep_group)
    assert t.item() == sum(m.group_ranks(["ep"]))
    assert "EP group ranks" in str(m)


def test_mapper_groups_gloo():
    from dist_utils import run_distributed
    run_distributed(_groups_worker, 4)
