import pytest
import torch

from optimus_lm_b200.schedules import make_schedule, max_in_flight, simulate


@pytest.mark.parametrize("scheme,PP,NMB,VPP", [("gpipe", 4, 8, 1), ("1f1b", 4, 8, 1), ("1f1b", 4, 8, 2),
                                               ("1f1b", 2, 4, 2), ("1f1b", 4, 4, 3), ("gpipe", 2, 4, 2),
                                               ("1f1b", 8, 16, 2), ("1f1b", 4, 2, 1), ("1f1b", 1, 3, 1)])
def test_schedules_complete_and_deadlock_free(scheme, PP, NMB, VPP):
    for p in range(PP):
        ops = make_schedule(scheme, p, PP, NMB, VPP)
        fs = [(o.mb, o.vp) for o in ops if o.kind == "F"]
        bs = [(o.mb, o.vp) for o in ops if o.kind == "B"]
        want = sorted((m, v) for m in range(NMB) for v in range(VPP))
        assert sorted(fs) == want and sorted(bs) == want
        seen = set()
        for o in ops:
            if o.kind == "F":
                seen.add((o.mb, o.vp))
            else:
                assert (o.mb, o.vp) in seen
        if scheme == "1f1b" and VPP == 1:
            assert max_in_flight(ops) == min(PP - p, NMB)
    simulate(scheme, PP, NMB, VPP)


def _toy_worker(rank, world, scheme, VPP):
    from optimus_lm_b200.trainer import self_test
    out_err, grad_err = self_test(pp_scheme=scheme, VPP=VPP, verbose=False)
    if out_err is not None:
        assert out_err < 1e-5
    if grad_err is not None:
        assert grad_err < 1e-5


@pytest.mark.parametrize("scheme,VPP,world", [("1f1b", 2, 2), ("gpipe", 1, 2), ("1f1b", 1, 4), ("1f1b", 2, 4)])
def test_toy_pipeline_matches_serial(scheme, VPP, world):
    from dist_utils import run_distributed
    run_distributed(_toy_worker, world, scheme, VPP)


def test_buffer_manager_follows_every_schedule_and_stays_within_the_reference_bound():
    """The slot plan of the activations in flight: replaying each stage's schedule never needs more slots than the
    schedule's peak, slots are reused lowest-first, the backward index maps to the forward it undoes, and for the
    interleaved schedule the peak is within the reference's buffer count (optimus/trainer.py:99-101)."""
    from types import SimpleNamespace

    from optimus_lm_b200.schedules import Interleaved1f1bBufferManager, make_schedule, max_in_flight

    for scheme, PP, NMB, VPP in [("1f1b", 2, 4, 1), ("1f1b", 4, 8, 1), ("1f1b", 2, 4, 2), ("1f1b", 4, 8, 2), ("1f1b", 4, 8, 4),
                                 ("1f1b", 3, 4, 1), ("gpipe", 2, 3, 1), ("gpipe", 3, 5, 2)]:
        for pp_ind in range(PP):
            pmap = SimpleNamespace(pp_ind=pp_ind, pp_ind_reverse=PP - 1 - pp_ind, rank=pp_ind)
            ops = make_schedule(scheme, pp_ind, PP, NMB, VPP)
            mgr = Interleaved1f1bBufferManager(pmap, VPP, PP, NMB, reuse_buffers_in_1f1b=True, pp_scheme=scheme)
            assert mgr.num_act_buffers == max_in_flight(ops) and mgr.num_ograd_buffers == 1
            if scheme == "1f1b" and VPP > 1:
                assert mgr.num_act_buffers <= VPP * PP - pp_ind + pmap.pp_ind_reverse + 1
            seen = set()
            n_b = 0
            for op in ops:
                idx = mgr.flat_index(op.mb, op.vp)
                assert 0 <= idx < VPP * NMB
                if op.kind == "F":
                    assert idx not in seen
                    seen.add(idx)
                    slot = mgr.add_forward_to_flight(idx)
                    assert slot == mgr.get_forward_buffer_id(idx) and 0 <= slot < mgr.num_act_buffers
                else:
                    if scheme == "1f1b" and VPP > 1:
                        assert mgr.get_forward_index_from_backward_index(n_b) == idx
                    n_b += 1
                    assert mgr.get_backward_buffer_id(idx) == 0
                    assert mgr.drain_forward_from_flight(idx) is not None
            assert len(seen) == VPP * NMB and mgr.peak_used == mgr.num_act_buffers and not mgr._slot_of
            full = Interleaved1f1bBufferManager(pmap, VPP, PP, NMB, reuse_buffers_in_1f1b=False, pp_scheme=scheme)
            assert full.num_act_buffers == VPP * NMB == full.num_ograd_buffers and full.get_backward_buffer_id(3 % (VPP * NMB)) == 3 % (VPP * NMB)
    assert mgr.get_forward_buffer_id(None) is None and mgr.get_forward_buffer_id(-1) is None
