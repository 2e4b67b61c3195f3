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
