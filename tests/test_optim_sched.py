"""Host logic around the layer that needs no GPU: the cross-layer prefetch assignment
(MOLE/cpp/core.cpp:1302-1345) through the C ABI, the host Adam of offloaded experts
(MOLE/optim/mixed_optim.py:28-152 with the arithmetic of MOLE/cpp/define.hpp:543-579) and the
scheduler's prefetch-count policy (MOLE/utils/Uscheduler.py:262-343) on stand-in layers."""
import types

import pytest
import torch
from hypothesis import given, settings, strategies as st

from mole_b200 import core
from mole_b200.optim.mixed_optim import CPUAdam


def assign_reference(P, F, E):
    """The greedy of MOLE/cpp/core.cpp:1302-1345 restated: a stack of lenders, most recent first."""
    n = len(E)
    gp, lp, stack, p_cur = [[] for _ in range(n)], [0] * n, [], P
    for i in range(n):
        fetchable = min(p_cur, F[i])
        if fetchable <= E[i]:
            need = E[i] - fetchable
            lp[i] = fetchable
            while stack and need > 0:
                top_id, top = stack[-1]
                take = min(top, need)
                gp[top_id].append([i, take])
                p_cur += take
                need -= take
                if take == top:
                    stack.pop()
                else:
                    stack[-1][1] = top - take
        else:
            lend = fetchable - E[i]
            p_cur -= lend
            stack.append([i, lend])
            lp[i] = E[i]
    return gp, lp


def test_fast_assign_prefetch_hand_cases():
    # one layer with time for 6 fetches but only 2 experts lends 4 slots to the next layer
    gp, lp = core.fast_assign_prefetch(8, [6, 1, 0], [2, 4, 4])
    assert lp == [2, 1, 0]
    assert gp == [[[1, 3], [2, 1]], [], []]
    # nothing to spare anywhere: purely local
    gp, lp = core.fast_assign_prefetch(4, [1, 2, 9], [4, 4, 4])
    assert lp == [1, 2, 4] and gp == [[], [], []]
    # the pool bounds what can be fetched at all
    gp, lp = core.fast_assign_prefetch(2, [5], [8])
    assert lp == [2] and gp == [[]]
    assert core.fast_assign_prefetch(3, [], []) == ([], [])


@settings(max_examples=200, deadline=None)
@given(st.integers(0, 20), st.lists(st.tuples(st.integers(0, 12), st.integers(0, 8)), min_size=0, max_size=12))
def test_fast_assign_prefetch_matches_restatement(P, layers):
    F = [a for a, _ in layers]
    E = [b for _, b in layers]
    gp, lp = core.fast_assign_prefetch(P, F, E)
    gp_ref, lp_ref = assign_reference(P, F, E)
    assert lp == lp_ref and gp == gp_ref
    # invariants: a layer never prefetches more than it owns; a lender lends only to later layers
    for i, (l, e) in enumerate(zip(lp, E)):
        assert 0 <= l <= e
        assert all(j > i and c > 0 for j, c in gp[i])


def _host_param(shape, seed):
    g = torch.Generator().manual_seed(seed)
    p = torch.randn(*shape, generator=g)
    p.grad_ = torch.randn(*shape, generator=g)
    p.momentum = torch.zeros(*shape)
    p.variance = torch.zeros(*shape)
    p.grad_.lazy_zero = False
    return p


@pytest.mark.parametrize("adamw,wd", [(False, 0.0), (False, 0.1), (True, 0.1)])
def test_cpu_adam_matches_torch_adam(adamw, wd):
    p = _host_param((3, 5, 7), 0)
    ref = p.clone().requires_grad_(True)
    opt_ref = (torch.optim.AdamW if adamw else torch.optim.Adam)([ref], lr=1e-2, betas=(0.9, 0.99),
                                                                  eps=1e-8, weight_decay=wd)
    opt = CPUAdam([p], lr=1e-2, betas=(0.9, 0.99), eps=1e-8, weight_decay=wd, adamw_mode=adamw)
    for step in range(4):
        g = torch.randn(3, 5, 7, generator=torch.Generator().manual_seed(10 + step))
        p.grad_.copy_(g)
        ref.grad = g.clone()
        opt.step()
        opt_ref.step()
        torch.testing.assert_close(p, ref.detach(), rtol=2e-6, atol=2e-7)
    torch.testing.assert_close(p.momentum, opt_ref.state[ref]["exp_avg"], rtol=1e-6, atol=1e-8)
    torch.testing.assert_close(p.variance, opt_ref.state[ref]["exp_avg_sq"], rtol=1e-6, atol=1e-8)
    assert opt.state[p]["step"] == 4


def test_cpu_adam_hybrid_split_only_steps_the_tail():
    """With the GPU stepping the first ``hybrid_adam_count`` experts, the host optimizer updates
    the rest and leaves the head alone; with all experts on the GPU it only counts steps."""
    p = _host_param((6, 4), 1)
    before = p.clone()
    opt = CPUAdam([p], lr=1e-2)
    opt.adv_adam, opt.hybrid_adam, opt.hybrid_adam_count = True, True, 4
    opt.step()
    assert torch.equal(p[:4], before[:4]) and not torch.equal(p[4:], before[4:])
    opt.hybrid_adam_count = -1
    mid = p.clone()
    opt.step()
    assert torch.equal(p, mid) and opt.state[p]["step"] == 2


class _Layer:
    def __init__(self, d_experts, pool_size):
        self.d_experts, self.pool_size = d_experts, pool_size
        self.global_prefetch = False
        self.local_prefetch_fwd_count = self.local_prefetch_bwd_count = 0
        self.global_prefetch_fwd_count = self.global_prefetch_bwd_count = 0


@pytest.fixture
def scheduler(monkeypatch):
    from mole_b200.utils import Uscheduler
    from mole_b200.moe import layer as L
    monkeypatch.setattr(Uscheduler.UniScheduler, "_instance", None)
    sched = Uscheduler.UniScheduler(local_rank=0, disable_overlap=True, adv_adam=False,
                                    gate_control_by_MOLE=True)
    layers = [_Layer(4, 8), _Layer(4, 8), _Layer(4, 8)]
    monkeypatch.setattr(L.MOLEModule, "_instance", layers)
    monkeypatch.setattr(Uscheduler.Udist.MOLEDist, "get_MOLE_world_size", staticmethod(lambda: 1))
    return Uscheduler.UniScheduler, sched, layers


def test_scheduler_local_prefetch_counts(scheduler):
    US, sched, layers = scheduler
    US.schedule_policy(profile_step=6, prefetch_on=True)
    sched.ftime = 0.010                        # one expert takes 10 ms to fetch
    sched.fwd_stat = [0.050, 0.021, 0.005]     # gaps in front of layers 0, 1, 2
    sched.bwd_stat = [0.030, 0.100, 0.009]     # gaps in front of layers 2, 1, 0 (backward order)
    US.set_prefetch_scheme("")
    assert sched.fwd_pf == [0, 3, 1]           # ceil(gap / fetch); the first layer's is switched off
    assert [m.local_prefetch_fwd_count for m in layers] == [0, 3, 1]
    assert [m.local_prefetch_bwd_count for m in layers] == [1, 4, 3]      # min(ceil, experts, pool)
    assert not any(m.global_prefetch for m in layers)
    US.schedule_policy(profile_step=6, prefetch_on=True, prefetch_floor=True,
                       deactivate_first_prefetch=False)
    US.set_prefetch_scheme("")
    assert sched.fwd_pf == [5, 2, 0]
    US.set_prefetch_scheme("[[1, 1, 1], [2, 2, 2]]")           # forced scheme
    assert [m.local_prefetch_fwd_count for m in layers] == [1, 1, 1]
    assert [m.local_prefetch_bwd_count for m in layers] == [2, 2, 2]


def test_scheduler_global_prefetch_assignment(scheduler):
    US, sched, layers = scheduler
    US.schedule_policy(profile_step=6, prefetch_on=True, global_prefetch=True,
                       deactivate_first_prefetch=False)
    sched.ftime = 0.010
    sched.fwd_stat = [0.065, 0.005, 0.000]     # layer 0 has time for 7 fetches, owns 4 experts
    sched.bwd_stat = [0.000, 0.000, 0.000]
    US.set_prefetch_scheme("")
    assert all(m.global_prefetch for m in layers)
    assert [m.local_prefetch_fwd_count for m in layers] == [4, 1, 0]
    # layer 0 lends its 3 spare fetches: all three to layer 1 (which needs 3 more)
    assert layers[0].global_prefetch_fwd_count == [[1, 3]]
    assert layers[1].global_prefetch_fwd_count == [] and layers[2].global_prefetch_fwd_count == []
    assert [m.local_prefetch_bwd_count for m in layers] == [0, 0, 0]


def test_scheduler_step_phases(scheduler):
    US, sched, layers = scheduler
    US.schedule_policy(profile_step=3, prefetch_on=True)
    sched.cur_step = 1
    assert US.time_it() and not US.prefetch_it()
    sched.cur_step = 3
    assert not US.time_it() and not US.prefetch_it()
    sched.cur_step = 4
    assert US.prefetch_it()
