"""Host-side logic of the fused data-parallel optimizer: bucket/slice/segment plan,
equivalence with torch AdamW + clip, sharded state <-> torch state dict, and
N gloo ranks == one process."""

import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dual_mod_public_b200.parallel.fused_optim import (FusedDPAdamW, NcclAdamW, decay_groups,
                                                       default_buckets)

from helpers import free_port, make_model, rand_idx, small_cfg


def _grads_like(params, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(p.shape, generator=g) * 0.1 for p in params]


def test_matches_torch_adamw_with_clip():
    cfg = small_cfg()
    m1, m2 = make_model(cfg), make_model(cfg)
    opt = FusedDPAdamW(decay_groups(m1, 0.1), default_buckets(m1), lr=1e-2, max_norm=0.5, use_kernel=False)
    G = opt.grad_buffers()
    ref = torch.optim.AdamW([{"params": g["params"], "weight_decay": g["weight_decay"]}
                             for g in decay_groups(m2, 0.1)], lr=1e-2, betas=(0.9, 0.95), eps=1e-8)
    uniq2 = [p for g in ref.param_groups for p in g["params"]]
    order1 = [p for g in decay_groups(m1, 0.1) for p in g["params"]]
    for step in range(3):
        gs = _grads_like(order1, step)
        opt.zero_grad()
        for p, g in zip(order1, gs):
            G.get(p).copy_(g)
        for p, g in zip(uniq2, gs):
            p.grad = g.clone()
        torch.nn.utils.clip_grad_norm_(uniq2, 0.5)
        ctrl = opt.step()
        ref.step()
        assert ctrl[2] == 0
    for a, b in zip(order1, uniq2):
        assert (a - b).abs().max() < 1e-6
    sd = opt.state_dict()
    rsd = ref.state_dict()
    for k in rsd["state"]:
        assert (sd["state"][k]["exp_avg"] - rsd["state"][k]["exp_avg"]).abs().max() < 1e-6
    # round trip through the torch layout
    opt2 = FusedDPAdamW(decay_groups(m2, 0.1), default_buckets(m2), lr=1e-2, use_kernel=False)
    opt2.load_state_dict(sd)
    assert (opt2.m - opt.m).abs().max() == 0 and opt2.step_count == 3


def test_skip_predicate_leaves_parameters_untouched():
    cfg = small_cfg()
    m = make_model(cfg)
    opt = FusedDPAdamW(decay_groups(m, 0.0), default_buckets(m), lr=1e-2, skip_norm=1e-3, use_kernel=False)
    before = opt.flat_params.clone()
    opt.flat_grads.fill_(1.0)
    ctrl = opt.step()
    assert ctrl[2] == 1 and torch.equal(before, opt.flat_params)
    opt.flat_grads[0] = float("nan")
    assert opt.step()[2] == 1 and torch.equal(before, opt.flat_params)


def test_skipped_steps_do_not_advance_adamw_time():
    """Two voided steps, then two applied ones: parameters, moments and the saved `step` equal
    torch.optim.AdamW's, whose step() is simply not called on a voided step."""
    cfg = small_cfg()
    m1, m2 = make_model(cfg), make_model(cfg)
    opt = FusedDPAdamW(decay_groups(m1, 0.1), default_buckets(m1), lr=1e-2, max_norm=0.0, use_kernel=False)
    G = opt.grad_buffers()
    ref = torch.optim.AdamW([{"params": g["params"], "weight_decay": g["weight_decay"]}
                             for g in decay_groups(m2, 0.1)], lr=1e-2, betas=(0.9, 0.95), eps=1e-8)
    uniq2 = [p for g in ref.param_groups for p in g["params"]]
    order1 = [p for g in decay_groups(m1, 0.1) for p in g["params"]]
    for step in range(4):
        gs = _grads_like(order1, step)
        opt.zero_grad()
        for p, g in zip(order1, gs):
            G.get(p).copy_(g)
        void = step < 2
        opt.skip_norm = 1e-30 if void else 0.0          # every finite norm exceeds 1e-30
        ctrl = opt.step()
        assert bool(ctrl[2]) == void
        if not void:
            for p, g in zip(uniq2, gs):
                p.grad = g.clone()
            ref.step()
    assert opt.applied_steps() == 2 and float(opt.ctrl[4]) == 2.0
    for a, b in zip(order1, uniq2):
        assert (a - b).abs().max() < 1e-6
    sd, rsd = opt.state_dict(), ref.state_dict()
    assert float(sd["state"][0]["step"]) == float(rsd["state"][0]["step"]) == 2.0


def test_expired_wait_is_reported_with_the_step_verdict():
    """The status word set by hand (as the kernels set it when a bounded wait runs out): the step is
    voided, the code rides in ctrl[7], and check_status names the peer and the phase."""
    from dual_mod_public_b200.parallel.fused_optim import PeerWaitExpired
    cfg = small_cfg()
    m = make_model(cfg)
    opt = FusedDPAdamW(decay_groups(m, 0.0), default_buckets(m), lr=1e-2, use_kernel=False)
    opt.flat_grads.fill_(1e-3)
    assert opt.step()[2] == 0
    opt.check_status(int(opt.ctrl[7]))
    before = opt.flat_params.clone()
    opt.status[0], opt.status[1] = 2, 5
    ctrl = opt.step()
    assert ctrl[2] == 1 and ctrl[7] == 2 and torch.equal(before, opt.flat_params)
    with pytest.raises(PeerWaitExpired, match="rank 5 at the norm exchange"):
        opt.check_status(int(ctrl[7]))


def _rank_main(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(0)
    cfg = small_cfg()
    m = make_model(cfg, seed=10 + rank)             # different inits: rank 0's must win
    opt = FusedDPAdamW(decay_groups(m, 0.1), default_buckets(m), lr=1e-2, max_norm=1.0, use_kernel=False)
    G = opt.grad_buffers()
    order = [p for g in decay_groups(m, 0.1) for p in g["params"]]
    for step in range(2):
        opt.zero_grad()
        for p, g in zip(order, _grads_like(order, 100 * step + rank)):
            G.get(p).copy_(g)
        opt.step()
    sd = opt.state_dict()
    if rank == 0:
        q.put((opt.flat_params.clone(), sd["state"][0]["exp_avg"].clone()))
    flat = opt.flat_params.clone()
    ref = flat.clone()
    dist.broadcast(ref, src=0)
    assert torch.equal(ref, flat), "ranks diverged"
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_gloo_ranks_equal_single_process(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    flat_dp, m0 = q.get(timeout=120)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    # single process, averaged gradients
    cfg = small_cfg()
    m = make_model(cfg, seed=10)
    opt = FusedDPAdamW(decay_groups(m, 0.1), default_buckets(m), lr=1e-2, max_norm=1.0, use_kernel=False)
    G = opt.grad_buffers()
    order = [p for g in decay_groups(m, 0.1) for p in g["params"]]
    for step in range(2):
        opt.zero_grad()
        for r in range(world):
            for p, g in zip(order, _grads_like(order, 100 * step + r)):
                G.get(p).add_(g / world)
        opt.step()
    # layouts differ in padding (bucket length depends on world): compare per parameter
    opt_dp_layout_world = world
    from dual_mod_public_b200.parallel.fused_optim import BucketLayout
    lay_dp = BucketLayout(default_buckets(m), opt_dp_layout_world)
    for p in order:
        assert (lay_dp.view(flat_dp, p) - p.detach()).abs().max() < 1e-5


def test_nccl_baseline_interface_single_process():
    cfg = small_cfg()
    m = make_model(cfg)
    opt = NcclAdamW(decay_groups(m, 0.1), lr=1e-2)
    G = opt.grad_buffers()
    for p in m.parameters():
        G.get(p).fill_(0.01)
    w0 = m.norm_f.weight.detach().clone()
    opt.step()
    assert not torch.equal(w0, m.norm_f.weight)
