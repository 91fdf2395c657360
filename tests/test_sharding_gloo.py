"""CPU: the multi-GPU host logic (packing plan, dealing packs to ranks, final gather) with
world_size-2 gloo processes.  No collective is on the data path; ranks only meet in the gather."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oasr_b200 import sharding


def _lengths(n=300, seed=5):
    rng = np.random.default_rng(seed)
    secs = np.clip(rng.lognormal(np.log(6.0), 0.6, size=n), 1.0, 30.0)
    return [int(round(100 * s)) for s in secs]


def test_plan_packs_follows_reference_rule():
    lens = [400, 650, 800, 1000, 33000, 120, 120]
    packs = sharding.plan_packs(lens, max_packed_frames=400)
    flat = [i for p in packs for i in p]
    assert sorted(flat) == list(range(len(lens)))
    assert [lens[i] for i in flat] == sorted(lens)                # ascending length, stable
    for p in packs:                                               # budget holds unless a single utterance exceeds it
        tok = sum(max(1, lens[i] // 4) for i in p)
        assert tok <= 400 or len(p) == 1
    assert packs[0] == [5, 6, 0, 1]                               # 30 + 30 + 100 + 162 <= 400; the next (200) does not fit

def test_assign_packs_is_balanced_and_deterministic():
    lens = _lengths()
    packs = sharding.plan_packs(lens)
    for world in (1, 2, 4, 8):
        plan = sharding.assign_packs(lens, packs, world)
        assert plan == sharding.assign_packs(lens, packs, world)
        assert sorted(j for r in plan for j in r) == list(range(len(packs)))
        loads = [sum(sharding.pack_cost(lens, packs[j]) for j in r) for r in plan]
        if len(packs) >= 4 * world:
            assert max(loads) / (sum(loads) / world) < 1.25


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, lens, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        packs = sharding.plan_packs(lens)
        mine = sharding.assign_packs(lens, packs, world)[rank]
        # stand-in for the GPU step: the "tokens" of utterance i are a function of i and its length
        local = {i: [i, lens[i] % 97, rank] for j in mine for i in packs[j]}
        if rank == 1 and ret.get("drop"):
            local.pop(next(iter(local)))
        try:
            out = sharding.gather_results(local, len(lens))
            if rank == 0:
                ret["out"] = out
        except RuntimeError as e:
            ret["err"] = str(e)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("drop", [False, True])
def test_two_rank_gloo_gather(drop):
    lens = _lengths(64)
    mgr = mp.Manager()
    ret = mgr.dict()
    ret["drop"] = drop
    port = _free_port()
    mp.spawn(_worker, args=(2, port, lens, ret), nprocs=2, join=True)
    if drop:
        assert "not processed by any rank" in ret["err"]           # a lost utterance is detected on the host
        return
    out = ret["out"]
    assert len(out) == len(lens)
    assert all(out[i][0] == i and out[i][1] == lens[i] % 97 for i in range(len(lens)))
    assert {t[2] for t in out} == {0, 1}                            # both ranks contributed
