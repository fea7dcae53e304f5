"""World-size-2 gloo tests of the data-parallel host logic, on the CPU oracle:
config 3's "local gradients -> all-reduce -> SGD" equals the single-program step."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))
sys.path.insert(0, os.path.join(ROOT, "tests"))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _load_fixture(name):
    from conftest import Golden
    return Golden(name)


def _worker(rank, world, port, q):
    import importlib
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import vmoracle
        dp = importlib.import_module("pjrt-ocl_b200.dataparallel")
        full = _load_fixture("c3_mlp_f32_small")
        grads = _load_fixture("c3_dp2_grads_f32_small")
        apply_ = _load_fixture("c3_dp2_apply_f32_small")
        blobs = {"full": full.blob, "grads": grads.blob, "apply": apply_.blob}
        plan = dp.DpPlan("full", "grads", batch_inputs=(0, 1), reduce_outputs=(0, 1, 2, 3),
                         apply_program="apply", apply_inputs=(2, 3, 4), apply_skip=1, scaling="strong")

        def run(name, ins):
            # every output of these f32 programs is f32; the oracle returns raw bytes
            outs = vmoracle.Program(blobs[name]).execute([np.ascontiguousarray(a) for a in ins], threads=1)
            return [o.view(np.float32) for o in outs]

        def all_reduce_sum(a):
            t = torch.from_numpy(np.array(a, copy=True))
            dist.all_reduce(t)
            return t.numpy()

        ins = dp.rank_inputs(plan, full.args, rank, world)
        assert ins[0].shape[0] == full.args[0].shape[0] // world
        got = dp.step(plan, world, run, all_reduce_sum, ins)
        want = run("full", full.args)
        ok = len(got) == len(want)
        err = 0.0
        for g, w in zip(got, want):
            g = np.asarray(g, np.float64).reshape(-1)
            w = np.asarray(w, np.float64).reshape(-1)
            err = max(err, float(np.max(np.abs(g - w) / (np.abs(w) + 1e-3))))
        q.put((rank, ok, err))
    finally:
        dist.destroy_process_group()


def test_c3_data_parallel_equals_single_program():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok, err in res:
        assert ok, f"rank {rank}: wrong number of results"
        assert err < 1e-4, f"rank {rank}: data-parallel step differs from the single-program step by {err}"


def _agree_worker(rank, world, port, q):
    import importlib
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        dp = importlib.import_module("pjrt-ocl_b200.dataparallel")
        # each rank would stop on its own after a different number of trips; the body holds a collective
        mine, trips, total = (3, 5)[rank], 0, 0.0
        while dp.ranks_agree(trips < mine):
            t = torch.ones(1)
            dist.all_reduce(t)
            total += float(t.item())
            trips += 1
        # the next collective still pairs up: nothing is left over from the loop
        t = torch.tensor([float(rank + 1)])
        dist.all_reduce(t)
        q.put((rank, trips, total, float(t.item())))
    finally:
        dist.destroy_process_group()


def test_loops_with_collectives_end_on_all_ranks_together():
    """The bench keeps its steps running while a per-rank sampler warms up; steps of replica and gradient plans
    hold all-reduces, so the loop condition is agreed between the ranks (dataparallel.ranks_agree)."""
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_agree_worker, args=(r, world, port, q)) for r in range(world)]
    for p_ in procs:
        p_.start()
    got = sorted(q.get(timeout=120) for _ in range(world))
    for p_ in procs:
        p_.join(60)
        assert p_.exitcode == 0
    assert [g[1] for g in got] == [5, 5]              # both ran until the slower-to-stop rank was done
    assert [g[2] for g in got] == [10.0, 10.0]        # every all-reduce in the body met its partner
    assert [g[3] for g in got] == [3.0, 3.0]
    dp = __import__("importlib").import_module("pjrt-ocl_b200.dataparallel")
    assert dp.ranks_agree(True) is True and dp.ranks_agree(False) is False      # no process group: the rank's own answer


def test_shard_rows_and_plan_names():
    import importlib
    dp = importlib.import_module("pjrt-ocl_b200.dataparallel")
    a = np.arange(24).reshape(8, 3)
    assert np.array_equal(dp.shard_rows(a, 1, 4), a[2:4])
    with pytest.raises(ValueError):
        dp.shard_rows(a, 0, 3)
    assert dp.PLANS["c3"].rank_program(1) == "c3_mlp_step_bf16"
    assert dp.PLANS["c3"].rank_program(4) == "c3_mlp_grads_bf16_dp4"
    assert dp.PLANS["c5_block"].rank_program(8) == "c5_block_bf16_dp8"
    assert dp.PLANS["c2"].rank_program(8) == "c2_chain_f32"
