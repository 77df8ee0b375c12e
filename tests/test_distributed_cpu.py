"""Host-side logic of the data-parallel gradient reducer, on two CPU ranks over gloo."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import sys
        from pathlib import Path
        sys.path.insert(0, str(Path(__file__).resolve().parents[1] / "sm120-nvfp4-training_b200"))
        from nvfp4_training.distributed import GradientReducer
        torch.manual_seed(0)
        params = [torch.nn.Parameter(torch.zeros(8 + i)) for i in range(5)]
        for p in params[:3]:
            p._v4_request_scale = True       # "converted layer weights": gradients live in reducer slots
        index = {id(p): i for i, p in enumerate(params)}
        red = GradientReducer(params, slot_dtype=torch.float32, depth=2, bucket_mb=0)
        assert red.world == world and red.grad_scale == 1.0 / world
        assert [red.has_slot(p) for p in params] == [True, True, True, False, False]

        # ---- streaming protocol: updates lag the submissions by `depth` --------------------------------
        red.begin(params, capturing=True)
        order, updated = [], []
        for i, p in reversed(list(enumerate(params))):          # backward order
            if red.has_slot(p):
                red.slot(p).fill_(float(rank + 1) * (i + 1))
                pack = (red.slot(p), None, None)
            else:
                p.grad = torch.full_like(p, float(rank + 1) * (i + 1))
                pack = (p.grad, None, None)
            ready = red.submit(p, "group", pack)
            order.append(i)
            assert len(red._queue) <= 2
            updated += [(index[id(q)], float(k[0][0])) for q, _, k in ready]
        updated += [(index[id(q)], float(k[0][0])) for q, _, k in red.drain()]
        assert [i for i, _ in updated] == order == [4, 3, 2, 1, 0]
        total = sum(r + 1 for r in range(world))
        assert all(abs(v - total * (i + 1)) < 1e-6 for i, v in updated)

        # ---- eager protocol: slots reduced when ready, dense gradients in finish() ---------------------
        red.begin(params)
        for i in (2, 1, 0):
            red.slot(params[i]).fill_(float(rank))
            red.ready(params[i])
        for p in params[3:]:
            p.grad = torch.full_like(p, 10.0 + rank)
        red.finish(params[3:])
        assert all(float(red.slot(p)[0]) == sum(range(world)) for p in params[:3])
        assert all(float(p.grad[0]) == sum(10.0 + r for r in range(world)) for p in params[3:])
        assert [index[id(p)] for p in red.launched] == [2, 1, 0]

        # ---- buckets: small dense gradients share one FP32 collective, slot gradients keep their own -------------
        red = GradientReducer(params, slot_dtype=torch.float32, depth=0, bucket_mb=1.0)
        red.begin(params, capturing=True)
        got = {}
        for i, p in reversed(list(enumerate(params))):
            if red.has_slot(p):
                red.slot(p).fill_(float(rank + 1) * (i + 1))
                pack = (red.slot(p), None, None)
            else:
                p.grad = torch.full_like(p, float(rank + 1) * (i + 1))
                pack = (p.grad, None, None)
            for q, _, k in red.submit(p, "group", pack):
                got[index[id(q)]] = k[0].clone()
        assert sorted(got) == [0, 1, 2]                      # the two dense gradients wait in the open bucket
        for q, _, k in red.drain():
            got[index[id(q)]] = k[0].clone()
        assert red.collectives == 4                          # three slots + one bucket for parameters 3 and 4
        assert all(got[i].shape == params[i].shape and abs(float(got[i].flatten()[0]) - total * (i + 1)) < 1e-6 for i in range(5))

        # ---- a parameter with a slot gradient and a second dense gradient: both are reduced ----------------------
        red.begin(params, capturing=True)
        p0 = params[0]
        red.slot(p0).fill_(float(rank + 1))
        second = torch.full_like(p0, 10.0 * (rank + 1))
        ready = red.submit(p0, "group", (red.slot(p0), None, None), extra=second) + red.drain()
        assert len(ready) == 1 and float(red.slot(p0)[0]) == total and float(second[0]) == 10.0 * total
        # an eager step after a captured one waits for its collectives again
        red.begin(params)
        assert red._streaming is False
        results[rank] = "ok"
    except Exception as e:  # pragma: no cover - reported to the parent
        results[rank] = repr(e)
    finally:
        dist.destroy_process_group()


def test_reducer_protocols_on_two_gloo_ranks():
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    assert dict(results) == {0: "ok", 1: "ok"}


# ---- failures are found on the host, between steps ---------------------------------------------------------------------
def _init(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import sys
    from pathlib import Path
    sys.path.insert(0, str(Path(__file__).resolve().parents[1] / "sm120-nvfp4-training_b200"))
    from nvfp4_training import distributed
    return distributed


def _guard_worker(rank, world, port, results):
    D = _init(rank, world, port)
    try:
        seen = {}
        # mismatched slot sizes: rank 1 converted a layer of another width
        params = [torch.nn.Parameter(torch.zeros(16 if rank == 0 else 24)), torch.nn.Parameter(torch.zeros(8))]
        params[0]._v4_request_scale = True
        try:
            D.verify_layout(D.GradientReducer(params, slot_dtype=torch.float32))
        except ValueError as e:
            seen["layout"] = str(e)
        # mismatched bucket size alone is found as well
        same = [torch.nn.Parameter(torch.zeros(16))]
        same[0]._v4_request_scale = True
        try:
            D.verify_layout(D.GradientReducer(same, slot_dtype=torch.float32, bucket_mb=1.0 + rank))
        except ValueError as e:
            seen["bucket"] = str(e)
        D.verify_layout(D.GradientReducer(same, slot_dtype=torch.float32))          # agreeing ranks pass
        # replicas that hold the same state agree; one changed weight (or moment) is found on every rank
        torch.manual_seed(0)
        model = torch.nn.Sequential(torch.nn.Linear(8, 8), torch.nn.LayerNorm(8))
        opt = torch.optim.AdamW(model.parameters(), lr=1e-2)
        model(torch.ones(2, 8)).sum().backward()
        opt.step()
        seen["digest"] = D.verify_replicas(model, opt)
        if rank == 1:
            with torch.no_grad():
                model[0].weight[3, 3] += 1e-3
        try:
            D.verify_replicas(model, opt)
        except RuntimeError as e:
            seen["diverged"] = str(e)
        if rank == 1:
            with torch.no_grad():
                model[0].weight[3, 3] -= 1e-3
                opt.state[model[0].bias]["exp_avg"][0] += 1.0
        try:
            D.verify_replicas(model, opt)
        except RuntimeError as e:
            seen["moment"] = str(e)
        results[rank] = seen
    except Exception as e:  # pragma: no cover - reported to the parent
        results[rank] = repr(e)
    finally:
        dist.destroy_process_group()


def test_layout_and_replica_guards_raise_on_every_rank():
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_guard_worker, args=(2, _free_port(), results), nprocs=2, join=True)
    got = dict(results)
    assert all(isinstance(got[r], dict) for r in (0, 1)), got
    for r in (0, 1):
        assert "ranks [1] differ from rank 0" in got[r]["layout"] and "ranks [1] differ" in got[r]["bucket"]
        assert "ranks [1] hold different state" in got[r]["diverged"] and "ranks [1]" in got[r]["moment"]
    assert got[0]["digest"] == got[1]["digest"] and len(got[0]["digest"]) == 64


def _leaver_worker(rank, world, port, results):
    D = _init(rank, world, port)
    try:
        watch = D.PeerWatch(timeout_s=4.0)
        watch.check()                      # step 1: everyone is there
        if rank == world - 1:
            results[rank] = "left"         # this rank leaves between steps, nothing of its in flight
            return
        try:
            watch.check()                  # step 2: the survivors learn of it before they launch anything
            results[rank] = "no error"
        except RuntimeError as e:
            results[rank] = str(e)
    except Exception as e:  # pragma: no cover - reported to the parent
        results[rank] = repr(e)
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_survivors_learn_of_a_rank_that_left_between_steps():
    world = 3
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_leaver_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    got = dict(results)
    assert got[2] == "left"
    for r in (0, 1):
        assert got[r].startswith("Data-parallel peer check failed before the step"), got
    assert "2" in got[0]                   # rank 0 names the rank that did not answer
