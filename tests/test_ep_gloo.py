"""CPU tests (gloo, world_size 2) of the expert-parallel plumbing in strixite_b200/ep.py: token / expert sharding,
the all-gather into the experts and the reduce-scatter out of them.  The per-rank device work is replaced by a
stand-in built on the CPU oracle, so what is tested is exactly the exchange logic the GPU ranks run."""
import datetime
import os
import socket
import sys
import pathlib

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = pathlib.Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

E, K_TOP, D, I, T, LAYERS = 8, 2, 128, 64, 12, 2


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def make_problem():
    from oracle import cpu
    rng = np.random.default_rng(7)
    x = torch.from_numpy(rng.standard_normal((T, D)).astype(np.float32)).to(torch.bfloat16)
    layers = []
    for _ in range(LAYERS):
        wr = (rng.standard_normal((E, D)) * 0.05).astype(np.float32)
        gu = cpu.quantize((rng.standard_normal((E * 2 * I, D)) * 0.05).astype(np.float32), 64, 4)
        dn = cpu.quantize((rng.standard_normal((E * D, I)) * 0.05).astype(np.float32), 64, 8)
        layers.append((wr, gu, dn))
    return x, layers


def oracle_compute(layers, e_lo, e_hi):
    """The per-rank work on the oracle: routing on local rows; expert math for experts [e_lo, e_hi) only."""
    from oracle import cpu
    from strixite_b200.ep import Compute

    def bits(t):
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)

    def route(l, x_loc):
        logits = (x_loc.to(torch.float32) @ torch.from_numpy(layers[l][0]).t()).numpy()
        ids, coef = cpu.moe_router(np.ascontiguousarray(logits), E, K_TOP)
        return torch.from_numpy(ids), torch.from_numpy(coef)

    def experts(l, x_all, ids, coef):
        _, gu, dn = layers[l]
        ids_np, coef_np = ids.numpy(), coef.numpy().copy()
        mine = (ids_np >= e_lo) & (ids_np < e_hi)
        local_ids = np.where(mine, ids_np - e_lo, 0).astype(np.int32)  # other ranks' slots: any valid expert, weight 0
        coef_np[~mine] = 0.0
        n = e_hi - e_lo
        gu_l, dn_l = gu.rows(e_lo * 2 * I, e_hi * 2 * I), dn.rows(e_lo * D, e_hi * D)
        h = cpu.experts_gather(bits(x_all), gu_l, n, local_ids, swiglu_mode=1, threads=1)
        y = cpu.experts_combine(h, dn_l, n, local_ids, coef_np, out_act=cpu.F32, threads=1)
        return torch.from_numpy(y)

    return Compute(route, experts)


def chunked(compute):
    """The same stand-in with the chunk argument of micro-batched runs (it needs no per-chunk buffers)."""
    from strixite_b200.ep import Compute
    return Compute(lambda l, x, c: compute.route(l, x), lambda l, xa, i, cf, c: compute.experts(l, xa, i, cf), chunked=True)


def worker(rank, world, port, out_dir, die, micro=1, exchange="reduce_scatter"):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    from strixite_b200.ep import ExpertParallelMoe, shard_bounds
    x, layers = make_problem()
    e_lo, e_hi = shard_bounds(E, world, rank)
    comp = oracle_compute(layers, e_lo, e_hi)
    ep = ExpertParallelMoe(chunked(comp) if micro > 1 else comp, LAYERS, T, D, K_TOP, "cpu", micro=micro, exchange=exchange)
    assert ep.micro == micro
    if die and rank == 1:
        os._exit(0)  # this rank never joins the first collective
    try:
        out = ep.forward(x[ep.t_lo:ep.t_hi])
        torch.save(out, os.path.join(out_dir, f"out{rank}.pt"))
    except Exception as e:  # the surviving rank must see an error, not hang
        with open(os.path.join(out_dir, f"err{rank}.txt"), "w") as f:
            f.write(f"{type(e).__name__}: {e}")
    finally:
        if not die:
            dist.destroy_process_group()


def single_rank_reference():
    from strixite_b200.ep import ExpertParallelMoe
    x, layers = make_problem()
    ep = ExpertParallelMoe(oracle_compute(layers, 0, E), LAYERS, T, D, K_TOP, "cpu")
    assert ep.world == 1
    return ep.forward(x)


def test_shard_bounds():
    from strixite_b200.ep import shard_bounds
    assert [shard_bounds(512, 8, r) for r in (0, 3, 7)] == [(0, 64), (192, 256), (448, 512)]
    assert shard_bounds(16384, 1, 0) == (0, 16384)
    with pytest.raises(ValueError):
        shard_bounds(10, 4, 0)


def test_two_ranks_equal_one_rank(tmp_path, oracle):
    want = single_rank_reference()
    mp.spawn(worker, args=(2, free_port(), str(tmp_path), False), nprocs=2, join=True)
    got = torch.cat([torch.load(tmp_path / f"out{r}.pt") for r in range(2)])
    # same slots, same per-slot values; only the order of the FP32 sum across ranks differs
    assert got.shape == want.shape
    assert torch.allclose(got.float(), want.float(), rtol=0, atol=2.0 ** -7 * float(want.float().abs().max()))
    assert (got != want).float().mean() < 0.02


def test_two_ranks_with_micro_batches_equal_one_rank(tmp_path, oracle):
    """Each rank's 6 rows as 2 and as 3 chunks: the chunks' stacks are independent, the result is the same rows."""
    want = single_rank_reference()
    for micro in (2, 3):
        out = tmp_path / f"m{micro}"
        out.mkdir()
        mp.spawn(worker, args=(2, free_port(), str(out), False, micro), nprocs=2, join=True)
        got = torch.cat([torch.load(out / f"out{r}.pt") for r in range(2)])
        assert got.shape == want.shape
        assert torch.allclose(got.float(), want.float(), rtol=0, atol=2.0 ** -7 * float(want.float().abs().max()))
        assert (got != want).float().mean() < 0.02


def test_two_ranks_all_to_all_exchange_equals_one_rank(tmp_path, oracle):
    """The partial rows returned by all-to-all + local sum instead of the reduce-scatter."""
    want = single_rank_reference()
    mp.spawn(worker, args=(2, free_port(), str(tmp_path), False, 1, "a2a"), nprocs=2, join=True)
    got = torch.cat([torch.load(tmp_path / f"out{r}.pt") for r in range(2)])
    assert torch.allclose(got.float(), want.float(), rtol=0, atol=2.0 ** -7 * float(want.float().abs().max()))
    assert (got != want).float().mean() < 0.02


def test_a_rank_that_never_joins_is_an_error_not_a_hang(tmp_path, oracle):
    """Failure made on the host: rank 1 exits before the layer's first collective; rank 0's collective ends with an
    error inside the process group's timeout."""
    ctx = mp.spawn(worker, args=(2, free_port(), str(tmp_path), True), nprocs=2, join=False)
    import time
    deadline = time.time() + 90
    while any(p.is_alive() for p in ctx.processes) and time.time() < deadline:
        time.sleep(0.5)
    for p in ctx.processes:
        if p.is_alive():
            p.terminate()
            pytest.fail("rank 0 is still waiting for the dead rank")
    assert (tmp_path / "err0.txt").exists() and not (tmp_path / "out0.pt").exists()
