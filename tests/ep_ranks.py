"""Worker of tests/test_gpu_ep.py: one rank of an expert-parallel run (launched by torch.distributed.run, one process per
GPU).  Every rank holds its slice of the experts of a small layer; the rows come back through each way the library
offers (NCCL reduce-scatter, peer stores of FP32 pieces, of BF16 pieces) and through the torch.distributed driver; rank 0
also holds ALL experts and compares every result with the unsharded layer."""
import os
import pathlib
import sys

import torch
import torch.distributed as dist

ROOT = pathlib.Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def main():
    from dataclasses import replace
    from strixite_b200 import kernels as K, workloads as W
    from strixite_b200.ep import shard_bounds
    from strixite_b200.kernels import MoeMath
    from strixite_b200.layer import MoeBuffers, MoeLayer

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    failures = []
    for T, math in ((96 * world, MoeMath.WmmaF16F32Partials), (8 * world, MoeMath.F32)):
        cfg = replace(W.C0, T=T, shared=False, name=f"c0_t{T}")
        x = W.activations(cfg, 1, dev)
        logits = W.router_logits(x, W.router_weight(cfg, 1, dev), W.expert_bias(cfg, 1, dev))
        e_lo, e_hi = shard_bounds(cfg.E, world, rank)
        t_lo, t_hi = shard_bounds(T, world, rank)
        w = W.make_layer_weights(cfg, 1, dev, e_lo=e_lo, e_hi=e_hi)
        buf = MoeBuffers(T, cfg.d, cfg.I, e_hi - e_lo, cfg.k, dev, False)
        xs = torch.empty((T * cfg.k, cfg.d), dtype=torch.float16, device=dev)
        want = None
        if rank == 0:
            full = MoeLayer(W.make_layer_weights(cfg, 1, dev), cfg.E, cfg.k, MoeBuffers(T, cfg.d, cfg.I, cfg.E, cfg.k, dev, False))
            want = torch.empty((T, cfg.d), dtype=torch.float32, device=dev)
            full.forward(x, logits, want, math=math)
            torch.cuda.synchronize()
            full.check_errors(cfg.name)
        x_loc, lg_loc = x[t_lo:t_hi].contiguous(), logits[t_lo:t_hi].contiguous()
        for rp in (0, 1, 2):
            box = [K.ep_unique_id() if rank == 0 else None]
            dist.broadcast_object_list(box, src=0)
            ctx = K.EpContext(box[0], world, rank, T, cfg.d, cfg.k, rp)
            y = torch.full((t_hi - t_lo, cfg.d), float("nan"), dtype=torch.float32, device=dev)
            for _ in range(2):  # twice: the receive buffers are reused
                ctx.layer(x_loc, lg_loc, y, w.gate_up, w.down, e_hi - e_lo, cfg.E, e_lo, cfg.k, buf.ids, buf.coef, buf.ws, buf.ws_bytes,
                          buf.h, buf.partial, buf.router_err, buf.expert_err, xs=xs, math=math)
            torch.cuda.synchronize()
            K.check_router_error(buf.router_err, cfg.name)
            K.check_expert_error(buf.expert_err, cfg.name)
            K.check_grouped_status(buf.ws, cfg.name)
            rows = [torch.empty_like(y) for _ in range(world)] if rank == 0 else None
            dist.gather(y, rows, dst=0)
            if rank == 0:
                got = torch.cat(rows)
                scale = want.abs().max().item()
                tol = (2e-5 if rp != 2 else 2.0 ** -10) * scale  # FP32 summation order; or one F16 rounding per piece
                err = (got - want).abs().max().item()
                if not (err <= tol):
                    failures.append(f"{cfg.name} return path {rp}: max |y - unsharded| = {err:.3e} > {tol:.3e}")
            ctx.close()
    ok = torch.tensor([0 if failures else 1], device=dev)
    dist.broadcast(ok, src=0)
    if rank == 0:
        print("\n".join(failures) if failures else f"ep ok on {world} ranks")
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if int(ok.item()) == 1 else 1)


if __name__ == "__main__":
    main()
