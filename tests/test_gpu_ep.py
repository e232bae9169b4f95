"""The library's expert-parallel entry point (sxb_moe_layer_ep) on GPUs: as a single rank in this process (the whole
exchange machinery - NCCL communicator, gathers, the rows' way back - with one participant), and as N processes on N
GPUs where the machine has them."""
import pathlib
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = pathlib.Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("T,tc", [(96, True), (8, False)])
def test_one_rank_equals_the_plain_layer(cuda, T, tc):
    from dataclasses import replace
    from strixite_b200 import kernels as K, workloads as W
    from strixite_b200.kernels import MoeMath
    from strixite_b200.layer import MoeBuffers, MoeLayer
    cfg = replace(W.C0, T=T, shared=False, name=f"c0_t{T}")
    math = MoeMath.WmmaF16F32Partials if tc else MoeMath.F32
    x = W.activations(cfg, 2, cuda)
    logits = W.router_logits(x, W.router_weight(cfg, 2, cuda), W.expert_bias(cfg, 2, cuda))
    w = W.make_layer_weights(cfg, 2, cuda)
    layer = MoeLayer(w, cfg.E, cfg.k, MoeBuffers(T, cfg.d, cfg.I, cfg.E, cfg.k, cuda, False))
    want = torch.empty((T, cfg.d), dtype=torch.float32, device=cuda)
    layer.forward(x, logits, want, math=math)
    buf = MoeBuffers(T, cfg.d, cfg.I, cfg.E, cfg.k, cuda, False)
    xs = torch.empty((T * cfg.k, cfg.d), dtype=torch.float16, device=cuda)
    for rp in (0, 1, 2):
        ctx = K.EpContext(K.ep_unique_id(), 1, 0, T, cfg.d, cfg.k, rp)
        for dt in (torch.float32, torch.bfloat16):
            y = torch.empty((T, cfg.d), dtype=dt, device=cuda)
            ctx.set_timing(True)
            ctx.layer(x, logits, y, w.gate_up, w.down, cfg.E, cfg.E, 0, cfg.k, buf.ids, buf.coef, buf.ws, buf.ws_bytes, buf.h,
                      buf.partial, buf.router_err, buf.expert_err, xs=xs, math=math)
            torch.cuda.synchronize()
            K.check_router_error(buf.router_err, cfg.name)
            K.check_expert_error(buf.expert_err, cfg.name)
            assert torch.equal(buf.ids, layer.buf.ids)
            piece = want if rp != 2 else want.to(torch.float16).float()  # one rank: its piece is the whole sum, sent as F16
            assert torch.equal(y, piece.to(dt)), f"return path {rp}, {dt}"
            tm = ctx.timing()
            assert tm["layers"] >= 1 and tm["experts"] > 0
        ctx.close()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_ranks_on_separate_gpus():
    n = min(4, torch.cuda.device_count())
    n = 2 if n == 3 else n
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
                          "--master-port", "29631", str(ROOT / "tests" / "ep_ranks.py")], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
