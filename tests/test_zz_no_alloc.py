"""The allocation-free combine (sxb_linear_q4_experts_combine_grouped_noalloc) against the caller-scratch entry point.

Some hosts cannot give the library scratch memory: their device memory was handed out in full when the engine started,
and a decode loop cannot call cudaMalloc without stalling its own stream.  For them the per-slot dots of the grouped
combine live in a fixed 16 MiB array inside the library.  This file is collected last on purpose: if it fails, a run that
stops at the first failure has already run everything else.  It calls the new entry point through the C ABI twice in
a row - different shapes, the second smaller than the first so stale contents of the shared array would show - and
expects outputs identical to the existing entry point's, which is fed a scratch buffer of its own."""
import ctypes as C

import numpy as np
import pytest
import torch

from helpers import bf16_tensor, random_weights, upload

pytestmark = pytest.mark.gpu


def run_both(lib, oracle, dev, M, A, E, I, d, seed, shared, math=None, out_dtype=torch.float32, measure_memory=False):
    from strixite_b200 import _lib, kernels as K
    rng = np.random.default_rng(seed)
    dn = upload(oracle.quantize(random_weights(rng, E * d, I), 128 if I % 128 == 0 else 64, 4), dev)
    h = bf16_tensor(oracle.f32_to_bf16(rng.standard_normal((M * A, I)).astype(np.float32)), dev)
    ids = torch.from_numpy(np.stack([rng.permutation(E)[:A] for _ in range(M)]).astype(np.int32)).to(dev)
    coef = torch.from_numpy(rng.random((M, A)).astype(np.float32)).to(dev)
    nbytes = K.moe_route_workspace_bytes(M, A, E)
    ws = torch.empty(nbytes // 4, dtype=torch.int32, device=dev)
    err = torch.zeros(4, dtype=torch.int32, device=dev)
    K.moe_group_routes(ids, M, A, E, ws, nbytes, err)
    sh = None
    if shared:
        s = torch.from_numpy(rng.standard_normal((M, d)).astype(np.float32)).to(dev)
        gate = torch.from_numpy(rng.standard_normal(M).astype(np.float32)).to(dev)
        sh = K.MoeSharedAdd(s, gate, 1, E, err)
    stream = torch.cuda.current_stream().cuda_stream
    math = K.MoeMath.F32 if math is None else math
    out_act = K.Act.F32 if out_dtype == torch.float32 else K.Act.BF16
    if shared and out_dtype != torch.float32:
        sh.s = sh.s.to(torch.bfloat16)
    # existing entry point, caller-owned scratch
    partial = torch.empty((M * A, d), dtype=torch.float32, device=dev)
    want = torch.empty((M, d), dtype=out_dtype, device=dev)
    K.linear_qw_experts_combine_grouped(h, dn, E, ids, coef, ws, nbytes, partial, M, A, want, K.Act.BF16, math,
                                        shared=sh, out_act=out_act)
    # new entry point, straight through the C ABI: no scratch argument
    got = torch.full((M, d), float("nan"), dtype=torch.float32, device=dev).to(out_dtype)
    view = dn.c()
    shc = sh.c() if sh is not None else None
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    rc = lib.sxb_linear_q4_experts_combine_grouped_noalloc(
        h.data_ptr(), C.byref(view), E, ids.data_ptr(), coef.data_ptr(), ws.data_ptr(), nbytes, M, A, got.data_ptr(),
        int(K.Act.BF16), int(out_act), int(math), stream, C.byref(shc) if shc is not None else None, 0)
    assert rc == 0, lib.sxb_last_error().decode()
    torch.cuda.synchronize()
    if measure_memory:  # a call after the first takes no device memory: the free byte count of the device does not move
        assert torch.cuda.mem_get_info()[0] == free_before
    assert int(err[0]) == 0
    K.check_grouped_status(ws, "noalloc combine")
    return got, want


def test_noalloc_combine_matches_twice_in_a_row(cuda, oracle, lib):
    # the same kernels run on both sides, so the outputs are equal bit for bit (the tolerance of the combine's own
    # tests, 3e-5 of the output RMS, is the fallback bar should a future kernel reorder its sums)
    got1, want1 = run_both(lib, oracle, cuda, M=48, A=6, E=16, I=256, d=512, seed=1, shared=True)
    got2, want2 = run_both(lib, oracle, cuda, M=9, A=4, E=16, I=128, d=256, seed=2, shared=False, measure_memory=True)
    for got, want in ((got1, want1), (got2, want2)):
        assert torch.isfinite(got).all()
        rms = float(want.double().pow(2).mean().sqrt())
        assert float((got - want).abs().max()) <= 3e-5 * rms
        assert torch.equal(got, want)


def test_noalloc_combine_other_forms(cuda, oracle, lib):
    """The tcgen05 form of the down projection (BF16 per-slot dots in the built-in array) and a BF16 output, at small
    shapes, each against the caller-scratch entry point; the second call of each also checks that no memory was taken."""
    from strixite_b200 import kernels as K
    for kw in (dict(math=K.MoeMath.WmmaF16), dict(math=K.MoeMath.WmmaF16F32Partials), dict(out_dtype=torch.bfloat16)):
        for seed in (3, 4):
            got, want = run_both(lib, oracle, cuda, M=40, A=4, E=8, I=128, d=256, seed=seed, shared=True, measure_memory=seed == 4,
                                 **kw)
            assert torch.isfinite(got.float()).all()
            assert torch.equal(got, want)


def test_noalloc_combine_refuses_oversize(cuda, lib):
    from strixite_b200 import _lib
    view = _lib.SxbQView(4096, 8192, 12288, 512 * 4096, 1024, 128)
    # 2048 tokens x 10 slots x 4096 columns = 80 Mi floats: far beyond the 4 Mi built in
    rc = lib.sxb_linear_q4_experts_combine_grouped_noalloc(1 << 20, C.byref(view), 512, 1 << 21, 1 << 22, 1 << 23, 1 << 20,
                                                           2048, 10, 1 << 24, 1, 1, 0, None, None, 0)
    assert rc == 1
    msg = lib.sxb_last_error().decode()
    assert "exceed the built-in scratch" in msg and "caller-owned scratch" in msg
