"""The steps either side of the expert kernels, and the boundary's remaining forms, on the GPU against the CPU oracle:
the router-logits projection (streaming and tcgen05), router + pack as one launch, the residual add, the dense tcgen05
projections (linear_q*_wmma), FP32 activations, and a C++ host that issues the reference's call block through the shim."""
import subprocess

import numpy as np
import pytest
import torch

from helpers import bf16_tensor, bits_of, max_abs_over_rms, random_weights, upload

pytestmark = pytest.mark.gpu


def logits_f64(oracle, x_bits, w, bias):
    return oracle.bf16_to_f32(x_bits).astype(np.float64) @ w.astype(np.float64).T + bias.astype(np.float64)


@pytest.mark.parametrize("M,N,K,w_bf16", [(16, 513, 4096, False), (1, 65, 1024, True), (37, 513, 4096, True), (64, 129, 512, False)])
def test_router_logits_streaming(cuda, oracle, M, N, K, w_bf16):
    """logits = x W^T + bias against a float64 evaluation: within 1e-5 of the largest logit (FP32 sums of exact products)."""
    from strixite_b200 import kernels as Kn
    rng = np.random.default_rng(M * 1000 + N)
    xb = oracle.f32_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    bias = (rng.standard_normal(N) * 0.5).astype(np.float32)
    if w_bf16:
        wb = oracle.f32_to_bf16(w)
        w = oracle.bf16_to_f32(wb)
        w_dev = bf16_tensor(wb, cuda)
    else:
        w_dev = torch.from_numpy(w).to(cuda)
    x = bf16_tensor(xb, cuda)
    ld = N + 3
    out = torch.full((M, ld), float("nan"), dtype=torch.float32, device=cuda)
    Kn.router_logits(x, w_dev, torch.from_numpy(bias).to(cuda), out)
    want = logits_f64(oracle, xb, w, bias)
    got = out.cpu().numpy()
    assert np.all(np.isnan(got[:, N:])), "columns past N must stay untouched"
    assert np.max(np.abs(got[:, :N] - want)) <= 1e-5 * np.max(np.abs(want))
    if w_bf16:  # the reference's launcher (kernels/linear.hpp:22-27): no bias, ld = N, F32 or BF16 out
        y32 = torch.empty((M, N), dtype=torch.float32, device=cuda)
        ybf = torch.empty((M, N), dtype=torch.bfloat16, device=cuda)
        Kn.linear_bf16w(x, w_dev, y32, M, N, K, Kn.Act.BF16, Kn.Act.F32)
        Kn.linear_bf16w(x, w_dev, ybf, M, N, K, Kn.Act.BF16)
        plain = logits_f64(oracle, xb, w, np.zeros(N, np.float32))
        assert np.max(np.abs(y32.cpu().numpy() - plain)) <= 1e-5 * np.max(np.abs(plain))
        assert torch.equal(ybf, y32.to(torch.bfloat16))


@pytest.mark.parametrize("M,N,K,planes,w_bf16", [(4096, 513, 4096, 3, False), (300, 513, 1024, 2, False), (1000, 129, 512, 1, True),
                                                   (128, 64, 256, 3, False)])
def test_router_logits_tcgen05(cuda, oracle, M, N, K, planes, w_bf16):
    """The tensor-core projection: three planes reproduce the FP32 weight exactly, two planes keep 16 bits of it, one plane
    is a BF16 weight.  What is left is the tensor cores' FP32 accumulation, which is not IEEE summation (the reference says
    the same of its matrix units, kernels/wmma.hpp:10-11): measured 1.3e-5 of the largest logit over K = 4096 x 3 planes,
    held to 3e-5 here (the streaming form, plain FP32 FMAs, is held to 1e-5)."""
    from strixite_b200 import kernels as Kn
    rng = np.random.default_rng(M + N + planes)
    xb = oracle.f32_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    bias = (rng.standard_normal(N) * 0.5).astype(np.float32)
    x = bf16_tensor(xb, cuda)
    if w_bf16:
        wb = oracle.f32_to_bf16(w)
        w = oracle.bf16_to_f32(wb)
        w_dev = bf16_tensor(wb, cuda)
    else:
        w_dev = torch.from_numpy(w).to(cuda)
    rp = Kn.router_prepare(w_dev, planes)
    out = torch.full((M, N + 1), float("nan"), dtype=torch.float32, device=cuda)
    Kn.router_logits_wmma(x, rp, torch.from_numpy(bias).to(cuda), out)
    torch.cuda.synchronize()
    Kn.check_dense_status("router_logits_wmma")
    want = logits_f64(oracle, xb, w, bias)
    got = out.cpu().numpy()
    assert np.all(np.isnan(got[:, N:]))
    tol = 3e-5 if planes != 2 else 6e-5
    assert np.max(np.abs(got[:, :N] - want)) <= tol * np.max(np.abs(want)), np.max(np.abs(got[:, :N] - want)) / np.max(np.abs(want))
    if w_bf16 and planes == 1:  # the unprepared BF16 weight as its own plane
        out2 = torch.empty((M, N), dtype=torch.float32, device=cuda)
        Kn.router_logits_wmma(x, Kn.RouterPlanes(w_dev.view(torch.int16), 1, N, K), None, out2)
        plain = logits_f64(oracle, xb, w, np.zeros(N, np.float32))
        assert np.max(np.abs(out2.cpu().numpy() - plain)) <= 1e-5 * np.max(np.abs(plain))


@pytest.mark.parametrize("M,E,k,shards", [(16, 512, 10, 1), (64, 512, 10, 1), (7, 64, 4, 1), (200, 1000, 10, 1), (16, 512, 10, 4)])
def test_route_small_equals_router_then_pack(cuda, M, E, k, shards):
    """sxb_moe_route_small writes the same ids, coef and workspace, word for word, as moe_router + moe_group_routes[_ep]."""
    from strixite_b200 import kernels as Kn
    g = torch.Generator(device="cpu").manual_seed(M * 31 + E)
    logits = torch.randn((M, E + 1), generator=g).to(cuda)
    logits[0, :4] = 0.5  # ties
    E_local = E // shards
    e_lo = E_local * (shards - 1)
    nbytes = Kn.moe_route_workspace_bytes(M, k, E_local)
    outs = []
    for fused in (False, True):
        ids = torch.full((M, k), -7, dtype=torch.int32, device=cuda)
        coef = torch.zeros((M, k), dtype=torch.float32, device=cuda)
        ws = torch.zeros(nbytes // 4, dtype=torch.int32, device=cuda)
        e1, e2 = torch.zeros(4, dtype=torch.int32, device=cuda), torch.zeros(4, dtype=torch.int32, device=cuda)
        if fused:
            Kn.moe_route_small(logits, E + 1, M, E, k, e_lo if shards > 1 else 0, E_local, ids, coef, ws, nbytes, e1, e2)
        else:
            Kn.moe_router(logits, E + 1, M, E, k, None, 1, 0, ids, coef, Kn.Act.F32, e1)
            if shards > 1:
                Kn.moe_group_routes_ep(ids, M, k, E, e_lo, E_local, ws, nbytes, e2)
            else:
                Kn.moe_group_routes(ids, M, k, E, ws, nbytes, e2)
        torch.cuda.synchronize()
        outs.append((ids.cpu(), coef.cpu(), ws.cpu(), e1.cpu(), e2.cpu()))
    for a, b in zip(*outs):
        assert torch.equal(a, b)


def test_route_small_reports_a_bad_logit(cuda):
    from strixite_b200 import kernels as Kn
    logits = torch.zeros((4, 65), device=cuda)
    logits[2, 9] = float("inf")
    ids = torch.zeros((4, 4), dtype=torch.int32, device=cuda)
    coef = torch.zeros((4, 4), device=cuda)
    nbytes = Kn.moe_route_workspace_bytes(4, 4, 64)
    ws = torch.zeros(nbytes // 4, dtype=torch.int32, device=cuda)
    e1, e2 = torch.zeros(4, dtype=torch.int32, device=cuda), torch.zeros(4, dtype=torch.int32, device=cuda)
    Kn.moe_route_small(logits, 65, 4, 64, 4, 0, 64, ids, coef, ws, nbytes, e1, e2)
    torch.cuda.synchronize()
    assert e1.tolist()[:3] == [1, 2, 9] and ids[2].tolist() == [-1] * 4
    assert e2.tolist()[0] == 1  # the pack sees the token's ids of -1 as out of range


@pytest.mark.parametrize("ydt", [torch.float32, torch.bfloat16])
def test_residual_add(cuda, ydt):
    from strixite_b200 import kernels as Kn
    g = torch.Generator(device="cpu").manual_seed(3)
    x = torch.randn((33, 1024), generator=g).to(torch.bfloat16).to(cuda)
    y = torch.randn((33, 1024), generator=g).to(ydt).to(cuda)
    out = torch.empty_like(x)
    Kn.residual_add(x, y, out)
    assert torch.equal(out, (x.float() + y.float()).to(torch.bfloat16))
    Kn.residual_add(x, y, x)  # in place
    assert torch.equal(x, out)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_hc_inject(cuda, oracle, dt):
    """kernels/hc.hpp:52-54 against the oracle's injection (the one inside moe_shared_add_inject, with s = 0 and a gate that
    does not matter), bit for bit."""
    from strixite_b200 import kernels as Kn
    rng = np.random.default_rng(9)
    T, d, H = 7, 320, 4
    y = rng.standard_normal((T, d)).astype(np.float32)
    x = rng.standard_normal((T, H * d)).astype(np.float32)
    w_in = (rng.random((T, H)) * 2).astype(np.float32)
    if dt == torch.bfloat16:
        yb, xb = oracle.f32_to_bf16(y), oracle.f32_to_bf16(x)
        _, want = oracle.moe_shared_add_inject(yb, np.zeros_like(yb), np.zeros(T, np.float32), 0, xb, w_in)
        xd, yd = bf16_tensor(xb, cuda), bf16_tensor(yb, cuda)
    else:
        _, want = oracle.moe_shared_add_inject(y, np.zeros_like(y), np.zeros(T, np.float32), 0, x, w_in)
        xd, yd = torch.from_numpy(x).to(cuda), torch.from_numpy(y).to(cuda)
    Kn.hc_inject(xd, torch.from_numpy(w_in).to(cuda), yd, T, H, d, Kn.Act.F32 if dt == torch.float32 else Kn.Act.BF16)
    got = xd.cpu().numpy() if dt == torch.float32 else bits_of(xd)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("bits,G,M,N,K", [(8, 64, 300, 2048, 1024), (4, 128, 129, 512, 2048), (8, 64, 5, 256, 256)])
def test_dense_tcgen05_projections(cuda, oracle, bits, G, M, N, K):
    """linear_q*_wmma: y = x W^T with the matrix-unit numerics, against oracle.linear_q(w_f16); then the fused SwiGLU form
    feeding a down projection in the tile-blocked layout (the prefill shared expert's launch sequence)."""
    from strixite_b200 import kernels as Kn
    rng = np.random.default_rng(bits * 100 + M)
    wq = oracle.quantize(random_weights(rng, N, K), G, bits)
    xb = oracle.f32_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
    w, x = upload(wq, cuda), bf16_tensor(xb, cuda)
    want = oracle.linear_q(xb, wq, out_act=oracle.F32, w_f16=True)
    y32 = torch.empty((M, N), dtype=torch.float32, device=cuda)
    ybf = torch.empty((M, N), dtype=torch.bfloat16, device=cuda)
    Kn.linear_qw_wmma(x, w, y32, M, Kn.Act.BF16, Kn.Act.F32)
    Kn.linear_qw_wmma(x, w, ybf, M, Kn.Act.BF16, Kn.Act.BF16)
    torch.cuda.synchronize()
    Kn.check_dense_status("linear_wmma")
    assert max_abs_over_rms(y32.cpu().numpy(), want) <= 2e-5
    assert torch.equal(ybf, y32.to(torch.bfloat16))
    # staged input gives the same bits
    xs = torch.empty((M, K), dtype=torch.float16, device=cuda)
    Kn.stage_f16_tiles(x, None, 0, M, 1, 1, K, bits, xs)
    y2 = torch.empty_like(y32)
    Kn.linear_qw_wmma(xs, w, y2, M, Kn.Act.F16_TILED, Kn.Act.F32)
    assert torch.equal(y2, y32)
    # [gate | up] -> h (tile-blocked) -> down
    I = N // 2
    dq = oracle.quantize(random_weights(rng, 256, I), 64, 8)
    dn = upload(dq, cuda)
    h = torch.empty((M, I), dtype=torch.bfloat16, device=cuda)
    Kn.linear_qw_wmma_swiglu(xs, w, h, M, Kn.Act.F16_TILED, h_f16=4)
    s32 = torch.empty((M, 256), dtype=torch.float32, device=cuda)
    Kn.linear_qw_wmma(h, dn, s32, M, Kn.Act.F16_TILED, Kn.Act.F32)
    torch.cuda.synchronize()
    Kn.check_dense_status("linear_wmma_swiglu")
    zero = np.zeros((M, 1), dtype=np.int32)
    hs = oracle.experts_gather(xb, wq, 1, zero, swiglu_mode=2, w_f16=True)[:, 0]
    want_s = oracle.linear_q(hs, dq, out_act=oracle.F32, w_f16=True)
    assert max_abs_over_rms(s32.cpu().numpy(), want_s) <= 1e-2


@pytest.mark.parametrize("bits,G,M,N,K", [(8, 64, 300, 400, 256), (4, 128, 300, 400, 2048), (4, 32, 193, 144, 2048)])
def test_dense_tcgen05_partial_row_blocks(cuda, oracle, bits, G, M, N, K):
    """Tile-blocked activations into a weight whose row count is not a multiple of the 128-row work item, with token counts
    that leave a partly filled last tile - on both shapes of the kernel for tile-blocked activations (K below and from 2048).
    A store for a row past N would land in the next token's output row, so the comparison sees it."""
    from strixite_b200 import kernels as Kn
    rng = np.random.default_rng(bits + M + N)
    wq = oracle.quantize(random_weights(rng, N, K), G, bits)
    xb = oracle.f32_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
    w, x = upload(wq, cuda), bf16_tensor(xb, cuda)
    xs = torch.empty((M, K), dtype=torch.float16, device=cuda)
    Kn.stage_f16_tiles(x, None, 0, M, 1, 1, K, bits, xs)
    y32 = torch.full((M + 1, N), 7.0, dtype=torch.float32, device=cuda)
    ybf = torch.empty((M, N), dtype=torch.bfloat16, device=cuda)
    Kn.linear_qw_wmma(xs, w, y32, M, Kn.Act.F16_TILED, Kn.Act.F32)
    Kn.linear_qw_wmma(xs, w, ybf, M, Kn.Act.F16_TILED, Kn.Act.BF16)
    torch.cuda.synchronize()
    Kn.check_dense_status("partial row blocks")
    want = oracle.linear_q(xb, wq, out_act=oracle.F32, w_f16=True)
    assert max_abs_over_rms(y32[:M].cpu().numpy(), want) <= 2e-5
    assert torch.all(y32[M] == 7.0)  # nothing past the last token's row
    assert torch.equal(ybf, y32[:M].to(torch.bfloat16))


@pytest.mark.parametrize("bits,G", [(4, 128), (8, 64)])
def test_fp32_activations(cuda, oracle, bits, G):
    """Act::F32 into the dense, per-slot and grouped entry points (kernels/linear_q4.hpp:26-30): FP32 in, FP32 out,
    against the oracle's FP32 mode."""
    from strixite_b200 import kernels as Kn
    rng = np.random.default_rng(bits)
    E, N, K, M, A = 6, 64, 256, 9, 3
    wq = oracle.quantize(random_weights(rng, E * N, K), G, bits)
    w = upload(wq, cuda)
    xf = rng.standard_normal((M, K)).astype(np.float32)
    x = torch.from_numpy(xf).to(cuda)
    ids_np = np.stack([rng.permutation(E)[:A] for _ in range(M)]).astype(np.int32)
    ids = torch.from_numpy(ids_np).to(cuda)
    err = torch.zeros(4, dtype=torch.int32, device=cuda)
    tol = 2e-5
    # dense: the stacked matrix as one [E*N, K] weight
    y = torch.empty((M, E * N), dtype=torch.float32, device=cuda)
    Kn.linear_qw(x, w, y, M, Kn.Act.F32)
    assert max_abs_over_rms(y.cpu().numpy(), oracle.linear_q(xf, wq)) <= tol
    # per-slot gather, SwiGLU gather, combine
    g = torch.empty((M, A, N), dtype=torch.float32, device=cuda)
    Kn.linear_qw_experts_gather(x, w, E, ids, M, A, g, Kn.Act.F32, err)
    assert max_abs_over_rms(g.cpu().numpy(), oracle.experts_gather(xf, wq, E, ids_np)) <= tol
    hh = torch.empty((M, A, N // 2), dtype=torch.float32, device=cuda)
    Kn.linear_qw_experts_gather_swiglu(x, w, E, ids, M, A, hh, Kn.Act.F32, err)
    assert max_abs_over_rms(hh.cpu().numpy(), oracle.experts_gather(xf, wq, E, ids_np, swiglu_mode=1)) <= tol
    dq = oracle.quantize(random_weights(rng, E * 32, N), 32, bits)
    dn = upload(dq, cuda)
    coef_np = rng.random((M, A)).astype(np.float32)
    coef = torch.from_numpy(coef_np).to(cuda)
    yc = torch.empty((M, 32), dtype=torch.float32, device=cuda)
    Kn.linear_qw_experts_combine(g, dn, E, ids, coef, M, A, yc, Kn.Act.F32, err)
    want_c = oracle.experts_combine(g.cpu().numpy(), dq, E, ids_np, coef_np)
    assert max_abs_over_rms(yc.cpu().numpy(), want_c) <= tol
    # grouped forms (any math: FP32 activations always take the plain path)
    nbytes = Kn.moe_route_workspace_bytes(M, A, E)
    ws = torch.empty(nbytes // 4, dtype=torch.int32, device=cuda)
    Kn.moe_group_routes(ids, M, A, E, ws, nbytes, err)
    hg = torch.empty_like(hh)
    Kn.linear_qw_experts_gather_grouped_swiglu(x, w, E, ws, nbytes, M, A, hg, Kn.Act.F32, Kn.MoeMath.WmmaF16)
    assert torch.equal(hg, hh)
    partial = torch.empty((M * A, 32), dtype=torch.float32, device=cuda)
    yg = torch.empty_like(yc)
    Kn.linear_qw_experts_combine_grouped(g, dn, E, ids, coef, ws, nbytes, partial, M, A, yg, Kn.Act.F32, Kn.MoeMath.F32)
    torch.cuda.synchronize()
    assert int(err[0]) == 0
    assert max_abs_over_rms(yg.cpu().numpy(), want_c) <= tol


def test_cxx_host_runs_the_call_block(cuda, oracle, tmp_path):
    """tests/cpp/call_block.cpp, linked against libstrix_b200.so, issues the reference's call block through the C++ shim;
    its ids, coef and y equal the Python launcher sequence's bit for bit."""
    from helpers_cpp import build_call_block
    from strixite_b200 import kernels as Kn
    exe = build_call_block(tmp_path)
    rng = np.random.default_rng(11)
    M, E, A, d, I, G = 12, 8, 2, 256, 128, 64
    xb = oracle.f32_to_bf16(rng.standard_normal((M, d)).astype(np.float32))
    logits = rng.standard_normal((M, E)).astype(np.float32)
    gu = oracle.quantize(random_weights(rng, E * 2 * I, d), G, 4)
    dn = oracle.quantize(random_weights(rng, E * d, I), G, 4)
    with open(tmp_path / "in.bin", "wb") as f:
        f.write(np.array([M, E, A, d, I, G, G], dtype=np.int64).tobytes())
        for a in (xb, logits, gu.q, gu.scale, gu.minv, dn.q, dn.scale, dn.minv):
            f.write(np.ascontiguousarray(a).tobytes())
    subprocess.run([str(exe), str(tmp_path / "in.bin"), str(tmp_path / "out.bin")], check=True, timeout=120)
    raw = (tmp_path / "out.bin").read_bytes()
    ids_c = np.frombuffer(raw[: M * A * 4], dtype=np.int32).reshape(M, A)
    coef_c = np.frombuffer(raw[M * A * 4: 2 * M * A * 4], dtype=np.float32).reshape(M, A)
    y_c = np.frombuffer(raw[2 * M * A * 4:], dtype=np.uint16).reshape(M, d)
    # the same launchers from Python
    x, lg = bf16_tensor(xb, cuda), torch.from_numpy(logits).to(cuda)
    wg, wd = upload(gu, cuda), upload(dn, cuda)
    ids = torch.empty((M, A), dtype=torch.int32, device=cuda)
    coef = torch.empty((M, A), dtype=torch.float32, device=cuda)
    err = torch.zeros(8, dtype=torch.int32, device=cuda)
    nbytes = Kn.moe_route_workspace_bytes(M, A, E)
    ws = torch.empty(nbytes // 4, dtype=torch.int32, device=cuda)
    h = torch.empty((M * A, I), dtype=torch.bfloat16, device=cuda)
    partial = torch.empty((M * A, d), dtype=torch.float32, device=cuda)
    y = torch.empty((M, d), dtype=torch.bfloat16, device=cuda)
    Kn.moe_router(lg, E, M, E, A, None, 1, 0, ids, coef, Kn.Act.F32, err)
    Kn.moe_group_routes(ids, M, A, E, ws, nbytes, err[4:])
    Kn.linear_qw_experts_gather_grouped_swiglu(x, wg, E, ws, nbytes, M, A, h, Kn.Act.BF16, Kn.MoeMath.F32)
    Kn.linear_qw_experts_combine_grouped(h, wd, E, ids, coef, ws, nbytes, partial, M, A, y, Kn.Act.BF16, Kn.MoeMath.F32)
    torch.cuda.synchronize()
    assert np.array_equal(ids_c, ids.cpu().numpy())
    assert np.array_equal(coef_c.view(np.uint32), coef.cpu().numpy().view(np.uint32))
    assert np.array_equal(y_c, bits_of(y))
    # and the oracle agrees with both
    ref = oracle.moe_layer(xb, np.concatenate([logits, np.zeros((M, 1), np.float32)], axis=1), oracle.LayerWeights(gu, dn), E, A)
    assert np.array_equal(ref["ids"], ids_c)


@pytest.mark.parametrize("tiled", [False, True])
def test_a_wait_that_runs_out_ends_the_kernel_with_a_status(cuda, oracle, lib, tiled):
    """The tcgen05 kernels (tiled: the one for tile-blocked activations) bound every device-side wait.  With the limit set to 2 ms and CTA 0 told to leave one fill of its
    weight-code ring out (nothing is issued for it, so nothing can fault), the producers' wait for those codes runs out:
    the kernel returns, the status words name the work item and the role, tensor memory is released - a normal launch on
    the same context right after gives the right answer."""
    from strixite_b200 import kernels as Kn
    rng = np.random.default_rng(5)
    M, N, K = 200, 512, 1024
    wq = oracle.quantize(random_weights(rng, N, K), 64, 8)
    xb = oracle.f32_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
    w, x = upload(wq, cuda), bf16_tensor(xb, cuda)
    y = torch.empty((M, N), dtype=torch.float32, device=cuda)
    act = Kn.Act.BF16
    if tiled:
        xs = torch.empty((M, K), dtype=torch.float16, device=cuda)
        Kn.stage_f16_tiles(x, None, 0, M, 1, 1, K, 8, xs)
        x, act = xs, Kn.Act.F16_TILED
    Kn.linear_qw_wmma(x, w, y, M, act, Kn.Act.F32)  # warm: module loaded, attributes set
    torch.cuda.synchronize()
    Kn.check_dense_status("warm-up")
    try:
        Kn.set_wait_limit(2_000_000)
        assert lib.sxb_test_skip_ring_slot(3) == 0
        Kn.linear_qw_wmma(x, w, y, M, act, Kn.Act.F32)
        torch.cuda.synchronize()
    finally:
        lib.sxb_test_skip_ring_slot(-1)
        Kn.set_wait_limit(2_000_000_000)
    # which role's limit fires first is a matter of microseconds (every role of the stalled CTA is waiting): any of them
    with pytest.raises(Kn.Error, match=r"a tcgen05 kernel gave up a wait at work item 0 \((a weight producer|an MMA warp|the epilogue|the activation copy|the weight-code copy)"):
        Kn.check_dense_status("skipped fill")
    Kn.check_dense_status("cleared by the read")  # the words are cleared by the failing check
    y2 = torch.empty_like(y)
    Kn.linear_qw_wmma(x, w, y2, M, act, Kn.Act.F32)
    torch.cuda.synchronize()
    Kn.check_dense_status("after")
    want = oracle.linear_q(xb, wq, out_act=oracle.F32, w_f16=True)
    assert max_abs_over_rms(y2.cpu().numpy(), want) <= 2e-5
