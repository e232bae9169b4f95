"""GPU parity of the quantizer, the dense linears, SwiGLU and the expert kernels (per-slot and grouped,
exact-product math) against the CPU oracle, through the C ABI.

Tolerances.  The kernels accumulate in FP32 in a different order than the oracle's float64 sums, so FP32 outputs
agree to ~1e-5 relative to the output scale; BF16 outputs are the rounding of almost-equal FP32 values and may
differ by one BF16 ulp where a value sits on a rounding boundary (a tiny fraction of the elements)."""
import numpy as np
import pytest
import torch

from helpers import bf16_tensor, bf16_ulps, bits_of, download, max_abs_over_rms, random_weights, upload

pytestmark = pytest.mark.gpu

FORMATS = [(4, 128), (4, 64), (4, 32), (8, 64), (8, 128), (8, 32)]


def assert_bf16_close(got_bits, ref_bits, oracle, what, frac_off=5e-2, ulps=1):
    """Both sides round nearly equal FP32 values to BF16: they agree except where the value sits on a rounding
    boundary (then one BF16 ulp apart), plus the FP32 summation-order noise (3e-5 of the output scale) that matters
    only for outputs near zero.  `ulps=2` is for the fused SwiGLU output, which is rounded three times (g and u as
    stored, silu(g) as stored, their product): one flipped rounding of g or u can move h by two ulps."""
    got, ref = oracle.bf16_to_f32(got_bits).astype(np.float64), oracle.bf16_to_f32(ref_bits).astype(np.float64)
    scale = np.sqrt(np.mean(ref ** 2))
    tol = np.abs(ref) * ulps * 2.0 ** -7 + 3e-5 * scale
    bad = np.abs(got - ref) > tol
    assert not bad.any(), f"{what}: {bad.sum()} elements beyond one BF16 ulp, worst {np.abs(got - ref).max():.3e}"
    frac = (got_bits != ref_bits).mean()
    assert frac <= frac_off, f"{what}: {frac:.2e} of the elements differ"


@pytest.mark.parametrize("bits,G", FORMATS)
def test_device_quantizer_bit_exact(cuda, oracle, golden, bits, G):
    from strixite_b200 import kernels as K
    tag = f"q{bits}g{G}"
    v = K.quantize(torch.from_numpy(golden[f"{tag}.w"]).to(cuda), G, bits)
    torch.cuda.synchronize()
    assert np.array_equal(v.q.cpu().numpy(), golden[f"{tag}.q"])
    assert np.array_equal(v.scale.cpu().numpy().view(np.uint16), golden[f"{tag}.scale"])
    assert np.array_equal(v.minv.cpu().numpy().view(np.uint16), golden[f"{tag}.minv"])
    w = random_weights(np.random.default_rng(G), 300, 1024)
    v = K.quantize(torch.from_numpy(w).to(cuda), G, bits)
    r = oracle.quantize(w, G, bits)
    assert np.array_equal(v.q.cpu().numpy(), r.q) and np.array_equal(v.scale.cpu().numpy().view(np.uint16), r.scale)
    assert np.array_equal(v.minv.cpu().numpy().view(np.uint16), r.minv)
    bad = torch.from_numpy(w).to(cuda)
    bad[7, 130] = float("nan")
    with pytest.raises(K.Error, match=r"non-finite weight at \[7, 13\d\]|non-finite weight at \[7, 128\]"):
        K.quantize(bad, G, bits)


@pytest.mark.parametrize("bits,G", FORMATS)
@pytest.mark.parametrize("M,N,Kd", [(1, 64, 256), (7, 200, 1024), (16, 2048, 4096), (19, 40, 128)])
def test_linear_dense(cuda, oracle, bits, G, M, N, Kd):
    from strixite_b200 import kernels as K
    rng = np.random.default_rng(bits * G + M)
    w = oracle.quantize(random_weights(rng, N, Kd), G, bits)
    x = oracle.f32_to_bf16(rng.standard_normal((M, Kd)).astype(np.float32))
    ref32 = oracle.linear_q(x, w, out_act=oracle.F32)
    refbf = oracle.linear_q(x, w)
    wd, xd = upload(w, cuda), bf16_tensor(x, cuda)
    y32 = torch.empty((M, N), dtype=torch.float32, device=cuda)
    ybf = torch.empty((M, N), dtype=torch.bfloat16, device=cuda)
    K.linear_qw(xd, wd, y32, M, K.Act.BF16, K.Act.F32)
    K.linear_qw(xd, wd, ybf, M, K.Act.BF16)
    torch.cuda.synchronize()
    assert max_abs_over_rms(y32.cpu().numpy(), ref32) < 2e-5
    assert_bf16_close(bits_of(ybf), refbf, oracle, "linear bf16")


@pytest.mark.parametrize("rows,I", [(1, 8), (5, 1000), (160, 1024), (3, 7)])
def test_swiglu(cuda, oracle, rows, I):
    from strixite_b200 import kernels as K
    rng = np.random.default_rng(rows)
    gu = (rng.standard_normal((rows, 2 * I)) * 2).astype(np.float32)
    gb = oracle.f32_to_bf16(gu)
    h = torch.empty((rows, I), dtype=torch.bfloat16, device=cuda)
    K.swiglu(bf16_tensor(gb, cuda), h, rows, I, K.Act.BF16)
    hf = torch.empty((rows, I), dtype=torch.float32, device=cuda)
    K.swiglu(torch.from_numpy(gu).to(cuda), hf, rows, I, K.Act.F32)
    torch.cuda.synchronize()
    assert_bf16_close(bits_of(h), oracle.swiglu(gb), oracle, "swiglu bf16", frac_off=5e-3)
    np.testing.assert_allclose(hf.cpu().numpy(), oracle.swiglu(gu), rtol=2e-6, atol=1e-7)


def make_experts(oracle, rng, E, N, Kd, G, bits):
    return oracle.quantize(random_weights(rng, E * N, Kd), G, bits)


@pytest.mark.parametrize("bits,G", [(4, 128), (8, 64), (4, 32)])
@pytest.mark.parametrize("M,A,E,N,Kd", [(1, 4, 8, 64, 256), (5, 3, 16, 48, 512), (16, 10, 64, 256, 1024)])
def test_per_slot_experts(cuda, oracle, bits, G, M, A, E, N, Kd):
    """linear_q*_experts_gather / _gather_swiglu / _combine (decode form), incl. an out-of-range id."""
    from strixite_b200 import kernels as K
    rng = np.random.default_rng(M * 100 + E)
    w = make_experts(oracle, rng, E, N, Kd, G, bits)
    wd = upload(w, cuda)
    x = oracle.f32_to_bf16(rng.standard_normal((M, Kd)).astype(np.float32))
    ids = np.stack([rng.permutation(E)[:A] for _ in range(M)]).astype(np.int32)
    if M > 1:
        ids[1, 0] = E + 2
    coef = rng.random((M, A)).astype(np.float32)
    idd, xd = torch.from_numpy(ids).to(cuda), bf16_tensor(x, cuda)
    err = torch.zeros(4, dtype=torch.int32, device=cuda)
    y = torch.empty((M, A, N), dtype=torch.bfloat16, device=cuda)
    K.linear_qw_experts_gather(xd, wd, E, idd, M, A, y, K.Act.BF16, err)
    h = torch.empty((M, A, N // 2), dtype=torch.bfloat16, device=cuda)
    K.linear_qw_experts_gather_swiglu(xd, wd, E, idd, M, A, h, K.Act.BF16, err)
    torch.cuda.synchronize()
    err_ref = np.zeros(3, dtype=np.uint32)
    y_ref = oracle.experts_gather(x, w, E, ids, 0, err_ref)
    h_ref = oracle.experts_gather(x, w, E, ids, 1)
    good = np.ones((M, A), bool)
    if M > 1:
        good[1, 0] = False
        assert list(err.cpu().numpy().view(np.uint32)[:3]) == [1, E + 2, A] == list(err_ref)
        assert np.all(np.isnan(oracle.bf16_to_f32(bits_of(y)[1, 0]))) and np.all(np.isnan(oracle.bf16_to_f32(bits_of(h)[1, 0])))
    assert_bf16_close(bits_of(y)[good], y_ref[good], oracle, "gather")
    assert_bf16_close(bits_of(h)[good], h_ref[good], oracle, "gather_swiglu", frac_off=1e-2, ulps=2)
    # combine: h [M, A, K] -> y [M, N]; weights reused as a [E*N, K] down matrix
    hin = oracle.f32_to_bf16(rng.standard_normal((M, A, Kd)).astype(np.float32))
    yc = torch.empty((M, N), dtype=torch.float32, device=cuda)
    ycb = torch.empty((M, N), dtype=torch.bfloat16, device=cuda)
    err.zero_()
    K.linear_qw_experts_combine(bf16_tensor(hin, cuda), wd, E, idd, torch.from_numpy(coef).to(cuda), M, A, yc, K.Act.BF16, err,
                                out_act=K.Act.F32)
    K.linear_qw_experts_combine(bf16_tensor(hin, cuda), wd, E, idd, torch.from_numpy(coef).to(cuda), M, A, ycb, K.Act.BF16, err)
    torch.cuda.synchronize()
    yc_ref = oracle.experts_combine(hin, w, E, ids, coef, out_act=oracle.F32)
    rows = [m for m in range(M) if m != 1 or M == 1]
    assert max_abs_over_rms(yc.cpu().numpy()[rows], yc_ref[rows]) < 3e-5
    assert_bf16_close(bits_of(ycb)[rows], oracle.f32_to_bf16(yc_ref)[rows], oracle, "combine bf16")
    if M > 1:
        assert np.all(np.isnan(yc.cpu().numpy()[1]))
        with pytest.raises(K.Error, match=f"expert id {E + 2} at slot {A}"):
            K.check_expert_error(err, "combine")


@pytest.mark.parametrize("bits,G", [(4, 128), (8, 64)])
@pytest.mark.parametrize("M,A,E,I,d", [(16, 10, 64, 128, 512), (37, 4, 16, 64, 256), (300, 2, 8, 64, 256)])
def test_grouped_experts_exact_math(cuda, oracle, bits, G, M, A, E, I, d):
    """moe_group_routes -> gather_grouped(_swiglu) -> combine_grouped with MoeMath.F32, incl. a hot expert (> 8 slots:
    several tiles) and an invalid id; and the combine's folded shared add."""
    from strixite_b200 import kernels as K
    rng = np.random.default_rng(M + E)
    gu = make_experts(oracle, rng, E, 2 * I, d, G, bits)
    dn = make_experts(oracle, rng, E, d, I, min(G, 64) if I < 128 else G, bits)
    x = oracle.f32_to_bf16(rng.standard_normal((M, d)).astype(np.float32))
    ids = np.stack([rng.permutation(E)[:A] for _ in range(M)]).astype(np.int32)
    ids[:, 0] = np.where(rng.random(M) < 0.7, 3, ids[:, 0])  # expert 3 is hot
    for m in range(M):  # keep a token's ids distinct
        if (ids[m, 1:] == ids[m, 0]).any():
            ids[m, 0] = ids[m, np.argmax(ids[m, 1:] == ids[m, 0]) + 1] ^ 1
    ids[2, 1] = -5
    coef = rng.random((M, A)).astype(np.float32)
    gud, dnd, xd = upload(gu, cuda), upload(dn, cuda), bf16_tensor(x, cuda)
    idd, cfd = torch.from_numpy(ids).to(cuda), torch.from_numpy(coef).to(cuda)
    nbytes = K.moe_route_workspace_bytes(M, A, E)
    ws = torch.empty(nbytes // 4, dtype=torch.int32, device=cuda)
    err = torch.zeros(4, dtype=torch.int32, device=cuda)
    K.moe_group_routes(idd, M, A, E, ws, nbytes, err)
    g = torch.empty((M * A, 2 * I), dtype=torch.bfloat16, device=cuda)
    K.linear_qw_experts_gather_grouped(xd, gud, E, ws, nbytes, M, A, g, K.Act.BF16, K.MoeMath.F32)
    h = torch.empty((M * A, I), dtype=torch.bfloat16, device=cuda)
    K.linear_qw_experts_gather_grouped_swiglu(xd, gud, E, ws, nbytes, M, A, h, K.Act.BF16, K.MoeMath.WmmaBf16)
    # the fused SwiGLU equals the gather followed by swiglu(), bit for bit (kernels/linear_q4.hpp:53-54)
    h2 = torch.empty_like(h)
    K.swiglu(g, h2, M * A, I, K.Act.BF16)
    torch.cuda.synchronize()
    ok = np.ones(M * A, bool)
    ok[2 * A + 1] = False
    assert list(err.cpu().numpy().view(np.uint32)[:3]) == [1, 0xFFFFFFFB, 2 * A + 1]
    assert np.array_equal(bits_of(h)[ok], bits_of(h2)[ok])
    g_ref = oracle.experts_gather(x, gu, E, ids, 0).reshape(M * A, -1)
    h_ref = oracle.experts_gather(x, gu, E, ids, 1).reshape(M * A, -1)
    assert_bf16_close(bits_of(g)[ok], g_ref[ok], oracle, "gather_grouped")
    assert_bf16_close(bits_of(h)[ok], h_ref[ok], oracle, "gather_grouped_swiglu", frac_off=1e-2, ulps=2)
    assert np.all(np.isnan(oracle.bf16_to_f32(bits_of(h)[~ok])))
    # combine on the oracle's h so the two sides see identical inputs
    hd = bf16_tensor(h_ref, cuda)
    partial = torch.empty((M * A, d), dtype=torch.float32, device=cuda)
    y = torch.empty((M, d), dtype=torch.float32, device=cuda)
    K.linear_qw_experts_combine_grouped(hd, dnd, E, idd, cfd, ws, nbytes, partial, M, A, y, K.Act.BF16, K.MoeMath.F32,
                                        out_act=K.Act.F32)
    torch.cuda.synchronize()
    y_ref, p_ref = oracle.experts_combine(h_ref.reshape(M, A, I), dn, E, ids, coef, out_act=oracle.F32, want_partial=True)
    rows = [m for m in range(M) if m != 2]
    assert max_abs_over_rms(partial.cpu().numpy()[ok], p_ref[ok]) < 3e-5
    assert max_abs_over_rms(y.cpu().numpy()[rows], y_ref[rows]) < 3e-5
    assert np.all(np.isnan(y.cpu().numpy()[2]))
    # folded shared add == combine then moe_shared_add (kernels/moe_grouped.hpp:71-74), BF16 outputs, bit for bit
    s = oracle.f32_to_bf16(rng.standard_normal((M, d)).astype(np.float32))
    gate = rng.standard_normal((M, 2)).astype(np.float32)
    sd, gd = bf16_tensor(s, cuda), torch.from_numpy(gate).to(cuda)
    ya = torch.empty((M, d), dtype=torch.bfloat16, device=cuda)
    yb = torch.empty((M, d), dtype=torch.bfloat16, device=cuda)
    err2 = torch.zeros(4, dtype=torch.int32, device=cuda)
    K.linear_qw_experts_combine_grouped(hd, dnd, E, idd, cfd, ws, nbytes, partial, M, A, ya, K.Act.BF16, K.MoeMath.F32,
                                        shared=K.MoeSharedAdd(sd, gd.data_ptr() + 4, 2, E, err2))
    K.linear_qw_experts_combine_grouped(hd, dnd, E, idd, cfd, ws, nbytes, partial, M, A, yb, K.Act.BF16, K.MoeMath.F32)
    K.moe_shared_add(yb, sd, gd.data_ptr() + 4, 2, M, d, E, K.Act.BF16, err2)
    torch.cuda.synchronize()
    assert np.array_equal(bits_of(ya)[rows], bits_of(yb)[rows])
    ref = oracle.moe_shared_add(oracle.f32_to_bf16(y_ref), s, gate[:, 1], E)
    assert_bf16_close(bits_of(ya)[rows], ref[rows], oracle, "combine + shared add", frac_off=5e-3)


@pytest.mark.parametrize("bits,G", [(4, 128), (8, 64), (4, 32)])
@pytest.mark.parametrize("M,A,E,I,d", [(40, 2, 4, 128, 256), (300, 2, 8, 128, 256), (700, 4, 8, 256, 384),
                                       (700, 2, 4, 128, 2048)])  # the last: a long contraction over well-filled experts
def test_grouped_experts_tcgen05(cuda, oracle, bits, G, M, A, E, I, d):
    """MoeMath.WmmaF16: tcgen05 grouped GEMMs (F16 operands, FP32 accumulation in tensor memory) against the oracle's
    matrix-unit semantics: weights as the F16 operand f16(code * scale + min), h = silu(g) * u rounded once.  Both
    sides then multiply the same operand values; only the order of the FP32 sums differs."""
    from strixite_b200 import kernels as K
    rng = np.random.default_rng(M + E + bits)
    gu = make_experts(oracle, rng, E, 2 * I, d, G, bits)
    dn = make_experts(oracle, rng, E, d, I, G if I % G == 0 else 64, bits)
    x = oracle.f32_to_bf16(rng.standard_normal((M, d)).astype(np.float32))
    ids = np.stack([rng.permutation(E)[:A] for _ in range(M)]).astype(np.int32)
    if M >= 300:
        ids[:200, 0] = 1  # one expert with > 128 slots: several token tiles
        for m in range(200):
            if (ids[m, 1:] == 1).any():
                ids[m, np.argmax(ids[m, 1:] == 1) + 1] = 0 if 0 not in ids[m] else 2
    ids[5, 1] = E + 9
    coef = rng.random((M, A)).astype(np.float32)
    gud, dnd, xd = upload(gu, cuda), upload(dn, cuda), bf16_tensor(x, cuda)
    idd, cfd = torch.from_numpy(ids).to(cuda), torch.from_numpy(coef).to(cuda)
    nbytes = K.moe_route_workspace_bytes(M, A, E)
    ws = torch.empty(nbytes // 4, dtype=torch.int32, device=cuda)
    err = torch.zeros(4, dtype=torch.int32, device=cuda)
    K.moe_group_routes(idd, M, A, E, ws, nbytes, err)
    g = torch.zeros((M * A, 2 * I), dtype=torch.bfloat16, device=cuda)
    K.linear_qw_experts_gather_grouped(xd, gud, E, ws, nbytes, M, A, g, K.Act.BF16, K.MoeMath.WmmaF16)
    h = torch.zeros((M * A, I), dtype=torch.bfloat16, device=cuda)
    K.linear_qw_experts_gather_grouped_swiglu(xd, gud, E, ws, nbytes, M, A, h, K.Act.BF16, K.MoeMath.WmmaF16)
    hf = torch.zeros((M * A, I), dtype=torch.float16, device=cuda)
    K.linear_qw_experts_gather_grouped_swiglu(xd, gud, E, ws, nbytes, M, A, hf, K.Act.BF16, K.MoeMath.WmmaF16, h_f16=True)
    torch.cuda.synchronize()
    K.check_grouped_status(ws, "tcgen05 gather")
    ok = np.ones(M * A, bool)
    ok[5 * A + 1] = False
    g_ref = oracle.experts_gather(x, gu, E, ids, 0, w_f16=True).reshape(M * A, -1)
    assert_bf16_close(bits_of(g)[ok], g_ref[ok], oracle, "tcgen05 gather")
    h_ref = oracle.experts_gather(x, gu, E, ids, 2, w_f16=True).reshape(M * A, -1)
    assert_bf16_close(bits_of(h)[ok], h_ref[ok], oracle, "tcgen05 gather + swiglu")
    assert np.all(np.isnan(oracle.bf16_to_f32(bits_of(h)[~ok])))
    # h_f16 holds the F16 rounding of the same BF16 values (equal except below F16's normal range)
    okd = torch.from_numpy(ok).to(cuda)
    assert torch.allclose(hf.float()[okd], h.float()[okd], rtol=0, atol=2.0 ** -25)
    # the staged form: x converted once by stage_f16, h written in the down operand's k order
    PERM = [0, 4, 1, 5, 2, 6, 3, 7]
    hk = 2 if bits == 4 else 1
    xh = torch.empty((M, d), dtype=torch.float16, device=cuda)
    K.stage_f16(xd, M, d, bits, xh)
    want_x = xd.float().view(M, d // 8, 8)[:, :, PERM].reshape(M, d) if bits == 4 else xd.float()
    assert torch.allclose(xh.float(), want_x, rtol=0, atol=2.0 ** -25)  # exact above F16's subnormal range
    hs = torch.zeros((M * A, I), dtype=torch.float16, device=cuda)
    K.linear_qw_experts_gather_grouped_swiglu(xh, gud, E, ws, nbytes, M, A, hs, K.Act.F16_STAGED, K.MoeMath.WmmaF16, h_f16=hk)
    torch.cuda.synchronize()
    K.check_grouped_status(ws, "tcgen05 staged gather")
    want_hs = hf.view(M * A, I // 8, 8)[:, :, PERM].reshape(M * A, I) if hk == 2 else hf
    assert torch.equal(hs[okd].view(torch.int16), want_hs[okd].view(torch.int16))
    # the tile-blocked form: x gathered by stage_f16_tiles, h written tile-blocked; same values again
    xt = torch.zeros((M * A, d), dtype=torch.float16, device=cuda)
    K.stage_f16_tiles(xd, ws, nbytes, M, A, E, d, bits, xt)
    ht = torch.zeros((M * A, I), dtype=torch.float16, device=cuda)
    K.linear_qw_experts_gather_grouped_swiglu(xt, gud, E, ws, nbytes, M, A, ht, K.Act.F16_TILED, K.MoeMath.WmmaF16,
                                              h_f16=3 if bits == 4 else 4)
    torch.cuda.synchronize()
    K.check_grouped_status(ws, "tcgen05 tiled gather")

    def untile(buf, width):
        """Tile-blocked [S, width] F16 -> natural [slot, width] (host-side inverse of the layout, for checking)."""
        L = K.route_layout(M, A, E)
        w_ = ws.cpu().numpy()
        offs, slots_ = w_[L["offsets"]:L["offsets"] + E + 2], w_[L["slots"]:L["slots"] + M * A]
        raw = buf.cpu().numpy().view(np.uint16).reshape(-1)
        out = np.zeros((M * A, width), dtype=np.uint16)
        S = M * A
        for b in range(E):
            for pos in range(int(offs[b]), int(offs[b + 1])):
                n = (pos - int(offs[b])) % 128
                for kb in range(width // 64):
                    line = raw[((kb * S + pos) * 128) // 2:((kb * S + pos) * 128) // 2 + 64].reshape(8, 8)
                    for c in range(8):
                        chunk = line[c ^ (n & 7)]
                        out[slots_[pos], kb * 64 + c * 8:kb * 64 + c * 8 + 8] = chunk[np.argsort(PERM)] if bits == 4 else chunk
        return torch.from_numpy(out.view(np.float16)).to(cuda)

    assert torch.equal(untile(ht, I)[okd].view(torch.int16), hf[okd].view(torch.int16))
    # down + combine on the oracle's h (identical inputs on both sides), from BF16 h and from F16 h
    y_ref, p_ref = oracle.experts_combine(h_ref.reshape(M, A, I), dn, E, ids, coef, out_act=oracle.F32, want_partial=True,
                                          w_f16=True)
    rows = [m for m in range(M) if m != 5]
    for f16 in (0, 1, 2, 34):
        if f16 == 2 and bits != 4:
            continue
        if f16 == 34:  # tile-blocked h as the tiled gather leaves it, from the GPU's own h (== oracle h up to rare flips)
            partial = torch.zeros((M * A, d), dtype=torch.float32, device=cuda)
            y = torch.empty((M, d), dtype=torch.float32, device=cuda)
            K.linear_qw_experts_combine_grouped(ht, dnd, E, idd, cfd, ws, nbytes, partial, M, A, y, K.Act.BF16, K.MoeMath.WmmaF16,
                                                out_act=K.Act.F16_TILED if False else K.Act.F32, h_f16=3 if bits == 4 else 4)
            y2 = torch.empty((M, d), dtype=torch.float32, device=cuda)
            K.linear_qw_experts_combine_grouped(hf, dnd, E, idd, cfd, ws, nbytes, partial, M, A, y2, K.Act.BF16, K.MoeMath.WmmaF16,
                                                out_act=K.Act.F32, h_f16=1)
            torch.cuda.synchronize()
            K.check_grouped_status(ws, "tcgen05 tiled combine")
            assert torch.equal(y[rows], y2[rows])  # the same values through the bulk-copy path and the per-row path
            continue
        hd = bf16_tensor(h_ref, cuda)
        if f16:
            hd = hd.float().to(torch.float16)
        if f16 == 2:
            hd = hd.view(M * A, I // 8, 8)[:, :, PERM].reshape(M * A, I).contiguous()
        # FP32 per-slot dots (this library's extra math kind): tight against the oracle
        partial = torch.zeros((M * A, d), dtype=torch.float32, device=cuda)
        y = torch.empty((M, d), dtype=torch.float32, device=cuda)
        K.linear_qw_experts_combine_grouped(hd, dnd, E, idd, cfd, ws, nbytes, partial, M, A, y, K.Act.BF16,
                                            K.MoeMath.WmmaF16F32Partials, out_act=K.Act.F32, h_f16=f16)
        torch.cuda.synchronize()
        K.check_grouped_status(ws, "tcgen05 combine")
        assert max_abs_over_rms(partial.cpu().numpy()[ok], p_ref[ok]) < 3e-5
        assert max_abs_over_rms(y.cpu().numpy()[rows], y_ref[rows]) < 3e-5
        assert np.all(np.isnan(y.cpu().numpy()[5]))
        # BF16 per-slot dots (the reference's WMMA_F16, kernels/moe_grouped.hip:47-57): the stored dots are the BF16 rounding
        # of the same sums - equal to the oracle's rounding except where a sum sits on a rounding boundary (one ulp) - and
        # y is the slot-order sum of exactly those stored values
        pb = torch.zeros((M * A, d), dtype=torch.float32, device=cuda)
        yb = torch.empty((M, d), dtype=torch.float32, device=cuda)
        K.linear_qw_experts_combine_grouped(hd, dnd, E, idd, cfd, ws, nbytes, pb, M, A, yb, K.Act.BF16, K.MoeMath.WmmaF16,
                                            out_act=K.Act.F32, h_f16=f16)
        torch.cuda.synchronize()
        got_p = bits_of(pb.view(torch.bfloat16).reshape(-1)[: M * A * d].view(M * A, d))
        want_p = oracle.f32_to_bf16(p_ref)
        gp, wp = oracle.bf16_to_f32(got_p[ok]).astype(np.float64), oracle.bf16_to_f32(want_p[ok]).astype(np.float64)
        p_rms = float(np.sqrt(np.mean(wp ** 2)))
        assert np.all(np.abs(gp - wp) <= 2.0 ** -7 * np.abs(wp) + 3e-5 * p_rms)  # one BF16 ulp, or FP32 summation noise near zero
        assert (got_p[ok] != want_p[ok]).mean() < 0.01
        stored = oracle.bf16_to_f32(got_p).astype(np.float64).reshape(M, A, d)
        y_from_stored = np.einsum("ma,mad->md", coef.astype(np.float64), np.where(np.isnan(stored), 0, stored))
        assert max_abs_over_rms(yb.cpu().numpy()[rows], y_from_stored[rows]) < 3e-6
        y_ref_b = oracle.experts_combine(h_ref.reshape(M, A, I), dn, E, ids, coef, out_act=oracle.F32, w_f16=True, partial_bf16=True)
        # a dot on a BF16 rounding boundary falls either way (one ulp = 2^-8 of the dot, times its coefficient): over M * d
        # outputs the largest such flip reaches ~1e-2 of the RMS, which is why this library's default keeps the dots in FP32
        assert max_abs_over_rms(yb.cpu().numpy()[rows], y_ref_b[rows]) < 2e-2
