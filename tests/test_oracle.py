"""CPU tests of the oracle: pinned against the reference's quantizers (golden vectors made by the reference's own
code, and the compiled reference itself when present), and checked for self-consistency on router / pack / layer."""
import numpy as np
import pytest

QUANT = [(4, 128), (4, 64), (4, 32), (8, 128), (8, 64), (8, 32)]


@pytest.mark.parametrize("bits,G", QUANT)
def test_quantizer_matches_reference_golden(oracle, golden, bits, G):
    tag = f"q{bits}g{G}"
    r = oracle.quantize(golden[f"{tag}.w"], G, bits)
    assert np.array_equal(r.q, golden[f"{tag}.q"])
    assert np.array_equal(r.scale, golden[f"{tag}.scale"])
    assert np.array_equal(r.minv, golden[f"{tag}.minv"])
    deq = oracle.dequantize(r)
    assert np.array_equal(deq.view(np.uint32), golden[f"{tag}.deq"].view(np.uint32))
    # the format's own definition: w = code * scale + min, two FP32 roundings
    codes = r.q.astype(np.float32) if bits == 8 else np.stack([r.q & 0xF, r.q >> 4], -1).reshape(r.N, r.K).astype(np.float32)
    s = np.repeat(oracle.bf16_to_f32(r.scale), G, axis=1)
    m = np.repeat(oracle.bf16_to_f32(r.minv), G, axis=1)
    assert np.array_equal((codes * s + m).view(np.uint32), deq.view(np.uint32))


@pytest.mark.parametrize("bits,G", QUANT)
def test_quantizer_matches_compiled_reference(oracle, bits, G):
    if oracle.ref_lib() is None:
        pytest.skip("the reference checkout is not on this machine; the golden vectors cover this")
    rng = np.random.default_rng(bits * 1000 + G)
    w = (rng.standard_normal((33, 512)) * 0.02).astype(np.float32)
    a, b = oracle.quantize(w, G, bits), oracle.ref_quantize(w, G, bits)
    assert np.array_equal(a.q, b.q) and np.array_equal(a.scale, b.scale) and np.array_equal(a.minv, b.minv)
    assert np.array_equal(oracle.dequantize(a).view(np.uint32), oracle.ref_dequantize(b).view(np.uint32))


def test_quantizer_rejects_bad_input(oracle):
    w = np.zeros((2, 64), dtype=np.float32)
    w[1, 3] = np.inf
    with pytest.raises(ValueError):
        oracle.quantize(w, 32, 4)
    with pytest.raises(ValueError):
        oracle.quantize(np.zeros((2, 48), dtype=np.float32), 32, 4)  # K % G != 0


def test_router_golden_and_properties(oracle, golden):
    logits = golden["router.logits"]
    E, k = 64, 4
    ids, coef = oracle.moe_router(logits, E, k)
    assert np.array_equal(ids, golden["router.ids"])
    assert np.array_equal(coef.view(np.uint32), golden["router.coef"].view(np.uint32))
    # order: larger logit first, a tie to the lower index
    for m in range(logits.shape[0]):
        order = sorted(range(E), key=lambda e: (-float(logits[m, e]), e))[:k]
        assert list(ids[m]) == order
    assert list(ids[1]) == [0, 1, 2, 3] and list(ids[2][:2]) == [10, 40] and list(ids[3]) == [0, 1, 2, 3]
    np.testing.assert_allclose(coef.sum(1), 1.0, rtol=1e-6)
    assert coef[4, 0] == 1.0 and ids[4, 0] == 5
    ids_s, coef_s = oracle.moe_router(logits, E, k, np.ascontiguousarray(logits[:, E:]), 1, E)
    assert np.array_equal(ids_s, golden["router.ids_shared"]) and np.array_equal(ids_s[:, :k], ids)
    assert np.all(ids_s[:, k] == E)
    np.testing.assert_allclose(coef_s[:, k], 1 / (1 + np.exp(-logits[:, E].astype(np.float64))), rtol=1e-6)


def test_router_non_finite_fails_the_token(oracle):
    logits = np.zeros((3, 9), dtype=np.float32)
    logits[1, 4] = np.nan
    err = np.zeros(3, dtype=np.uint32)
    ids, coef = oracle.moe_router(logits, 8, 2, err=err)
    assert list(err) == [1, 1, 4]
    assert np.all(ids[1] == -1) and np.all(np.isnan(coef[1])) and np.all(ids[0] >= 0)
    bf = oracle.f32_to_bf16(logits)
    ids2, _ = oracle.moe_router(bf, 8, 2)
    assert np.all(ids2[1] == -1)


def test_pack_golden_and_is_a_stable_counting_sort(oracle, golden):
    ids = golden["pack.ids"]
    E = 16
    err = np.zeros(3, dtype=np.uint32)
    offsets, slots = oracle.moe_group_routes(ids, E, err)
    assert np.array_equal(offsets, golden["pack.offsets"]) and np.array_equal(slots, golden["pack.slots"])
    assert np.array_equal(err, golden["pack.err"]) and list(err) == [1, 0xFFFFFFFF, 3 * 4 + 1]
    flat = ids.reshape(-1)
    bucket = np.where((flat < 0) | (flat >= E), E, flat)
    assert np.array_equal(slots, np.argsort(bucket, kind="stable"))
    assert np.array_equal(np.diff(offsets), np.bincount(bucket, minlength=E + 1))


def test_layer_golden(oracle, golden):
    E, k = 4, 2
    def qw(name, N, K, G, bits):
        return oracle.QWeight(golden[f"layer.{name}.q"], golden[f"layer.{name}.scale"], golden[f"layer.{name}.minv"], N, K, G, bits)
    w = oracle.LayerWeights(qw("gu", E * 128, 128, 64, 4), qw("dn", E * 128, 64, 32, 8), qw("sgu", 128, 128, 64, 8),
                            qw("sdn", 128, 64, 64, 8))
    for sem in ("decode", "grouped", "grouped_f32_partials"):
        r = oracle.moe_layer(golden["layer.x"], golden["layer.logits"], w, E, k, semantics=sem, threads=2)
        assert np.array_equal(r["ids"], golden[f"layer.{sem}.ids"])
        assert np.array_equal(r["h"], golden[f"layer.{sem}.h"])
        assert np.array_equal(r["y_bf16"], golden[f"layer.{sem}.y_bf16"])
        np.testing.assert_array_equal(r["y_f32"], golden[f"layer.{sem}.y_f32"])


def test_layer_against_plain_numpy(oracle):
    """The oracle's C0-shaped layer against a direct float64 numpy evaluation of the same formulas."""
    rng = np.random.default_rng(0)
    T, d, E, k, I = 4, 1024, 64, 4, 256
    x = oracle.f32_to_bf16(rng.standard_normal((T, d)).astype(np.float32))
    wr = (rng.standard_normal((E + 1, d)) * 0.02).astype(np.float32)
    logits = (oracle.bf16_to_f32(x) @ wr.T).astype(np.float32)
    gu = oracle.quantize((rng.standard_normal((E * 2 * I, d)) * 0.02).astype(np.float32), 64, 8)
    dn = oracle.quantize((rng.standard_normal((E * d, I)) * 0.02).astype(np.float32), 64, 8)
    out = oracle.moe_layer(x, logits, oracle.LayerWeights(gu, dn), E, k)
    W, Wd = oracle.dequantize(gu).astype(np.float64), oracle.dequantize(dn).astype(np.float64)
    xf = oracle.bf16_to_f32(x).astype(np.float64)
    rt = lambda v: oracle.bf16_to_f32(oracle.f32_to_bf16(np.asarray(v, dtype=np.float32)))
    y = np.zeros((T, d))
    for m in range(T):
        for a in range(k):
            e = int(out["ids"][m, a])
            g, u = rt(W[e * 2 * I:e * 2 * I + I] @ xf[m]), rt(W[e * 2 * I + I:(e + 1) * 2 * I] @ xf[m])
            h = rt(rt(g / (1 + np.exp(-g))) * u)
            assert np.array_equal(oracle.f32_to_bf16(h), out["h"][m, a])
            y[m] += float(out["coef"][m, a]) * (Wd[e * d:(e + 1) * d] @ h.astype(np.float64))
    assert np.max(np.abs(y - out["y_f32"])) < 1e-6
    # rows are independent: a subset of the tokens gives the same rows
    sub = oracle.moe_layer(x[1:3], logits[1:3], oracle.LayerWeights(gu, dn), E, k)
    assert np.array_equal(sub["y_f32"], out["y_f32"][1:3])


def test_invalid_ids_poison_outputs(oracle):
    rng = np.random.default_rng(1)
    E, N, K = 4, 32, 64
    w = oracle.quantize((rng.standard_normal((E * N, K)) * 0.02).astype(np.float32), 32, 4)
    x = oracle.f32_to_bf16(rng.standard_normal((3, K)).astype(np.float32))
    ids = np.array([[0, 1], [7, 2], [3, 3]], dtype=np.int32)
    err = np.zeros(3, dtype=np.uint32)
    y = oracle.bf16_to_f32(oracle.experts_gather(x, w, E, ids, err=err))
    assert list(err) == [1, 7, 2] and np.all(np.isnan(y[1, 0])) and not np.any(np.isnan(y[1, 1]))
    h = oracle.f32_to_bf16(rng.standard_normal((3, 2, K)).astype(np.float32))
    yc = oracle.experts_combine(h, w, E, ids, np.ones((3, 2), np.float32), out_act=oracle.F32)
    assert np.all(np.isnan(yc[1])) and not np.any(np.isnan(yc[[0, 2]]))


@pytest.mark.parametrize("bits,G", [(4, 64), (8, 32), (4, 128)])
def test_chunk_major_matches_compiled_reference(oracle, bits, G):
    """The chunk-major re-layout the hyper-connection up projection reads (formats/q4.hpp:41-55) against the reference's own
    to_chunk_major, byte for byte."""
    if oracle.ref_lib() is None:
        pytest.skip("the reference checkout is not available here")
    rng = np.random.default_rng(bits * G)
    w = oracle.quantize((rng.standard_normal((37, 256)) * 0.02).astype(np.float32), G, bits)
    a, b = oracle.to_chunk_major(w), oracle.ref_to_chunk_major(w)
    assert np.array_equal(a.q, b.q) and np.array_equal(a.scale, b.scale) and np.array_equal(a.minv, b.minv)


def test_hc_mix_oracle_against_plain_loops(oracle):
    """The vectorised float64 hc_mix oracle against the definition written out element by element on a tiny case."""
    rng = np.random.default_rng(3)
    H, d, r, T, eps = 4, 32, 32, 2, 1e-6
    wd = oracle.quantize((rng.standard_normal((r + H, H * d)) * 0.05).astype(np.float32), 32, 4)
    x = rng.standard_normal((T, H * d)).astype(np.float32)
    h, w_in, inv = oracle.hc_mix_down(x, wd, H, d, r, True, eps)
    W = oracle.affine_weights(wd)
    for t in range(T):
        iv = [1.0 / np.sqrt(np.mean(x[t, s * d:(s + 1) * d].astype(np.float64) ** 2) + eps) for s in range(H)]
        assert np.allclose(inv[t], iv, rtol=1e-12)
        for n in range(r + H):
            a = sum(iv[s] * float(np.dot(x[t, s * d:(s + 1) * d].astype(np.float64), W[n, s * d:(s + 1) * d])) for s in range(H))
            z = a / H
            if n < r:
                assert np.isclose(h[t, n], z / (1 + np.exp(-z)), rtol=1e-10, atol=1e-12)
            else:
                assert np.isclose(w_in[t, n - r], 2 / (1 + np.exp(-z)), rtol=1e-10)
    wu = oracle.quantize((rng.standard_normal((H * d, r)) * 0.2).astype(np.float32), 32, 8)
    nw = (rng.standard_normal(H * d) * 0.1).astype(np.float32)
    u = oracle.hc_mix_up(h, wu, x, nw, inv, H, d)
    Wu = oracle.affine_weights(wu)
    for t in range(T):
        for j in range(d):
            tot = 0.0
            for s in range(H):
                row = s * d + j
                tot += 1 / (1 + np.exp(-float(np.dot(Wu[row], h[t])))) * float(x[t, row]) * inv[t, s] * (1 + float(nw[row]))
            assert np.isclose(u[t, j], tot / H, rtol=1e-10, atol=1e-12)


def test_hc_mix_oracle_f16_operands(oracle):
    """The matrix-unit form of the mix (kernels/hc_wmma.hpp:3-8): products of x, h and the weights each rounded once to F16,
    written out element by element with numpy's half type; inv comes from the unrounded x.  The rounding moves the result by
    about one part in a thousand, not more."""
    rng = np.random.default_rng(4)
    H, d, r, T, eps = 4, 32, 32, 2, 1e-6
    wd = oracle.quantize((rng.standard_normal((r + H, H * d)) * 0.05).astype(np.float32), 32, 8)
    x = (rng.standard_normal((T, H * d)) * 3).astype(np.float32)
    h, w_in, inv = oracle.hc_mix_down(x, wd, H, d, r, True, eps, f16_operands=True)
    h_exact, w_in_exact, inv_exact = oracle.hc_mix_down(x, wd, H, d, r, True, eps)
    assert np.array_equal(inv, inv_exact)
    W16 = oracle.affine_weights(wd).astype(np.float16).astype(np.float64)
    x16 = x.astype(np.float16).astype(np.float64)
    for t in range(T):
        for n in range(r + H):
            a = sum(inv[t, s] * float(np.dot(x16[t, s * d:(s + 1) * d], W16[n, s * d:(s + 1) * d])) for s in range(H))
            z = a / H
            got = h[t, n] if n < r else w_in[t, n - r]
            want = z / (1 + np.exp(-z)) if n < r else 2 / (1 + np.exp(-z))
            assert np.isclose(got, want, rtol=1e-10, atol=1e-12)
    assert 0 < np.max(np.abs(h - h_exact)) <= 1e-2 * np.sqrt(np.mean(h_exact ** 2))
    wu = oracle.quantize((rng.standard_normal((H * d, r)) * 0.2).astype(np.float32), 32, 4)
    nw = (rng.standard_normal(H * d) * 0.1).astype(np.float32)
    u = oracle.hc_mix_up(h, wu, x, nw, inv, H, d, f16_operands=True)
    Wu16 = oracle.affine_weights(wu).astype(np.float16).astype(np.float64)
    h16 = h.astype(np.float16).astype(np.float64)
    for t in range(T):
        for j in range(d):
            tot = 0.0
            for s in range(H):
                row = s * d + j
                tot += 1 / (1 + np.exp(-float(np.dot(Wu16[row], h16[t])))) * float(x[t, row]) * inv[t, s] * (1 + float(nw[row]))
            assert np.isclose(u[t, j], tot / H, rtol=1e-10, atol=1e-12)
    u_exact = oracle.hc_mix_up(h, wu, x, nw, inv, H, d)
    assert 0 < np.max(np.abs(u - u_exact)) <= 1e-2 * np.sqrt(np.mean(u_exact ** 2))
