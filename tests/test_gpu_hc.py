"""The hyper-connection mix either side of the MoE block (kernels/hc.hpp:36-54) against the float64 oracle, through the
C ABI: hc_mix_down, hc_mix_up (chunk-major weight) and the device-side chunk-major re-layout."""
import numpy as np
import pytest
import torch

from helpers import bf16_tensor, bits_of, max_abs_over_rms, random_weights, upload

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("bits,G", [(4, 64), (8, 128), (4, 32)])
def test_to_chunk_major_on_the_device(cuda, oracle, bits, G):
    """sxb_to_chunk_major equals the host re-layout, which test_oracle pins to the reference's own to_chunk_major."""
    from strixite_b200 import kernels as K
    rng = np.random.default_rng(bits + G)
    wq = oracle.quantize(random_weights(rng, 1300, 320), G if 320 % G == 0 else 64, bits)
    cm = K.to_chunk_major(upload(wq, cuda))
    want = oracle.to_chunk_major(wq)
    assert np.array_equal(cm.q.cpu().numpy().reshape(-1), want.q.reshape(-1))
    assert np.array_equal(cm.scale.cpu().numpy().view(np.uint16).reshape(-1), want.scale.reshape(-1))
    assert np.array_equal(cm.minv.cpu().numpy().view(np.uint16).reshape(-1), want.minv.reshape(-1))


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("bits,G,T,d,r,inject", [(4, 64, 1, 256, 64, True), (8, 128, 5, 512, 96, True), (4, 128, 16, 1024, 320, True),
                                                  (8, 64, 37, 256, 32, False), (4, 32, 300, 128, 64, True)])
def test_hc_mix(cuda, oracle, dt, bits, G, T, d, r, inject):
    """hc_mix_down then hc_mix_up, each against the oracle on the same inputs: h, w_in and inv within FP32 summation noise of the
    float64 values, u within it (F32 streams) or within one BF16 rounding of it (BF16 streams)."""
    from strixite_b200 import kernels as K
    H, eps = 4, 1e-6
    rng = np.random.default_rng(T * 7 + d + bits)
    R = r + (H if inject else 0)
    wd = oracle.quantize(random_weights(rng, R, H * d, std=0.05), G, bits)
    wu = oracle.quantize(random_weights(rng, H * d, r, std=0.2), 32 if r % G else G, bits)
    norm_w = (rng.standard_normal(H * d) * 0.1).astype(np.float32)
    x = (rng.standard_normal((T, H * d)) * np.repeat(rng.random((T, H)) * 3 + 0.2, d, axis=1)).astype(np.float32)  # streams of different RMS
    if dt == torch.bfloat16:
        xb = oracle.f32_to_bf16(x)
        x = oracle.bf16_to_f32(xb)
        xd, act = bf16_tensor(xb, cuda), K.Act.BF16
    else:
        xd, act = torch.from_numpy(x).to(cuda), K.Act.F32
    h = torch.full((T, r), float("nan"), dtype=torch.float32, device=cuda)
    w_in = torch.full((T, H), float("nan"), dtype=torch.float32, device=cuda) if inject else None
    inv = torch.full((T, H), float("nan"), dtype=torch.float32, device=cuda)
    K.hc_mix_down(xd, upload(wd, cuda), T, H, d, r, inject, eps, h, w_in, inv, act)
    h_ref, w_in_ref, inv_ref = oracle.hc_mix_down(x, wd, H, d, r, inject, eps)
    assert max_abs_over_rms(inv.cpu().numpy(), inv_ref) <= 1e-5
    assert max_abs_over_rms(h.cpu().numpy(), h_ref) <= 1e-4
    if inject:
        assert max_abs_over_rms(w_in.cpu().numpy(), w_in_ref) <= 1e-4
    # the up half on the GPU's own h and inv (so that its error is its own)
    u = torch.empty((T, d), dtype=dt, device=cuda)
    K.hc_mix_up(h, K.to_chunk_major(upload(wu, cuda)), xd, torch.from_numpy(norm_w).to(cuda), inv, T, H, d, u, act)
    torch.cuda.synchronize()
    u_ref = oracle.hc_mix_up(h.cpu().numpy(), wu, x, norm_w, inv.cpu().numpy(), H, d)
    if dt == torch.float32:
        assert max_abs_over_rms(u.cpu().numpy(), u_ref) <= 1e-4
    else:
        got = oracle.bf16_to_f32(bits_of(u)).astype(np.float64)
        assert np.all(np.abs(got - u_ref) <= 2.0 ** -8 * np.abs(u_ref) + 1e-5 * np.sqrt(np.mean(u_ref ** 2)))  # one BF16 rounding


def test_hc_mix_argument_checks(cuda, oracle):
    from strixite_b200 import kernels as K
    rng = np.random.default_rng(1)
    H, d, r, T = 4, 64, 32, 3
    wd = upload(oracle.quantize(random_weights(rng, r + H, H * d), 64, 4), cuda)
    x = torch.zeros((T, H * d), dtype=torch.bfloat16, device=cuda)
    h, w_in, inv = (torch.zeros((T, n), dtype=torch.float32, device=cuda) for n in (r, H, H))
    with pytest.raises(K.Error, match="w_in must be given exactly when inject"):
        K.hc_mix_down(x, wd, T, H, d, r, True, 1e-6, h, None, inv, K.Act.BF16)
    with pytest.raises(K.Error, match="rows, expected r"):
        K.hc_mix_down(x, wd, T, H, d, r, False, 1e-6, h, None, inv, K.Act.BF16)
    with pytest.raises(K.Error, match="streams, only 4"):
        K.hc_mix_down(x, wd, T, 2, 2 * d, r, True, 1e-6, h, w_in, inv, K.Act.BF16)
    with pytest.raises(K.Error, match="eps must be finite"):
        K.hc_mix_down(x, wd, T, H, d, r, True, 0.0, h, w_in, inv, K.Act.BF16)


def _ws(nbytes, device):
    return torch.empty(nbytes, dtype=torch.uint8, device=device)  # the caching allocator hands out 512-byte aligned blocks


# (bits, G, T, d, r, inject): short and long contractions, few and many tokens a stream (the two tcgen05 kernels and both
# tile widths of the second), an up mix of more than one block of 1024 tokens, one token
WMMA_CASES = [(4, 64, 40, 256, 64, True), (8, 128, 200, 512, 320, True), (4, 128, 700, 2560, 320, True), (8, 64, 50, 2560, 64, False),
              (4, 32, 1100, 128, 32, True), (8, 32, 1, 128, 64, True)]


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("bits,G,T,d,r,inject", WMMA_CASES)
def test_hc_mix_wmma(cuda, oracle, dt, bits, G, T, d, r, inject):
    """hc_mix_down_wmma then hc_mix_up_wmma against the oracle with the matrix-unit path's operand roundings (x, h and the
    weights once to F16): what remains is FP32 summation order.  Also within 1e-2 x RMS of the unrounded math."""
    from strixite_b200 import kernels as K
    H, eps = 4, 1e-6
    rng = np.random.default_rng(T * 11 + d + bits)
    R = r + (H if inject else 0)
    wd = oracle.quantize(random_weights(rng, R, H * d, std=0.05), G, bits)
    wu = oracle.quantize(random_weights(rng, H * d, r, std=0.2), 32 if r % G else G, bits)
    norm_w = (rng.standard_normal(H * d) * 0.1).astype(np.float32)
    x = (rng.standard_normal((T, H * d)) * np.repeat(rng.random((T, H)) * 3 + 0.2, d, axis=1)).astype(np.float32)
    if dt == torch.bfloat16:
        xb = oracle.f32_to_bf16(x)
        x = oracle.bf16_to_f32(xb)
        xd, act = bf16_tensor(xb, cuda), K.Act.BF16
    else:
        xd, act = torch.from_numpy(x).to(cuda), K.Act.F32
    h = torch.full((T, r), float("nan"), dtype=torch.float32, device=cuda)
    w_in = torch.full((T, H), float("nan"), dtype=torch.float32, device=cuda) if inject else None
    inv = torch.full((T, H), float("nan"), dtype=torch.float32, device=cuda)
    ws = _ws(K.hc_wmma_workspace_bytes(T, H, d, R, bits, G), cuda)
    K.hc_mix_down_wmma(xd, upload(wd, cuda), T, H, d, r, inject, eps, h, w_in, inv, ws, act)
    K.check_grouped_status(ws, "hc_mix_down_wmma")
    # the grouping workspace the mix wrote without ids (streams as experts) is the pack's own for ids[t * H + s] = s
    S = T * H
    ids = (torch.arange(S, device=cuda) % H).to(torch.int32)
    nbytes = K.moe_route_workspace_bytes(S, 1, H)
    ws_pack, err = torch.zeros(nbytes // 4, dtype=torch.int32, device=cuda), torch.zeros(4, dtype=torch.int32, device=cuda)
    K.moe_group_routes(ids, S, 1, H, ws_pack, nbytes, err)
    got_ws, want_ws, lay = ws[:nbytes].view(torch.int32).cpu().numpy(), ws_pack.cpu().numpy(), K.route_layout(S, 1, H)
    assert np.array_equal(got_ws[:5], want_ws[:5])
    assert np.array_equal(got_ws[lay["offsets"]:lay["offsets"] + H + 2], want_ws[lay["offsets"]:lay["offsets"] + H + 2])
    assert np.array_equal(got_ws[lay["slots"]:lay["slots"] + S], want_ws[lay["slots"]:lay["slots"] + S])
    for rows, n_at in ((8, 0), (128, 3)) + tuple((rows, lay[f"tile{rows}_n"]) for rows in K.TC_TILES):
        n = int(want_ws[n_at])
        assert int(got_ws[n_at]) == n
        for part in ("bucket", "start"):
            at = lay[f"tile{rows}_{part}"]
            assert np.array_equal(got_ws[at:at + n], want_ws[at:at + n])
    h_ref, w_in_ref, inv_ref = oracle.hc_mix_down(x, wd, H, d, r, inject, eps, f16_operands=True)
    h_exact, _, _ = oracle.hc_mix_down(x, wd, H, d, r, inject, eps)
    assert max_abs_over_rms(inv.cpu().numpy(), inv_ref) <= 1e-5
    assert max_abs_over_rms(h.cpu().numpy(), h_ref) <= 2e-4
    assert max_abs_over_rms(h.cpu().numpy(), h_exact) <= 1e-2
    if inject:
        assert max_abs_over_rms(w_in.cpu().numpy(), w_in_ref) <= 2e-4
    # inv_ready: the same result from an inv the caller already holds, which must not be rewritten
    h2 = torch.full_like(h, float("nan"))
    inv_before = inv.clone()
    K.hc_mix_down_wmma(xd, upload(wd, cuda), T, H, d, r, inject, eps, h2, w_in, inv, ws, act, inv_ready=True)
    assert torch.equal(h2, h) and torch.equal(inv, inv_before)
    # the up half on the GPU's own h and inv
    u = torch.empty((T, d), dtype=dt, device=cuda)
    wu_dev = K.to_chunk_major(upload(wu, cuda))
    ws_up = _ws(K.hc_mix_up_wmma_workspace_bytes(T, H, d, r, bits, wu.G), cuda)
    K.hc_mix_up_wmma(h, wu_dev, xd, torch.from_numpy(norm_w).to(cuda), inv, T, H, d, u, ws_up, act)
    K.check_dense_status("hc_mix_up_wmma")
    u_ref = oracle.hc_mix_up(h.cpu().numpy(), wu, x, norm_w, inv.cpu().numpy(), H, d, f16_operands=True)
    u_exact = oracle.hc_mix_up(h.cpu().numpy(), wu, x, norm_w, inv.cpu().numpy(), H, d)
    if dt == torch.float32:
        assert max_abs_over_rms(u.cpu().numpy(), u_ref) <= 2e-4
        assert max_abs_over_rms(u.cpu().numpy(), u_exact) <= 1e-2
    else:
        got = oracle.bf16_to_f32(bits_of(u)).astype(np.float64)
        assert np.all(np.abs(got - u_ref) <= 2.0 ** -8 * np.abs(u_ref) + 2e-4 * np.sqrt(np.mean(u_ref ** 2)))  # one BF16 rounding
    # and the tensor-core mix agrees with the per-token kernels of the same library
    u_pt = torch.empty_like(u)
    K.hc_mix_up(h, wu_dev, xd, torch.from_numpy(norm_w).to(cuda), inv, T, H, d, u_pt, act)
    # (two roundings to BF16 of values a few times the RMS may differ by one unit in the last place each)
    assert max_abs_over_rms(u.float().cpu().numpy(), u_pt.float().cpu().numpy().astype(np.float64)) <= (5e-2 if dt == torch.bfloat16 else 1e-2)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("T,d", [(1, 64), (37, 2560), (300, 136)])
def test_hc_inject_inv(cuda, oracle, dt, T, d):
    """hc_inject_inv leaves X bit-identical to hc_inject, and inv = 1 / sqrt(mean(stored X_s^2) + eps)."""
    from strixite_b200 import kernels as K
    H, eps = 4, 1e-6
    rng = np.random.default_rng(T + d)
    x = torch.from_numpy(rng.standard_normal((T, H * d)).astype(np.float32)).to(cuda).to(dt)
    y = torch.from_numpy(rng.standard_normal((T, d)).astype(np.float32)).to(cuda).to(dt)
    w_in = torch.from_numpy((rng.random((T, H)) * 2).astype(np.float32)).to(cuda)
    act = K.Act.BF16 if dt == torch.bfloat16 else K.Act.F32
    want = x.clone()
    K.hc_inject(want, w_in, y, T, H, d, act)
    inv = torch.full((T, H), float("nan"), dtype=torch.float32, device=cuda)
    K.hc_inject_inv(x, w_in, y, T, H, d, eps, inv, act)
    torch.cuda.synchronize()
    assert torch.equal(x, want)
    xs = want.double().cpu().numpy().reshape(T, H, d)
    inv_ref = 1.0 / np.sqrt((xs * xs).mean(axis=2) + eps)
    assert max_abs_over_rms(inv.cpu().numpy(), inv_ref) <= 1e-5


def test_hc_mix_wmma_argument_checks(cuda, oracle):
    from strixite_b200 import kernels as K
    rng = np.random.default_rng(2)
    H, d, r, T = 4, 128, 32, 3
    wd = upload(oracle.quantize(random_weights(rng, r + H, H * d), 64, 4), cuda)
    x = torch.zeros((T, H * d), dtype=torch.bfloat16, device=cuda)
    h, w_in, inv = (torch.zeros((T, n), dtype=torch.float32, device=cuda) for n in (r, H, H))
    need = K.hc_wmma_workspace_bytes(T, H, d, r + H, 4, 64)
    with pytest.raises(K.Error, match="workspace of"):
        K.hc_mix_down_wmma(x, wd, T, H, d, r, True, 1e-6, h, w_in, inv, _ws(need - 256, cuda), K.Act.BF16)
    with pytest.raises(K.Error, match="w_in must be given exactly when inject"):
        K.hc_mix_down_wmma(x, wd, T, H, d, r, True, 1e-6, h, None, inv, _ws(need, cuda), K.Act.BF16)
    with pytest.raises(K.Error, match="hc_mix_down_wmma_workspace_bytes: T = 3, H = 4, d = 96"):
        K.hc_wmma_workspace_bytes(T, H, 96, r + H, 4, 32)
    wu = K.to_chunk_major(upload(oracle.quantize(random_weights(rng, H * d, r), 32, 8), cuda))
    u = torch.zeros((T, d), dtype=torch.bfloat16, device=cuda)
    nw = torch.zeros(H * d, dtype=torch.float32, device=cuda)
    with pytest.raises(K.Error, match="workspace of"):
        K.hc_mix_up_wmma(h, wu, x, nw, inv, T, H, d, u, _ws(256, cuda), K.Act.BF16)
    with pytest.raises(K.Error, match="u overlaps"):
        K.hc_mix_up_wmma(h, wu, x, nw, inv, T, H, d, x, _ws(K.hc_mix_up_wmma_workspace_bytes(T, H, d, r, 8, 32), cuda), K.Act.BF16)
