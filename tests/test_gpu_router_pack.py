"""GPU parity of the router, the shared add and the pack against the CPU oracle, through the C ABI.
Router ids and the whole pack workspace are bit-exact; coefficients differ only by the device's expf (a few ulp)."""
import numpy as np
import pytest
import torch

from helpers import bf16_tensor, bits_of

pytestmark = pytest.mark.gpu


def run_router(K, logits_np, E, k, shared, dev, act_bf16=False):
    M, ld = logits_np.shape
    logits = bf16_tensor(logits_np, dev) if act_bf16 else torch.from_numpy(logits_np).to(dev)
    A = k + (1 if shared else 0)
    ids = torch.full((M, A), -7, dtype=torch.int32, device=dev)
    coef = torch.zeros((M, A), dtype=torch.float32, device=dev)
    err = torch.zeros(4, dtype=torch.int32, device=dev)
    es = 2 if act_bf16 else 4
    sl = logits.data_ptr() + es * E if shared else None
    K.moe_router(logits, ld, M, E, k, sl, ld, E, ids, coef, K.Act.BF16 if act_bf16 else K.Act.F32, err)
    torch.cuda.synchronize()
    return ids.cpu().numpy(), coef.cpu().numpy(), err.cpu().numpy().view(np.uint32)[:3]


def test_router_golden(cuda, oracle, golden):
    from strixite_b200 import kernels as K
    logits = golden["router.logits"]
    ids, coef, err = run_router(K, logits, 64, 4, False, cuda)
    assert np.array_equal(ids, golden["router.ids"]) and err[0] == 0
    np.testing.assert_allclose(coef, golden["router.coef"], rtol=4e-7 * 4, atol=0)
    ids, coef, err = run_router(K, logits, 64, 4, True, cuda)
    assert np.array_equal(ids, golden["router.ids_shared"])
    np.testing.assert_allclose(coef, golden["router.coef_shared"], rtol=2e-6, atol=0)


@pytest.mark.parametrize("M,E,k", [(1, 512, 10), (7, 512, 10), (512, 512, 10), (16, 64, 4), (33, 1024, 32), (5, 1, 1),
                                   (9, 100, 7), (4096, 512, 10)])
def test_router_ids_bit_exact(cuda, oracle, M, E, k):
    """The reference's method: bit for bit at T = 1, 7, 512 (tutorial/first-kernel), plus the limits of E and k."""
    from strixite_b200 import kernels as K
    rng = np.random.default_rng(M * 7919 + E)
    logits = (rng.standard_normal((M, E + 1)) * 1.3).astype(np.float32)
    if M > 3:
        logits[1, : min(E, 40)] = 0.5  # ties
        logits[2] = np.round(logits[2] * 2) / 2  # many ties
    ref_ids, ref_coef = oracle.moe_router(logits, E, k)
    ids, coef, err = run_router(K, logits, E, k, False, cuda)
    assert err[0] == 0
    assert np.array_equal(ids, ref_ids)
    np.testing.assert_allclose(coef, ref_coef, rtol=2e-6, atol=1e-30)
    # BF16 logits (Act.BF16): the same picks as the oracle on the same bits
    lb = oracle.f32_to_bf16(logits)
    ref_ids_b, ref_coef_b = oracle.moe_router(lb, E, k)
    ids_b, coef_b, _ = run_router(K, lb, E, k, False, cuda, act_bf16=True)
    assert np.array_equal(ids_b, ref_ids_b)
    np.testing.assert_allclose(coef_b, ref_coef_b, rtol=2e-6, atol=1e-30)


def test_router_mutation_is_caught(cuda, oracle):
    """A deliberately wrong expectation must fail: guards against a comparison that passes vacuously."""
    from strixite_b200 import kernels as K
    rng = np.random.default_rng(3)
    logits = rng.standard_normal((8, 513)).astype(np.float32)
    ref_ids, _ = oracle.moe_router(logits, 512, 10)
    mutated = logits.copy()
    mutated[4, ref_ids[4, 9]] -= 10.0  # token 4's last pick drops out
    ids, _, _ = run_router(K, mutated, 512, 10, False, cuda)
    assert not np.array_equal(ids, ref_ids) and np.array_equal(ids[:4], ref_ids[:4])


def test_router_non_finite(cuda, oracle):
    from strixite_b200 import kernels as K
    rng = np.random.default_rng(5)
    logits = rng.standard_normal((6, 513)).astype(np.float32)
    logits[3, 77] = np.inf
    logits[3, 300] = np.nan
    ids, coef, err = run_router(K, logits, 512, 10, True, cuda)
    assert list(err) == [1, 3, 77]
    assert np.all(ids[3] == -1) and np.all(np.isnan(coef[3]))
    ref_ids, _ = oracle.moe_router(logits, 512, 10, np.ascontiguousarray(logits[:, 512:]), 1, 512)
    assert np.array_equal(ids, ref_ids)
    logits[3, 77] = 0.0
    logits[3, 300] = 0.0
    logits[3, 512] = -np.inf  # the shared gate
    ids, coef, err = run_router(K, logits, 512, 10, True, cuda)
    assert list(err) == [1, 3, 512]
    e = torch.tensor([1, 3, 512, 0], dtype=torch.int32, device=cuda)
    with pytest.raises(K.Error, match="token 3, expert 512"):
        K.check_router_error(e, "test")


@pytest.mark.parametrize("act", ["bf16", "f32"])
def test_shared_add_and_inject(cuda, oracle, act):
    from strixite_b200 import kernels as K
    rng = np.random.default_rng(11)
    M, N, H = 5, 1000, 4
    yf, sf = rng.standard_normal((M, N)).astype(np.float32), rng.standard_normal((M, N)).astype(np.float32)
    xf, w_in = rng.standard_normal((M, H * N)).astype(np.float32), rng.standard_normal((M, H)).astype(np.float32)
    gate = rng.standard_normal((M, 3)).astype(np.float32)
    gate[2, 1] = np.nan
    if act == "bf16":
        y0, s0, x0 = oracle.f32_to_bf16(yf), oracle.f32_to_bf16(sf), oracle.f32_to_bf16(xf)
        up = lambda a: bf16_tensor(a, cuda)
        down = bits_of
        A = K.Act.BF16
    else:
        y0, s0, x0 = yf, sf, xf
        up = lambda a: torch.from_numpy(a).to(cuda)
        down = lambda t: t.cpu().numpy()
        A = K.Act.F32
    g = torch.from_numpy(gate).to(cuda)
    err_ref = np.zeros(3, dtype=np.uint32)
    y_ref = oracle.moe_shared_add(y0, s0, gate[:, 1], 512, err_ref)
    y, s, err = up(y0), up(s0), torch.zeros(4, dtype=torch.int32, device=cuda)
    K.moe_shared_add(y, s, g.data_ptr() + 4, 3, M, N, 512, A, err)
    torch.cuda.synchronize()
    got = down(y)
    ok = [0, 1, 3, 4]
    if act == "bf16":
        assert np.array_equal(got[ok], y_ref[ok])
    else:
        np.testing.assert_allclose(got[ok], y_ref[ok], rtol=3e-7)
    assert np.all(np.isnan(oracle.bf16_to_f32(got[2]) if act == "bf16" else got[2]))
    assert list(err.cpu().numpy().view(np.uint32)[:3]) == [1, 2, 512] == list(err_ref)
    # the fused add + residual injection equals the add then the injection (kernels/moe_router.hpp:56-60)
    y_ref2, x_ref2 = oracle.moe_shared_add_inject(y0, s0, gate[:, 1], 512, x0, w_in)
    y, x, err = up(y0), up(x0), torch.zeros(4, dtype=torch.int32, device=cuda)
    K.moe_shared_add_inject(y, s, g.data_ptr() + 4, 3, M, N, 512, x, torch.from_numpy(w_in).to(cuda), H, A, err)
    torch.cuda.synchronize()
    if act == "bf16":
        assert np.array_equal(down(y)[ok], y_ref2[ok]) and np.array_equal(down(x)[ok], x_ref2[ok])
    else:
        np.testing.assert_allclose(down(x)[ok], x_ref2[ok], rtol=1e-6, atol=1e-6)


def pack_on_gpu(K, ids_np, E, dev, ep=None):
    M, A = ids_np.shape
    ids = torch.from_numpy(ids_np).to(dev)
    nbytes = K.moe_route_workspace_bytes(M, A, E)
    ws = torch.full((nbytes // 4,), -1, dtype=torch.int32, device=dev)
    err = torch.zeros(4, dtype=torch.int32, device=dev)
    if ep is None:
        K.moe_group_routes(ids, M, A, E, ws, nbytes, err)
    else:
        K.moe_group_routes_ep(ids, M, A, ep[0], ep[1], E, ws, nbytes, err)
    torch.cuda.synchronize()
    return ws.cpu().numpy(), err.cpu().numpy().view(np.uint32)[:3], K.route_layout(M, A, E)


def check_tiles(ws, L, offsets, E, rows, n_key, b_key, s_key, skip_last_bucket=False):
    n = int(ws[n_key])
    want_b, want_s = [], []
    for b in range(E + (0 if skip_last_bucket else 1)):
        for s in range(int(offsets[b]), int(offsets[b + 1]), rows):
            want_b.append(b)
            want_s.append(s)
    assert n == len(want_b)
    assert np.array_equal(ws[L[b_key]:L[b_key] + n], np.array(want_b, dtype=np.int32))
    assert np.array_equal(ws[L[s_key]:L[s_key] + n], np.array(want_s, dtype=np.int32))


@pytest.mark.parametrize("M,A,E", [(1, 10, 512), (16, 10, 512), (37, 10, 512), (64, 11, 513), (200, 10, 512),
                                   (205, 10, 512), (4096, 10, 512), (16384, 10, 512), (5, 64, 1023), (3000, 1, 1)])
def test_pack_bit_exact(cuda, oracle, M, A, E):
    """offsets and, thanks to the stable order, slots and the four tile lists equal the CPU counting sort word for word -
    through both the single-CTA path (S <= 2048) and the three-launch path."""
    from strixite_b200 import kernels as K
    rng = np.random.default_rng(M * 31 + A)
    p = 1.0 / np.arange(1, E + 1) ** 1.1
    ids = rng.choice(E, size=(M, A), p=p / p.sum()).astype(np.int32)  # skewed load
    if M * A > 50:
        ids.reshape(-1)[17] = -3
        ids.reshape(-1)[41] = E
    err_ref = np.zeros(3, dtype=np.uint32)
    offsets, slots = oracle.moe_group_routes(ids, E, err_ref)
    ws, err, L = pack_on_gpu(K, ids, E, cuda)
    assert np.array_equal(ws[L["offsets"]:L["offsets"] + E + 2], offsets)
    assert np.array_equal(ws[L["slots"]:L["slots"] + M * A], slots)
    assert list(err) == list(err_ref)
    assert ws[1] == M * A and ws[2] == E and ws[4] == 0
    check_tiles(ws, L, offsets, E, 8, 0, "tile8_bucket", "tile8_start")
    check_tiles(ws, L, offsets, E, 128, 3, "tile128_bucket", "tile128_start")
    for rows in K.TC_TILES:
        check_tiles(ws, L, offsets, E, rows, L[f"tile{rows}_n"], f"tile{rows}_bucket", f"tile{rows}_start")


def test_pack_golden(cuda, golden):
    from strixite_b200 import kernels as K
    ws, err, L = pack_on_gpu(K, golden["pack.ids"], 16, cuda)
    assert np.array_equal(ws[L["offsets"]:L["offsets"] + 18], golden["pack.offsets"])
    assert np.array_equal(ws[L["slots"]:L["slots"] + 160], golden["pack.slots"])
    assert np.array_equal(err, golden["pack.err"])


@pytest.mark.parametrize("M", [16, 1000])
def test_pack_expert_parallel(cuda, oracle, M):
    """Rank view: experts [e_lo, e_lo + E_local) of E_total; everything else lands in the last bucket, untiled."""
    from strixite_b200 import kernels as K
    rng = np.random.default_rng(M)
    E_total, e_lo, E_local, A = 512, 128, 64, 10
    ids = rng.integers(0, E_total, size=(M, A)).astype(np.int32)
    ids[M // 2, 3] = 600  # invalid everywhere
    local = np.where((ids >= e_lo) & (ids < e_lo + E_local), ids - e_lo, E_local).astype(np.int32)
    offsets, slots = oracle.moe_group_routes(local, E_local)
    ws, err, L = pack_on_gpu(K, ids, E_local, cuda, ep=(E_total, e_lo))
    assert np.array_equal(ws[L["offsets"]:L["offsets"] + E_local + 2], offsets)
    assert np.array_equal(ws[L["slots"]:L["slots"] + M * A], slots)
    assert list(err) == [1, 600, (M // 2) * A + 3] and ws[4] == 1
    check_tiles(ws, L, offsets, E_local, 8, 0, "tile8_bucket", "tile8_start", skip_last_bucket=True)
    check_tiles(ws, L, offsets, E_local, 128, 3, "tile128_bucket", "tile128_start", skip_last_bucket=True)
    for rows in K.TC_TILES:
        check_tiles(ws, L, offsets, E_local, rows, L[f"tile{rows}_n"], f"tile{rows}_bucket", f"tile{rows}_start", skip_last_bucket=True)
