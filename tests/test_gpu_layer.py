"""Whole MoE sublayer on the GPU against the CPU oracle, on the benchmark configurations.

Gate (the acceptance rule of the path): router ids bit-exact given identical FP32 logits; layer output within
max-abs error <= 1e-2 x output RMS of the oracle's FP32 output.  The streaming (exact-product) path is in practice
three orders of magnitude inside that bar; its own, tighter bar is asserted too."""
import numpy as np
import pytest
import torch

from helpers import bits_of, download, max_abs_over_rms, oracle_layer_on_touched_experts

pytestmark = pytest.mark.gpu

TOL = 1e-2  # max |y - y_ref| <= TOL * rms(y_ref), the path's stated tolerance


def run_layer(cfg, seed, dev, math=None):
    from strixite_b200 import workloads as W
    from strixite_b200.layer import MoeBuffers, MoeLayer
    w = W.make_layer_weights(cfg, seed, dev)
    x = W.activations(cfg, seed, dev)
    logits = W.router_logits(x, W.router_weight(cfg, seed, dev), W.expert_bias(cfg, seed, dev))
    buf = MoeBuffers(cfg.T, cfg.d, cfg.I, cfg.E, cfg.k, dev, cfg.shared)
    layer = MoeLayer(w, cfg.E, cfg.k, buf)
    y32 = torch.empty((cfg.T, cfg.d), dtype=torch.float32, device=dev)
    ybf = torch.empty((cfg.T, cfg.d), dtype=torch.bfloat16, device=dev)
    layer.forward(x, logits, y32, math=math)
    layer.forward(x, logits, ybf, math=math)
    torch.cuda.synchronize()
    layer.check_errors(cfg.name)
    return w, x, logits, buf, y32, ybf


@pytest.mark.parametrize("name", ["c0", "c1", "c2"])
def test_layer_streaming_path(cuda, oracle, name):
    from strixite_b200 import workloads as W
    from strixite_b200.kernels import MoeMath
    cfg = W.c2_config(0) if name == "c2" else W.CONFIGS[name]
    w, x, logits, buf, y32, ybf = run_layer(cfg, 0, cuda, math=MoeMath.F32)
    xb, lg = bits_of(x), logits.cpu().numpy()
    ref = oracle_layer_on_touched_experts(oracle, cfg, w, xb, lg, np.arange(cfg.T), "decode")
    assert np.array_equal(buf.ids[: cfg.T].cpu().numpy(), ref["ids"]), "router ids must be bit-exact"
    np.testing.assert_allclose(buf.coef[: cfg.T].cpu().numpy(), ref["coef"], rtol=2e-6)
    # pack offsets: bit-exact against the CPU counting sort of the same ids
    offsets, slots = oracle.moe_group_routes(ref["ids"], cfg.E)
    from strixite_b200 import kernels as K
    L = K.route_layout(cfg.T, cfg.k, cfg.E)
    ws = buf.ws.cpu().numpy()
    assert np.array_equal(ws[L["offsets"]:L["offsets"] + cfg.E + 2], offsets)
    assert np.array_equal(ws[L["slots"]:L["slots"] + cfg.T * cfg.k], slots)
    err = max_abs_over_rms(y32.cpu().numpy(), ref["y_f32"])
    assert err <= TOL, f"{cfg.name}: max-abs error {err:.3e} x RMS exceeds the path's tolerance {TOL}"
    assert err <= 2e-3, f"{cfg.name}: the exact-product path should be far inside the tolerance, got {err:.3e}"
    # BF16 output: the reference's roundings (s, y, y + g s) of almost the same FP32 values - equal except where one of
    # them sits on a rounding boundary, which moves y by at most one BF16 ulp of y plus one of s
    got, want = oracle.bf16_to_f32(bits_of(ybf)).astype(np.float64), oracle.bf16_to_f32(ref["y_bf16"]).astype(np.float64)
    s_mag = np.abs(oracle.bf16_to_f32(ref["shared_s"])) if "shared_s" in ref else 0.0
    bound = 1.5 * 2.0 ** -7 * (np.abs(want) + np.abs(ref["y_routed_f32"]) + s_mag) + 5e-4 * np.sqrt(np.mean(want ** 2))
    worst = float(np.max(np.abs(got - want) - bound))
    assert worst <= 0, f"{cfg.name}: a BF16 output is {worst:.3e} beyond the rounding bound"
    assert (bits_of(ybf) != ref["y_bf16"]).mean() < 0.05


def test_layer_rows_do_not_depend_on_batch(cuda):
    """A conversation's rows give the same outputs alone or packed with others (runtime/qwen4exp.hpp:804-809:
    a batch of one equals forward())."""
    from strixite_b200 import workloads as W
    from strixite_b200.kernels import MoeMath
    from strixite_b200.layer import MoeBuffers, MoeLayer
    cfg = W.c2_config(0)
    w = W.make_layer_weights(cfg, 0, cuda)
    x = W.activations(cfg, 0, cuda)
    logits = W.router_logits(x, W.router_weight(cfg, 0, cuda), W.expert_bias(cfg, 0, cuda))
    layer = MoeLayer(w, cfg.E, cfg.k, MoeBuffers(cfg.T, cfg.d, cfg.I, cfg.E, cfg.k, cuda, cfg.shared))
    y_all = torch.empty((cfg.T, cfg.d), dtype=torch.float32, device=cuda)
    layer.forward(x, logits, y_all, math=MoeMath.F32)
    start = 0
    for n in cfg.runs[:3]:
        y_run = torch.empty((n, cfg.d), dtype=torch.float32, device=cuda)
        layer.forward(x[start:start + n].contiguous(), logits[start:start + n].contiguous(), y_run, math=MoeMath.F32)
        torch.cuda.synchronize()
        assert torch.equal(y_run, y_all[start:start + n])
        start += n


def edge_rows(buf, cfg):
    """Token rows that sit at the edges of the pack: the first and the last slot of the fullest and of the emptiest
    non-empty expert, and the first slot of a partly filled 128-slot tile."""
    from strixite_b200 import kernels as K
    L = K.route_layout(cfg.T, cfg.k, cfg.E)
    ws = buf.ws.cpu().numpy()
    off = ws[L["offsets"]:L["offsets"] + cfg.E + 2].astype(np.int64)
    slots = ws[L["slots"]:L["slots"] + cfg.T * cfg.k]
    cnt = np.diff(off)[: cfg.E]
    live = np.nonzero(cnt)[0]
    hot, cold = live[np.argmax(cnt[live])], live[np.argmin(cnt[live])]
    pos = [off[hot], off[hot + 1] - 1, off[cold], off[cold + 1] - 1]
    ragged = [e for e in live if cnt[e] % 128 != 0 and cnt[e] > 128]
    if ragged:
        e = ragged[0]
        pos += [off[e] + (cnt[e] // 128) * 128, off[e + 1] - 1]
    return sorted({int(slots[p]) // cfg.k for p in pos}), int(cnt[hot]), int(cnt[cold])


def tc_layer_case(cuda, oracle, cfg, n_check, seed=0, math=None):
    """Runs the layer on the tcgen05 path and checks `n_check` seeded token rows - the pack's edge rows among them -
    against the oracle's matrix-unit semantics (rows are independent, so a subset is a valid check of the full-size
    run).  Returns (error vs the reference's numerics, error vs the FP32-partials variant, the two variants' distance)."""
    from strixite_b200.kernels import MoeMath
    math = MoeMath.WmmaF16F32Partials if math is None else math
    w, x, logits, buf, y32, ybf = run_layer(cfg, seed, cuda, math=math)
    edges, hot, cold = edge_rows(buf, cfg)
    rnd = [int(r) for r in np.random.default_rng(seed).permutation(cfg.T) if int(r) not in set(edges)]
    rows = np.array(sorted(edges + rnd[: max(0, min(n_check, cfg.T) - len(edges))]))
    xb, lg = bits_of(x), logits.cpu().numpy()
    ref = oracle_layer_on_touched_experts(oracle, cfg, w, xb, lg, rows, "grouped")
    alt = oracle_layer_on_touched_experts(oracle, cfg, w, xb, lg, rows, "grouped_f32_partials")
    assert np.array_equal(buf.ids.cpu().numpy()[rows], ref["ids"]), "router ids must be bit-exact"
    got = y32.cpu().numpy()[rows]
    err_ref, err_alt = max_abs_over_rms(got, ref["y_f32"]), max_abs_over_rms(got, alt["y_f32"])
    dist = max_abs_over_rms(ref["y_f32"], alt["y_f32"])
    print(f"{cfg.name} {math.name}: {len(rows)} rows (fullest expert {hot} slots, emptiest {cold}); max-abs error / RMS "
          f"{err_ref:.3e} vs the reference's numerics (BF16 per-slot dots), {err_alt:.3e} vs FP32 per-slot dots; "
          f"the two oracle variants differ by {dist:.3e}")
    if math == MoeMath.WmmaF16F32Partials:
        assert err_alt <= TOL, f"{cfg.name}: max-abs error {err_alt:.3e} x RMS exceeds the path's tolerance {TOL}"
    else:
        # BF16 per-slot dots: a dot that falls the other side of a rounding boundary than the oracle's (FP32 against float64
        # accumulation) moves y by coef x one BF16 ulp of the dot; the rounding itself is `dist` away from FP32 dots
        assert err_ref <= 5 * TOL, f"{cfg.name}: max-abs error {err_ref:.3e} x RMS with BF16 per-slot dots"
    return err_ref, err_alt, dist


def test_layer_tcgen05_small(cuda, oracle):
    """C0's layer (Q8 experts, no shared expert) with enough tokens for every expert to be hit, all rows checked, both
    forms of the per-slot dots."""
    from dataclasses import replace
    from strixite_b200 import workloads as W
    from strixite_b200.kernels import MoeMath
    cfg = replace(W.C0, T=96, name="c0_t96")
    tc_layer_case(cuda, oracle, cfg, 96)
    tc_layer_case(cuda, oracle, cfg, 96, math=MoeMath.WmmaF16)


def test_layer_tcgen05_c3_prefill(cuda, oracle):
    """C3 at full size (T = 4096, 512 Q4 experts + Q8 shared expert) on the tcgen05 path; 512 rows against the oracle,
    the pack's edge rows among them."""
    from strixite_b200 import workloads as W
    tc_layer_case(cuda, oracle, W.C3, 512)


def test_layer_tcgen05_rows_do_not_depend_on_batch(cuda):
    """A full-size property of the tcgen05 path: rows computed in the big batch (C3, T = 4096) equal, bit for bit, the same
    rows computed as a batch of their own (320 of them: other tiles, other tile fill, same per-row arithmetic)."""
    from strixite_b200 import workloads as W
    from strixite_b200.kernels import MoeMath
    from strixite_b200.layer import MoeBuffers, MoeLayer
    cfg = W.C3
    w = W.make_layer_weights(cfg, 0, cuda)
    x = W.activations(cfg, 0, cuda)
    logits = W.router_logits(x, W.router_weight(cfg, 0, cuda), W.expert_bias(cfg, 0, cuda))
    layer = MoeLayer(w, cfg.E, cfg.k, MoeBuffers(cfg.T, cfg.d, cfg.I, cfg.E, cfg.k, cuda, cfg.shared))
    y_all = torch.empty((cfg.T, cfg.d), dtype=torch.float32, device=cuda)
    layer.forward(x, logits, y_all, math=MoeMath.WmmaF16)
    sel = torch.arange(100, 100 + 320, device=cuda)
    y_sub = torch.empty((320, cfg.d), dtype=torch.float32, device=cuda)
    layer.forward(x[sel].contiguous(), logits[sel].contiguous(), y_sub, math=MoeMath.WmmaF16)
    torch.cuda.synchronize()
    layer.check_errors(cfg.name)
    assert torch.equal(y_sub, y_all[sel])


@pytest.mark.gpu
def test_layer_tcgen05_c4_layer(cuda, oracle):
    """One layer of C4 at full size (T = 16384, Q4 gate/up, Q8 down, Zipf-biased routing: tiles from a few tokens to full)
    on the tcgen05 path; 256 rows against the oracle, the pack's edge rows among them."""
    from strixite_b200 import workloads as W
    from strixite_b200.kernels import MoeMath
    tc_layer_case(cuda, oracle, W.C4, 256)
    tc_layer_case(cuda, oracle, W.C4, 64, math=MoeMath.WmmaF16)


@pytest.mark.gpu
@pytest.mark.parametrize("name,T,tc", [("c0", 96, True), ("c0", 4, False), ("c2", 0, False)])
def test_expert_parallel_shards_add_up(cuda, name, T, tc):
    """The expert-parallel entry points on ONE GPU: every shard of the experts (2 and 4 shards), run with all tokens and the
    full router output, yields its partial rows; their sum is the unsharded layer's output up to FP32 summation order."""
    from dataclasses import replace
    from strixite_b200 import kernels as K, workloads as W
    from strixite_b200.kernels import MoeMath
    from strixite_b200.layer import MoeBuffers, MoeLayer
    cfg = W.CONFIGS[name]
    cfg = replace(cfg, shared=False, **({"T": T} if T else {}))
    math = MoeMath.WmmaF16 if tc else None
    x = W.activations(cfg, 3, cuda)
    logits = W.router_logits(x, W.router_weight(cfg, 3, cuda), W.expert_bias(cfg, 3, cuda))
    # reference: all experts on one rank
    w = W.make_layer_weights(cfg, 3, cuda)
    buf = MoeBuffers(cfg.T, cfg.d, cfg.I, cfg.E, cfg.k, cuda, False)
    full = MoeLayer(w, cfg.E, cfg.k, buf)
    y_ref = torch.empty((cfg.T, cfg.d), dtype=torch.float32, device=cuda)
    full.forward(x, logits, y_ref, math=math)
    torch.cuda.synchronize()
    full.check_errors(cfg.name)
    ids, coef = buf.ids[:cfg.T].clone(), buf.coef[:cfg.T].clone()
    for shards in (2, 4):
        total = torch.zeros_like(y_ref)
        n = cfg.E // shards
        for r in range(shards):
            wl = W.make_layer_weights(cfg, 3, cuda, e_lo=r * n, e_hi=(r + 1) * n)
            bl = MoeBuffers(cfg.T, cfg.d, cfg.I, n, cfg.k, cuda, False)
            bl.ids[:cfg.T].copy_(ids)
            bl.coef[:cfg.T].copy_(coef)
            part = MoeLayer(wl, n, cfg.k, bl, E_total=cfg.E, e_lo=r * n)
            y = torch.empty_like(y_ref)
            part.run_experts(x, cfg.T, y, part.math_for(cfg.T, math), logits)
            torch.cuda.synchronize()
            part.check_errors(f"{cfg.name} shard {r}/{shards}")
            total += y
        scale = y_ref.abs().max().item()
        assert (total - y_ref).abs().max().item() <= 2e-5 * scale, f"{cfg.name}: {shards} shards do not add up to the whole"


@pytest.mark.gpu
@pytest.mark.parametrize("name,T,tc,shared", [("c0", 4, False, False), ("c1", 16, False, True), ("c0", 96, True, False),
                                               ("c2", 0, False, False), ("c1e", 320, True, True)])
def test_one_call_layer_equals_the_launch_sequence(cuda, name, T, tc, shared):
    """sxb_moe_layer (the whole block enqueued by one C call) against the same block issued launcher by launcher:
    the same kernels with the same arguments, so the outputs are bit-identical (BF16 and FP32 outputs)."""
    from dataclasses import replace
    from strixite_b200 import kernels as K, workloads as W
    from strixite_b200.kernels import MoeMath
    from strixite_b200.layer import MoeBuffers, MoeLayer
    cfg = replace(W.C1, E=32, name="c1e") if name == "c1e" else W.CONFIGS[name]
    cfg = replace(cfg, shared=shared, **({"T": T} if T else {}))
    math = MoeMath.WmmaF16 if tc else MoeMath.F32
    x = W.activations(cfg, 5, cuda)
    logits = W.router_logits(x, W.router_weight(cfg, 5, cuda), W.expert_bias(cfg, 5, cuda))
    w = W.make_layer_weights(cfg, 5, cuda)
    buf = MoeBuffers(cfg.T, cfg.d, cfg.I, cfg.E, cfg.k, cuda, shared)
    layer = MoeLayer(w, cfg.E, cfg.k, buf)
    b2 = MoeBuffers(cfg.T, cfg.d, cfg.I, cfg.E, cfg.k, cuda, shared)
    S = cfg.T * cfg.k
    xs = torch.empty((S, cfg.d), dtype=torch.float16, device=cuda) if tc else None
    sh_xs = torch.empty((cfg.T, cfg.d), dtype=torch.float16, device=cuda) if (tc and shared) else None
    for dt in (torch.float32, torch.bfloat16):
        want = torch.empty((cfg.T, cfg.d), dtype=dt, device=cuda)
        got = torch.empty_like(want)
        layer.forward(x, logits, want, math=math)
        extra = {}
        if shared:
            extra = dict(shared_gate_up=w.shared_gate_up, shared_down=w.shared_down, sh_gu=b2.sh_gu, sh_h=b2.sh_h,
                         sh_y=b2.sh_y32 if dt == torch.float32 else b2.sh_y, sh_xs=sh_xs)
        K.moe_layer(x, logits, got, w.gate_up, w.down, cfg.E, cfg.k, b2.ids, b2.coef, b2.ws, b2.ws_bytes, b2.h, b2.partial,
                    b2.router_err, b2.expert_err, xs=xs, math=math, **extra)
        torch.cuda.synchronize()
        K.check_router_error(b2.router_err, cfg.name)
        K.check_expert_error(b2.expert_err, cfg.name)
        assert torch.equal(b2.ids, buf.ids)
        assert torch.equal(got.view(torch.int32 if dt == torch.float32 else torch.int16),
                           want.view(torch.int32 if dt == torch.float32 else torch.int16)), f"{cfg.name} {dt}"
