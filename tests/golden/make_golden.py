"""Generates tests/golden/moe_golden.npz.  Run in a container that has the reference checkout:

    make -C oracle all ref REF=<reference checkout> && python tests/golden/make_golden.py

Quantizer known answers come from the REFERENCE's own formats/q4.cpp / formats/q8.cpp (compiled unchanged by
oracle/Makefile); router, pack and layer vectors come from the oracle (the reference ships no CPU code and no vectors
for those), so they pin the oracle against regressions rather than against the reference.
"""
import pathlib
import sys

import numpy as np

ROOT = pathlib.Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
from oracle import cpu  # noqa: E402


def quant_cases(rng):
    out = {}
    for bits, G in [(4, 128), (4, 64), (4, 32), (8, 128), (8, 64), (8, 32)]:
        N, K = 10, 256
        w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
        w[1, :] = 0.0137                                   # constant row: scale 0, every code 0
        w[2, :] = np.linspace(-1.0, 1.0, K)                # ramp: exercises every code and half-way cases
        w[3, :] = (rng.standard_normal(K) * 300).astype(np.float32)   # large magnitudes
        w[4, :] = (rng.standard_normal(K) * 1e-30).astype(np.float32)  # tiny magnitudes
        w[5, :G] = np.arange(G) % 2                        # two-valued group
        w[6, :] = np.round(rng.standard_normal(K) * 4) / 8  # many exact ties
        w[7, 0] = -0.0
        r = cpu.ref_quantize(w, G, bits)
        tag = f"q{bits}g{G}"
        out[f"{tag}.w"] = w
        out[f"{tag}.q"] = r.q
        out[f"{tag}.scale"] = r.scale
        out[f"{tag}.minv"] = r.minv
        out[f"{tag}.deq"] = cpu.ref_dequantize(r)
    return out


def router_cases(rng):
    E, k, M = 64, 4, 12
    logits = (rng.standard_normal((M, E + 1))).astype(np.float32)
    logits[1, :E] = 0.25                     # all tied: picks 0, 1, 2, 3
    logits[2, 10] = logits[2, 40] = 9.0      # a tie for first place
    logits[3, :E] = np.where(np.arange(E) % 2 == 0, 0.0, -0.0)  # +0 / -0 compare equal
    logits[4, 5] = 80.0                      # one dominant logit: softmax underflows the rest
    logits[5, :E] = -1e30
    logits[5, 63] = -1e29
    ids, coef = cpu.moe_router(logits, E, k)
    ids_s, coef_s = cpu.moe_router(logits, E, k, shared_logit=np.ascontiguousarray(logits[:, E:]), shared_ld=1,
                                   shared_id=E)
    return {"router.logits": logits, "router.ids": ids, "router.coef": coef, "router.ids_shared": ids_s,
            "router.coef_shared": coef_s}


def pack_cases(rng):
    E, M, A = 16, 40, 4
    ids = rng.integers(0, E, size=(M, A)).astype(np.int32)
    ids[3, 1] = -1
    ids[7, 2] = E + 5
    ids[20:30, 0] = 2  # a hot expert
    err = np.zeros(3, dtype=np.uint32)
    offsets, slots = cpu.moe_group_routes(ids, E, err)
    return {"pack.ids": ids, "pack.offsets": offsets, "pack.slots": slots, "pack.err": err}


def layer_case(rng):
    """A miniature layer: E=4, d=128, I=64, top-2, T=5; gate/up Q4 G64, down Q8 G32, shared expert Q8 G64."""
    E, d, I, k, T = 4, 128, 64, 2, 5
    x = cpu.f32_to_bf16(rng.standard_normal((T, d)).astype(np.float32))
    wr = (rng.standard_normal((E + 1, d)) * 0.02).astype(np.float32)
    logits = (cpu.bf16_to_f32(x) @ wr.T).astype(np.float32)
    gu = cpu.ref_quantize((rng.standard_normal((E * 2 * I, d)) * 0.02).astype(np.float32), 64, 4)
    dn = cpu.ref_quantize((rng.standard_normal((E * d, I)) * 0.02).astype(np.float32), 32, 8)
    sgu = cpu.ref_quantize((rng.standard_normal((2 * I, d)) * 0.02).astype(np.float32), 64, 8)
    sdn = cpu.ref_quantize((rng.standard_normal((d, I)) * 0.02).astype(np.float32), 64, 8)
    out = {"layer.x": x, "layer.logits": logits}
    for name, w in [("gu", gu), ("dn", dn), ("sgu", sgu), ("sdn", sdn)]:
        out[f"layer.{name}.q"], out[f"layer.{name}.scale"], out[f"layer.{name}.minv"] = w.q, w.scale, w.minv
    for sem in ("decode", "grouped", "grouped_f32_partials"):
        r = cpu.moe_layer(x, logits, cpu.LayerWeights(gu, dn, sgu, sdn), E, k, semantics=sem, threads=1)
        out[f"layer.{sem}.ids"], out[f"layer.{sem}.coef"] = r["ids"], r["coef"]
        out[f"layer.{sem}.h"], out[f"layer.{sem}.y_f32"], out[f"layer.{sem}.y_bf16"] = r["h"], r["y_f32"], r["y_bf16"]
    return out


def main():
    cpu.build()
    if cpu.ref_lib() is None:
        raise SystemExit("the reference quantizers are not built: make -C oracle ref REF=<reference checkout>")
    rng = np.random.default_rng(20261125)
    data = {}
    data.update(quant_cases(rng))
    data.update(router_cases(rng))
    data.update(pack_cases(rng))
    data.update(layer_case(rng))
    path = pathlib.Path(__file__).resolve().parent / "moe_golden.npz"
    np.savez_compressed(path, **data)
    print(path, path.stat().st_size, "bytes,", len(data), "arrays")


if __name__ == "__main__":
    main()
