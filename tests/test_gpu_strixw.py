"""A strixw file made resident on the GPU (sxb_strixw_load) and its stacked expert tensors cut into the views the MoE
kernels take: the layer computed from the file's bytes equals, bit for bit, the layer computed from the weights the file
was written from."""
import numpy as np
import pytest
import torch

from helpers import download

pytestmark = pytest.mark.gpu


def test_layer_from_a_loaded_file(cuda, oracle, tmp_path):
    from dataclasses import replace
    from oracle import strixw_file as S
    from strixite_b200 import kernels as K, workloads as W
    from strixite_b200.kernels import MoeMath
    from strixite_b200.layer import MoeBuffers, MoeLayer, MoeWeights
    from strixite_b200.strixw import DATA, StrixwFile
    cfg = replace(W.C0, T=40, E=16, name="c0_e16")
    w = W.make_layer_weights(cfg, 7, cuda)
    # the shared expert's gate_up stacked as expert #E (same format as the routed ones); its down kept apart (other format)
    sh_gu = K.quantize(W.expert_weight_f32(cfg, 7, cuda, "shared_gate_up", 0), 64, 8)
    sh_dn = K.quantize(W.expert_weight_f32(cfg, 7, cuda, "shared_down", 0), 32, 4)
    gu, dn, sgu, sdn = (download(v, oracle) for v in (w.gate_up, w.down, sh_gu, sh_dn))
    stacked = oracle.QWeight(np.concatenate([gu.q, sgu.q]), np.concatenate([gu.scale, sgu.scale]), np.concatenate([gu.minv, sgu.minv]),
                             gu.N + sgu.N, gu.K, gu.G, gu.bits)
    router = W.router_weight(cfg, 7, cuda).cpu().numpy()
    path = tmp_path / "layer.strixw"
    size = S.write(path, {"arch": "qwen4_exp"}, [
        S.quantized("layers.0.mlp.experts_gate_up", stacked, cfg.E + 1),
        S.quantized("layers.0.mlp.experts_down", dn, cfg.E),
        S.quantized("layers.0.mlp.shared_down", sdn),
        S.Tensor("layers.0.mlp.router", S.F32, router.shape, {S.DATA: router.tobytes()}),
    ])
    f = StrixwFile(path)
    f.verify(4)
    seconds = f.load(read_threads=4)
    assert seconds > 0 and size > 10e6
    r_gu, s_gu, bits_gu = f.expert_views("layers.0.mlp.experts_gate_up", cfg.E)
    r_dn, s_dn, bits_dn = f.expert_views("layers.0.mlp.experts_down", cfg.E)
    assert bits_gu == 8 and bits_dn == 8 and s_gu is not None and s_dn is None
    assert r_gu.N == cfg.E * 2 * cfg.I and s_gu.N == 2 * cfg.I and r_gu.q % 256 == 0
    v_sdn, bits_sdn = f.qview("layers.0.mlp.shared_down", cfg.d, cfg.I)
    assert bits_sdn == 4
    with pytest.raises(K.Error, match=r"is \[1024, 256\], expected \[1024, 128\]"):
        f.qview("layers.0.mlp.shared_down", cfg.d, 128)
    x = W.activations(cfg, 7, cuda)
    logits = W.router_logits(x, W.router_weight(cfg, 7, cuda), W.expert_bias(cfg, 7, cuda))
    # the router projection straight from the file's FP32 weight on the device: the same bits as from the original tensor
    from strixite_b200 import _lib
    lg_file = torch.empty((cfg.T, cfg.E + 1), dtype=torch.float32, device=cuda)
    lg_orig = torch.empty_like(lg_file)
    rc = _lib.load().sxb_router_logits(x.data_ptr(), f.device_ptr("layers.0.mlp.router", DATA), int(K.Act.F32), None, cfg.T, cfg.E + 1,
                                       cfg.d, lg_file.data_ptr(), cfg.E + 1, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, _lib.load().sxb_last_error().decode()
    K.router_logits(x, W.router_weight(cfg, 7, cuda), None, lg_orig)
    assert torch.equal(lg_file, lg_orig)
    for math in (MoeMath.F32, MoeMath.WmmaF16F32Partials):
        want_w = MoeWeights(w.gate_up, w.down, sh_gu, sh_dn)
        got_w = MoeWeights(K.QRawView(r_gu, bits_gu, f), K.QRawView(r_dn, bits_dn, f), K.QRawView(s_gu, bits_gu, f), K.QRawView(v_sdn, bits_sdn, f))
        ys = []
        for weights in (want_w, got_w):
            layer = MoeLayer(weights, cfg.E, cfg.k, MoeBuffers(cfg.T, cfg.d, cfg.I, cfg.E, cfg.k, cuda, True))
            y = torch.empty((cfg.T, cfg.d), dtype=torch.float32, device=cuda)
            layer.forward(x, logits, y, math=math)
            torch.cuda.synchronize()
            layer.check_errors("strixw layer")
            ys.append(y)
        assert torch.equal(ys[0], ys[1])
    f.close()
