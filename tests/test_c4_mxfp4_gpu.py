"""Config 4 of the benchmark description, as stated: the 120b-shape layer (128 experts,
top-4, hidden = intermediate = 2880) with MXFP4 expert weights (e2m1 codes uniform over
the 16 values, e8m0 scales uniform in 2^-8 .. 2^-4), decode batches T = 64 / 256 / 1024,
router biased so that expert popularity follows Zipf(1.1) over a seeded permutation.

The inputs are drawn by the same function the benchmark uses (bench.c4_layer).  Checked:
the router on every token against the oracle's router; 32 seeded tokens end to end
against the oracle fed the bf16 dequantisation of the same weights (what the reference's
exporter stores, export_model_bin/gpt-oss-120b/export_model_bin.py:100-137).  Only the
experts those tokens use are dequantised for the oracle; the others stay zero pages.

Tolerance: expert indices exact (1e-6 tie exemption); block output (zero residual)
max-abs <= 2e-2 * (output std / 0.6), mean-rel <= 1e-2.  The absolute limit is the stated
2e-2 scaled to the output magnitude of this configuration: the stated figure belongs to
outputs of std 0.6 (bf16 weights N(0, 0.02)), while these weights have an rms of 0.094
and give outputs of std ~3, whose bf16 output format alone rounds by up to 0.03.

A last case has more than 128 rows per expert on average, which selects the wide-tile
instantiation of the MXFP4 kernel (token tiles of up to 256) instead of the decode one.
"""
import ctypes

import numpy as np
import pytest

import helpers
from gpt_oss_b200 import synth

pytestmark = pytest.mark.gpu

N_SAMPLE = 32


def _dequant_expert(codes_e, scales_e):
    """[rows, k/2] packed codes + [rows, k/32] scales of one expert (CUDA tensors) -> float32
    numpy [rows, k]; exact (every value is a bf16 number)."""
    import torch

    lut = torch.tensor(synth.E2M1_VALUES, device=codes_e.device)
    lo = lut[(codes_e & 15).long()]
    hi = lut[(codes_e >> 4).long()]
    vals = torch.stack([lo, hi], dim=-1).reshape(codes_e.shape[0], -1)
    s = torch.exp2(scales_e.float() - 127.0).repeat_interleave(32, dim=1)
    return (vals * s).cpu().numpy()


def _oracle_router(oracle, t, pos, w_router, b_router, K):
    T, H = t.shape
    E = w_router.shape[0]
    lib = ctypes.CDLL(str(oracle.ORACLE_LIB))
    fp, ip = ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_int)
    lg = np.zeros((T, E), np.float32)
    ti = np.full((T, K), -1, np.int32)
    tv = np.zeros((T, K), np.float32)
    lib.oracle_router.argtypes = [fp, ip] + [ctypes.c_int] * 4 + [fp, fp, fp, ip, fp]
    rc = lib.oracle_router(t.ctypes.data_as(fp), pos.ctypes.data_as(ip), T, H, E, K,
                           w_router.ctypes.data_as(fp), b_router.ctypes.data_as(fp),
                           lg.ctypes.data_as(fp), ti.ctypes.data_as(ip), tv.ctypes.data_as(fp))
    assert rc == 0
    return lg, ti, tv


def _check_case(pkg, oracle, case, T, n_sample):
    import torch

    eng, w = case["engine"], case["weights"]
    H, IM, E, K = case["H"], case["IM"], case["E"], case["K"]
    dev = w["w_router"].device
    g = torch.Generator(device=dev)
    g.manual_seed(40 + T)
    import bench

    t, _ = bench.c4_tokens(T, H, g, dev)
    x = torch.zeros((T, H), dtype=torch.bfloat16, device=dev)  # zero residual: the block's output
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    pos[7::31] = -1
    eng.forward(0, t, x, pos, T, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert eng.device_status() == 0
    got = x.float().cpu().numpy()
    r = eng.get_routing(T)
    t_h, pos_h = t.float().cpu().numpy(), pos.cpu().numpy()
    active = pos_h >= 0
    w_router = w["w_router"].float().cpu().numpy()
    b_router = w["b_router"].cpu().numpy()
    # router on every token
    lg, ti, tv = _oracle_router(oracle, t_h, pos_h, w_router, b_router, K)
    helpers.check_indices(r["topk_i"], ti, lg, active)
    same = (r["topk_i"] == ti).all(axis=1) & active
    np.testing.assert_allclose(r["topk_v"][same], tv[same], rtol=0, atol=3e-5)
    assert (r["topk_i"][~active] == -1).all() and (got[~active] == 0).all()
    # the skew is there: the most popular expert gets several times the mean share
    counts = np.bincount(ti[ti >= 0], minlength=E)
    if E >= 64 and T >= 256:
        assert counts.max() > 4 * counts.mean()
    # a seeded sample end to end
    rng = np.random.default_rng(T)
    idx = np.sort(rng.choice(np.nonzero(active)[0], min(n_sample, int(active.sum())), replace=False))
    used = np.unique(ti[idx])
    w1 = np.zeros((E, 2 * IM, H), np.float32)  # untouched experts: never committed pages
    w2 = np.zeros((E, H, IM), np.float32)
    for e in used:
        w1[e] = _dequant_expert(w["w1_codes"][e], w["w1_scales"][e])
        w2[e] = _dequant_expert(w["w2_codes"][e], w["w2_scales"][e])
    d = {"t": t_h[idx], "x": np.zeros((idx.size, H), np.float32), "pos": None,
         "w_router": w_router, "b_router": b_router, "w_mlp1": w1,
         "b_mlp1": w["b_mlp1"].cpu().numpy(), "w_mlp2": w2, "b_mlp2": w["b_mlp2"].cpu().numpy()}
    want = oracle.moe_layer(d, synth.MoeShape("c4", idx.size, H, IM, E, K, 7.0, 0))
    np.testing.assert_array_equal(want["topk_i"], ti[idx])
    scale = max(1.0, float(want["e_agg"].std()) / 0.6)
    m_abs, m_rel = helpers.check_activations(got[idx], want["e_agg"], f"c4 T={T} block output",
                                             max_abs=helpers.MAX_ABS * scale,
                                             mean_rel=helpers.MEAN_REL)
    print(f"c4 T={T}: experts touched {int((counts > 0).sum())}, output std "
          f"{want['e_agg'].std():.2f}, max_abs {m_abs:.3e} (limit {helpers.MAX_ABS * scale:.3e}), "
          f"mean_rel {m_rel:.3e}")


def test_config4_as_stated(pkg, oracle):
    import torch

    import bench

    case = bench.c4_layer(pkg, torch.device("cuda:0"), max_tokens=1024)
    try:
        for T in (64, 256, 1024):
            _check_case(pkg, oracle, case, T, N_SAMPLE)
    finally:
        case["engine"].close()


def test_mxfp4_wide_token_tiles(pkg, oracle):
    """More than 128 rows per expert on average: token tiles of up to 256."""
    import torch

    import bench

    case = bench.c4_layer(pkg, torch.device("cuda:0"), max_tokens=1200, n_experts=8)
    try:
        assert 1200 * 4 > 128 * 8
        _check_case(pkg, oracle, case, 1200, 24)
    finally:
        case["engine"].close()
