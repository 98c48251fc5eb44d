"""MXFP4 expert weights: packed e2m1 codes + e8m0 scales stay packed in HBM and are
expanded to bf16 inside the GEMM's load path.  The CPU oracle is fed the bf16
dequantisation of the same weights (exact: every e2m1 value times a power of two
is a bf16 number), as the reference's exporter does
(export_model_bin/gpt-oss-120b/export_model_bin.py:100-137).
"""
import numpy as np
import pytest

import helpers
from gpt_oss_b200 import synth

pytestmark = pytest.mark.gpu


def _case(pkg, oracle, T, H, IM, E, K, inactive=0, on_device=False, scale_range=(119, 123), seed=0,
          input_scale=0.25, mx_tmem=None):
    import torch

    shape = synth.MoeShape("mx", T, H, IM, E, K, 7.0, 500 + seed)
    d = synth.make_layer(shape, inactive_every=inactive)
    rng = np.random.default_rng(900 + seed)
    b1, s1 = synth.mxfp4_random(rng, (E, 2 * IM), H, *scale_range)
    b2, s2 = synth.mxfp4_random(rng, (E, H), IM, *scale_range)
    d["w_mlp1"] = synth.mxfp4_dequant(b1, s1)
    d["w_mlp2"] = synth.mxfp4_dequant(b2, s2)
    # N(0,1) inputs against weights of magnitude up to 6 * 2^-4 make huge activations;
    # scale the inputs so pre-activations stay around the clamp
    d["t"] = synth.bf16_round(d["t"] * np.float32(input_scale))
    want = oracle.moe_layer(d, shape)

    dev = torch.device("cuda:0")
    eng = pkg.MoeEngine(H, IM, E, K, max_tokens=max(T, 1), weight_format=pkg.WEIGHTS_MXFP4)
    try:
        wr = synth.bf16_bits(d["w_router"])
        args = [wr, d["b_router"], b1, s1, d["b_mlp1"], b2, s2, d["b_mlp2"]]
        if on_device:
            keep = [torch.from_numpy(np.ascontiguousarray(a).view(np.int16) if a.dtype == np.uint16
                                     else np.ascontiguousarray(a)).to(dev) for a in args]
            eng.load_layer_mxfp4(0, *keep, on_device=True)
        else:
            eng.load_layer_mxfp4(0, *[np.ascontiguousarray(a) for a in args], on_device=False)
        with pytest.raises(pkg.MoeError):
            eng.set_option("gemm_impl", pkg.GEMM_TCGEN05)
        if mx_tmem is not None:
            eng.set_option("mx_tmem", mx_tmem)
        t = helpers.to_dev_bf16(d["t"], dev)
        x = helpers.to_dev_bf16(np.zeros_like(d["x"]), dev)
        pos = torch.from_numpy(d["pos"]).to(dev)
        eng.forward(0, t, x, pos, T, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert eng.device_status() == 0
        got = x.float().cpu().numpy()
        r = eng.get_routing(T)
    finally:
        eng.close()
    active = d["pos"] >= 0
    np.testing.assert_array_equal(r["topk_i"][active], want["topk_i"][active])
    # block output (zero residual); its magnitude here is larger than in the bf16 cases, so
    # the absolute limit is the stated 2e-2 scaled to it (the stated figure goes with outputs
    # of std 0.6)
    scale = max(1.0, float(want["e_agg"][active].std()) / 0.6)
    helpers.check_activations(got[active], want["e_agg"][active], "mxfp4 block output",
                              max_abs=helpers.MAX_ABS * scale, mean_rel=helpers.MEAN_REL)
    assert (got[~active] == 0).all()


@pytest.mark.parametrize("T,H,IM,E,K,inactive", [
    (200, 256, 192, 8, 4, 7),
    (64, 96, 160, 8, 2, 0),       # K tails: 96 and 160 are not multiples of the 64-deep K block
    (300, 128, 64, 16, 4, 0),     # down weights: 128 rows = half a CTA pair
    (40, 2880, 2880, 4, 2, 0),    # the real hidden sizes (23 / 12 weight-row pairs, 45 K blocks)
])
def test_mxfp4_layer_against_oracle(pkg, oracle, T, H, IM, E, K, inactive):
    _case(pkg, oracle, T, H, IM, E, K, inactive)


@pytest.mark.parametrize("T,H,IM,E,K", [
    (64, 96, 160, 8, 2),
    (40, 2880, 2880, 4, 2),
])
def test_mxfp4_decode_tiles_expanded_into_shared_memory(pkg, oracle, T, H, IM, E, K):
    # decode-sized batches expand the weights into tensor memory, three K blocks per pipeline
    # stage, by default (every other case of this file); the variant with one K block per
    # stage and the weights expanded into the shared-memory operand ring stays selectable
    _case(pkg, oracle, T, H, IM, E, K, mx_tmem=0)


def test_mxfp4_device_side_upload_and_all_scale_codes(pkg, oracle):
    # scales over a wide range, including small exponents whose values are bf16 subnormals' neighbours
    _case(pkg, oracle, 100, 128, 96, 8, 4, on_device=True, scale_range=(110, 126), seed=3)


def test_mxfp4_scales_above_one(pkg, oracle):
    # block scales up to 2^4 (e8m0 131): weights up to 96, past the exponent one bf16 multiply
    # of the expansion can carry; inputs scaled down to keep the pre-activations near the clamp
    _case(pkg, oracle, 96, 128, 96, 8, 4, scale_range=(125, 131), seed=5, input_scale=2.0 ** -8)
    _case(pkg, oracle, 96, 128, 96, 8, 4, scale_range=(125, 131), seed=5, input_scale=2.0 ** -8,
          mx_tmem=0)
