"""The CPU oracle (C restatement) against the reference's own outputs.

The fixtures under tests/golden/ were produced by the reference's compiled CPU
code (see tests/golden/make_golden.py).  The restatement must reproduce them bit
for bit: both sum exact float products in double in the same order.
"""
import numpy as np
import pytest

import helpers


@pytest.mark.parametrize("name", helpers.GOLDEN_CASES)
def test_oracle_matches_reference_fixture(oracle, name):
    shape, d, ref = helpers.load_golden(name)
    got = oracle.moe_layer(d, shape, which="oracle")
    active = d["pos"] >= 0
    assert active.sum() > 0
    np.testing.assert_array_equal(got["logits"][active], ref["logits"][active])
    # reference tie order is unspecified (qsort); fixtures hold no exact ties
    np.testing.assert_array_equal(got["topk_i"][active], ref["topk_i"][active])
    np.testing.assert_array_equal(got["topk_v"][active], ref["topk_v"][active])
    np.testing.assert_array_equal(got["e_agg"][active], ref["e_agg"][active])
    np.testing.assert_array_equal(got["x_out"], ref["x_out"])
    # inactive rows keep their residual
    np.testing.assert_array_equal(got["x_out"][~active], d["x"][~active])


def test_fixtures_cover_clamp_and_inactive_rows():
    shape, d, ref = helpers.load_golden("layer_e16_k2_big_acts")
    assert shape.experts_per_token == 2 and (d["pos"] < 0).any()
    # with the scaled inputs some pre-activations exceed the clamp on both sides
    t = d["t"][d["pos"] >= 0]
    pre = t @ d["w_mlp1"][int(ref["topk_i"][d["pos"] >= 0][0, 0])].T
    assert (pre > shape.swiglu_limit).any() and (pre < -shape.swiglu_limit).any()


def test_oracle_against_live_reference_if_present(oracle):
    """Where the reference's compiled code is available, compare on a fresh seed too."""
    if not oracle.have_ref():
        pytest.skip("oracle/_ref not built on this machine")
    from gpt_oss_b200 import synth

    shape = synth.MoeShape("live", 10, 96, 48, 16, 4, 7.0, 777)
    d = synth.make_layer(shape, inactive_every=3)
    a = oracle.moe_layer(d, shape, which="oracle")
    b = oracle.moe_layer(d, shape, which="ref")
    for k in ("topk_i", "topk_v", "e_agg", "x_out"):
        np.testing.assert_array_equal(a[k], b[k])
    w = np.abs(synth.bf16_round(np.random.default_rng(0).standard_normal(96).astype(np.float32)))
    np.testing.assert_array_equal(oracle.rmsnorm_rows(d["x"], w, "oracle"),
                                  oracle.rmsnorm_rows(d["x"], w, "ref"))


def test_oracle_tie_break_lowest_index_first(oracle):
    from gpt_oss_b200 import synth

    shape = synth.MoeShape("ties", 4, 32, 16, 8, 4, 7.0, 5)
    d = synth.make_layer(shape)
    d["w_router"][:] = 0.0  # all logits equal the bias
    d["b_router"][:] = 0.25
    got = oracle.moe_layer(d, shape, which="oracle")
    np.testing.assert_array_equal(got["topk_i"], np.tile(np.arange(4, dtype=np.int32), (4, 1)))
    np.testing.assert_allclose(got["topk_v"], 0.25)


def test_bf16_helpers_round_to_nearest_even():
    from gpt_oss_b200 import synth

    a = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.0e-39], np.float32)
    bits = synth.bf16_bits(a)
    back = synth.bf16_to_f32(bits)
    assert back[0] == 1.0 and back[3] == -2.5
    assert back[1] == 1.0            # exactly half way: ties to even mantissa
    assert back[2] == np.float32(1.015625)  # half way, rounds up to the even neighbour
