"""gptoss_moe_permute_static: the permutation stage for hosts that cannot allocate.

Some callers of this library must not call cudaMalloc: an engine that has already
handed all free HBM to its own pool, or a serving loop that cannot take the
device-wide synchronisation an allocation implies.  For them the library offers
the per-expert counting sort with its scratch in a fixed array inside the
library image.  This test drives it through the C ABI and compares it with what
the ordinary, handle-based permutation (gptoss_moe_permute) produced for the
same routing, on two calls in a row - the second one smaller than the first, so
anything the first call left in the shared scratch would show.

The file name sorts last on purpose: if this extra entry point breaks, a run that
stops at the first failure has already run every other test.
"""
import numpy as np
import pytest

import helpers
from gpt_oss_b200 import synth

pytestmark = pytest.mark.gpu


def _one_call(pkg, shape, inactive_every):
    import torch

    d = synth.make_layer(shape, inactive_every=inactive_every)
    # existing entry points: route + permute inside the engine, read back through the taps
    want = helpers.run_gpu_layer(pkg, shape, d)["routing"]
    T, K, E = shape.n_tokens, shape.experts_per_token, shape.n_experts
    dev = torch.device("cuda:0")
    slot_expert = torch.from_numpy(want["topk_i"]).to(dev)
    slot_weight = torch.from_numpy(want["topk_v"]).to(dev)
    offsets = torch.full((E + 1,), -7, dtype=torch.int32, device=dev)
    sorted_row = torch.full((T * K,), -7, dtype=torch.int32, device=dev)
    sorted_weight = torch.full((T * K,), -7.0, dtype=torch.float32, device=dev)
    row_of = torch.full((T * K,), -7, dtype=torch.int32, device=dev)
    pkg.permute_static(slot_expert, slot_weight, T, K, E, offsets, sorted_row, sorted_weight,
                       row_of, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    offsets, sorted_row = offsets.cpu().numpy(), sorted_row.cpu().numpy()
    sorted_weight, row_of = sorted_weight.cpu().numpy(), row_of.cpu().numpy().reshape(T, K)

    n = int(want["expert_offsets"][-1])
    np.testing.assert_array_equal(offsets, want["expert_offsets"])          # integers: exact
    np.testing.assert_array_equal(sorted_row[:n], want["sorted_token"])
    assert (sorted_row[n:] == -7).all(), "nothing may be written past the last assignment"
    # inverse map and weights: slot (row, k) sits at row_of[row, k] in sorted order
    valid = want["topk_i"] >= 0
    assert (row_of[~valid] == -1).all()
    rows, ks = np.nonzero(valid)
    dst = row_of[rows, ks]
    assert sorted(dst.tolist()) == list(range(n))
    np.testing.assert_array_equal(sorted_row[dst], rows)
    np.testing.assert_array_equal(sorted_weight[dst], want["topk_v"][rows, ks])  # copied bits
    e_of_dst = np.searchsorted(offsets, dst, side="right") - 1
    np.testing.assert_array_equal(e_of_dst, want["topk_i"][rows, ks])


def test_static_permutation_matches_engine_permutation_twice(pkg):
    _one_call(pkg, synth.MoeShape("static_big", 1000, 128, 64, 32, 4, 7.0, 51), inactive_every=9)
    _one_call(pkg, synth.MoeShape("static_small", 300, 128, 64, 8, 2, 7.0, 52), inactive_every=0)


def test_static_permutation_rejects_sizes_beyond_its_scratch(pkg):
    import torch

    dev = torch.device("cuda:0")
    buf = torch.zeros(16, dtype=torch.int32, device=dev)
    fbuf = torch.zeros(16, dtype=torch.float32, device=dev)
    for rows, k, e in ((8193, 4, 32), (128, 4, 257), (128, 9, 32)):
        with pytest.raises(pkg.MoeError) as ei:
            pkg.permute_static(buf, fbuf, rows, k, e, buf, buf, fbuf, buf)
        assert ei.value.code == pkg.GPTOSS_E_CAPACITY
        assert "8192 rows" in str(ei.value)
