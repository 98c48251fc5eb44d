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


def _numpy_permutation(slot_expert, n_experts):
    """Stable counting sort of the flat (row, slot) pairs by expert; ids outside
    [0, n_experts) are skipped."""
    flat = slot_expert.reshape(-1)
    valid = (flat >= 0) & (flat < n_experts)
    order = np.nonzero(valid)[0]
    order = order[np.argsort(flat[order], kind="stable")]
    offsets = np.zeros(n_experts + 1, np.int64)
    np.add.at(offsets, flat[valid] + 1, 1)
    offsets = np.cumsum(offsets)
    row_of = np.full(flat.shape, -1, np.int64)
    row_of[order] = np.arange(order.size)
    return offsets, order, row_of


@pytest.mark.parametrize("rows,k,e", [(8192, 8, 256), (8192, 1, 256), (8191, 8, 255), (1, 8, 256)])
def test_static_permutation_at_its_limits(pkg, rows, k, e):
    """The largest sizes the fixed scratch takes, against a numpy counting sort; some
    slots empty (-1) and some with ids past the last expert (skipped without a report)."""
    import torch

    rng = np.random.default_rng(rows + k + e)
    slot_expert = rng.integers(-1, e + 3, size=(rows, k)).astype(np.int32)
    slot_weight = rng.random((rows, k), dtype=np.float32)
    dev = torch.device("cuda:0")
    se, sw = torch.from_numpy(slot_expert).to(dev), torch.from_numpy(slot_weight).to(dev)
    offsets = torch.full((e + 1,), -7, dtype=torch.int32, device=dev)
    sorted_row = torch.full((rows * k,), -7, dtype=torch.int32, device=dev)
    sorted_weight = torch.full((rows * k,), -7.0, dtype=torch.float32, device=dev)
    row_of = torch.full((rows * k,), -7, dtype=torch.int32, device=dev)
    for _ in range(2):  # twice in a row: the scratch keeps the first call's contents
        pkg.permute_static(se, sw, rows, k, e, offsets, sorted_row, sorted_weight, row_of,
                           torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    want_off, want_order, want_row_of = _numpy_permutation(slot_expert, e)
    n = int(want_off[-1])
    np.testing.assert_array_equal(offsets.cpu().numpy(), want_off)
    np.testing.assert_array_equal(sorted_row.cpu().numpy()[:n], want_order // k)
    np.testing.assert_array_equal(sorted_weight.cpu().numpy()[:n], slot_weight.reshape(-1)[want_order])
    np.testing.assert_array_equal(row_of.cpu().numpy(), want_row_of)
    assert (sorted_row.cpu().numpy()[n:] == -7).all()


def test_static_permutation_of_nothing(pkg):
    import torch

    dev = torch.device("cuda:0")
    offsets = torch.full((33,), -7, dtype=torch.int32, device=dev)
    pkg.permute_static(None, None, 0, 4, 32, offsets, None, None, None,
                       torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert (offsets.cpu().numpy() == 0).all()


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
