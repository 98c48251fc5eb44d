"""Expert parallelism over peer memory with all ranks on ONE GPU.

The ranks are engines on the same device, wired in-process (gptoss_moe_ep_init_local),
and the layer is driven part by part through one stream - every rank's publish, then
every rank's owner stage, then every rank's combine (gptoss_moe_forward_part) - so no
kernel is launched before the kernels whose flags it polls: the flag waits inside the
kernels always find their flags set.  That is the whole data path of the peer-memory
transport (routing results written into every rank's control block, owners sorting all
ranks' rows and pulling them from the homes' buffers, homes pulling the expert outputs
of their tokens' slots from the owners' buffers),
checked against the CPU oracle on every rank's own tokens, on a box with one GPU.

Also here: a bounded wait that runs out.  One rank runs its owner stage although the
other never published: the kernel gives up after the (shortened) limit, records status
106, the stream drains on mapped memory, and the calls that synchronise report
GPTOSS_E_DEVICE.  Nothing faults or hangs: the wait is bounded by construction.
"""
import numpy as np
import pytest

import helpers
from gpt_oss_b200 import ep_plan, synth

pytestmark = pytest.mark.gpu


def _make_rank_inputs(rank, T, H, seed):
    rng = np.random.default_rng(seed + rank)
    t = synth.bf16_round(rng.standard_normal((T, H)).astype(np.float32))
    x = synth.bf16_round(rng.standard_normal((T, H)).astype(np.float32))
    pos = np.arange(T, dtype=np.int32)
    pos[3::13] = -1
    return t, x, pos


def _engines(pkg, world, H, IM, E, K, max_tokens, weights):
    engs = []
    for r in range(world):
        eng = pkg.MoeEngine(H, IM, E, K, max_tokens=max_tokens, ep_rank=r, ep_size=world, device=0)
        eng.load_layer_f32(0, weights["w_router"], weights["b_router"], weights["w_mlp1"],
                           weights["b_mlp1"], weights["w_mlp2"], weights["b_mlp2"])
        engs.append(eng)
    pkg.MoeEngine.ep_init_local(engs)
    assert all(e.ep_transport == 1 for e in engs)
    return engs


def _layer_in_parts(engs, ts, xs, poss, Ts, stream):
    for part in range(3):
        for eng, t, x, pos, T in zip(engs, ts, xs, poss, Ts):
            eng.forward_part(0, part, t, x, pos, T, stream)


@pytest.mark.parametrize("world,H,IM,E,K,sizes", [
    (2, 128, 64, 8, 4, [[90, 101], [40, 0], [0, 77]]),           # a rank without tokens, both ways
    (4, 256, 192, 32, 4, [[300, 311, 322, 333], [5, 0, 129, 1]]),
    (8, 128, 64, 128, 4, [[64, 70, 1, 128, 0, 33, 90, 17]]),     # 16 experts per rank
])
def test_ranks_on_one_gpu_match_the_oracle(pkg, oracle, world, H, IM, E, K, sizes):
    import torch

    dev = torch.device("cuda:0")
    weights = synth.make_layer(synth.MoeShape("ep", 8, H, IM, E, K, 7.0, 4242))
    max_tokens = max(max(s) for s in sizes)
    engs = _engines(pkg, world, H, IM, E, K, max_tokens, weights)
    stream = torch.cuda.current_stream().cuda_stream
    try:
        for round_no, Ts in enumerate(sizes):  # consecutive layers reuse the published buffers
            ins = [_make_rank_inputs(r, Ts[r], H, 100 * round_no + 7) for r in range(world)]
            ts = [helpers.to_dev_bf16(i[0], dev) for i in ins]
            xs = [helpers.to_dev_bf16(i[1], dev) for i in ins]
            poss = [torch.from_numpy(i[2]).to(dev) for i in ins]
            _layer_in_parts(engs, ts, xs, poss, Ts, stream)
            torch.cuda.synchronize()
            for r, eng in enumerate(engs):
                assert eng.device_status() == 0
                T = Ts[r]
                if T == 0:
                    continue
                t, x, pos = ins[r]
                d = dict(weights)
                d["t"], d["x"], d["pos"] = t, x, pos
                shape = synth.MoeShape("ep", T, H, IM, E, K, 7.0, 0)
                want = oracle.moe_layer(d, shape)
                got = xs[r].float().cpu().numpy()
                active = pos >= 0
                routing = eng.get_routing(T)
                helpers.check_indices(routing["topk_i"], want["topk_i"], want["logits"], active)
                helpers.check_activations(got[active], want["x_out"][active], f"rank {r} x_out",
                                          bf16_quantum=True)
                np.testing.assert_array_equal(got[~active], x[~active])
                # the homes add the same K expert outputs in the same order as one GPU with
                # all experts does; what still differs is the GEMMs' own last bits (an
                # expert's rows share token tiles of other widths with other ranks' rows)
                single = helpers.run_gpu_layer(pkg, shape, d)["x_out"]
                helpers.check_activations(got, single, f"rank {r} vs one GPU", max_abs=4e-2,
                                          mean_rel=1e-3)
                mine = ep_plan.local_expert_slice(E, r, world)
                assert routing["expert_offsets"].shape[0] == len(mine) + 1
    finally:
        torch.cuda.synchronize()
        for eng in engs:
            eng.close()


def test_zero_residual_block_output_under_expert_parallelism(pkg, oracle):
    """The strict bar (max-abs 2e-2, mean-rel 1e-2) on the block's own output, 4 ranks."""
    import torch

    dev = torch.device("cuda:0")
    world, H, IM, E, K, T = 4, 256, 192, 32, 4, 200
    weights = synth.make_layer(synth.MoeShape("ep", 8, H, IM, E, K, 7.0, 999))
    engs = _engines(pkg, world, H, IM, E, K, T, weights)
    stream = torch.cuda.current_stream().cuda_stream
    try:
        ins = [_make_rank_inputs(r, T, H, 31) for r in range(world)]
        ts = [helpers.to_dev_bf16(i[0], dev) for i in ins]
        xs = [torch.zeros((T, H), dtype=torch.bfloat16, device=dev) for _ in ins]
        poss = [torch.from_numpy(i[2]).to(dev) for i in ins]
        _layer_in_parts(engs, ts, xs, poss, [T] * world, stream)
        torch.cuda.synchronize()
        for r in range(world):
            t, _, pos = ins[r]
            d = dict(weights)
            d["t"], d["x"], d["pos"] = t, np.zeros_like(t), pos
            want = oracle.moe_layer(d, synth.MoeShape("ep", T, H, IM, E, K, 7.0, 0))
            active = pos >= 0
            helpers.check_activations(xs[r].float().cpu().numpy()[active], want["e_agg"][active],
                                      f"rank {r} e_agg")
    finally:
        torch.cuda.synchronize()
        for eng in engs:
            eng.close()


def test_pushed_return_and_single_fetch_leave_the_results_unchanged(pkg):
    """The down GEMM storing its rows into the homes' memory (ep_push) and the single fetch of
    a token with several experts on one owner (ep_dedup) move the same bits as the plain
    fetch-everything path."""
    import torch

    dev = torch.device("cuda:0")
    world, H, IM, E, K, T = 4, 256, 192, 16, 4, 150
    weights = synth.make_layer(synth.MoeShape("ep", 8, H, IM, E, K, 7.0, 77))
    engs = _engines(pkg, world, H, IM, E, K, T, weights)
    stream = torch.cuda.current_stream().cuda_stream
    try:
        ins = [_make_rank_inputs(r, T, H, 5) for r in range(world)]
        ts = [helpers.to_dev_bf16(i[0], dev) for i in ins]
        poss = [torch.from_numpy(i[2]).to(dev) for i in ins]
        outs = {}
        for push, dedup in ((1, 1), (0, 0), (1, 0), (0, 1)):
            for eng in engs:
                eng.set_option("ep_push", push)
                eng.set_option("ep_dedup", dedup)
            xs = [helpers.to_dev_bf16(i[1], dev) for i in ins]
            _layer_in_parts(engs, ts, xs, poss, [T] * world, stream)
            torch.cuda.synchronize()
            assert all(e.device_status() == 0 for e in engs)
            outs[(push, dedup)] = [x.cpu() for x in xs]
        for key, got in outs.items():
            for r in range(world):
                assert torch.equal(got[r], outs[(1, 1)][r]), f"options {key}, rank {r}"
    finally:
        torch.cuda.synchronize()
        for eng in engs:
            eng.close()


def test_engines_that_disagree_are_refused(pkg):
    a = pkg.MoeEngine(128, 64, 8, 4, max_tokens=64, ep_rank=0, ep_size=2, device=0)
    b = pkg.MoeEngine(128, 64, 8, 4, max_tokens=96, ep_rank=1, ep_size=2, device=0)
    try:
        with pytest.raises(pkg.MoeError) as ei:
            pkg.MoeEngine.ep_init_local([a, b])
        assert ei.value.code == pkg.GPTOSS_E_INVALID
        assert "different max_tokens" in str(ei.value)
        with pytest.raises(pkg.MoeError):  # ranks out of order
            pkg.MoeEngine.ep_init_local([b, a])
    finally:
        a.close()
        b.close()


def test_a_flag_that_never_comes_ends_in_a_status_not_a_hang(pkg):
    import time

    import torch

    dev = torch.device("cuda:0")
    H, IM, E, K, T = 128, 64, 8, 4, 48
    weights = synth.make_layer(synth.MoeShape("ep", 8, H, IM, E, K, 7.0, 5))
    engs = _engines(pkg, 2, H, IM, E, K, T, weights)
    stream = torch.cuda.current_stream().cuda_stream
    try:
        t, x, pos = _make_rank_inputs(0, T, H, 1)
        td, xd = helpers.to_dev_bf16(t, dev), helpers.to_dev_bf16(x, dev)
        posd = torch.from_numpy(pos).to(dev)
        engs[0].set_option("wait_limit_ms", 20)
        # rank 0 publishes and runs its owner stage; rank 1 never publishes
        engs[0].forward_part(0, 0, td, xd, posd, T, stream)
        t0 = time.perf_counter()
        engs[0].forward_part(0, 1, td, xd, posd, T, stream)
        torch.cuda.synchronize()
        waited = time.perf_counter() - t0
        assert 0.015 < waited < 1.5, f"the wait took {waited:.3f} s for a 20 ms limit"
        assert engs[0].device_status() == 106  # kStatusWaitTimeoutPeer; reading clears it
        assert engs[0].device_status() == 0
        # the one-call host path synchronises by itself and must report the problem
        xh = synth.bf16_bits(x)
        with pytest.raises(pkg.MoeError) as ei:
            engs[0].forward_host(0, synth.bf16_bits(t), xh, pos, T)
        assert ei.value.code == pkg.GPTOSS_E_DEVICE and "106" in str(ei.value)
        assert engs[1].device_status() == 0
        # the context is intact: a plain engine still computes
        shape = synth.MoeShape("after", 32, H, IM, E, K, 7.0, 5)
        helpers.run_gpu_layer(pkg, shape, synth.make_layer(shape))
    finally:
        torch.cuda.synchronize()
        for eng in engs:
            eng.close()
