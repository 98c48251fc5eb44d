"""Expert parallelism on real GPUs: one process per GPU; rows travel by NCCL send/recv
or are read from the peers' memory.

Every rank has its own tokens and 1/N of the experts; each rank's result must
equal the CPU oracle (all experts) on that rank's tokens.  Needs >= 2 GPUs, so it
is skipped on a one-GPU box.
"""
import os
import pathlib
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = pathlib.Path(__file__).resolve().parents[1]

CASES = [
    # H, IM, E, K, tokens on rank r = base + 11 * r
    (128, 64, 8, 4, 90),
    (256, 192, 32, 4, 300),
]


def _worker(rank, world, uid, tmp):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch

    import __graft_entry__ as entry

    pkg = entry.load_package()
    from gpt_oss_b200 import ep_plan, synth

    import helpers

    oracle = entry.load_oracle()
    torch.cuda.set_device(rank)
    report = []
    try:
        for (H, IM, E, K, base) in CASES:
            d = synth.make_layer(synth.MoeShape("ep", 8, H, IM, E, K, 7.0, 4242))
            T = base + 11 * rank
            shape = synth.MoeShape("ep", T, H, IM, E, K, 7.0, 4242)
            rng = np.random.default_rng(99 + rank)
            d["t"] = synth.bf16_round(rng.standard_normal((T, H)).astype(np.float32))
            d["x"] = synth.bf16_round(rng.standard_normal((T, H)).astype(np.float32))
            d["pos"] = np.arange(T, dtype=np.int32)
            d["pos"][3::13] = -1
            want = oracle.moe_layer(d, shape)
            eng = pkg.MoeEngine(H, IM, E, K, max_tokens=base + 11 * world, ep_rank=rank,
                                ep_size=world, device=rank)
            eng.load_layer_f32(0, d["w_router"], d["b_router"], d["w_mlp1"], d["b_mlp1"],
                               d["w_mlp2"], d["b_mlp2"])
            eng.ep_init(uid[len(report)])
            dev = torch.device("cuda", rank)
            t = helpers.to_dev_bf16(d["t"], dev)
            x = helpers.to_dev_bf16(d["x"], dev)
            pos = torch.from_numpy(d["pos"]).to(dev)
            stream = torch.cuda.current_stream().cuda_stream
            # both transports (NCCL send/recv; peer memory where the ranks could map each
            # other's buffers)
            # (transport, overlap of the second half's gather with the first half's GEMM)
            transports = [(0, 0), (1, 0), (1, 1)] if eng.ep_transport == 1 else [(0, 0)]
            outs = []
            for tr, ov in transports:
                eng.set_option("ep_transport", tr)
                eng.set_option("ep_overlap", ov)
                for rep in range(2):  # twice: buffers are reused between layers
                    x.copy_(helpers.to_dev_bf16(d["x"], dev))
                    eng.forward(0, t, x, pos, T, stream)
                torch.cuda.synchronize()
                assert eng.device_status() == 0
                outs.append(x.float().cpu().numpy())
            # peer memory with and without the overlapped gather: the same bits; the NCCL
            # transport rounds once more per owner (the owner's per-row sum goes back as
            # bf16), so it agrees with them within the tolerance, not bit for bit
            if len(outs) == 3:
                np.testing.assert_array_equal(outs[2], outs[1])
                helpers.check_activations(outs[0][d["pos"] >= 0], outs[1][d["pos"] >= 0],
                                          "NCCL transport vs peer memory", bf16_quantum=True)
            got = outs[-1]
            # one GPU with all experts: the same sum of the same K rows per token; only the
            # GEMMs' own last bits differ (other tile widths)
            if len(outs) == 3:
                single = helpers.run_gpu_layer(pkg, shape, d)["x_out"]
                helpers.check_activations(got, single, "peer memory vs one GPU", max_abs=4e-2,
                                          mean_rel=1e-3)
            active = d["pos"] >= 0
            r = eng.get_routing(T)
            helpers.check_indices(r["topk_i"], want["topk_i"], want["logits"], active)
            helpers.check_activations(got[active], want["x_out"][active], "ep x_out",
                                      bf16_quantum=True)
            np.testing.assert_array_equal(got[~active], d["x"][~active])
            # this rank's expert groups hold exactly the rows routed to its experts
            mine = ep_plan.local_expert_slice(E, rank, world)
            assert r["expert_offsets"].shape[0] == len(mine) + 1
            report.append("ok transports=%s" % transports)
            eng.close()
    except Exception as exc:  # noqa: BLE001
        report.append(f"fail: {exc!r}")
    (pathlib.Path(tmp) / f"rank{rank}.txt").write_text("\n".join(report))


def test_expert_parallel_two_or_more_gpus(pkg, tmp_path):
    import torch
    import torch.multiprocessing as mp

    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    uids = [pkg.MoeEngine.ep_unique_id() for _ in CASES]
    mp.spawn(_worker, args=(world, uids, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        lines = (tmp_path / f"rank{r}.txt").read_text().splitlines()
        assert len(lines) == len(CASES) and all(l.startswith("ok") for l in lines), \
            f"rank {r}: {lines}"
        print(f"rank {r}: {lines}")
