"""The decode step with the experts sharded over 2+ GPUs (one process per GPU): every
rank decodes its own copy of the golden sequence, started a few steps apart, and must
reproduce the reference's logits like the single-GPU engine does.  Skipped on a one-GPU
box."""
import os
import pathlib
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = pathlib.Path(__file__).resolve().parents[1]


def _worker(rank, world, uid, tmp):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch

    import __graft_entry__ as entry

    pkg = entry.load_package()
    from gpt_oss_b200 import synth

    import test_decode_gpu as single

    report = "ok"
    try:
        torch.cuda.set_device(rank)
        g = np.load(ROOT / "tests" / "golden" / "model_mini.npz")
        cfg = synth.MINI_MODEL
        tokens = g["tokens"]
        path = pathlib.Path(tmp) / f"model{rank}.bin"
        synth.write_model_bin(path, cfg, int(g["seed"]))
        eng = pkg.DecodeEngine(cfg, 3, device=rank, ep_rank=rank, ep_size=world)
        eng.load_bin(np.asarray(np.memmap(path, dtype=np.uint8, mode="r")))
        moe = eng.moe(ep_rank=rank, ep_size=world, device=rank)
        moe.ep_init(uid)
        n, late = len(tokens), 3 * rank  # rank r starts 3r steps late (inactive rows before)
        logits, nexts = [], []
        for step in range(n + 3 * (world - 1)):  # every rank makes every call
            p = step - late
            tok = np.full(3, -1, np.int32)
            pos = np.full(3, -1, np.int32)
            if 0 <= p < n:
                tok[1], pos[1] = tokens[p], p
            nxt = eng.step(tok, pos)
            if 0 <= p < n:
                nexts.append(int(nxt[1]))
                logits.append(eng.logits(1))
        single._check_against_golden(g, np.stack(logits), nexts)
        report += f" transport={moe.ep_transport}"
        eng.close()
    except Exception as exc:  # noqa: BLE001
        report = f"fail: {exc!r}"
    (pathlib.Path(tmp) / f"rank{rank}.txt").write_text(report)


def test_decode_with_sharded_experts(pkg, tmp_path):
    import torch
    import torch.multiprocessing as mp

    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    uid = pkg.MoeEngine.ep_unique_id()
    mp.spawn(_worker, args=(world, uid, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        text = (tmp_path / f"rank{r}.txt").read_text()
        assert text.startswith("ok"), f"rank {r}: {text}"
        print(f"rank {r}: {text}")
