"""Host-side logic of expert parallelism that needs no GPU.

* Rank-agreed termination (gpt-oss_b200/host/step_agreement.h): host threads with very
  different amounts of work all make the longest one's number of steps and stop together,
  so no GPU leaves the step loop while its experts are still needed - the hang the
  reference's loop has (getp-csrc/getp_run.cpp:942-943 against expert.cpp:145-171).
* The capacity check of the NCCL transport: every rank takes the go / no-go decision
  from the whole all-gathered count matrix, so two ranks (gloo, world size 2) that hold
  the same matrix decide alike also when only one of them is over its limits.
"""
import ctypes
import os
import pathlib
import subprocess
import sys

import numpy as np

ROOT = pathlib.Path(__file__).resolve().parents[1]


def test_step_agreement_threads_stop_together(pkg):
    from gpt_oss_b200 import build as native_build

    if not native_build.AGREEMENT_TEST.exists():
        native_build.build_host()
    res = subprocess.run([str(native_build.AGREEMENT_TEST)], capture_output=True, text=True,
                         timeout=120)
    assert res.returncode == 0, res.stdout + res.stderr
    assert res.stdout.strip() == "ok"


def _check(lib, counts, n, max_tokens, top_k):
    fn = lib.gptoss_internal_ep_counts_problem
    fn.restype = ctypes.c_char_p
    fn.argtypes = [ctypes.POINTER(ctypes.c_int), ctypes.c_int, ctypes.c_int, ctypes.c_int]
    c = np.ascontiguousarray(counts, dtype=np.int32)
    out = fn(c.ctypes.data_as(ctypes.POINTER(ctypes.c_int)), n, max_tokens, top_k)
    return None if out is None else out.decode()


def test_counts_check_single_process(pkg):
    lib = pkg.load_library()
    ok = np.array([[10, 20], [30, 5]])
    assert _check(lib, ok, 2, 32, 4) is None
    assert "out of range" in _check(lib, np.array([[10, 33], [0, 0]]), 2, 32, 4)
    assert "out of range" in _check(lib, np.array([[10, -1], [0, 0]]), 2, 32, 4)
    # a rank may send each token once per owner: 4 ranks, top-2 => at most 2 * max_tokens rows
    over = np.zeros((4, 4), np.int32)
    over[1] = [32, 32, 1, 0]
    assert "more rows" in _check(lib, over, 4, 32, 2)
    full = np.full((2, 2), 32, np.int32)  # everything to everybody: exactly at capacity
    assert _check(lib, full, 2, 32, 4) is None


def _worker(rank, world, port, tmp):
    sys.path.insert(0, str(ROOT))
    import torch
    import torch.distributed as dist

    import __graft_entry__ as entry

    pkg = entry.load_package()
    lib = pkg.load_library()
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    max_tokens, top_k = 64, 4
    verdicts = []
    # case 0: fine; case 1: rank 1 alone claims more rows than fit; case 2: a corrupt count
    for case, mine in enumerate([[20 + rank, 30], [64, 64] if rank == 0 else [65, 3],
                                 [10, 10] if rank == 0 else [-5, 10]]):
        row = torch.tensor(mine, dtype=torch.int32)
        rows = [torch.zeros(world, dtype=torch.int32) for _ in range(world)]
        dist.all_gather(rows, row)
        counts = torch.stack(rows).numpy()
        verdicts.append(_check(lib, counts, world, max_tokens, top_k))
    (pathlib.Path(tmp) / f"rank{rank}.txt").write_text(repr(verdicts))
    dist.destroy_process_group()


def test_counts_check_gives_every_rank_the_same_verdict(pkg, tmp_path):
    import torch.multiprocessing as mp

    port = 29000 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    a = (tmp_path / "rank0.txt").read_text()
    b = (tmp_path / "rank1.txt").read_text()
    assert a == b, f"ranks disagree: {a} vs {b}"
    verdicts = eval(a)  # noqa: S307 - our own repr of a list of str / None
    assert verdicts[0] is None
    assert verdicts[1] is not None and verdicts[2] is not None
