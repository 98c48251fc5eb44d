"""The C++ getp entry points (warm_up / inference / finish) driven by a host program the
way the reference's getp() drives them, on the tiny model of the benchmark description.

Prompts are lines of token ids (the test host's encode() parses them).  The first request
is the golden prompt: its greedy continuation must follow the reference's until the first
position where the reference's own two best logits are closer than the tolerance band.
"""
import os
import pathlib
import subprocess

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = pathlib.Path(__file__).resolve().parents[1]
BAND = 4e-2  # twice the logit tolerance of the teacher-forced test


def test_getp_entry_points_on_tiny_model(pkg, tmp_path):
    from gpt_oss_b200 import build as native_build
    from gpt_oss_b200 import synth

    if not native_build.HARNESS.exists():
        native_build.build_host()
    g = np.load(ROOT / "tests" / "golden" / "model_tiny.npz")
    cfg = synth.TINY_MODEL
    n_prompt = int(g["n_prompt"])
    bin_path = tmp_path / "tiny.bin"
    synth.write_model_bin(bin_path, cfg, int(g["seed"]))
    rng = np.random.default_rng(5)
    prompts = [list(g["tokens"][:n_prompt]),
               list(rng.integers(0, cfg["vocab_size"], size=9)),
               list(rng.integers(0, cfg["vocab_size"], size=1)),
               [17, 199999, 5]]  # an end-of-sequence id inside the prompt stops the request
    req = tmp_path / "requests.txt"
    req.write_text(f"{len(prompts)}\n" + "\n".join(" ".join(str(int(t)) for t in p) for p in prompts) + "\n")
    out = tmp_path / "out.txt"
    env = dict(os.environ, GPTOSS_GETP_GPUS="1", GPTOSS_GETP_BATCH="3")  # two batches: 3 + 1
    res = subprocess.run([str(native_build.HARNESS), str(bin_path), str(req), str(out)],
                         capture_output=True, text=True, env=env, timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr
    rows = [[int(t) for t in line.split()] for line in out.read_text().splitlines()]
    assert len(rows) == len(prompts)
    # every request runs to the end of the KV cache unless it meets an end-of-sequence id
    for p, r in zip(prompts[:3], rows[:3]):
        assert all(0 <= t < cfg["vocab_size"] for t in r)
        if not any(t in (199999, 200002) for t in r):
            assert len(p) + len(r) == cfg["seq_len"]
    assert rows[3] == []
    total = int(res.stdout.split("generated ")[1].split()[0])
    assert total == sum(len(r) for r in rows)
    # the golden request against the reference's greedy continuation
    want = g["tokens"][n_prompt:]
    got = rows[0][:len(want)]
    for i, (a, b) in enumerate(zip(got, want)):
        if a == b:
            continue
        p = n_prompt - 1 + i  # position whose logits chose this token
        ids, vals = g["top_ids"][p], g["top_logits"][p]
        where = np.nonzero(ids == a)[0]
        assert where.size and vals[0] - vals[where[0]] <= BAND, (
            f"generated token {i}: {a} instead of {b}, outside the tie band")
        break  # the sequences differ from here on by construction
    else:
        assert len(got) == len(want)
    # the reference's static batches (a batch starts when the previous one is all done) give
    # every request the same tokens as the default schedule, where a finished row is handed
    # to the next waiting request at once
    out_static = tmp_path / "out_static.txt"
    res = subprocess.run([str(native_build.HARNESS), str(bin_path), str(req), str(out_static)],
                         capture_output=True, text=True, env=dict(env, GPTOSS_GETP_STATIC="1"),
                         timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr
    assert out_static.read_text() == out.read_text()


def _run_host(native_build, bin_path, req, out, env_extra):
    env = dict(os.environ, **env_extra)
    res = subprocess.run([str(native_build.HARNESS), str(bin_path), str(req), str(out)],
                         capture_output=True, text=True, env=env, timeout=900)
    assert res.returncode == 0, res.stdout + res.stderr
    rows = [[int(t) for t in line.split()] for line in out.read_text().splitlines()]
    return rows, res.stdout


def test_getp_entry_points_expert_parallel(pkg, tmp_path):
    """warm_up / inference / finish with the experts sharded over 2 GPUs (the reference's
    GETP_FORCE_EP switch), one host thread per GPU.  The second GPU's requests end after
    two steps (an end-of-sequence id in the prompt) while the first GPU decodes two full
    batches: the idle GPU must keep stepping for its experts' sake and all threads must
    stop together.  The generated ids must equal the one-GPU run's; where they part, the
    one-GPU engine's own logits at that step must be a near tie (sharding adds one bf16
    rounding per owner to the block's output)."""
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    from gpt_oss_b200 import build as native_build
    from gpt_oss_b200 import synth

    if not native_build.HARNESS.exists():
        native_build.build_host()
    g = np.load(ROOT / "tests" / "golden" / "model_tiny.npz")
    cfg = synth.TINY_MODEL
    n_prompt = int(g["n_prompt"])
    bin_path = tmp_path / "tiny.bin"
    synth.write_model_bin(bin_path, cfg, int(g["seed"]))
    rng = np.random.default_rng(11)
    prompts = [list(g["tokens"][:n_prompt]),
               list(rng.integers(0, cfg["vocab_size"], size=5)),
               [23, 199999, 7],      # these two go to the second GPU and end at once
               [1234, 200002]]
    req = tmp_path / "requests.txt"
    req.write_text(f"{len(prompts)}\n" + "\n".join(" ".join(str(int(t)) for t in p) for p in prompts) + "\n")
    one, _ = _run_host(native_build, bin_path, req, tmp_path / "one.txt",
                       {"GPTOSS_GETP_GPUS": "1", "GPTOSS_GETP_BATCH": "1"})
    two, log = _run_host(native_build, bin_path, req, tmp_path / "two.txt",
                         {"GPTOSS_GETP_GPUS": "2", "GPTOSS_GETP_BATCH": "1", "GETP_FORCE_EP": "1",
                          "NCCL_NVLS_ENABLE": "0"})
    assert "experts sharded over the GPUs" in log
    assert len(one) == len(two) == len(prompts)
    assert two[2] == [] and two[3] == []
    assert len(prompts[0]) + len(two[0]) == cfg["seq_len"] or any(t in (199999, 200002) for t in two[0])
    image = np.fromfile(bin_path, dtype=np.uint8)
    eng = pkg.DecodeEngine(cfg, 1)
    eng.load_bin(image)
    try:
        for p, a, b in zip(prompts, one, two):
            if a == b:
                continue
            i = next(k for k in range(min(len(a), len(b))) if a[k] != b[k])
            seq = list(p) + a[:i]
            for pos_i, tok in enumerate(seq):
                eng.step(np.array([tok], np.int32), np.array([pos_i], np.int32))
            lg = eng.logits(0)
            gap = abs(float(lg[a[i]]) - float(lg[b[i]]))
            assert gap <= 2e-2, (f"generated token {i}: {a[i]} on one GPU, {b[i]} with sharded "
                                 f"experts, logits {gap:.4f} apart")
    finally:
        eng.close()
