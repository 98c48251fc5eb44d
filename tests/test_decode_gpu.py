"""Whole-model decode step on the GPU against the reference's forward().

Teacher forcing: the golden record (tests/golden/make_golden_model.py) holds the token
fed at every position and the reference's logits there; the GPU is fed the same tokens
and must reproduce the logits within tolerance and pick the same next token unless the
reference's own top logits are closer than the tolerance band (greedy ids of a
random-init model sit on near-flat logits).
"""
import pathlib

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = pathlib.Path(__file__).resolve().parents[1]

# logits have std 0.23; activations pass through bf16 between kernels
LOGIT_MAX_ABS = 2e-2
LOGIT_MEAN_ABS = 2e-3


def _golden(name):
    return np.load(ROOT / "tests" / "golden" / f"model_{name}.npz")


def _run_teacher_forced(pkg, cfg, seed, tokens, tmp_path, rows=(0,), max_batch=4,
                        stagger=0):
    """Feeds `tokens` position by position to every row in `rows` (row r starts
    r * stagger steps late, idle rows and late rows are inactive) and returns the logits
    of rows[0] at every position plus the next-token ids of every row."""
    from gpt_oss_b200 import synth

    path = tmp_path / "model.bin"
    synth.write_model_bin(path, cfg, seed)
    image = np.memmap(path, dtype=np.uint8, mode="r")
    eng = pkg.DecodeEngine(cfg, max_batch)
    eng.load_bin(np.asarray(image))
    n = len(tokens)
    probe_logits, nexts = [], {r: [] for r in rows}
    for step in range(n + stagger * (len(rows) - 1)):
        tok = np.full(max_batch, -1, np.int32)
        pos = np.full(max_batch, -1, np.int32)
        for j, r in enumerate(rows):
            p = step - j * stagger
            if 0 <= p < n:
                tok[r], pos[r] = tokens[p], p
        nxt = eng.step(tok, pos)
        for j, r in enumerate(rows):
            p = step - j * stagger
            if 0 <= p < n:
                nexts[r].append(int(nxt[r]))
                if j == 0:
                    probe_logits.append(eng.logits(r))
            else:
                assert nxt[r] == -1
    eng.close()
    return np.stack(probe_logits), nexts


def _check_against_golden(g, logits, nexts):
    probes = g["probes"]
    err = np.abs(logits[:, probes].astype(np.float64) - g["probe_logits"])
    assert err.max() <= LOGIT_MAX_ABS, f"logits max-abs {err.max():.3e}"
    assert err.mean() <= LOGIT_MEAN_ABS, f"logits mean-abs {err.mean():.3e}"
    top_ids, top_logits = g["top_ids"], g["top_logits"]
    # the reference's best logits are reproduced at their ids
    got_top = np.take_along_axis(logits, top_ids.astype(np.int64), axis=1)
    assert np.abs(got_top - top_logits).max() <= LOGIT_MAX_ABS
    mismatches = 0
    for p, nx in enumerate(nexts):
        if nx == top_ids[p, 0]:
            continue
        mismatches += 1
        where = np.nonzero(top_ids[p] == nx)[0]
        assert where.size, f"position {p}: token {nx} is not among the reference's top 8"
        gap = top_logits[p, 0] - top_logits[p, where[0]]
        assert gap <= 2 * LOGIT_MAX_ABS, f"position {p}: picked a logit {gap:.4f} below the best"
    assert mismatches <= len(nexts) // 8


@pytest.mark.parametrize("name", ["tiny", "mini"])
def test_decode_matches_reference_logits(pkg, tmp_path, name):
    from gpt_oss_b200 import synth

    g = _golden(name)
    cfg = synth.TINY_MODEL if name == "tiny" else synth.MINI_MODEL
    logits, nexts = _run_teacher_forced(pkg, cfg, int(g["seed"]), g["tokens"], tmp_path)
    _check_against_golden(g, logits, nexts[0])


def test_rows_are_independent_and_inactive_rows_idle(pkg, tmp_path):
    """Three sequences in one batch, started 5 steps apart in rows 0, 2, 3 (row 1 never
    used): every row reproduces the single-sequence result bit for bit."""
    from gpt_oss_b200 import synth

    g = _golden("mini")
    tokens = g["tokens"][:24]
    cfg = synth.MINI_MODEL
    _, solo = _run_teacher_forced(pkg, cfg, int(g["seed"]), tokens, tmp_path)
    _, multi = _run_teacher_forced(pkg, cfg, int(g["seed"]), tokens, tmp_path, rows=(0, 2, 3),
                                   stagger=5)
    for r in (0, 2, 3):
        assert multi[r] == solo[0], f"row {r}"


@pytest.mark.parametrize("heads", [(4, 2), (8, 1), (6, 2)])
def test_live_reference_when_present(pkg, oracle, tmp_path, heads):
    """Fresh seed, full logits against the compiled reference where it travelled along;
    2, 8 and 3 query heads per KV head, contexts longer than one 16-position block and a
    window that cuts into them."""
    from gpt_oss_b200 import synth

    if not oracle.have_ref():
        pytest.skip("compiled reference not present")
    # every expert is selected (top-4 of 4), so no near-tie in the router can make the bf16
    # pipeline and the fp32 reference pick different experts
    cfg = dict(synth.MINI_MODEL, vocab_size=777, sliding_window=21, n_layers=2,
               n_attn_heads=heads[0], n_kv_heads=heads[1], n_experts=4, experts_per_token=4)
    rng = np.random.default_rng(77 + heads[0])
    tokens = rng.integers(0, cfg["vocab_size"], size=40, dtype=np.int32)
    logits, _ = _run_teacher_forced(pkg, cfg, 9, tokens, tmp_path)
    want = oracle.model_logits(tmp_path / "model.bin", tokens, cfg["vocab_size"])
    err = np.abs(logits - want)
    assert err.max() <= LOGIT_MAX_ABS and err.mean() <= LOGIT_MEAN_ABS, (err.max(), err.mean())


def test_decode_argument_errors(pkg):
    from gpt_oss_b200 import synth

    bad = dict(synth.MINI_MODEL, head_dim=48)
    with pytest.raises(pkg.MoeError) as ei:
        pkg.DecodeEngine(bad, 2)
    assert ei.value.code == pkg.GPTOSS_E_INVALID
    eng = pkg.DecodeEngine(synth.MINI_MODEL, 2)
    with pytest.raises(pkg.MoeError) as ei:  # weights not loaded
        eng.step(np.zeros(2, np.int32), np.zeros(2, np.int32))
    assert ei.value.code == pkg.GPTOSS_E_STATE
    eng.close()


def test_per_tensor_loading_and_cache_transfer(pkg, tmp_path):
    """An engine filled tensor by tensor (fp32 from the host, or bf16 / fp32 already on the
    device) and handed another engine's KV cache continues a sequence exactly as the engine
    that loaded the .bin image and ran the sequence itself."""
    import torch

    from gpt_oss_b200 import synth

    cfg = synth.MINI_MODEL
    path = tmp_path / "model.bin"
    W = synth.write_model_bin(path, cfg, 12)
    a = pkg.DecodeEngine(cfg, 3)
    a.load_bin(np.asarray(np.memmap(path, dtype=np.uint8, mode="r")))
    rng = np.random.default_rng(8)
    tokens = rng.integers(0, cfg["vocab_size"], size=11, dtype=np.int32)
    idle = np.full(3, -1, np.int32)
    for p, t in enumerate(tokens[:-1]):
        tok, pos = idle.copy(), idle.copy()
        tok[2], pos[2] = t, p
        a.step(tok, pos)

    b = pkg.DecodeEngine(cfg, 3)
    dev = torch.device("cuda:0")
    L = cfg["n_layers"]
    for name in ("token_embedding_table", "out"):
        b.set_tensor(name, 0, W[name])                                   # fp32 from the host
    b.set_tensor("rms_out_w", 0, torch.from_numpy(W["rms_out_w"]).to(dev))  # fp32 on the device
    for l in range(L):
        b.set_tensor("w_qkv", l, torch.from_numpy(W["w_qkv"][l]).to(dev).bfloat16())  # bf16 on the device
        b.set_tensor("w_o", l, np.ascontiguousarray(W["w_o"][l]))
        for name in ("b_qkv", "b_o", "attn_sinks", "rms_attn_w", "rms_ffn_w"):
            b.set_tensor(name, l, np.ascontiguousarray(W[name][l]))
    with pytest.raises(pkg.MoeError):  # the MoE layers are still missing
        b.step(np.zeros(3, np.int32), np.zeros(3, np.int32))
    moe = b.moe()
    for l in range(L):
        moe.load_layer_f32(l, W["w_router"][l], W["b_router"][l], W["w_mlp1"][l], W["b_mlp1"][l],
                           W["w_mlp2"][l], W["b_mlp2"][l])
    dkv = cfg["n_kv_heads"] * cfg["head_dim"]
    n_ctx = len(tokens) - 1
    for l in range(L):
        k = torch.empty((1, n_ctx, dkv), device=dev, dtype=torch.bfloat16)
        v = torch.empty_like(k)
        a.get_kv(l, 2, 0, k, v)       # row 2 of engine a ...
        b.set_kv(l, 1, 0, k, v)       # ... becomes row 1 of engine b
    tok, pos = idle.copy(), idle.copy()
    tok[2], pos[2] = tokens[-1], n_ctx
    na = a.step(tok, pos)
    nb = b.step(np.array([-1, tokens[-1], -1], np.int32), np.array([-1, n_ctx, -1], np.int32))
    assert na[2] == nb[1] and nb[0] == -1
    np.testing.assert_array_equal(a.logits(2), b.logits(1))
    a.close()
    b.close()
