"""Golden vectors for the whole-model decode step, made with the reference's own
forward() (the compiled reference under oracle/_ref, present only where the reference
tree is mounted).  Run from the repository root:

    python tests/golden/make_golden_model.py

For each model (gpt_oss_b200.synth.TINY_MODEL = the tiny model of the benchmark
description, MINI_MODEL = a variant whose sliding window bites) it writes the checkpoint
to a temporary .bin, picks 16 seeded prompt tokens, lets the model continue greedily for
32 steps and stores a compact record of the reference's teacher-forced logits over the
48 positions: the tokens fed, per position the 8 largest logits with their ids, and the
logits at 512 fixed probe ids.

A bf16 pipeline cannot be compared with the fp32 reference at a position where the
router's 4th and 5th logits nearly tie: the two would pick different experts and differ
by far more than rounding from there on (through the KV cache).  (Positions stop short
of seq_len - 1: there the reference writes the sink logit one past its per-head score
row, run.cpp:626, into the next head's row while the heads run in parallel.)  The prompt seed is
therefore searched until the smallest such gap over all positions and layers is at least
MIN_ROUTER_GAP.  The gaps come from a float64 numpy restatement of forward()
(run.cpp:536-766) in this file, which is itself checked against the reference's logits
before anything is written.
"""
import math
import pathlib
import sys
import tempfile

import numpy as np

ROOT = pathlib.Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

N_PROMPT, N_GEN, N_PROBE, TOP = 16, 32, 512, 8
MIN_ROUTER_GAP = 4e-3


def rope_tables(cfg):
    """compute_concentration_and_inv_freq (run.cpp:423-474) with ntk_beta 32, ntk_alpha 1."""
    D = cfg["head_dim"]
    half = D // 2
    base, sf = np.float32(cfg["rope_theta"]), np.float32(cfg["rope_scaling_factor"])
    ctx = np.float32(cfg["initial_context_length"])
    freq = np.array([base ** (np.float32(2 * i) / np.float32(D)) for i in range(half)], np.float32)
    if sf <= 1:
        return 1.0 / freq.astype(np.float64), 1.0
    conc = 0.1 * math.log(sf) + 1.0
    low = half * math.log(ctx / (32.0 * 2 * math.pi)) / math.log(base)
    high = half * math.log(ctx / (1.0 * 2 * math.pi)) / math.log(base)
    inv = np.zeros(half)
    for i in range(half):
        ramp = min(max((i - low) / (high - low), 0.0), 1.0)
        inv[i] = (1.0 / (sf * freq[i])) * ramp + (1.0 / freq[i]) * (1.0 - ramp)
    return inv, conc


def emulate(cfg, W, prompt, n_total):  # W: float64 except the embedding table
    """Greedy decode in float64: tokens fed, logits per position, smallest gap between the
    router's K-th and (K+1)-th logits per position."""
    V, H, L, D = cfg["vocab_size"], cfg["hidden_dim"], cfg["n_layers"], cfg["head_dim"]
    Hq, Hkv, K = cfg["n_attn_heads"], cfg["n_kv_heads"], cfg["experts_per_token"]
    half, limit = D // 2, cfg["swiglu_limit"]
    inv, conc = rope_tables(cfg)

    def rms(x, w):
        return w * (x / math.sqrt((x * x).mean() + 1e-5))

    def rot(a, nh, c, s):
        a = a.reshape(nh, D).copy()
        x1, x2 = a[:, :half].copy(), a[:, half:].copy()
        a[:, :half], a[:, half:] = x1 * c - x2 * s, x2 * c + x1 * s
        return a.reshape(-1)

    kc = np.zeros((L, n_total, Hkv * D))
    vc = np.zeros((L, n_total, Hkv * D))
    tokens, logits, gaps = list(prompt), [], []
    for pos in range(n_total):
        x = W["token_embedding_table"][tokens[pos]].astype(np.float64)
        gap = np.inf
        c, s = np.cos(pos * inv) * conc, np.sin(pos * inv) * conc
        for l in range(L):
            t = rms(x, W["rms_attn_w"][l])
            qkv = W["w_qkv"][l] @ t + W["b_qkv"][l]
            q = rot(qkv[:Hq * D], Hq, c, s)
            kc[l, pos] = rot(qkv[Hq * D:(Hq + Hkv) * D], Hkv, c, s)
            vc[l, pos] = qkv[(Hq + Hkv) * D:]
            win = cfg["sliding_window"] if (cfg["sliding_window"] > 0 and l % 2 == 0) else 0
            t0 = max(0, pos - win + 1) if win else 0
            tb = np.zeros(Hq * D)
            for h in range(Hq):
                kv = (h // (Hq // Hkv)) * D
                sc = np.append(kc[l, t0:pos + 1, kv:kv + D] @ q[h * D:(h + 1) * D] / math.sqrt(D),
                               W["attn_sinks"][l, h])
                p = np.exp(sc - sc.max())
                p /= p.sum()
                tb[h * D:(h + 1) * D] = p[:-1] @ vc[l, t0:pos + 1, kv:kv + D]
            x = x + W["w_o"][l] @ tb + W["b_o"][l]
            t = rms(x, W["rms_ffn_w"][l])
            lg = W["w_router"][l] @ t + W["b_router"][l]
            order = np.argsort(-lg, kind="stable")
            gap = min(gap, lg[order[K - 1]] - lg[order[K]])
            idx = order[:K]
            wv = np.exp(lg[idx] - lg[idx].max())
            wv /= wv.sum()
            agg = np.zeros(H)
            for e, we in zip(idx, wv):
                m1 = W["w_mlp1"][l, e] @ t + W["b_mlp1"][l, e]
                g, u = np.minimum(m1[0::2], limit), np.clip(m1[1::2], -limit, limit)
                agg += we * (W["w_mlp2"][l, e] @ (g / (1 + np.exp(-1.702 * g)) * (u + 1)) + W["b_mlp2"][l, e])
            x = x + agg
        lg_out = W["out"] @ rms(x, W["rms_out_w"])
        logits.append(lg_out)
        gaps.append(gap)
        if len(tokens) == pos + 1:
            tokens.append(int(np.argmax(lg_out)))
    return np.array(tokens[:n_total], np.int32), np.array(logits), np.array(gaps)


def main():
    entry.load_package()
    from gpt_oss_b200 import synth

    oracle = entry.load_oracle()
    assert oracle.have_ref(), "needs the compiled reference (oracle/_ref)"
    n_total = N_PROMPT + N_GEN
    for name, cfg, seed in (("tiny", synth.TINY_MODEL, 0), ("mini", synth.MINI_MODEL, 5)):
        V = cfg["vocab_size"]
        with tempfile.TemporaryDirectory() as tmp:
            path = pathlib.Path(tmp) / f"{name}.bin"
            W = synth.write_model_bin(path, cfg, seed)
            W = {k: (v if k == "token_embedding_table" else v.astype(np.float64))
                 for k, v in W.items()}
            for prompt_seed in range(2000):
                rng = np.random.Generator(np.random.PCG64(1000 + prompt_seed))
                prompt = rng.integers(0, V, size=N_PROMPT, dtype=np.int32)
                tokens, emu, gaps = emulate(cfg, W, prompt, n_total)
                if gaps.min() >= MIN_ROUTER_GAP:
                    break
            else:
                raise SystemExit(f"{name}: no prompt with router gaps >= {MIN_ROUTER_GAP}")
            logits = oracle.model_logits(path, tokens, V)
        diff = np.abs(logits - emu).max()
        assert diff < 1e-5, f"the restatement does not follow the reference ({diff:.3e})"
        assert (np.argmax(logits[N_PROMPT - 1:-1], axis=1) == tokens[N_PROMPT:]).all()
        rng = np.random.Generator(np.random.PCG64(77))
        probes = np.sort(rng.choice(V, size=min(N_PROBE, V), replace=False)).astype(np.int32)
        order = np.argsort(-logits, axis=1, kind="stable")[:, :TOP].astype(np.int32)
        out = ROOT / "tests" / "golden" / f"model_{name}.npz"
        np.savez_compressed(out, tokens=tokens, n_prompt=np.int32(N_PROMPT), probes=probes,
                            probe_logits=logits[:, probes], top_ids=order,
                            top_logits=np.take_along_axis(logits, order, axis=1),
                            seed=np.int32(seed), router_gap=gaps.astype(np.float32))
        print(out, "prompt seed", prompt_seed, "min router gap %.4f" % gaps.min(),
              "logit std %.4f" % logits.std())


if __name__ == "__main__":
    main()
