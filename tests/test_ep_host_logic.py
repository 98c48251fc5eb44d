"""Expert-parallel exchange among CPU ranks (gloo, world size 2).

The dispatch plan (owner = e % N, one row per (token, owner), owner-local expert
ids), the owner-side per-row pre-reduction and the home-side sum are run with
numpy as the experts' arithmetic and torch.distributed(gloo) as the transport;
each rank's result must equal the single-rank oracle on its own tokens.
"""
import os
import pathlib
import sys

import numpy as np
import pytest

ROOT = pathlib.Path(__file__).resolve().parents[1]


def _expert_rows(rows, se, sw, w1, b1, w2, b2, limit):
    """Owner side: sum over the row's local slots of w * (W2 . swiglu(W1 . t + b1) + b2)."""
    out = np.zeros((rows.shape[0], w2.shape[1]), np.float64)
    for r in range(rows.shape[0]):
        for k in range(se.shape[1]):
            e = int(se[r, k])
            if e < 0:
                continue
            pre = w1[e].astype(np.float64) @ rows[r].astype(np.float64) + b1[e]
            gate, up = pre[0::2], pre[1::2]
            gate = np.minimum(gate, limit)
            up = np.clip(up, -limit, limit)
            act = gate / (1.0 + np.exp(-1.702 * gate)) * (up + 1.0)
            out[r] += float(sw[r, k]) * (w2[e].astype(np.float64) @ act + b2[e])
    return out


def _worker(rank, world, port, tmp):
    sys.path.insert(0, str(ROOT))
    import torch.distributed as dist

    import __graft_entry__ as entry

    entry.load_package()
    from gpt_oss_b200 import ep_plan, synth

    oracle = entry.load_oracle()
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    # every rank: the same weights (same seed, same draw order), its own tokens
    d = synth.make_layer(synth.MoeShape("ep", 8, 48, 24, 8, 4, 7.0, 900))
    shape = synth.MoeShape("ep", 37 + 5 * rank, 48, 24, 8, 4, 7.0, 900)
    rng = np.random.default_rng(1234 + rank)
    d["t"] = synth.bf16_round(rng.standard_normal((shape.n_tokens, 48)).astype(np.float32))
    d["x"] = synth.bf16_round(rng.standard_normal((shape.n_tokens, 48)).astype(np.float32))
    d["pos"] = np.arange(shape.n_tokens, dtype=np.int32)
    d["pos"][::6] = -1
    want = oracle.moe_layer(d, shape)

    plans = ep_plan.dispatch_plan(want["topk_i"], want["topk_v"], world)
    # dispatch: every rank learns what every home sends to it
    outbox = [{"rows": d["t"][p["tokens"]], "se": p["slot_expert"], "sw": p["slot_weight"]}
              for p in plans]
    gathered = [None] * world
    dist.all_gather_object(gathered, outbox)
    mine = ep_plan.local_expert_slice(shape.n_experts, rank, world)
    w1, b1 = d["w_mlp1"][mine], d["b_mlp1"][mine]
    w2, b2 = d["w_mlp2"][mine], d["b_mlp2"][mine]
    back = []
    for home in range(world):
        msg = gathered[home][rank]
        assert (msg["se"] < len(mine)).all()
        back.append(_expert_rows(msg["rows"], msg["se"], msg["sw"], w1, b1, w2, b2,
                                 shape.swiglu_limit))
    returned = [None] * world
    dist.all_gather_object(returned, back)
    # combine at home
    e_agg = np.zeros_like(want["e_agg"], dtype=np.float64)
    for owner in range(world):
        e_agg[plans[owner]["tokens"]] += returned[owner][rank]
    ok = np.allclose(e_agg, want["e_agg"], rtol=0, atol=2e-5)
    inactive = d["pos"] < 0
    ok = ok and (e_agg[inactive] == 0).all()
    # every (token, owner) pair is sent once, even with several experts on one owner
    sent = sum(len(p["tokens"]) for p in plans)
    pairs = {(t, int(e) % world) for t in range(shape.n_tokens) for e in want["topk_i"][t]
             if e >= 0}
    ok = ok and sent == len(pairs)
    (pathlib.Path(tmp) / f"rank{rank}.txt").write_text("ok" if ok else "mismatch")
    dist.destroy_process_group()


def _peer_worker(rank, world, port, tmp):
    """The peer-memory protocol with gloo standing in for the mapped buffers: every rank
    publishes activations and routing result; owners work on global rows src * max_t + t
    and fill a row of sums only where they have a slot; homes add the owners' sums in
    ascending owner order."""
    sys.path.insert(0, str(ROOT))
    import torch.distributed as dist

    import __graft_entry__ as entry

    entry.load_package()
    from gpt_oss_b200 import ep_plan, synth

    oracle = entry.load_oracle()
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    max_t, H, K, E = 48, 48, 4, 8
    d = synth.make_layer(synth.MoeShape("ep", 8, H, 24, E, K, 7.0, 901))
    T = 31 + 9 * rank
    shape = synth.MoeShape("ep", T, H, 24, E, K, 7.0, 901)
    rng = np.random.default_rng(4321 + rank)
    d["t"] = synth.bf16_round(rng.standard_normal((T, H)).astype(np.float32))
    d["x"] = synth.bf16_round(rng.standard_normal((T, H)).astype(np.float32))
    d["pos"] = np.arange(T, dtype=np.int32)
    d["pos"][2::7] = -1
    want = oracle.moe_layer(d, shape)
    # publish (rows past T: id -1, as the publishing kernel writes them)
    ids = np.full((max_t, K), -1, np.int32)
    wts = np.zeros((max_t, K), np.float32)
    act = np.zeros((max_t, H), np.float32)
    ids[:T], wts[:T], act[:T] = want["topk_i"], want["topk_v"], d["t"]
    published = [None] * world
    dist.all_gather_object(published, {"ids": ids, "wts": wts, "act": act})
    all_i = np.stack([p["ids"] for p in published])
    all_v = np.stack([p["wts"] for p in published])
    all_t = np.concatenate([p["act"] for p in published])  # global rows
    # owner
    se, sw = ep_plan.owner_view(all_i, all_v, rank, world)
    mine = ep_plan.local_expert_slice(E, rank, world)
    rows = np.nonzero((se >= 0).any(axis=1))[0]
    sums = np.zeros((world * max_t, H), np.float64)
    sums[rows] = _expert_rows(all_t[rows], se[rows], sw[rows], d["w_mlp1"][mine], d["b_mlp1"][mine],
                              d["w_mlp2"][mine], d["b_mlp2"][mine], shape.swiglu_limit)
    everyone = [None] * world
    dist.all_gather_object(everyone, sums)
    # home: pull in owner order
    e_agg = np.zeros((T, H), np.float64)
    for t in range(T):
        for o in ep_plan.owners_of_token(want["topk_i"][t], world):
            e_agg[t] += everyone[o][rank * max_t + t]
    ok = np.allclose(e_agg, want["e_agg"], rtol=0, atol=2e-5)
    ok = ok and (e_agg[d["pos"] < 0] == 0).all()
    # an owner touches exactly the global rows that have one of its experts
    expect = {s * max_t + t for s in range(world) for t in range(max_t)
              for e in all_i[s, t] if e >= 0 and e % world == rank}
    ok = ok and set(rows.tolist()) == expect
    (pathlib.Path(tmp) / f"peer{rank}.txt").write_text("ok" if ok else "mismatch")
    dist.destroy_process_group()


def test_peer_memory_protocol_two_cpu_ranks(tmp_path):
    import torch.multiprocessing as mp

    port = 31500 + os.getpid() % 2000
    mp.spawn(_peer_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert (tmp_path / f"peer{r}.txt").read_text() == "ok"


def test_ep_exchange_two_cpu_ranks(tmp_path):
    import torch.multiprocessing as mp

    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert (tmp_path / f"rank{r}.txt").read_text() == "ok"


def test_ownership_rule():
    import __graft_entry__ as entry

    entry.load_package()
    from gpt_oss_b200 import ep_plan

    for n in (2, 4, 8):
        owned = [ep_plan.local_expert_slice(128, r, n) for r in range(n)]
        assert sorted(np.concatenate(owned).tolist()) == list(range(128))
        for r in range(n):
            for j, e in enumerate(owned[r]):
                assert ep_plan.owner_of(int(e), n) == r and ep_plan.local_id(int(e), n) == j
