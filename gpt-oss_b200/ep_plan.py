"""Host-side model of the expert-parallel exchange (numpy).

States in a few lines what `csrc/ep.cu` does on the device, so that tests can
check the GPU taps against it and run the exchange among CPU ranks:
ownership `e % n_ranks` with local id `e // n_ranks` (the reference's rule,
getp-csrc/expert.cpp:18, :1191-1213), one row per (token, owner) however many
of the token's experts live there, slots rewritten to owner-local expert ids.
"""
from __future__ import annotations

import numpy as np


def owner_of(expert: int, n_ranks: int) -> int:
    return expert % n_ranks


def local_id(expert: int, n_ranks: int) -> int:
    return expert // n_ranks


def dispatch_plan(topk_i: np.ndarray, topk_v: np.ndarray, n_ranks: int):
    """Per-owner send lists for one home rank.

    topk_i [T,K] global expert ids (-1 = inactive slot), topk_v [T,K].
    Returns a list over owners of dicts: tokens (ascending token ids),
    slot_expert [n,K] (owner-local id or -1), slot_weight [n,K].
    """
    T, K = topk_i.shape
    plans = []
    for o in range(n_ranks):
        mine = (topk_i >= 0) & (topk_i % n_ranks == o)
        tokens = np.nonzero(mine.any(axis=1))[0].astype(np.int32)
        se = np.where(mine[tokens], topk_i[tokens] // n_ranks, -1).astype(np.int32)
        sw = np.where(mine[tokens], topk_v[tokens], 0.0).astype(np.float32)
        plans.append({"tokens": tokens, "slot_expert": se, "slot_weight": sw})
    return plans


def local_expert_slice(n_experts: int, rank: int, n_ranks: int) -> np.ndarray:
    """Global ids of the experts a rank owns, in local-id order."""
    return np.arange(rank, n_experts, n_ranks, dtype=np.int32)


def owner_view(all_topk_i: np.ndarray, all_topk_v: np.ndarray, rank: int, n_ranks: int):
    """Peer-memory transport, owner side: what rank `rank` makes of every rank's routing
    result.  all_topk_i / all_topk_v [N, max_t, K] (ids of rows past a rank's batch = -1).
    Returns slot_expert, slot_weight [N * max_t, K] over global rows g = src * max_t + t:
    owner-local ids of the slots whose expert lives here, -1 elsewhere."""
    N, max_t, K = all_topk_i.shape
    ids = all_topk_i.reshape(N * max_t, K)
    mine = (ids >= 0) & (ids % n_ranks == rank)
    se = np.where(mine, ids // n_ranks, -1).astype(np.int32)
    sw = np.where(mine, all_topk_v.reshape(N * max_t, K), 0.0).astype(np.float32)
    return se, sw


def owners_of_token(topk_row: np.ndarray, n_ranks: int):
    """Ranks a home pulls partial sums from for one token, in the order it adds them."""
    return sorted({int(e) % n_ranks for e in topk_row if e >= 0})
