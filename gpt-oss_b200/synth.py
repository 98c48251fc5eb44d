"""Seeded synthetic inputs for the MoE block.

The reference is benchmarked on real gpt-oss checkpoints and prompt files that
are not available offline; every workload here is random data with the shapes,
dtypes and value distributions of those runs: activations bf16 N(0,1) (as after
RMSNorm), weights bf16 N(0,0.02), biases N(0,0.01) (router bias N(0,0.02)).
All values are rounded to bf16 and carried as float32, so the CPU oracle (fp32
arithmetic) and the GPU path (bf16 storage) see identical numbers.
"""
from __future__ import annotations

import dataclasses

import numpy as np


def bf16_bits(a: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns (uint16), round to nearest even."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    rounded = u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))
    return (rounded >> np.uint32(16)).astype(np.uint16)


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    """bf16 bit patterns (uint16) -> float32."""
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(
        np.float32
    )


def bf16_round(a: np.ndarray) -> np.ndarray:
    """Round float32 values to the nearest bf16, keep float32 storage."""
    return bf16_to_f32(bf16_bits(a))


@dataclasses.dataclass
class MoeShape:
    """One MoE layer workload (names follow the reference's Config, run.cpp:26-46)."""

    name: str
    n_tokens: int
    hidden_dim: int
    intermediate_dim: int
    n_experts: int
    experts_per_token: int = 4
    swiglu_limit: float = 7.0
    seed: int = 0


# The workloads of the benchmark description.  "c2" is the 20b-shape layer the
# single-GPU metric is quoted on, "c3" the 120b-shape layer.
SHAPES = {
    "tiny": MoeShape("tiny", 16, 128, 128, 8, 4, 7.0, 0),
    "c2": MoeShape("gpt-oss-20b-moe-layer-T7168", 7168, 2880, 2880, 32, 4, 7.0, 1),
    "c3": MoeShape("gpt-oss-120b-moe-layer-T6144", 6144, 2880, 2880, 128, 4, 7.0, 2),
    # c2 cut to 8 experts and a quarter of the tokens: the same 896 rows per expert
    # and the same tiles, 0.4 GB of weights (still larger than L2); the case that
    # profiler captures with many passes are taken on
    "c2s": MoeShape("gpt-oss-20b-moe-layer-8experts-T1792", 1792, 2880, 2880, 8, 4, 7.0, 1),
    # c3 cut to 16 experts and an eighth of the tokens: the same 192 rows per expert,
    # 0.8 GB of weights (larger than L2); the weight-streaming case for profiler captures
    "c3s": MoeShape("gpt-oss-120b-moe-layer-16experts-T768", 768, 2880, 2880, 16, 4, 7.0, 2),
    # c3's routing problem (6144 tokens, 128 experts, hidden 2880) with narrow experts
    # (intermediate 64: 0.14 GB of weights): the case that captures of the router,
    # permutation and combine kernels are taken on
    "c3r": MoeShape("gpt-oss-120b-routing-T6144-narrow-experts", 6144, 2880, 64, 128, 4, 7.0, 2),
}


def make_layer(shape: MoeShape, n_tokens: int | None = None, inactive_every: int = 0):
    """Host tensors of one layer, float32 arrays holding bf16-exact values.

    Returns a dict with t, x (residual stream; a second N(0,1) draw), pos,
    w_router, b_router, w_mlp1 (gate rows even, up rows odd), b_mlp1, w_mlp2,
    b_mlp2.  inactive_every > 0 marks every n-th token inactive (pos = -1).
    """
    T = shape.n_tokens if n_tokens is None else n_tokens
    H, IM, E = shape.hidden_dim, shape.intermediate_dim, shape.n_experts
    rng = np.random.Generator(np.random.PCG64(shape.seed))

    def normal(size, std):
        return bf16_round((rng.standard_normal(size, dtype=np.float32) * np.float32(std)))

    d = {
        "t": normal((T, H), 1.0),
        "x": normal((T, H), 1.0),
        "w_router": normal((E, H), 0.02),
        "b_router": normal((E,), 0.02),
        "w_mlp1": normal((E, 2 * IM, H), 0.02),
        "b_mlp1": normal((E, 2 * IM), 0.01),
        "w_mlp2": normal((E, H, IM), 0.02),
        "b_mlp2": normal((E, H), 0.01),
    }
    pos = np.arange(T, dtype=np.int32)
    if inactive_every > 0:
        pos[::inactive_every] = -1
    d["pos"] = pos
    return d


# ---------------------------------------------------------------- MXFP4
E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
                        -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], dtype=np.float32)


def mxfp4_random(rng, rows_shape, k, scale_lo=119, scale_hi=123):
    """Random MXFP4 tensor [..., k]: packed codes [..., k/2] (uniform over the 16 e2m1
    codes, low nibble = even element) and e8m0 scales [..., k/32] (uniform in
    [scale_lo, scale_hi], i.e. 2^-8 .. 2^-4 by default)."""
    codes = rng.integers(0, 16, size=(*rows_shape, k), dtype=np.uint8)
    blocks = (codes[..., 0::2] | (codes[..., 1::2] << 4)).astype(np.uint8)
    scales = rng.integers(scale_lo, scale_hi + 1, size=(*rows_shape, k // 32), dtype=np.uint8)
    return blocks, scales


def mxfp4_dequant(blocks, scales):
    """Packed codes + e8m0 scales -> float32 (exact; every value is a bf16 number)."""
    lo = E2M1_VALUES[blocks & 0x0F]
    hi = E2M1_VALUES[blocks >> 4]
    vals = np.stack([lo, hi], axis=-1).reshape(*blocks.shape[:-1], blocks.shape[-1] * 2)
    s = np.exp2(scales.astype(np.float32) - 127.0)
    return (vals.reshape(*scales.shape, 32) * s[..., None]).reshape(vals.shape).astype(np.float32)


# ---------------------------------------------------------------- whole models (.bin)
# Field order of the reference's Config = header of the .bin file (run.cpp:26-46).
MODEL_CONFIG_FIELDS = (
    ("vocab_size", "i"), ("hidden_dim", "i"), ("n_experts", "i"), ("experts_per_token", "i"),
    ("intermediate_dim", "i"), ("n_layers", "i"), ("head_dim", "i"), ("n_attn_heads", "i"),
    ("n_kv_heads", "i"), ("seq_len", "i"), ("initial_context_length", "i"), ("rope_theta", "f"),
    ("rope_scaling_factor", "f"), ("sliding_window", "i"), ("swiglu_limit", "f"),
)

# The tiny GPT-OSS-architecture model of the benchmark description (2 layers, hidden 128,
# 4 query / 2 KV heads of 32, 8 experts top-4, vocabulary 201088); rope constants of the
# reference's 7m export.
TINY_MODEL = dict(vocab_size=201088, hidden_dim=128, n_experts=8, experts_per_token=4,
                  intermediate_dim=128, n_layers=2, head_dim=32, n_attn_heads=4, n_kv_heads=2,
                  seq_len=64, initial_context_length=4096, rope_theta=150000.0,
                  rope_scaling_factor=32.0, sliding_window=128, swiglu_limit=7.0)
# Same architecture with a small vocabulary, wider heads and a window short enough to bite.
MINI_MODEL = dict(vocab_size=1000, hidden_dim=128, n_experts=8, experts_per_token=4,
                  intermediate_dim=64, n_layers=3, head_dim=64, n_attn_heads=4, n_kv_heads=2,
                  seq_len=64, initial_context_length=4096, rope_theta=150000.0,
                  rope_scaling_factor=32.0, sliding_window=8, swiglu_limit=7.0)


def model_tensors(cfg: dict, seed: int = 0):
    """Random-init tensors of a whole model in the order of the .bin file
    (memory_map_weights, run.cpp:207-248): weights bf16-exact N(0, 0.02), biases
    N(0, 0.01), norm scales 1, sinks N(0, 0.02).  List of (name, float32 array)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    V, H, L = cfg["vocab_size"], cfg["hidden_dim"], cfg["n_layers"]
    D, Hq, Hkv = cfg["head_dim"], cfg["n_attn_heads"], cfg["n_kv_heads"]
    E, IM = cfg["n_experts"], cfg["intermediate_dim"]
    dqkv = (Hq + 2 * Hkv) * D

    def w(*shape):
        return bf16_round(rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02))

    def b(*shape):
        return bf16_round(rng.standard_normal(shape, dtype=np.float32) * np.float32(0.01))

    return [
        ("token_embedding_table", w(V, H)), ("out", w(V, H)),
        ("rms_attn_w", np.ones((L, H), np.float32)), ("rms_ffn_w", np.ones((L, H), np.float32)),
        ("rms_out_w", np.ones((H,), np.float32)),
        ("w_qkv", w(L, dqkv, H)), ("b_qkv", b(L, dqkv)),
        ("w_o", w(L, H, Hq * D)), ("b_o", b(L, H)), ("attn_sinks", w(L, Hq)),
        ("w_router", w(L, E, H)), ("b_router", b(L, E)),
        ("w_mlp1", w(L, E, 2 * IM, H)), ("b_mlp1", b(L, E, 2 * IM)),
        ("w_mlp2", w(L, E, H, IM)), ("b_mlp2", b(L, E, H)),
    ]


def write_model_bin(path, cfg: dict, seed: int = 0):
    """Writes a checkpoint in the reference's .bin layout: the 60-byte Config header, then
    little-endian fp32 tensors.  Returns the tensors as a dict."""
    import struct

    tensors = model_tensors(cfg, seed)
    with open(path, "wb") as f:
        for name, kind in MODEL_CONFIG_FIELDS:
            f.write(struct.pack("<" + kind, cfg[name]))
        for _, a in tensors:
            f.write(np.ascontiguousarray(a, dtype="<f4").tobytes())
    return dict(tensors)
