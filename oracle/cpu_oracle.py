"""ctypes access to the CPU checkers.  TEST INFRASTRUCTURE ONLY.

``liboracle.so`` is the C restatement (oracle/moe_oracle.c); ``_ref`` is the
reference's own CPU code compiled by oracle/Makefile when the reference tree is
present.  Only tests, the smoke check and the benchmark's CPU-baseline /
reference arm may import this module; the product library never does.
"""
from __future__ import annotations

import ctypes
import os
import pathlib
import subprocess

import numpy as np

HERE = pathlib.Path(__file__).resolve().parent
ORACLE_LIB = HERE / "liboracle.so"
REF_LIB = HERE / "_ref" / "libgptoss_ref.so"

_f = ctypes.POINTER(ctypes.c_float)
_i = ctypes.POINTER(ctypes.c_int)


def build(native: bool = False) -> None:
    """Compile liboracle.so (and _ref when the reference tree exists)."""
    args = ["make", "-C", str(HERE), "-s"]
    if native:
        args.append("ORACLE_MARCH=native")
    subprocess.run(args, check=True)


def _fp(a):
    return None if a is None else a.ctypes.data_as(_f)


def _ip(a):
    return None if a is None else a.ctypes.data_as(_i)


def _load(path):
    if not path.exists():
        raise RuntimeError(f"{path} not built (make -C oracle)")
    return ctypes.CDLL(str(path))


_layer_args = [_f, _f, _i] + [ctypes.c_int] * 5 + [_f] * 6 + [ctypes.c_float, _f, _i, _f, _f]


def have_ref() -> bool:
    return REF_LIB.exists()


def num_threads(which: str = "oracle") -> int:
    lib = _load(ORACLE_LIB if which == "oracle" else REF_LIB)
    fn = lib.oracle_num_threads if which == "oracle" else lib.ref_num_threads
    fn.restype = ctypes.c_int
    return int(fn())


def moe_layer(d, shape, which: str = "oracle", taps: bool = True):
    """Run one MoE block on the CPU.

    d: dict from gpt_oss_b200.synth.make_layer (float32 arrays); shape: MoeShape.
    which: "oracle" (C restatement) or "ref" (the reference's compiled code).
    Returns dict with x_out, and when taps: logits, topk_i, topk_v, e_agg.
    """
    lib = _load(ORACLE_LIB if which == "oracle" else REF_LIB)
    fn = lib.oracle_moe_layer if which == "oracle" else lib.ref_moe_layer
    fn.restype = ctypes.c_int
    fn.argtypes = _layer_args
    T = d["t"].shape[0]
    H, IM, E, K = shape.hidden_dim, shape.intermediate_dim, shape.n_experts, shape.experts_per_token
    t = np.ascontiguousarray(d["t"], dtype=np.float32)
    x = np.array(d["x"], dtype=np.float32, order="C", copy=True)
    pos = None if d.get("pos") is None else np.ascontiguousarray(d["pos"], dtype=np.int32)
    logits = np.zeros((T, E), np.float32) if taps else None
    topk_i = np.full((T, K), -1, np.int32) if taps else None
    topk_v = np.zeros((T, K), np.float32) if taps else None
    e_agg = np.zeros((T, H), np.float32) if taps else None
    w = [np.ascontiguousarray(d[k], dtype=np.float32)
         for k in ("w_router", "b_router", "w_mlp1", "b_mlp1", "w_mlp2", "b_mlp2")]
    rc = fn(_fp(t), _fp(x), _ip(pos), T, H, IM, E, K, *[_fp(a) for a in w],
            ctypes.c_float(shape.swiglu_limit), _fp(logits), _ip(topk_i), _fp(topk_v), _fp(e_agg))
    if rc != 0:
        raise RuntimeError(f"{which} moe layer returned {rc}")
    out = {"x_out": x}
    if taps:
        out.update(logits=logits, topk_i=topk_i, topk_v=topk_v, e_agg=e_agg)
    return out


def rmsnorm_rows(x, w, which: str = "oracle"):
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    out = np.empty_like(x)
    if which == "ref":
        lib = _load(REF_LIB)
        lib.ref_rmsnorm_rows.argtypes = [_f, _f, _f, ctypes.c_int, ctypes.c_int]
        lib.ref_rmsnorm_rows(_fp(out), _fp(x), _fp(w), x.shape[0], x.shape[1])
    else:
        lib = _load(ORACLE_LIB)
        lib.oracle_rmsnorm.argtypes = [_f, _f, _f, ctypes.c_int]
        for r in range(x.shape[0]):
            lib.oracle_rmsnorm(_fp(out[r]), _fp(x[r]), _fp(w), x.shape[1])
    return out


def model_logits(bin_path, tokens, vocab_size: int):
    """Teacher-forced fp32 logits [len(tokens), vocab_size] of the whole model from the
    reference's own forward() (only with the compiled reference, ``_ref``)."""
    lib = _load(REF_LIB)
    toks = np.ascontiguousarray(tokens, dtype=np.int32)
    out = np.empty((toks.shape[0], vocab_size), dtype=np.float32)
    lib.ref_model_logits.argtypes = [ctypes.c_char_p, _i, ctypes.c_int, _f]
    lib.ref_model_logits.restype = ctypes.c_int
    rc = lib.ref_model_logits(str(bin_path).encode(), _ip(toks), toks.shape[0], _fp(out))
    if rc != 0:
        raise RuntimeError(f"ref_model_logits returned {rc}")
    return out


def set_threads(n: int) -> None:
    os.environ["OMP_NUM_THREADS"] = str(n)
