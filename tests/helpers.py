"""Shared test helpers: golden fixtures, tolerances, GPU runs through the C ABI."""
import pathlib

import numpy as np

import __graft_entry__ as entry

entry.load_package()
from gpt_oss_b200 import synth  # noqa: E402

GOLDEN_DIR = pathlib.Path(__file__).resolve().parent / "golden"
GOLDEN_CASES = sorted(p.stem for p in GOLDEN_DIR.glob("layer_*.npz"))  # model_*.npz: whole-model records

# Tolerances stated by the benchmark description for bf16 activations.
MAX_ABS = 2e-2
MEAN_REL = 1e-2
# Expert indices must match bit for bit unless the deciding logits are this close.
TIE_EPS = 1e-6


def load_golden(name):
    z = np.load(GOLDEN_DIR / f"{name}.npz")
    T, H, IM, E, K = (int(v) for v in z["dims"])
    shape = synth.MoeShape(name, T, H, IM, E, K, float(z["swiglu_limit"]), 0)
    d = {k: synth.bf16_to_f32(z[k + "_bf16"])
         for k in ("t", "x", "w_router", "b_router", "w_mlp1", "b_mlp1", "w_mlp2", "b_mlp2")}
    d["pos"] = z["pos"].astype(np.int32)
    ref = {k[4:]: z[k] for k in z.files if k.startswith("ref_")}
    return shape, d, ref


def check_indices(got_i, want_i, want_logits, active):
    """Bit-exact expert indices, except where the logits that decide the order
    are within TIE_EPS of each other (then any order of the tied experts is
    accepted)."""
    bad = []
    for tok in np.nonzero(active)[0]:
        if np.array_equal(got_i[tok], want_i[tok]):
            continue
        lg = want_logits[tok]
        ok = True
        for r in range(got_i.shape[1]):
            a, b = int(got_i[tok, r]), int(want_i[tok, r])
            if a == b:
                continue
            if a < 0 or a >= lg.shape[0] or abs(float(lg[a]) - float(lg[b])) > TIE_EPS:
                ok = False
        if not ok:
            bad.append(int(tok))
    assert not bad, f"expert indices differ beyond the tie exemption on tokens {bad[:10]}"


def check_activations(got, want, what, max_abs=MAX_ABS, mean_rel=MEAN_REL, bf16_quantum=False):
    """max-abs / mean-rel check.  bf16_quantum=True is for the residual stream,
    whose magnitude is set by the caller's residual and not by the block: the
    limit on each element then grows by half a bf16 ulp of the expected value
    (|want| * 2^-9), the part of the error the output format itself imposes."""
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    if bf16_quantum:
        err = np.maximum(err - np.abs(want.astype(np.float64)) * 2.0 ** -9, 0.0)
    denom = max(float(np.abs(want).mean()), 1e-30)
    m_abs, m_rel = float(err.max()) if err.size else 0.0, float(err.mean() / denom) if err.size else 0.0
    assert m_abs <= max_abs and m_rel <= mean_rel, (
        f"{what}: max_abs={m_abs:.4e} (limit {max_abs}), mean_rel={m_rel:.4e} (limit {mean_rel})")
    return m_abs, m_rel


def to_dev_bf16(a, dev):
    import torch

    return torch.from_numpy(synth.bf16_bits(a).view(np.int16)).to(dev).view(torch.bfloat16)


def run_gpu_layer(pkg, shape, d, max_tokens=None, gemm_impl=None, zero_residual=False,
                  keep_logits=True, via="forward"):
    """One MoE block on cuda:0 through the C ABI.  Returns x_out (float32),
    routing taps and the engine's launch count."""
    import torch

    dev = torch.device("cuda:0")
    T = d["t"].shape[0]
    eng = pkg.MoeEngine(shape.hidden_dim, shape.intermediate_dim, shape.n_experts,
                        shape.experts_per_token, n_layers=1,
                        max_tokens=max_tokens or max(T, 1), swiglu_limit=shape.swiglu_limit)
    try:
        eng.load_layer_f32(0, d["w_router"], d["b_router"], d["w_mlp1"], d["b_mlp1"],
                           d["w_mlp2"], d["b_mlp2"])
        if gemm_impl is not None:
            eng.set_option("gemm_impl", gemm_impl)
        if keep_logits:
            eng.set_option("keep_logits", 1)
        x_in = np.zeros_like(d["x"]) if zero_residual else d["x"]
        pos_np = d.get("pos")
        if via == "host":
            t_h = synth.bf16_bits(d["t"])
            x_h = synth.bf16_bits(x_in)
            eng.forward_host(0, t_h, x_h, pos_np, T)
            x_out = synth.bf16_to_f32(x_h)
        else:
            t = to_dev_bf16(d["t"], dev)
            x = to_dev_bf16(x_in, dev)
            pos = None if pos_np is None else torch.from_numpy(pos_np).to(dev)
            stream = torch.cuda.current_stream().cuda_stream
            if via == "stages":
                eng.route(0, t, pos, T, stream)
                eng.permute(t, T, stream)
                eng.experts(0, stream)
                eng.combine(x, T, stream)
            else:
                eng.forward(0, t, x, pos, T, stream)
            torch.cuda.synchronize()
            x_out = x.float().cpu().numpy()
        status = eng.device_status()
        assert status == 0, f"device status {status}"
        routing = eng.get_routing(T, want_logits=keep_logits) if T > 0 else None
        return {"x_out": x_out, "routing": routing, "launches": eng.launch_count(),
                "x_in": x_in}
    finally:
        eng.close()
