"""Regenerates the golden fixtures in this directory.

Each fixture is one small MoE layer: seeded synthetic inputs (bf16 bit patterns)
and the outputs of the REFERENCE's own CPU code on them (oracle/_ref, compiled
from the reference tree by oracle/Makefile: its matmul / topk / softmax driven
token by token exactly as run.cpp:662-750 does).  Needs the reference tree, so
it only runs where that tree is mounted; the .npz files are committed.

    python tests/golden/make_golden.py
"""
import pathlib
import sys

import numpy as np

ROOT = pathlib.Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

entry.load_package()
from gpt_oss_b200 import synth  # noqa: E402

oracle = entry.load_oracle()

# name -> (shape, inactive_every)
CASES = {
    "layer_e8_h64": (synth.MoeShape("layer_e8_h64", 24, 64, 32, 8, 4, 7.0, 101), 5),
    "layer_e8_h128": (synth.MoeShape("layer_e8_h128", 9, 128, 64, 8, 4, 7.0, 102), 0),
    "layer_e32_h64": (synth.MoeShape("layer_e32_h64", 33, 64, 24, 32, 4, 7.0, 103), 0),
    "layer_e16_k2_big_acts": (synth.MoeShape("layer_e16_k2_big_acts", 12, 64, 16, 16, 2, 1.5, 104), 4),
}


def main():
    oracle.build()
    if not oracle.have_ref():
        raise SystemExit("reference tree not available: cannot regenerate fixtures")
    out_dir = pathlib.Path(__file__).resolve().parent
    for name, (shape, inactive) in CASES.items():
        d = synth.make_layer(shape, inactive_every=inactive)
        if name.endswith("big_acts"):
            # scale the inputs so pre-activations pass the clamp on both sides
            d["t"] = synth.bf16_round(d["t"] * np.float32(24.0))
        ref = oracle.moe_layer(d, shape, which="ref")
        np.savez_compressed(
            out_dir / f"{name}.npz",
            dims=np.array([shape.n_tokens, shape.hidden_dim, shape.intermediate_dim,
                           shape.n_experts, shape.experts_per_token], np.int32),
            swiglu_limit=np.float32(shape.swiglu_limit),
            pos=d["pos"],
            **{k + "_bf16": synth.bf16_bits(d[k])
               for k in ("t", "x", "w_router", "b_router", "w_mlp1", "b_mlp1", "w_mlp2", "b_mlp2")},
            ref_logits=ref["logits"], ref_topk_i=ref["topk_i"], ref_topk_v=ref["topk_v"],
            ref_e_agg=ref["e_agg"], ref_x_out=ref["x_out"],
        )
        print(name, "written; |e_agg| mean", float(np.abs(ref["e_agg"]).mean()))


if __name__ == "__main__":
    main()
