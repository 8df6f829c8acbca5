"""Generates tests/golden/*.npz by running the reference's own code (oracle/_ref, built from the
reference headers by oracle/Makefile) on the seeded inputs of tests/cases.py.

Run from the repository root where the reference sources are mounted:
    make -C oracle && python tests/golden/make_golden.py
The outputs are small float32 arrays; the inputs are regenerated from their seeds.
"""
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
import cases  # noqa: E402
import oracle_lib as ol  # noqa: E402


def main():
    ref = ol.ref_oracle()
    if ref is None:
        raise SystemExit("oracle/_ref/libjasmine_ref.so is missing: run `make -C oracle` where the reference is mounted")
    out = {}
    for name, op, sa, sb, s in cases.EXPR_CASES:
        A, B = cases.expr_inputs(name, op, sa, sb, s)
        out[f"expr_{name}"] = ref.expr(op, A, B, s)
    R = cases.reduce_input()
    for k, nm in enumerate(cases.REDUCE_KINDS):
        out[f"reduce_{nm}"] = ref.reduce(k, R)
    A, B = cases.softmax_inputs()
    out["hsoftmax_axpb"] = ref.hsoftmax(A, B, 0.125)
    out["hsoftmax_plain"] = ref.hsoftmax(A)
    out["softmax_full"] = ref.softmax_full(A[:6, :10])
    x, x2, g, b = cases.norm_inputs()
    out["layer_norm_ref"] = ref.layer_norm(x)
    out["layer_norm_eps"] = ref.layer_norm(x, x2, g, b, 1e-5)
    out["rms_norm"] = ref.rms_norm(x, g, 1e-5)
    A, B = cases.dot_inputs()
    out["dot"] = ref.dot(A, B)[1]
    X, W, bb = cases.linear_inputs()
    out["linear"] = ref.linear(X, W, bb)
    out["relu_net"] = ref.activation(0, X)
    out["sigmoid_net"] = ref.activation(1, X)
    w, xx = cases.mha_inputs()
    out["mha_causal"] = ref.mha(w, xx, cases.MHA["H"], True)
    out["mha_full"] = ref.mha(w, xx, cases.MHA["H"], False)
    out["rope"] = ref.rope(cases.rope_input())
    w, xx = cases.encoder_inputs()
    e = cases.ENC
    out["encoder_causal_rope"] = ref.encoder(w, xx, e["L"], e["H"], True, True)
    out["encoder_plain"] = ref.encoder(w, xx, e["L"], e["H"], False, False)
    np.savez_compressed(HERE / "ops.npz", **out)

    g = cases.GPT
    logits, gen, gl = ref.gpt(cases.gpt_weights(), g["L"], g["d"], g["H"], g["ffn"], g["vocab"], g["max_pos"], g["eps"],
                              cases.gpt_ids(), g["n_gen"])
    np.savez_compressed(HERE / "gpt_tiny.npz", logits=logits, tokens=gen, gen_logits=gl)
    print("wrote", HERE / "ops.npz", HERE / "gpt_tiny.npz")




def make_dropin_expected(reference_root="/root/reference"):
    """Expected output of tests/dropin/dropin_program.cpp: the program compiled against the reference's headers."""
    import subprocess
    import tempfile
    src = HERE.parent / "dropin" / "dropin_program.cpp"
    with tempfile.TemporaryDirectory() as tmp:
        exe = Path(tmp) / "dropin_ref"
        subprocess.run(["g++", "-std=c++20", "-O2", "-w", "-ffp-contract=off", f"-I{reference_root}", str(src), "-o", str(exe)],
                       check=True)
        out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    (HERE / "dropin_expected.txt").write_text(out)
    print("wrote", HERE / "dropin_expected.txt")


if __name__ == "__main__":
    main()
    make_dropin_expected()
