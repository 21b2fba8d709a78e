"""Generates the golden vectors in this directory by running the reference's own ggml-cpu code.

The reference ships no tests, fixtures or known-answer vectors for this path, so these files are the
pin: they are produced by the reference compiled unmodified from its sources (oracle/_ref, built by
oracle/Makefile with -O3 -mavx2 -mfma -mf16c) on seeded inputs.  Run from the repository root on a
machine that has a checkout of the reference:

    python tests/golden/make_golden.py

Inputs are regenerated from the seeds by tests/inputs.py, so only outputs (or small samples of large
outputs) are stored.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import inputs  # noqa: E402
from oracle.binding import Q4_0, Q8_0, Q8_AVX2, Q8_SCALAR, Reference  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    ref = Reference.load()
    assert ref is not None, "the reference must be compiled (oracle/_ref) to generate golden vectors"
    out = {}

    # --- quantisers ---------------------------------------------------------------------------
    x = inputs.quantizer_rows()
    out["q8_avx2"] = ref.quantize_q8_0(x, Q8_AVX2)
    out["q8_scalar"] = ref.quantize_q8_0(x, Q8_SCALAR)
    w = inputs.small_weights()
    out["wq4"] = ref.quantize_weights(Q4_0, w)
    out["wq8"] = ref.quantize_weights(Q8_0, w)

    # --- small mul_mat, full outputs, plus exact block dots ---------------------------------------
    xa = inputs.small_activations()
    for name, t in (("q4", Q4_0), ("q8", Q8_0)):
        wq = out["w" + name]
        dst, _ = ref.mul_mat(t, wq, xa, n_threads=2)
        out[f"mm_{name}"] = dst
        # integer dots: with both block scales forced to 1.0 the reference's vec_dot over one block
        # returns the int32 dot exactly
        aq = ref.quantize_q8_0(xa, Q8_AVX2)
        K = xa.shape[1]
        bw = 18 if t == Q4_0 else 34
        dots = np.empty((xa.shape[0], wq.shape[0], K // 32), np.int32)
        one = np.array([0x3C00], np.uint16).view(np.uint8)
        for n in range(xa.shape[0]):
            for m in range(wq.shape[0]):
                for b in range(K // 32):
                    wb = wq[m, b * bw:(b + 1) * bw].copy()
                    ab = aq[n, b * 34:(b + 1) * 34].copy()
                    wb[:2] = one
                    ab[:2] = one
                    dots[n, m, b] = int(ref.vec_dot(t, wb, ab, 32))
        out[f"dots_{name}"] = dots

    # --- config 1 (4096 x 4096 Q4_0, N in {1, 8, 512}): samples of the outputs -----------------------
    W = inputs.cfg1_weights()
    wq = ref.quantize_weights(Q4_0, W)
    out["cfg1_wq_crc"] = np.array([inputs.checksum(wq)], np.uint64)
    for N in (1, 8, 512):
        X = inputs.cfg1_activations(N)
        dst, _ = ref.mul_mat(Q4_0, wq, X, n_threads=8)
        out[f"cfg1_n{N}_sample"] = dst[:, ::inputs.CFG1_SAMPLE_STRIDE].copy() if N > 8 else dst
        out[f"cfg1_n{N}_sum"] = np.array([dst.astype(np.float64).sum(), np.abs(dst).astype(np.float64).sum()])

    # --- Q8_0 weights at an lm_head-like shape --------------------------------------------------
    W8 = inputs.head_weights()
    wq8 = ref.quantize_weights(Q8_0, W8)
    X8 = inputs.head_activations()
    dst, _ = ref.mul_mat(Q8_0, wq8, X8, n_threads=8)
    out["head_q8"] = dst

    # --- flash attention ------------------------------------------------------------------------
    for name, case in inputs.fattn_cases().items():
        o, _ = ref.flash_attn_ext(case["q"], case["kc"], case["vc"], case["mask"], case["scale"], n_kv=case["n_kv"],
                                  max_bias=case.get("max_bias", 0.0), softcap=case.get("softcap", 0.0), n_threads=8)
        valid = case["valid_rows"]
        out[f"fa_{name}"] = o[valid]

    # --- row ops ---------------------------------------------------------------------------------
    r = inputs.row_op_inputs()
    out["rms"] = ref.row_op(0, r["x"], r["w"], 1e-5)
    out["silu_mul"] = ref.row_op(1, r["x"], r["y"])
    out["add"] = ref.row_op(2, r["x"], r["y"])
    out["rope"] = ref.row_op(3, r["xr"], r["pos"], 500000.0)
    out["cpy_f16"] = ref.row_op(4, r["x"], None, out_dtype=np.uint16)
    out["rope_f16"] = ref.row_op(5, r["kf16"], r["shift"], 500000.0, out_dtype=np.uint16)

    path = os.path.join(HERE, "golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes;", len(out), "arrays")


if __name__ == "__main__":
    main()
