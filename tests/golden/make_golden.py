"""Generates tests/golden/ref_vectors.npz by running the reference's own C code.

    python tests/golden/make_golden.py

Needs oracle/_ref/librpl_ref.so (``make -C oracle``, which compiles the
reference's sources where they lie).  Inputs come from a seeded numpy
generator and are stored with the outputs, so the checks that read the file
need neither the reference nor this script.  The reference ships no golden
vectors of its own for this path; these are facts about what its scalar
x86-64 branch computes.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle.loader import Ref  # noqa: E402


def main():
    R = Ref()
    rng = np.random.default_rng(20240607)
    out = {}

    # --- known-answer vectors: rounding, clamp, zero point ----------------
    kat = np.array([0.5, -0.5, 1.5, 2.5, -2.5, 127.5, -128.5, 300.0], np.float32)
    out["kat_x"] = kat
    out["kat_q_s1_z0"] = R.quantize(kat, 1.0, 0)
    out["kat_q_s1_z5"] = R.quantize(kat, 1.0, 5)
    out["kat_dq_s1_z5"] = R.dequantize(out["kat_q_s1_z5"], 1.0, 5)
    q, s = R.quantize_symmetric(kat)
    out["kat_q_sym"], out["kat_scale_sym"] = q, np.float32(s)

    # --- degenerate and non-finite inputs ----------------------------------
    zeros = np.zeros(8, np.float32)
    q, s = R.quantize_symmetric(zeros)
    out["zeros_q_sym"], out["zeros_scale_sym"] = q, np.float32(s)
    odd = np.array([np.nan, np.inf, -np.inf, 1e20, -1e20, 3e9, -3e9, 1.0], np.float32)
    out["odd_x"] = odd
    out["odd_q_s1_z0"] = R.quantize(odd, 1.0, 0)
    out["odd_q_s1_z7"] = R.quantize(odd, 1.0, 7)
    out["odd_q_s1_zm7"] = R.quantize(odd, 1.0, -7)
    withnan = np.array([1.0, np.nan, -3.0, 2.0, np.nan, 0.25, -0.75, 2.5], np.float32)
    out["withnan_x"] = withnan
    q, s = R.quantize_symmetric(withnan)
    out["withnan_q_sym"], out["withnan_scale_sym"] = q, np.float32(s)
    mn, mx = R.minmax(withnan)
    out["withnan_minmax"] = np.array([mn, mx], np.float32)

    # --- a ragged tensor: N(0,3) with outliers at +/-50 ---------------------
    x = (rng.standard_normal((7, 1031)) * 3.0).astype(np.float32)
    flat = x.reshape(-1)
    idx = rng.choice(flat.size, 8, replace=False)
    flat[idx] = np.where(rng.random(8) < 0.5, -50.0, 50.0).astype(np.float32)
    out["x"] = x
    out["x_minmax"] = np.array(R.minmax(x), np.float32)
    out["x_q_explicit"] = R.quantize(x, 0.05, 3)
    q, s = R.quantize_symmetric(x)
    out["x_q_sym"], out["x_scale_sym"] = q, np.float32(s)
    q, s, z = R.quantize_asymmetric(x)
    out["x_q_asym"], out["x_scale_asym"], out["x_zp_asym"] = q, np.float32(s), np.int32(z)
    q, sc, zp = R.quantize_per_channel(x, 0)
    out["x_q_pc"], out["x_scales_pc"], out["x_zps_pc"] = q, sc, zp
    out["x_dq_sym"] = R.dequantize(out["x_q_sym"], out["x_scale_sym"], 0)
    out["x_dq_asym"] = R.dequantize(out["x_q_asym"], out["x_scale_asym"], int(out["x_zp_asym"]))

    # weights of a small Linear: N(0,0.05), rows of 784 (quantized per output row)
    w = (rng.standard_normal((10, 784)) * 0.05).astype(np.float32)
    out["w"] = w
    q, sc, zp = R.quantize_per_channel(w, 0)
    out["w_q_pc"], out["w_scales_pc"] = q, sc

    # --- contraction ---------------------------------------------------------
    A = rng.integers(-128, 128, (37, 129), dtype=np.int8)
    W = rng.integers(-128, 128, (23, 129), dtype=np.int8)
    bias = rng.integers(-128, 128, 23, dtype=np.int8)
    out["A"], out["W"], out["bias_i8"] = A, W, bias
    out["linear_raw"] = R.linear(A, W)
    out["linear_bias"] = R.linear(A, W, bias)
    B = np.ascontiguousarray(W.T)                       # [K,N] for gemm_int8
    out["gemm_unit"] = R.gemm_requant(A, B)
    out["gemm_scaled"] = R.gemm_requant(A, B, 0.013, 0.021, 0.37)
    out["gemm_zp"] = R.gemm_requant(A, B, 0.013, 0.021, 0.37, 3, -7)
    out["gemm_params"] = np.array([0.013, 0.021, 0.37], np.float32)
    two = np.array([[127, 127]], np.int8)
    twoT = np.array([[127], [127]], np.int8)
    out["gemm_kat"] = np.array([R.gemm_requant(two, twoT)[0, 0], R.gemm_requant(two, twoT, 0.5, 0.5, 2.0)[0, 0],
                                R.gemm_requant(two, twoT, 1, 1, 1, 3, -2)[0, 0]], np.int32)
    relu_in = np.array([-1.0, -0.0, 0.0, 2.5, -np.inf, np.inf, -1e-30, 1e-30], np.float32)
    out["relu_in"], out["relu_out"] = relu_in, R.relu(relu_in)

    path = os.path.join(HERE, "ref_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
