"""Writes tests/golden/golden.npz: (1) the literal known-answer fixtures of the reference's own tests, (2) oracle outputs on
small seeded inputs for every op of the path.  Run from the repository root:  python tests/golden/make_golden.py

The reference is Go and cannot run in the build image, so (1) is transcribed from its test sources (cited per entry) and
(2) is produced by the CPU oracle after it has been pinned against (1) (tests/test_oracle_golden.py).  The file freezes the
oracle: tests/test_golden_fixtures.py fails if a later oracle edit changes any output, and the GPU tests compare the
kernels with the frozen arrays.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle as O  # noqa: E402


def cases():
    g = {}
    # ---- (1) literal fixtures of the reference ----
    # execution/math_gated_residual_intrinsic_test.go:17-65
    g["ref_gated_residual_res"] = np.arange(1, 13, dtype=np.float32)
    g["ref_gated_residual_mod"] = np.array([0, 0, 0, 0, 0, 0, 0.5, 1, 2, 0, 0, 0, 0, 0, 0, 3, 4, 5], np.float32)
    g["ref_gated_residual_want"] = np.array([1.5, 3, 5, 4.5, 6, 8, 10, 12, 14, 13, 15, 17], np.float32)
    # device/metal/attention/multihead_parity_darwin_test.go:16-37
    g["ref_decode_v"] = np.array([[1, 10], [2, 20], [3, 30]], np.float32)
    g["ref_decode_want"] = np.array([2, 20, 2, 20], np.float32)
    # device/metal/attention/multihead_parity_darwin_test.go:39-67 (inputs; expected = CPU semantics)
    g["ref_prefill_q"] = np.array([0.25, -0.50, 0.75, 0.10, -0.30, 0.20, 0.40, -0.80, 0.60, 0.90, -0.20, 0.35], np.float32).reshape(3, 4)
    g["ref_prefill_k"] = np.array([0.10, 0.20, -0.40, 0.30, 0.50, -0.70], np.float32).reshape(3, 2)
    g["ref_prefill_v"] = np.array([1, 10, 2, 20, 3, 30], np.float32).reshape(3, 2)
    g["ref_prefill_want"] = O.mha(O.F32, g["ref_prefill_q"], g["ref_prefill_k"], g["ref_prefill_v"], 3, 3, 2, 1, 2, True)
    # device/cpu/attention/softmax_test.go:10-40
    g["ref_softmax_in"] = np.array([[1, np.inf, 2], [np.inf, 1, np.inf]], np.float32)
    g["ref_softmax_want"] = np.array([[0, 1, 0], [0.5, 0, 0.5]], np.float32)

    # ---- (2) seeded inputs, oracle outputs ----
    rng = np.random.default_rng(1234)
    x32 = (rng.standard_normal(1024) * 3).astype(np.float32)
    y32 = rng.standard_normal(1024).astype(np.float32)
    g["x32"], g["y32"] = x32, y32
    xb, yb = O.from_f32(x32, O.BF16), O.from_f32(y32, O.BF16)
    g["xb"], g["yb"] = xb, yb
    for name, code in (("silu", O.SILU), ("gelu", O.GELU), ("gelu_tanh", O.GELU_TANH)):
        g[f"{name}_f32"] = O.unary(code, O.F32, x32)
        g[f"{name}_bf16"] = O.unary(code, O.BF16, xb)
    g["swiglu_f32"] = O.gated_tensors(O.SWIGLU, O.F32, x32, y32)
    g["swiglu_bf16"] = O.gated_tensors(O.SWIGLU, O.BF16, xb, yb)
    g["add_bf16"] = O.binary(O.ADD, O.BF16, xb, yb)
    gamma = rng.uniform(0.5, 1.5, 128).astype(np.float32)
    g["gamma"] = gamma
    g["rmsnorm_f32"] = O.rmsnorm(O.F32, x32.reshape(8, 128), gamma, 1e-5)
    g["rmsnorm_bf16"] = O.rmsnorm(O.BF16, xb.reshape(8, 128), O.from_f32(gamma, O.BF16), 1e-6)
    g["rope_f32_llama3_half"] = O.rope(O.F32, x32, 8, 2, 64, base=500000.0, start=3, mode=1, scaling=1, factor=32.0, low=1.0, high=4.0,
                                       orig_ctx=8192)
    g["rope_bf16_interleaved"] = O.rope(O.BF16, xb, 8, 2, 64, base=10000.0)
    f = rng.integers(0, 2**32, 4096, dtype=np.uint64).astype(np.uint32).view(np.float32)
    g["conv_src_f32"] = f
    for name, dt in (("bf16", O.BF16), ("f16", O.F16), ("e4m3", O.E4M3), ("e5m2", O.E5M2)):
        g[f"conv_f32_to_{name}"] = O.convert(f, O.F32, dt)
    g["conv_bf16_all"] = O.convert(np.arange(65536, dtype=np.uint16), O.BF16, O.F32)
    g["conv_f16_all"] = O.convert(np.arange(65536, dtype=np.uint16), O.F16, O.F32)
    g["conv_e4m3_all"] = O.convert(np.arange(256, dtype=np.uint8), O.E4M3, O.F32)
    g["conv_e5m2_all"] = O.convert(np.arange(256, dtype=np.uint8), O.E5M2, O.F32)
    # attention: f32 MHA (GQA, causal), bf16 MHA, flash
    q = rng.standard_normal((16, 4 * 32)).astype(np.float32)
    k = rng.standard_normal((24, 2 * 32)).astype(np.float32)
    v = rng.standard_normal((24, 2 * 32)).astype(np.float32)
    g["att_q"], g["att_k"], g["att_v"] = q, k, v
    g["mha_f32"] = O.mha(O.F32, q, k, v, 16, 24, 4, 2, 32, True)
    g["mha_bf16"] = O.mha(O.BF16, O.from_f32(q, O.BF16), O.from_f32(k, O.BF16), O.from_f32(v, O.BF16), 16, 24, 4, 2, 32, True)
    g["sdpa_f32"] = O.sdpa(O.F32, q[:, :32].copy(), k[:, :32].copy(), v[:, :32].copy(), 16, 24, 32, 32, True)
    # paged decode: 3 sequences, page 16, 8 query heads / 2 KV heads, head_dim 128
    ctx = np.array([40, 7, 100], np.int32)
    pages = int(((ctx + 15) // 16).sum()) + 1
    table = np.zeros((3, 7), np.int32)
    perm = rng.permutation(pages).astype(np.int32)
    at = 0
    for b, n in enumerate((ctx + 15) // 16):
        table[b, :n] = perm[at:at + n]
        at += n
    kp = O.from_f32(rng.standard_normal((pages, 16, 256)).astype(np.float32), O.BF16)
    vp = O.from_f32(rng.standard_normal((pages, 16, 256)).astype(np.float32), O.BF16)
    qd = O.from_f32(rng.standard_normal((3, 8 * 128)).astype(np.float32), O.BF16)
    g["dec_ctx"], g["dec_table"], g["dec_k"], g["dec_v"], g["dec_q"] = ctx, table, kp, vp, qd
    g["dec_out"] = O.paged_decode(O.BF16, O.BF16, qd, kp, vp, table, ctx, 16, 8, 2, 128)
    return g


if __name__ == "__main__":
    O.build()
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden.npz")
    np.savez_compressed(out, **cases())
    print("wrote", out, os.path.getsize(out), "bytes")
