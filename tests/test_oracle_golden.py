"""The plain-C oracle against the golden vectors produced by the reference's own ggml-cpu (AVX2 build).

Integer and byte results must be identical; float results of the mul_mat and attention restatements are
bit-identical too, because the oracle follows the accumulation order of the AVX2 branch.
"""
import numpy as np

import inputs
from oracle.binding import Q4_0, Q8_0, Q8_AVX2, Q8_SCALAR


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def test_q8_0_activation_quantiser_both_variants(oracle, golden):
    x = inputs.quantizer_rows()
    assert np.array_equal(oracle.quantize_q8_0(x, Q8_AVX2), golden["q8_avx2"])
    assert np.array_equal(oracle.quantize_q8_0(x, Q8_SCALAR), golden["q8_scalar"])
    # the two variants really differ on the tie rows, so the test can tell them apart
    assert not np.array_equal(golden["q8_avx2"], golden["q8_scalar"])


def test_weight_quantisers(oracle, golden):
    w = inputs.small_weights()
    assert np.array_equal(oracle.quantize_weights(Q4_0, w), golden["wq4"])
    assert np.array_equal(oracle.quantize_weights(Q8_0, w), golden["wq8"])


def test_block_dots_exact(oracle, golden):
    xa = inputs.small_activations()
    aq = oracle.quantize_q8_0(xa, Q8_AVX2)
    for name, t in (("q4", Q4_0), ("q8", Q8_0)):
        dots = oracle.block_dots(t, golden["w" + name], aq, xa.shape[1])
        assert np.array_equal(dots, golden["dots_" + name])


def test_small_mul_mat_bit_exact(oracle, golden):
    xa = inputs.small_activations()
    for name, t in (("q4", Q4_0), ("q8", Q8_0)):
        dst, _ = oracle.mul_mat(t, golden["w" + name], xa)
        assert np.array_equal(bits(dst), bits(golden["mm_" + name]))


def test_cfg1_mul_mat(oracle, golden):
    wq = oracle.quantize_weights(Q4_0, inputs.cfg1_weights())
    assert inputs.checksum(wq) == int(golden["cfg1_wq_crc"][0])
    for N in (1, 8):
        dst, _ = oracle.mul_mat(Q4_0, wq, inputs.cfg1_activations(N))
        assert np.array_equal(bits(dst), bits(golden[f"cfg1_n{N}_sample"]))
    # N = 512: the oracle is scalar C, so check a column sample only
    X = inputs.cfg1_activations(512)
    cols = np.arange(0, 4096, inputs.CFG1_SAMPLE_STRIDE)
    dst, _ = oracle.mul_mat(Q4_0, wq[cols], X[:64])
    assert np.array_equal(bits(dst), bits(golden["cfg1_n512_sample"][:64]))


def test_head_q8_0_mul_mat(oracle, golden):
    wq = oracle.quantize_weights(Q8_0, inputs.head_weights())
    dst, _ = oracle.mul_mat(Q8_0, wq, inputs.head_activations())
    assert np.array_equal(bits(dst), bits(golden["head_q8"]))


def test_flash_attn_cases(oracle, golden):
    for name, c in inputs.fattn_cases().items():
        o = oracle.flash_attn_ext(c["q"], c["kc"], c["vc"], c["mask"], c["scale"], n_kv=c["n_kv"],
                                  max_bias=c.get("max_bias", 0.0), softcap=c.get("softcap", 0.0))
        g = golden["fa_" + name]
        assert np.isfinite(g).all()
        # expf/tanhf/powf come from libm on both sides; allow an ulp-level difference across libm builds
        np.testing.assert_allclose(o[c["valid_rows"]], g, rtol=0, atol=2e-6, err_msg=name)


def test_flash_attn_fp16_accumulator_is_visible(oracle):
    """The reference accumulates V in fp16; the double-accumulating mode shows how far that is from the truth."""
    c = inputs.fattn_cases()["d128_gqa4"]
    a = oracle.flash_attn_ext(c["q"], c["kc"], c["vc"], c["mask"], c["scale"], n_kv=c["n_kv"], acc_mode=0)
    b = oracle.flash_attn_ext(c["q"], c["kc"], c["vc"], c["mask"], c["scale"], n_kv=c["n_kv"], acc_mode=1)
    err = np.abs(a - b).max() / np.abs(b).max()
    assert 1e-5 < err < 5e-3


def test_kq_mask_matches_numpy(oracle):
    c = inputs.fattn_cases()["d128_gqa4"]
    m = oracle.build_kq_mask(c["n_kv"], c["cell_pos"][:c["n_kv"]], c["cell_seq"][:c["n_kv"]], c["tok_pos"], c["tok_seq"])
    assert np.array_equal(m, c["mask"])


def test_row_ops(oracle, golden):
    r = inputs.row_op_inputs()
    assert np.array_equal(bits(oracle.rms_norm_mul(r["x"], r["w"], 1e-5)), bits(golden["rms"]))
    assert np.array_equal(bits(oracle.add(r["x"], r["y"])), bits(golden["add"]))
    np.testing.assert_allclose(oracle.rope_norm(r["xr"], r["pos"], 500000.0), golden["rope"], rtol=0, atol=1e-6)
    assert np.array_equal(oracle.cpy_f32_f16(r["x"]), golden["cpy_f16"])
    # K-shift of cached f16 keys: the f32 rotation differs from the reference's by at most the last bit before rounding to
    # f16, so nearly every f16 result is identical and none is more than one f16 step away
    got, want = oracle.rope_norm_f16(r["kf16"], r["shift"], 500000.0), golden["rope_f16"]
    gf, wf = got.view(np.float16).astype(np.float32), want.view(np.float16).astype(np.float32)
    assert (got == want).mean() > 0.999
    assert np.all(np.abs(gf - wf) <= np.spacing(np.abs(wf).astype(np.float16)).astype(np.float32))
    unshifted = r["shift"] == 0
    assert np.array_equal(want[unshifted], r["kf16"][unshifted])   # a zero shift leaves the row as it was
    # the reference's SIMD silu uses a polynomial exp: tolerance only
    np.testing.assert_allclose(oracle.silu_mul(r["x"], r["y"]), golden["silu_mul"], rtol=0, atol=1e-5)


def test_fp16_conversion_against_numpy(oracle):
    rng = np.random.default_rng(7)
    xs = np.concatenate([rng.standard_normal(4000).astype(np.float32) * s for s in (1, 1e-3, 1e-5, 1e-7, 100, 6e4)]
                        + [np.array([0, -0.0, 65504, 65519.99, 65520, 2**-24, 2**-25, 2**-25 * 1.0001, np.inf, -np.inf], np.float32)])
    with np.errstate(over="ignore"):
        want = xs.astype(np.float16).view(np.uint16)
    got = np.array([oracle.L.orc_fp32_to_fp16(float(v)) for v in xs], np.uint16)
    assert np.array_equal(got, want)
    hs = np.arange(0, 0x7C00, dtype=np.uint16)  # all finite non-negative halves
    back = np.array([oracle.L.orc_fp16_to_fp32(int(h)) for h in hs], np.float32)
    assert np.array_equal(back, hs.view(np.float16).astype(np.float32))
