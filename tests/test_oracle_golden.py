"""Pin the CPU oracle against outputs of the reference itself.

The ``.npz`` fixtures were produced by ``tests/golden/make_golden.py`` calling
the reference's functions; every comparison on integer/fp16 elementwise work
is bit for bit.  The int4 known-answer vector is the one the reference's own
``tests/test_vllm_real_quant_export.py:30-40`` uses.
"""
import numpy as np
import pytest

from oracle import pseudo_quant as O


def bits(a):
    return np.ascontiguousarray(a).view(np.uint16)


@pytest.mark.parametrize("suffix", ["", "_ragged", "_const"])
def test_w4_group_asym_matches_reference_bitwise(golden, suffix):
    g = golden("w4a16_small.npz")
    wdq, s, z, u = O.w4_group_asym_quantize(g["w" + suffix], 128)
    assert np.array_equal(bits(wdq), bits(g["wdq" + suffix]))
    assert np.array_equal(bits(s), bits(g["scales" + suffix]))
    assert np.array_equal(bits(z), bits(g["zeros" + suffix]))
    assert u.min() >= 0 and u.max() <= 15


def test_w4_pack_dequant_round_trip_is_reference_wdq(golden):
    g = golden("w4a16_small.npz")
    wdq, s, z, u = O.w4_group_asym_quantize(g["w"], 128)
    packed = O.pack_int4_unsigned(u)
    zp = O.pack_int4_unsigned(z.astype(np.uint8))
    assert packed.dtype == np.int32 and packed.shape == (24, 48)
    back = O.w4_dequant(packed, s, zp, 24, 384, 128)
    assert np.array_equal(bits(back), bits(g["wdq"]))
    y = O.linear_f16(g["x"], back)
    assert O.rel_frobenius(y, g["y"]) < 1e-3


def test_int4_pack_known_answer_vectors(golden):
    g = golden("int4_pack.npz")
    kat = g["kat"]
    assert kat.tolist() == [[-8, -7, -1, 0, 1, 6, 7, -3, 4, 2]]
    p = O.pack_int4_signed(kat)
    assert p.dtype == np.int32 and p.shape == (1, 2)
    assert np.array_equal(p, g["kat_packed"])
    assert np.array_equal(O.unpack_int4_signed(p, 10), kat)
    assert np.array_equal(O.pack_int4_signed(g["q"]), g["q_packed"])
    assert np.array_equal(O.unpack_int4_signed(g["q_packed"], 40), g["q_unpacked"])
    with pytest.raises(ValueError):
        O.pack_int4_signed(np.array([[9]], dtype=np.int8))
    with pytest.raises(ValueError):
        O.pack_int4_signed(np.zeros((2, 2, 2), dtype=np.int8))


def test_symmetric_export_dequant_matches_reference(golden):
    g = golden("int4_pack.npz")
    w = O.w4_dequant(g["q_packed"], g["scale"], None, 6, 40, 8)
    assert np.array_equal(bits(w), bits(g["q_dequant_f32"].astype(np.float16)))


def test_gptq_artifact_reconstructs_fake_weight(golden):
    g = golden("gptq_artifact.npz")
    assert g["int_weight"].min() >= -8 and g["int_weight"].max() <= 7
    assert np.array_equal(O.pack_int4_signed(g["int_weight"]), g["packed"])
    rec = g["int_weight"].astype(np.float32) * np.repeat(g["scale"], 32, axis=1)
    assert np.allclose(rec, g["fake_weight"], atol=1e-6, rtol=0)
    w16 = O.w4_dequant(g["packed"], g["scale"].astype(np.float16), None, 16, 64, 32)
    ref16 = (g["int_weight"].astype(np.float32)
             * np.repeat(g["scale"].astype(np.float16).astype(np.float32), 32, axis=1)).astype(np.float16)
    assert np.array_equal(bits(w16), bits(ref16))


def test_act_and_weight_absmax_quant_bitwise(golden):
    g = golden("w8a8_small.npz")
    fake, codes, s = O.absmax_quant_last_dim(g["x"])
    assert np.array_equal(bits(fake), bits(g["x_fake"]))
    assert np.abs(codes.astype(np.int32)).max() <= 127
    # through int8 the sign of a zero code is lost, so compare values, not bit patterns
    assert np.array_equal((codes.astype(np.float16) * s).astype(np.float16), g["x_fake"])
    assert float(s[5, 0]) == float(np.float16(np.float16(1e-5) / np.float16(127)))   # all-zero token
    wfake, _, _ = O.absmax_quant_last_dim(g["w"])
    assert np.array_equal(bits(wfake), bits(g["w_fake"]))
    q, sc, off = O.weight_quant_per_channel_fp32(g["w"])
    assert np.array_equal(q, g["exp_q"])
    assert np.array_equal(bits(sc), bits(g["exp_scale"]))
    assert np.array_equal(bits(off), bits(g["exp_offset"]))


def test_smoothquant_linear_forward(golden):
    g = golden("w8a8_small.npz")
    wfake, qw, sw = O.absmax_quant_last_dim(g["w"])
    y = O.smoothquant_linear_forward(g["x"], wfake, g["bias"])
    assert O.rel_frobenius(y, g["y"]) < 1e-3
    yq = O.smoothquant_linear_forward(g["x"], wfake, g["bias"], quantize_output=True)
    assert O.rel_frobenius(yq, g["y_outq"]) < 5e-3
    # the real-int pipeline (int32 accumulate, scale epilogue) stays within the stated 1e-2
    _, qx, sx = O.absmax_quant_last_dim(g["x"])
    yi = O.w8a8_int_forward(qx, sx, qw, sw, g["bias"])
    assert O.rel_frobenius(yi, g["y"]) < 1e-2


def test_router_top2_matches_reference(golden):
    g = golden("moe_small.npz")
    idx, w = O.router_top2(g["logits"], 2)
    assert np.array_equal(idx, g["top_k_index"])
    assert np.allclose(w.astype(np.float32), g["top_k_weights"].astype(np.float32), atol=1e-3)
    assert (idx != 3).all()


def test_moe_experts_forward(golden):
    g = golden("moe_small.npz")
    guf, _, _ = O.absmax_quant_last_dim(g["gate_up"])
    dnf, _, _ = O.absmax_quant_last_dim(g["down"])
    assert np.array_equal(bits(guf), bits(g["gate_up_fake"]))
    assert np.array_equal(bits(dnf), bits(g["down_fake"]))
    out = O.moe_experts_forward(g["hidden"], g["top_k_index"], g["top_k_weights"], guf, dnf)
    assert O.rel_frobenius(out, g["out"]) < 2e-3


def test_omniquant_affine_quantizer_bitwise(golden):
    g = golden("omniquant_small.npz")
    for key in ("x", "w"):
        fake, codes, s, zp = O.affine_quant_last_dim(g[key])
        assert np.array_equal(bits(fake), bits(g[key + "_fake"]))
        assert np.array_equal(bits(s), bits(g[key + "_scale"]))
        assert np.array_equal(bits(zp), bits(g[key + "_zp"]))
        assert codes.min() >= 0 and codes.max() <= 255
    y = O.omniquant_linear_forward(g["x"], g["w"], g["bias"])
    assert O.rel_frobenius(y, g["y"]) < 1e-3
