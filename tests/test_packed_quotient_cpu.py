"""The packed f16x2 quotient the int8 quantisation kernels use, replayed in numpy for every pair of
11-bit significands: q = x' * r; rem = fma(-q, s', x'); q' = fma(rem, r, q) with r = f16(1 / s') must
be the correctly rounded fp16 quotient wherever it decides an int8 code (0.25 <= |x'/s'| <= 128)."""
import numpy as np

F16 = np.float16


def _rn16(a64):
    return a64.astype(F16)


def _fma16(a, b, c):
    # 11-bit x 11-bit + 11-bit of similar magnitude is exact in float64, so this rounds once
    return _rn16(a.astype(np.float64) * b.astype(np.float64) + c.astype(np.float64))


def test_packed_quotient_is_correctly_rounded_for_all_significands():
    sig = np.arange(1024, 2048, dtype=np.float64) / 1024.0
    sp = sig.astype(F16)[:, None]                                   # s' in [1, 2)
    r = (np.float32(1.0) / sp.astype(np.float32)).astype(F16)        # f16(1 / s') as the kernel forms it
    checked = 0
    for e in range(-3, 8):
        xp = (sig * 2.0 ** e).astype(F16)[None, :]
        t = xp.astype(np.float64) / sp.astype(np.float64)
        want = _rn16(t)
        q = _rn16(xp.astype(np.float64) * r.astype(np.float64))
        rem = _fma16(-q, np.broadcast_to(sp, q.shape), np.broadcast_to(xp, q.shape))
        q2 = _fma16(rem, np.broadcast_to(r, q.shape), q)
        sel = (t >= 0.25) & (t <= 128.0)
        assert not np.any((q2 != want) & sel), f"exponent {e}"
        checked += int(sel.sum())
    assert checked > 9_000_000


def test_fp32_rounding_in_the_middle_is_harmless():
    """torch divides in fp32 and then rounds to fp16; for fp16 operands that equals rounding once."""
    rng = np.random.default_rng(0)
    x = rng.standard_normal(1 << 20).astype(F16)
    s = np.abs(rng.standard_normal(1 << 20)).astype(F16) + F16(1e-3)
    twice = (x.astype(np.float32) / s.astype(np.float32)).astype(F16)
    once = (x.astype(np.float64) / s.astype(np.float64)).astype(F16)
    assert np.array_equal(twice.view(np.uint16), once.view(np.uint16))
