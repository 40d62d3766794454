"""Host-side checks of two identities the kernels' dropout path rests on
(flash-attention_b200/csrc/fa_dropout.cuh): the float keep factor and the mirrored Philox state."""
import numpy as np

from oracle import attention_oracle as orc


def _keep_factor(bits16, threshold, junk_byte):
    """What fa_keep_factor_lo / _hi compute: the 16 random bits become bytes 2..1 of a float whose
    top byte is 0x3F (byte 0 is filler: zero for the low half, the neighbour's top byte for the
    high half), then sat(x * -2^24 + T * 2^24) in fp32 with a single rounding (fma)."""
    x = (np.uint32(0x3F000000) + (bits16.astype(np.uint32) << 8) + np.uint32(junk_byte)).astype(np.uint32)
    t = np.array([0x3F000000 + ((threshold + 1) << 8)], dtype=np.uint32).view(np.float32)[0]
    thr_term = np.float32(t) * np.float32(16777216.0)
    assert float(thr_term) == float(t) * 16777216.0          # exact: a power-of-two scale
    exact = x.view(np.float32).astype(np.float64) * -16777216.0 + np.float64(thr_term)   # exact in fp64
    return np.clip(exact.astype(np.float32), 0.0, 1.0)


def test_keep_factor_is_exactly_the_integer_compare():
    u = np.arange(65536, dtype=np.uint32)
    for p_drop in (0.0, 0.1, 0.17, 0.5, 0.9, 0.999):
        thr = orc.dropout_threshold(p_drop)
        for junk in (0x00, 0x5A, 0xFF):
            k = _keep_factor(u, thr, junk)
            assert np.array_equal(k, (u <= thr).astype(np.float32)), (p_drop, junk)
    for thr in (0, 1, 0x7BFF, 0x7C00, 0x7FFF, 0x8000, 0xFBFF, 0xFC00, 65534, 65535):
        assert np.array_equal(_keep_factor(u, thr, 0xA7), (u <= thr).astype(np.float32)), thr


M0, M1 = 0xD2511F53, 0xCD9E8D57
W0, W1 = 0x9E3779B9, 0xBB67AE85
MASK = 0xFFFFFFFF


def _lane_round(s, mul_a, mul_b, key_a, key_b):
    """LanePhilox::round: word 0 is multiplied by mul_a, word 2 by mul_b."""
    p0, p1 = mul_a * s[0], mul_b * s[2]
    return [(p1 >> 32) ^ s[1] ^ key_a, p1 & MASK, (p0 >> 32) ^ s[3] ^ key_b, p0 & MASK]


def test_mirrored_state_runs_the_same_generator():
    """Running the rounds on (c2, c3, c0, c1) with multipliers and keys swapped yields the mirror
    of the ordinary result, so the lane of the upper row can keep words 0, 1 like its partner."""
    rng = np.random.RandomState(7)
    for _ in range(200):
        c = [int(v) for v in rng.randint(0, 2 ** 32, size=4, dtype=np.uint64)]
        k0, k1 = (int(v) for v in rng.randint(0, 2 ** 32, size=2, dtype=np.uint64))
        a, s = list(c), [c[2], c[3], c[0], c[1]]
        for r in range(7):
            ka, kb = (k0 + r * W0) & MASK, (k1 + r * W1) & MASK
            a = _lane_round(a, M0, M1, ka, kb)
            s = _lane_round(s, M1, M0, kb, ka)
        assert s == [a[2], a[3], a[0], a[1]]
        # and the ordinary orientation is the oracle's generator
        want = orc.philox4x32(np.array(c, dtype=np.uint32), (k0, k1), rounds=7)
        assert a == [int(v) for v in want]
