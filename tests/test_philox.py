"""The numpy Philox4x32-10 restatement against the known-answer vectors published with the
Random123 library (kat_vectors: philox4x32 with 10 rounds), and the uniform mapping."""
import numpy as np

from oracle.philox import philox4x32_10, uniforms

KAT = [
    ((0, 0, 0, 0), (0, 0), (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)),
    ((0xffffffff,) * 4, (0xffffffff, 0xffffffff), (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)),
    ((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0),
     (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1)),
]


def test_known_answers():
    for ctr, key, want in KAT:
        got = philox4x32_10(*[[c] for c in ctr], *key)
        assert tuple(int(w[0]) for w in got) == want


def test_uniforms_layout_and_range():
    u = uniforms(1 << 16, 0x123456789abcdef, 1)
    assert u.dtype == np.float32 and u.shape == (1 << 16,)
    assert 0.0 <= u.min() and u.max() < 1.0 and abs(u.mean() - 0.5) < 0.01
    # element e comes from call e // 4, word e % 4, with the mask number in counter word 2
    words = philox4x32_10([5], [0], [1], [0], 0x89abcdef, 0x1234567)
    assert u[21] == np.float32(int(words[1][0]) >> 8) * np.float32(2.0 ** -24)
    assert not np.array_equal(u, uniforms(1 << 16, 0x123456789abcdef, 0))
    assert np.array_equal(uniforms(13, 7, 0), uniforms(16, 7, 0)[:13])
