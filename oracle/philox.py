"""TEST INFRASTRUCTURE - Philox4x32-10 counter-based generator in numpy.

Restates the published algorithm (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy
as 1, 2, 3", SC'11): ten rounds of two 32x32->64 multiplications (constants 0xD2511F53,
0xCD9E8D57) with the key bumped by the Weyl constants 0x9E3779B9 / 0xBB67AE85 after each round.
The reference's dropout-fused oracles draw their masks with Triton's ``tl.rand`` (the same
generator; e.g. repros/canonical/mean_014afd4984e6/oracle.py:60-75); its eager modules draw with
``prims.inductor_random``, so masks are stochastic outputs for the reference's check and the
counter layout below is this backend's own: counter = (element index // 4 as 64 bits, mask
number, 0), key = the 64-bit seed, the four words of one call going to four consecutive elements,
uniform = (word >> 8) * 2^-24.

Only tests may import this module.
"""
import numpy as np

_M0, _M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
_W0, _W1 = 0x9E3779B9, 0xBB67AE85
_LO = np.uint64(0xFFFFFFFF)
_S32 = np.uint64(32)


def philox4x32_10(c0, c1, c2, c3, k0: int, k1: int):
    """Arrays of 32-bit counter words (held in uint64) and a scalar key -> four arrays of 32-bit words."""
    c0, c1, c2, c3 = (np.asarray(c, dtype=np.uint64) for c in (c0, c1, c2, c3))
    for _ in range(10):
        p0, p1 = _M0 * c0, _M1 * c2
        c0, c1, c2, c3 = ((p1 >> _S32) ^ c1 ^ np.uint64(k0), p1 & _LO,
                          (p0 >> _S32) ^ c3 ^ np.uint64(k1), p0 & _LO)
        k0, k1 = (k0 + _W0) & 0xFFFFFFFF, (k1 + _W1) & 0xFFFFFFFF
    return c0, c1, c2, c3


def uniforms(numel: int, seed: int, which: int) -> np.ndarray:
    """float32 uniforms in [0, 1) for elements 0..numel-1 of mask number ``which``."""
    seed &= 0xFFFFFFFFFFFFFFFF
    groups = np.arange((numel + 3) // 4, dtype=np.uint64)
    words = philox4x32_10(groups & _LO, groups >> _S32, np.full_like(groups, which), np.zeros_like(groups),
                          seed & 0xFFFFFFFF, seed >> 32)
    bits = np.stack(words, axis=1).reshape(-1)[:numel]
    return ((bits >> np.uint64(8)).astype(np.float32) * np.float32(2.0 ** -24)).astype(np.float32)
