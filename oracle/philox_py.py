"""Pure-Python Philox4x32-10 (Salmon et al., SC'11) and the cuRAND-style per-row state model.

TEST INFRASTRUCTURE ONLY.  Written from the published algorithm; used for known-answer tests of
the C oracle and of the GPU ``setup_rand`` (reference: sampling.cu:9, :136-144; one 4-word block
is consumed per sampling call, sampling.cu:383).
"""
M0, M1 = 0xD2511F53, 0xCD9E8D57
W0, W1 = 0x9E3779B9, 0xBB67AE85
MASK = 0xFFFFFFFF


def philox4x32_10(ctr, key):
    c0, c1, c2, c3 = ctr
    k0, k1 = key
    for _ in range(10):
        p0 = M0 * c0
        p1 = M1 * c2
        c0, c1, c2, c3 = ((p1 >> 32) ^ c1 ^ k0) & MASK, p1 & MASK, ((p0 >> 32) ^ c3 ^ k1) & MASK, p0 & MASK
        k0 = (k0 + W0) & MASK
        k1 = (k1 + W1) & MASK
    return (c0, c1, c2, c3)


def block(seed, row, n):
    """The n-th 4-word block handed to row ``row`` of a state created with ``setup_rand(seed, B)``."""
    ctr = (n & MASK, (n >> 32) & MASK, row & MASK, (row >> 32) & MASK)
    return philox4x32_10(ctr, (seed & MASK, (seed >> 32) & MASK))


def state_bytes(seed, row, n=0):
    """64-byte state of ``row`` after n sampling calls (layout: ctr[4] out[4] key[2] pos + 5 zero words)."""
    import struct
    ctr = (n & MASK, (n >> 32) & MASK, row & MASK, (row >> 32) & MASK)
    key = (seed & MASK, (seed >> 32) & MASK)
    return struct.pack("<10I", *ctr, *philox4x32_10(ctr, key), *key) + b"\0" * 24
