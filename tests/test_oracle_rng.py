"""CPU: Philox4x32-10 known answers and the per-row state model (reference: sampling.cu:9, :136-144, :383)."""
import struct

import numpy as np

from oracle import c_oracle as co
from oracle import philox_py as pp

# Known-answer vectors published with the Philox paper's reference implementation (counter, key, output).
KATS = [
    ((0, 0, 0, 0), (0, 0), (0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8)),
    ((0xFFFFFFFF,) * 4, (0xFFFFFFFF,) * 2, (0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD)),
    ((0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344), (0xA4093822, 0x299F31D0),
     (0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1)),
]


def test_philox_known_answers():
    for ctr, key, exp in KATS:
        assert pp.philox4x32_10(ctr, key) == exp
        assert co.philox4x32_10(ctr, key) == exp


def test_state_layout_and_subsequence():
    seed = 0x1234_5678_9ABC_DEF0
    st = co.setup_rand(seed, 5)
    assert st.dtype == np.int8 and st.size == 5 * 64
    for row in range(5):
        raw = st[64 * row:64 * row + 64].tobytes()
        assert raw == pp.state_bytes(seed, row)
        words = struct.unpack("<16I", raw)
        assert words[0:4] == (0, 0, row, 0)                       # counter: subsequence in the high half
        assert words[8:10] == (seed & 0xFFFFFFFF, seed >> 32)     # key = seed
        assert words[10:] == (0,) * 6                             # pos and the unused Box-Muller words


def test_first_row_offset_matches_unsharded():
    full = co.setup_rand(7, 16)
    part = co.setup_rand(7, 4, row0=8)
    assert np.array_equal(full[8 * 64:12 * 64], part)


def test_draw_sequence_and_state_advance():
    seed, row = 42, 3
    st = co.setup_rand(seed, 4)
    for n in range(5):
        assert co.draw4(st, row) == pp.block(seed, row, n)
        assert st[64 * row:64 * row + 64].tobytes() == pp.state_bytes(seed, row, n + 1)
    # other rows untouched
    assert st[0:64].tobytes() == pp.state_bytes(seed, 0)


def test_uniform_mapping_is_half_open_at_zero():
    assert co.uniform(0) == 2.0 ** -33
    assert co.uniform(0xFFFFFFFF) == 1.0          # rounds up to exactly 1.0f: the range is (0, 1]
    assert co.uniform(1 << 31) == np.float32(0.5) + np.float32(2.0 ** -33)
