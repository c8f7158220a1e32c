"""The decode work list's cuts (host arithmetic of the library, no GPU): the fixed cuts depend on a sequence's own length only
and still deal the benchmark's ragged batch evenly over the warps."""
import ctypes as C

import numpy as np

from straydog_b200 import _lib
from straydog_b200.synthetic import ragged_lengths


def cuts(lengths, probe=0, warps=148 * 8, fixed=1, kv_heads=2):
    lib = _lib.load()
    n = len(lengths)
    begins = (C.c_uint32 * 4096)()
    stats = (C.c_uint64 * 4)()
    count = lib.sdx_qsa_cuts((C.c_uint64 * n)(*lengths), n, kv_heads, warps, fixed, probe, begins, 4096, stats)
    assert count >= 0, lib.sd_error()
    return list(begins[:count]), dict(zip(("pieces", "warps", "most", "total"), [int(x) for x in stats]))


def test_a_sequences_cuts_do_not_depend_on_its_batch():
    lengths = ragged_lengths(7, 64)
    for probe in (0, 13, 63):
        alone, _ = cuts([lengths[probe]])
        together, _ = cuts(lengths, probe)
        reordered, _ = cuts(lengths[::-1], 63 - probe)
        assert alone == together == reordered
    # the moving cuts do depend on it (which is why they are not the default)
    alone, _ = cuts([lengths[5]], fixed=0)
    together, _ = cuts(lengths, 5, fixed=0)
    assert alone != together


def test_the_cuts_cover_every_key_once_in_tile_steps():
    for length in (1, 15, 16, 17, 100, 511, 8191, 8192, 8193, 32767, 32768):
        begins, stats = cuts([length])
        assert begins[0] == 0 and all(b % 16 == 0 for b in begins) and sorted(set(begins)) == begins
        assert stats["total"] == 2 * ((length + 15) // 16)
        assert begins[-1] < length


def test_the_ragged_batch_is_dealt_evenly():
    lengths = ragged_lengths(20261125, 64)
    _, stats = cuts(lengths)
    mean = stats["total"] / stats["warps"]
    assert stats["warps"] == 148 * 8
    assert stats["most"] <= 1.03 * mean + 1, (stats, mean)
    _, moving = cuts(lengths, fixed=0)
    assert stats["pieces"] < 4 * moving["pieces"]
    # a short batch still spreads over many warps
    _, small = cuts([4096])
    assert small["warps"] >= 48 and small["most"] <= 16
