"""The oracle's drafter block attention (orc_dspark_attention) against an independent numpy F64 restatement of the reference
test's own oracle (crates/straydog-engine/tests/dspark_attention_gpu.rs:25-39), on that test's inputs."""
import numpy as np

import oracle
from straydog_b200.synthetic import dspark_case


def numpy_reference(q, ring, block, sinks, heads, slots, anchor, history):
    keys = np.concatenate([ring[[p % 128 for p in range(anchor - history, anchor)]], block[:slots]]).astype(np.float64)
    out = np.empty((slots, heads, 512))
    for s in range(slots):
        for h in range(heads):
            scores = keys @ q[s, h].astype(np.float64) / np.sqrt(512.0)
            top = max(float(sinks[h]), scores.max())
            w = np.exp(scores - top)
            out[s, h] = w @ keys / (w.sum() + np.exp(float(sinks[h]) - top))
    return out


def test_matches_the_reference_tests_f64_oracle():
    c = dspark_case()
    for slots, history, anchor, heads in [(1, 0, 0, 64), (5, 37, 149, 64), (3, 128, 389, 64), (4, 37, 149, 32)]:
        # (a device's half of the heads reads q as [slots][32][512]: the first slots * 32 rows of the buffer)
        q = c["q"].reshape(-1, 512)[:slots * heads].reshape(slots, heads, 512)
        want = numpy_reference(q, c["ring"], c["block"], c["sinks"], heads, slots, anchor, history)
        for f64 in (True, False):
            got = oracle.dspark_attention(q, c["ring"], c["block"], c["sinks"], heads, slots, anchor, history, f64=f64)
            error = np.abs(got - want) / (1.0 + np.abs(want))
            assert error.max() <= (1e-6 if f64 else 2e-5), (slots, history, f64, error.max())


def test_the_sink_takes_its_share_of_the_denominator():
    # zero queries: every key scores 0; five keys 1..5 and a sink of 0 give (1 + 2 + 3 + 4 + 5) / 6
    q = np.zeros((5, 2, 512), np.float32)
    ring = np.full((128, 512), 23.0, np.float32)
    block = np.repeat(np.arange(1, 6, dtype=np.float32)[:, None], 512, 1)
    assert np.allclose(oracle.dspark_attention(q, ring, block, np.zeros(2, np.float32), 2, 5, 0, 0), 2.5)
    assert np.allclose(oracle.dspark_attention(q, ring, block, np.full(2, 1000.0, np.float32), 2, 5, 0, 0), 0.0)
    assert np.allclose(oracle.dspark_attention(q, ring, block, np.full(2, -1000.0, np.float32), 2, 5, 0, 0), 3.0)
