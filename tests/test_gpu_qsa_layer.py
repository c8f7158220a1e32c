"""The Qwen attention layer behind its projections, held to the reference's own library: tests/golden/reference_b200_qsa.npz holds what
sd_qsa_sequence (gpu/sparse_attention.hpp:441-512) left behind on a B200 when its six weight matrices are selection matrices (a 1 a row: the
projections are then exact copies of input columns, whatever order its GEMV sums in, and the output is the first ten heads' gated attention).
This library's three calls over the same projections (sdx_qsa_normalize_chunk, sdx_qsa_index_select, sdx_qsa_attention_rows) must leave the
same K/V rows, the same indexer columns and ring bit for bit, choose the blocks the reference's block scores choose, and give its output
(within FP32 summation order for one token; within the FP16 rounding of the reference's own prompt kernel for a chunk)."""
import os

import numpy as np
import pytest

from util import QSA_SEQUENCE_CASES, close, qsa_sequence_case

pytestmark = pytest.mark.gpu
GOLDEN = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_b200_qsa.npz"))
SELECTED, HEADS, KV_HEADS = 2052, 24, 2


def lists_from(scores, position):
    """The rule of gpu/sparse_attention.hpp:172-243 over given block scores: (positions listed, count)."""
    complete = (position + 1) // 4
    if complete <= 512:
        return np.arange(position + 1), position + 1
    order = np.argsort(-scores[:complete].astype(np.float64), kind="stable")[:512]   # (stable: equal scores by lowest block)
    kept = np.sort(order)
    listed = np.concatenate([(kept[:, None] * 4 + np.arange(4)).ravel(), np.arange(complete * 4, position + 1)])
    return listed, len(listed)


@pytest.mark.parametrize("context,position,steps,seed", QSA_SEQUENCE_CASES)
def test_the_layer_behind_its_projections_equals_the_reference_librarys(gpu, context, position, steps, seed):
    c = qsa_sequence_case(context, position, steps, seed)
    key = f"qsa_{context}_{position}_{steps}_{seed}"
    names = ("qgate", "key", "value", "iq", "ik", "state", "index_state")
    bufs = {n: gpu.upload(c[n]) for n in names}
    norms = [gpu.upload(n) for n in c["norms"]]
    packed = gpu.buffer(steps * (HEADS * 256 + KV_HEADS * 512 + SELECTED + 1) * 4)
    out = gpu.buffer(steps * HEADS * 256 * 4)
    gpu.qsa_normalize_chunk(bufs["qgate"].pointer, bufs["key"].pointer, bufs["value"].pointer, bufs["iq"].pointer, bufs["ik"].pointer, steps, position,
                            HEADS, KV_HEADS, *[n.pointer for n in norms], packed.pointer, SELECTED, bufs["state"], context, bufs["index_state"].pointer)
    gpu.qsa_index_select(bufs["iq"].pointer, 512, bufs["index_state"].pointer, c["pool"], position, None, steps, SELECTED, HEADS, KV_HEADS, packed.pointer)
    gpu.qsa_attention_rows(bufs["state"], context, position, None, steps, SELECTED, HEADS, KV_HEADS, 0.0625, packed.pointer, out.pointer,
                           gates=(bufs["qgate"].pointer, HEADS * 512))
    assert gpu.decode_status() == 0
    rows = gpu.read(bufs["state"], np.uint8, (4, context, 272))[:, position:position + steps]
    assert np.array_equal(rows, GOLDEN[key + "_rows"]), "the K/V rows of the chunk: normalised, rotated keys and the values, Q8_0, bit for bit"
    index_after = gpu.read(bufs["index_state"], np.float32, c["index_state"].shape)
    blocks = index_after[:c["pool"] * 128].reshape(128, c["pool"])[:, position // 4:(position + steps) // 4]
    assert np.array_equal(blocks.view(np.uint32), GOLDEN[key + "_blocks"].view(np.uint32)), "the pooled blocks the chunk completed"
    assert np.array_equal(index_after[c["pool"] * 128:].view(np.uint32), GOLDEN[key + "_ring"].view(np.uint32)), "the history ring"
    got_packed = gpu.read(packed, np.float32, (steps * (HEADS * 256 + KV_HEADS * 512 + SELECTED + 1),))
    start = steps * (HEADS * 256 + KV_HEADS * 512)
    if key + "_scores" in GOLDEN:   # the block choice ran: this library's lists are the rule's over the reference's block scores
        for t in range(steps):
            listed, count = lists_from(GOLDEN[key + "_scores"][t], position + t)
            assert got_packed[start + steps * SELECTED + t] == count
            assert np.array_equal(got_packed[start + t * SELECTED:start + t * SELECTED + count], listed.astype(np.float32)), t
    got = gpu.read(out, np.float32, (steps, HEADS, 256))[:, :10].reshape(steps, 2560)
    # one token: the reference attends in FP32 (qsa_decode_parts) and the two differ by summation order; a chunk: its prompt kernel rounds
    # K, V and the weights to FP16 (qsa_flash_mma, gpu/sparse_attention_compute.hpp:416-584; its own figure: 4.8e-4 at worst), this
    # library's selection kernel does not
    ok, worst = close(got, GOLDEN[key + "_out"])
    assert ok and worst < (1e-4 if steps == 1 else 2e-3), worst
    for b in list(bufs.values()) + norms + [packed, out]:
        gpu.release(b)


def test_the_dense_decode_at_the_reference_layers_heads_equals_its_output(gpu):
    # sdx_qsa_decode at Qwen's own geometry (24 query / 2 K/V heads: groups of 12, taken as two halves of six) over every position of a
    # sequence is the layer's decode step while it lists every position (up to 512 blocks): the reference's output for such a step, after
    # the front has written the token's row; the queries reach the dense kernel as FP16, which is what separates the two
    context, position, steps, seed = 2048, 1500, 1, 5
    c = qsa_sequence_case(context, position, steps, seed)
    key = f"qsa_{context}_{position}_{steps}_{seed}"
    bufs = {n: gpu.upload(c[n]) for n in ("qgate", "key", "value", "iq", "ik", "state", "index_state")}
    norms = [gpu.upload(n) for n in c["norms"]]
    packed = gpu.buffer((HEADS * 256 + KV_HEADS * 512 + SELECTED + 1) * 4)
    gpu.qsa_normalize_chunk(bufs["qgate"].pointer, bufs["key"].pointer, bufs["value"].pointer, bufs["iq"].pointer, bufs["ik"].pointer, 1, position,
                            HEADS, KV_HEADS, *[n.pointer for n in norms], packed.pointer, SELECTED, bufs["state"], context, bufs["index_state"].pointer)
    queries = gpu.read(packed, np.float32, (HEADS * 256,))
    q16, out = gpu.upload(queries.astype(np.float16)), gpu.buffer(HEADS * 256 * 4)
    gpu.qsa_decode([bufs["state"]], [context], [position + 1], HEADS, KV_HEADS, 0.0625, q16.pointer, out.pointer)
    assert gpu.decode_status() == 0
    gate = c["qgate"].reshape(HEADS, 512)[:, 256:].astype(np.float64)
    got = (gpu.read(out, np.float32, (HEADS, 256)) / (1 + np.exp(-gate)))[:10].reshape(1, 2560)
    ok, worst = close(got, GOLDEN[key + "_out"])
    assert ok and worst < 5e-4, worst
    for b in list(bufs.values()) + norms + [packed, q16, out]:
        gpu.release(b)


def test_the_prompt_kernel_at_the_reference_layers_heads_equals_its_output(gpu):
    # sdx_qsa_prompt (tcgen05) at 24 query / 2 K/V heads (groups of 12: ten tokens a block of 120 rows) over a chunk whose every position is
    # listed is the layer's prompt attention: the reference's output for the chunk, after the front has written the chunk's rows. Both sides
    # round on the way (the reference's prompt kernel K, V and the weights to FP16; this one the queries and the weights)
    context, position, steps, seed = 1024, 100, 60, 6
    c = qsa_sequence_case(context, position, steps, seed)
    key = f"qsa_{context}_{position}_{steps}_{seed}"
    bufs = {n: gpu.upload(c[n]) for n in ("qgate", "key", "value", "iq", "ik", "state", "index_state")}
    norms = [gpu.upload(n) for n in c["norms"]]
    packed = gpu.buffer(steps * (HEADS * 256 + KV_HEADS * 512 + SELECTED + 1) * 4)
    gpu.qsa_normalize_chunk(bufs["qgate"].pointer, bufs["key"].pointer, bufs["value"].pointer, bufs["iq"].pointer, bufs["ik"].pointer, steps, position,
                            HEADS, KV_HEADS, *[n.pointer for n in norms], packed.pointer, SELECTED, bufs["state"], context, bufs["index_state"].pointer)
    queries = gpu.read(packed, np.float32, (steps * HEADS * 256,))
    q16, out = gpu.upload(queries.astype(np.float16)), gpu.buffer(steps * HEADS * 256 * 4)
    gpu.qsa_prompt(bufs["state"], context, position, steps, HEADS, KV_HEADS, 0.0625, q16.pointer, out.pointer)
    assert gpu.decode_status() == 0
    gate = c["qgate"].reshape(steps, HEADS, 512)[:, :, 256:].astype(np.float64)
    got = (gpu.read(out, np.float32, (steps, HEADS, 256)) / (1 + np.exp(-gate)))[:, :10].reshape(steps, 2560)
    ok, worst = close(got, GOLDEN[key + "_out"])
    assert ok and worst < 2e-3, worst
    for b in list(bufs.values()) + norms + [packed, q16, out]:
        gpu.release(b)
