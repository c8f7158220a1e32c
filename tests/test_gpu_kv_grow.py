"""sdx_kv_grow: the data movement of sd_kv_grow (gpu/kernels.cpp:4048-4203). A grown state holds every plane's old positions at the
new plane stride and zeros behind them, the indexer's blocks sit at their new pitch with the ring behind them, and attention over
the grown state gives the bits it gave over the old one."""
import numpy as np
import pytest

from straydog_b200.backend import StraydogError
from util import q8_state, queries_f16

pytestmark = pytest.mark.gpu


def index_state_of(rng, context):
    pool = context // 4 + 1
    return rng.normal(0, 1, pool * 128 + 2048).astype(np.float32)


def check_index(before, after, from_context, to_context, valid):
    old_pool, pool = from_context // 4 + 1, to_context // 4 + 1
    keep = min(old_pool, valid // 4 + 1)
    want = np.zeros(pool * 128 + 2048, np.float32)
    want[:pool * 128].reshape(128, pool)[:, :keep] = before[:old_pool * 128].reshape(128, old_pool)[:, :keep]
    want[pool * 128:] = before[old_pool * 128:]
    assert np.array_equal(after.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("kv_heads,from_context,to_context,valid", [(2, 1000, 4096, 1000), (2, 64, 65, 10), (1, 4096, 8192, 4000), (4, 37, 262144, 37)])
def test_a_grown_state_holds_the_old_positions_at_the_new_stride(gpu, kv_heads, from_context, to_context, valid):
    rng = np.random.default_rng(from_context)
    state_np = rng.integers(0, 256, (2 * kv_heads, from_context, 272), dtype=np.uint8)
    index_np = index_state_of(rng, from_context)
    state, index = gpu.upload(state_np), gpu.upload(index_np)
    old_pointer, used_before = state.pointer, gpu.memory()[0]
    grown, grown_index = gpu.kv_grow(kv_heads, from_context, to_context, valid, state, index)
    assert grown.pointer != old_pointer and state.pointer is None
    planes = gpu.read(grown, np.uint8, (2 * kv_heads, to_context, 272))
    assert np.array_equal(planes[:, :from_context], state_np) and not planes[:, from_context:].any()
    check_index(index_np, gpu.read(grown_index, np.float32, ((to_context // 4 + 1) * 128 + 2048,)), from_context, to_context, valid)
    # the old allocations are gone, the budget holds the new ones in their place
    grew = (to_context - from_context) * 2 * kv_heads * 272 + ((to_context // 4 + 1) - (from_context // 4 + 1)) * 128 * 4
    assert gpu.memory()[0] - used_before == grew
    with pytest.raises(StraydogError):
        gpu.read(type(grown)(gpu, old_pointer, 16), np.uint8, (16,))
    gpu.release(grown)
    gpu.release(grown_index)


def test_attention_over_a_grown_state_gives_the_same_bits(gpu):
    rng = np.random.default_rng(5)
    length, from_context, to_context = 3000, 3072, 16384
    state_np = q8_state(rng, from_context, 2)
    q = queries_f16(rng, 1, 16, 256)
    state, index, q_dev = gpu.upload(state_np), gpu.upload(index_state_of(rng, from_context)), gpu.upload(q)
    out = gpu.buffer(16 * 256 * 4)
    gpu.qsa_decode([state], [from_context], [length], 16, 2, 1 / 16, q_dev.pointer, out.pointer)
    before = gpu.read(out, np.uint32, (16 * 256,))
    grown, grown_index = gpu.kv_grow(2, from_context, to_context, length, state, index)
    gpu.qsa_decode([grown], [to_context], [length], 16, 2, 1 / 16, q_dev.pointer, out.pointer)
    assert np.array_equal(before, gpu.read(out, np.uint32, (16 * 256,)))
    for b in (grown, grown_index, q_dev, out):
        gpu.release(b)


def test_an_index_state_with_room_is_grown_in_place_and_a_host_state_in_host_memory(gpu):
    rng = np.random.default_rng(6)
    from_context, to_context, valid, kv_heads = 512, 2048, 300, 2
    index_np = index_state_of(rng, from_context)
    roomy = gpu.buffer(((to_context // 4 + 1) * 128 + 2048) * 4 + 4096)
    gpu.write_buffer(roomy, 0, index_np)
    state_np = rng.integers(0, 256, (2 * kv_heads, from_context, 272), dtype=np.uint8)
    host = gpu.host_state(state_np.nbytes)
    gpu.write_buffer(host, 0, state_np)
    pointer, used = roomy.pointer, gpu.memory()[0]
    grown, same = gpu.kv_grow(kv_heads, from_context, to_context, valid, host, roomy)
    assert same is roomy and roomy.pointer == pointer and gpu.memory()[0] == used, "a host-resident state and a roomy index state take no VRAM"
    check_index(index_np, gpu.read(roomy, np.float32, ((to_context // 4 + 1) * 128 + 2048,)), from_context, to_context, valid)
    planes = gpu.read(grown, np.uint8, (2 * kv_heads, to_context, 272))
    assert np.array_equal(planes[:, :valid], state_np[:, :valid]) and not planes[:, valid:].any(), "the CPU copies the written positions"
    # the grown state is still a host-resident one: the gathered attention accepts it, the plain decode reads it in place
    gpu.release(grown)
    gpu.release(roomy)


def test_a_refused_growth_leaves_both_states_as_they_were(gpu):
    rng = np.random.default_rng(7)
    state_np = rng.integers(0, 256, (4, 256, 272), dtype=np.uint8)
    index_np = index_state_of(rng, 256)
    state, index = gpu.upload(state_np), gpu.upload(index_np)
    for kwargs in (dict(to_context=256), dict(to_context=100), dict(valid=257), dict(to_context=262145), dict(kv_heads=0), dict(from_context=128),
                   dict(kv_heads=1)):
        a = dict(kv_heads=2, from_context=256, to_context=1024, valid=200)
        a.update(kwargs)
        with pytest.raises(StraydogError, match="invalid Straydog K/V growth"):
            gpu.kv_grow(a["kv_heads"], a["from_context"], a["to_context"], a["valid"], state, index)
    used, budget = gpu.memory()
    small = type(gpu)(0, 64 << 20)   # a handle whose budget cannot hold the grown state
    s2, i2 = small.upload(state_np), small.upload(index_np)
    with pytest.raises(StraydogError, match="budget|VRAM|memory"):
        small.kv_grow(2, 256, 262144, 200, s2, i2)
    assert np.array_equal(small.read(s2, np.uint8, state_np.shape), state_np) and np.array_equal(small.read(i2, np.float32, index_np.shape), index_np)
    small.close()
    assert np.array_equal(gpu.read(state, np.uint8, state_np.shape), state_np) and gpu.memory()[0] == used
    gpu.release(state)
    gpu.release(index)
