"""Property tests (hypothesis) of the shard geometry against the oracle, on host memory."""

import numpy as np
from hypothesis import given, settings
from hypothesis import strategies as st

from fastsafetensors_b200 import _native as nat
from fastsafetensors_b200 import shard_plan
from oracle import st_oracle

DTYPES = ["U8", "F16", "F32", "F64"]


@st.composite
def shard_cases(draw):
    world = draw(st.integers(1, 8))
    rank_count = draw(st.integers(1, 4))
    dim = draw(st.integers(0, rank_count - 1))
    shape = [draw(st.integers(0, 6)) for _ in range(rank_count)]
    shape[dim] = world * draw(st.integers(0, 5))          # even split, possibly empty
    return tuple(shape), draw(st.sampled_from(DTYPES)), dim, world


@settings(max_examples=80, deadline=None)
@given(shard_cases())
def test_scatter_ops_equal_numpy_slicing(case):
    shape, dtype, dim, world = case
    bits = st_oracle.BITS[dtype]
    n = int(np.prod(shape, dtype=np.int64)) * bits // 8
    src = np.random.default_rng(n + dim).integers(0, 256, max(n, 1), dtype=np.uint8)[:n]
    ops, shard_bytes = shard_plan.scatter_ops(src.ctypes.data if n else 4096, 0, shape, bits, dim, world)
    packed = np.full(shard_bytes * world + 8, 0x77, dtype=np.uint8)
    nat.gather_host([(o[0], o[1] + packed.ctypes.data) + o[2:] for o in ops], 2)
    assert (packed[shard_bytes * world:] == 0x77).all()
    for r in range(world):
        want, new_shape = st_oracle.shard(src, shape, dtype, dim, r, world)
        assert new_shape[dim] == shape[dim] // world
        assert np.array_equal(packed[r * shard_bytes:(r + 1) * shard_bytes], want)


@st.composite
def column_groups(draw):
    world = draw(st.integers(1, 4))
    dim = draw(st.integers(0, 1))
    other = draw(st.integers(1, 5))
    k = draw(st.integers(1, 4))
    extents = [world * draw(st.integers(1, 4)) for _ in range(k)]
    shapes = [((e, other) if dim == 0 else (other, e)) for e in extents]
    return shapes, dim, world


@settings(max_examples=60, deadline=None)
@given(column_groups())
def test_multi_col_ops_equal_numpy_concatenation(case):
    shapes, dim, world = case
    raws = [np.random.default_rng(i).integers(0, 256, int(np.prod(s)) * 2, dtype=np.uint8)
            for i, s in enumerate(shapes)]
    ops, per_rank, shape = shard_plan.multi_col_ops([r.ctypes.data for r in raws], 0, shapes, 16, dim, world)
    packed = np.zeros(per_rank * world, dtype=np.uint8)
    nat.gather_host([(o[0], o[1] + packed.ctypes.data) + o[2:] for o in ops], 1)
    for r in range(world):
        want, want_shape = st_oracle.multi_cols(raws, shapes, "F16", dim, r, world)
        assert shape == want_shape
        assert np.array_equal(packed[r * per_rank:(r + 1) * per_rank], want)


def test_store_orders_of_an_owner_are_permutations_of_each_other():
    """BatchLayout.fill_ops: region by region, rotated region by region, and tensor by tensor to
    all destinations emit the same copies in different orders; the own region always comes first
    in the two orders meant for peers' memory."""
    from fastsafetensors_b200.batch import BatchLayout
    from fastsafetensors_b200.common import TensorFrame
    from fastsafetensors_b200.st_types import DType

    world, me = 4, 2
    lay = BatchLayout(world)
    frames, src = {}, {}
    specs = [("q", (8, 16), ("shard", 0)), ("o", (8, 16), ("shard", 1)), ("norm", (16,), ("replicate",)),
             ("expert", (4, 4), ("push", 1)), ("mine", (4, 4), ("push", me)), ("empty", (0, 4), ("shard", 0))]
    off = 0
    for i, (name, shape, action) in enumerate(specs):
        n = int(np.prod(shape)) * 2
        frames[name] = TensorFrame.from_buffer({"dtype": "BF16", "shape": list(shape), "data_offsets": [off, off + n]})
        src[name] = 0x10000 + off
        off += n
        lay.add(name, frames[name], me, action)
    region = [0x1000000 * (d + 1) for d in range(world)]
    plain = lay.fill_ops(me, frames, src, region)
    rotated = lay.fill_ops(me, frames, src, region, rotate=True)
    interleaved = lay.fill_ops(me, frames, src, region, rotate="interleave")
    assert sorted(plain) == sorted(rotated) == sorted(interleaved) and len(plain) == len(set(plain))
    own = [o for o in plain if region[me] <= o[1] < region[me] + 0x1000000]
    assert rotated[: len(own)] == own and interleaved[: len(own)] == own
    # tensor by tensor: the three peers' slots of "q" are adjacent, starting with rank me + 1
    peers = interleaved[len(own):]
    firsts = [(o[1] >> 24) - 1 for o in peers[:3]]
    assert firsts == [(me + 1) % world, (me + 2) % world, (me + 3) % world]
