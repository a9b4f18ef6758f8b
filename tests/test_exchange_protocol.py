"""The one-shot all-reduce's exchange protocol on CPU ranks.

muser_b200/csrc/oneshot_exchange.h holds the protocol once, for the GPU kernel and for tests/exchange_harness.cpp, in
which every rank is a host thread.  Faults are made on the host: a rank that never joins a call, a rank that
brings fewer elements.  No GPU is involved."""
import ctypes as C
import subprocess
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
GAVE_UP = 401


@pytest.fixture(scope="module")
def harness(tmp_path_factory):
    out = tmp_path_factory.mktemp("xchg") / "libxchg.so"
    subprocess.run(["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-pthread", str(ROOT / "tests" / "exchange_harness.cpp"), "-o", str(out)],
                   check=True, capture_output=True)
    lib = C.CDLL(str(out))
    lib.xchg_box_create.restype = C.c_void_p
    lib.xchg_box_create.argtypes = [C.c_uint32]
    lib.xchg_box_destroy.argtypes = [C.c_void_p]
    u32p, f32p, i32p = C.POINTER(C.c_uint32), C.POINTER(C.c_float), C.POINTER(C.c_int)
    lib.xchg_call.argtypes = [C.c_void_p, f32p, C.c_uint32, u32p, u32p, u32p, C.c_uint32, i32p]
    lib.xchg_run.argtypes = [C.c_void_p, f32p, C.c_uint32, C.c_uint32, u32p, C.c_uint32, i32p]
    return lib


def _u32(values):
    return (C.c_uint32 * len(values))(*values)


def call(lib, box, data, joins=None, counts=None, lead=None, wait_limit=1 << 22):
    world, count = data.shape
    status = (C.c_int * world)()
    lib.xchg_call(box, data.ctypes.data_as(C.POINTER(C.c_float)), count, _u32(joins or [1] * world), _u32(counts or [count] * world),
                  _u32(lead or [0] * world), wait_limit, status)
    return list(status)


def rank_order_sum(parts):
    total = np.zeros(parts.shape[1], dtype=np.float32)
    for p in parts:
        total = total + p  # f32, rank 0 first: the order every rank uses
    return total


@pytest.mark.parametrize("world,count", [(2, 5120), (4, 40960), (8, 20480), (3, 1), (8, 65536)])
def test_all_ranks_end_with_the_same_bits(harness, world, count):
    rng = np.random.default_rng(world * 1000 + count)
    box = harness.xchg_box_create(world)
    try:
        for k in range(5):  # five calls: both slots, wrapped around twice
            parts = (rng.standard_normal((world, count)) * 10.0 ** rng.integers(-3, 4)).astype(np.float32)
            data = parts.copy()
            assert call(harness, box, data, lead=[(50 * ((r + k) % 3)) for r in range(world)]) == [0] * world
            want = rank_order_sum(parts)
            for r in range(world):
                assert np.array_equal(data[r].view(np.uint32), want.view(np.uint32)), (k, r)
    finally:
        harness.xchg_box_destroy(box)


def test_back_to_back_calls_with_ranks_running_ahead(harness):
    """No host join between calls: a fast rank starts call k + 1 while a slow one still reads call k's cells.  Two
    slots are enough because nobody gets further ahead than that without the slow rank's values of call k + 1."""
    world, count, calls = 4, 6000, 40
    rng = np.random.default_rng(5)
    parts = rng.standard_normal((calls, world, count)).astype(np.float32)
    data = parts.copy()
    status = (C.c_int * world)()
    box = harness.xchg_box_create(world)
    try:
        harness.xchg_run(box, data.ctypes.data_as(C.POINTER(C.c_float)), count, calls, _u32([0, 300, 0, 120]), 1 << 24, status)
    finally:
        harness.xchg_box_destroy(box)
    assert list(status) == [0] * world
    for k in range(calls):
        want = rank_order_sum(parts[k])
        for r in range(world):
            assert np.array_equal(data[k, r].view(np.uint32), want.view(np.uint32)), (k, r)


def test_a_rank_that_never_joins(harness):
    """Rank 2 skips a call.  The others give up after their bounded wait, report it, and every output they hold is
    either a complete rank-order sum (none can be: rank 2's values never came) or their own untouched partial sum;
    nothing stale from the two earlier calls leaks in.  The group is then rebuilt and works again."""
    world, count = 4, 5000
    rng = np.random.default_rng(9)
    box = harness.xchg_box_create(world)
    try:
        for _ in range(2):  # two good calls first, so that both slots hold old values
            parts = rng.standard_normal((world, count)).astype(np.float32)
            data = parts.copy()
            assert call(harness, box, data) == [0] * world
        parts = rng.standard_normal((world, count)).astype(np.float32)
        data = parts.copy()
        status = call(harness, box, data, joins=[1, 1, 0, 1], wait_limit=2000)
        assert status == [GAVE_UP, GAVE_UP, 0, GAVE_UP]
        for r in (0, 1, 3):
            assert np.array_equal(data[r].view(np.uint32), parts[r].view(np.uint32)), r  # own partial sums, untouched
        assert np.array_equal(data[2], parts[2])
    finally:
        harness.xchg_box_destroy(box)
    box = harness.xchg_box_create(world)  # what comm set-up does: fresh buffers, sequence numbers from zero
    try:
        parts = rng.standard_normal((world, count)).astype(np.float32)
        data = parts.copy()
        assert call(harness, box, data) == [0] * world
        assert np.array_equal(data[0].view(np.uint32), rank_order_sum(parts).view(np.uint32))
    finally:
        harness.xchg_box_destroy(box)


def test_a_rank_with_a_short_count(harness):
    """Rank 1 brings 3000 of 5000 elements.  Where its values exist the sums are complete on every rank; the wait
    for the first missing element gives up, and from there on the other ranks keep their own partial sums."""
    world, count, short = 3, 5000, 3000
    rng = np.random.default_rng(13)
    parts = rng.standard_normal((world, count)).astype(np.float32)
    data = parts.copy()
    box = harness.xchg_box_create(world)
    try:
        status = call(harness, box, data, counts=[count, short, count], wait_limit=2000)
    finally:
        harness.xchg_box_destroy(box)
    assert status == [GAVE_UP, 0, GAVE_UP]
    want = rank_order_sum(parts)
    # rank 1 saw everything it asked for
    assert np.array_equal(data[1, :short].view(np.uint32), want[:short].view(np.uint32))
    assert np.array_equal(data[1, short:], parts[1, short:])
    for r in (0, 2):
        # every chunk below element 3000 is complete, the chunk that holds it stops there, the chunks behind give up at once
        assert np.array_equal(data[r, :short].view(np.uint32), want[:short].view(np.uint32)), r
        assert np.array_equal(data[r, short:].view(np.uint32), parts[r, short:].view(np.uint32)), r
