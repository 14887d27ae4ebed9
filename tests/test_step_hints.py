"""Host-side hints of a step: the class of context length that decides which captured decode
graph may be replayed, and its bound on the keys a row may see."""

from thing_htn_2026_b200 import ops


def test_context_class_bounds_every_length_of_its_class():
    first = ops.CONTEXT_CLASS_BASE
    assert ops.context_class(0) == (0, first - 1)
    assert ops.context_class(first - 1) == (0, first - 1)
    assert ops.context_class(first) == (1, 2 * first - 1)
    assert ops.context_class(2 * first - 1) == (1, 2 * first - 1)
    assert ops.context_class(2 * first) == (2, 4 * first - 1)
    last = (-1, -1)
    for longest in list(range(0, 5 * first, 97)) + [10 ** 6]:
        k, bound = ops.context_class(longest)
        assert bound >= longest, "a step's bound must hold for the step itself"
        assert (k, bound) >= last, "classes follow the length"
        if k:
            assert bound < 2 * longest + 1, "a class spans one doubling"
        last = (k, bound)


def test_few_classes_over_a_long_generation():
    seen = {ops.context_class(n)[0] for n in range(1, 200_000, 13)}
    assert len(seen) <= 9, "one captured graph per class and batch size: the classes stay few"


def test_row_tiles_cover_every_row_once_fewest_keys_first():
    counts, held, size = [5, 300, 128, 1], [0, 64, 1000, 7], 128
    row0, rows = ops.row_tiles_of(counts, held, size)
    covered = sorted(r for a, n in zip(row0, rows) for r in range(a, a + n))
    assert covered == list(range(sum(counts))) and max(rows) <= size
    starts = [0, 5, 305, 433]
    def keys(a, n):
        i = max(j for j, s in enumerate(starts) if s <= a)
        return held[i] + (a - starts[i]) + n
    seen = [keys(a, n) for a, n in zip(row0, rows)]
    assert seen == sorted(seen), "the kernels start at the end of the list: longest tiles last"
    for a, n in zip(row0, rows):                      # a tile never crosses into another sequence
        i = max(j for j, s in enumerate(starts) if s <= a)
        assert a + n <= starts[i] + counts[i]


def test_counter_buffer_refuses_to_grow():
    import pytest
    with pytest.raises(ops.KernelError, match="arrival counters"):
        ops._counter_buffer(ops.COUNTER_SLOTS + 1, "cpu")


def test_lengths_differ_is_a_coarse_class():
    assert not ops.lengths_differ([640] * 8)
    assert not ops.lengths_differ([640, 600, 520, 481])         # within a quarter of the longest
    assert ops.lengths_differ([640, 479])
    assert ops.lengths_differ([2048, 64, 1000])
    assert not ops.lengths_differ([1])
