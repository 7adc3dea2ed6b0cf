"""Plain-Python restatement of the reference's interval allocator, used only to check the C++
planner on random inputs.  TEST INFRASTRUCTURE ONLY.

Follows details::allocateIntervals (graph/interval_memory_planner.cpp:170-216 of the reference):
intervals sorted by (first ascending, size descending, order ascending); allocations that ended
before the interval starts move to a free list in end order; the smallest free block that fits is
taken (ties: the one freed first) and split without merging; otherwise the arena grows; tensors
never touched get unique storage at the end.  Pinned by the six cases of
tests/graph/interval_memory_planner_tests.cpp:17-106 (see tests/test_planner.py).
"""


def _round_up(v, a):
    return (v + a - 1) // a * a


def allocate_intervals(intervals, unseen, alignment):
    ordered = sorted(intervals, key=lambda iv: (iv[1], -iv[3], iv[4]))
    offsets, memory = {}, 0
    active, free = [], []  # active: (last, order, offset, size); free: (size, free_order, offset)
    free_order = 0
    for ident, first, last, size, order in ordered:
        active.sort()
        while active and active[0][0] < first:
            l, o, off, sz = active.pop(0)
            free.append((sz, free_order, off))
            free_order += 1
        fits = sorted(b for b in free if b[0] >= size)
        if fits:
            sz, fo, off = fits[0]
            free.remove(fits[0])
            if sz > size:
                free.append((sz - size, fo, off + size))
            offset = off
        else:
            offset = _round_up(memory, alignment)
            memory = offset + size
        offsets[ident] = offset
        active.append((last, order, offset, size))
    for ident, size in unseen:
        offset = _round_up(memory, alignment)
        offsets[ident] = offset
        memory = offset + size
    return offsets, _round_up(memory, alignment)
