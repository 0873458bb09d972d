"""Host-side logic of the host-buffer front end that needs no GPU."""
import ops


def test_chunk_schedule_covers_the_batch_once():
    sched = ops.backend.host.chunk_schedule
    for B in (1, 2, 5, 7, 32, 33):
        for chunk in (1, 2, 3, 4, 8, 64):
            ranges = sched(B, chunk)
            assert ranges[0][0] == 0 and ranges[-1][1] == B
            assert all(a1 == b0 for (_, a1), (b0, _) in zip(ranges, ranges[1:]))
            assert all(0 < b1 - b0 <= chunk for b0, b1 in ranges)
            # the first copy in and the last copy out are the shortest
            assert ranges[0][1] - ranges[0][0] == min(b1 - b0 for b0, b1 in ranges)
            assert ranges[-1][1] - ranges[-1][0] == min(b1 - b0 for b0, b1 in ranges)


def test_pipeline_schedule_cuts_both_ends_into_head_groups():
    import pytest
    sched = ops.backend.host.pipeline_schedule
    # every (batch element, head) exactly once, in order
    for B, Hh, parts in ((1, 16, 4), (4, 16, 4), (32, 16, 4), (2, 5, 3), (3, 2, 8), (5, 7, 1)):
        chunks = sched(B, Hh, head_parts=parts)
        seen = [(b, h) for b0, b1, h0, h1 in chunks for b in range(b0, b1) for h in range(h0, h1)]
        assert seen == [(b, h) for b in range(B) for h in range(Hh)]
        cut = [c for c in chunks if (c[2], c[3]) != (0, Hh)]
        # only the first and the last batch element are cut, into min(parts, heads) groups each
        assert {c[0] for c in cut} <= {0, B - 1}
        want = min(parts, Hh)
        assert len(cut) == (0 if want == 1 else want if B == 1 else 2 * want)
        assert all(h1 - h0 in (Hh // want, Hh // want + 1) for _, _, h0, h1 in cut)
    assert sched(4, 16, head_parts=4)[:5] == [(0, 1, 0, 4), (0, 1, 4, 8), (0, 1, 8, 12), (0, 1, 12, 16), (1, 2, 0, 16)]
    # given batch sizes: ends that are more than one element stay whole
    assert sched(5, 4, sizes=[2, 3], head_parts=2) == [(0, 2, 0, 4), (2, 5, 0, 4)]
    assert sched(3, 4, sizes=[1, 2], head_parts=2) == [(0, 1, 0, 2), (0, 1, 2, 4), (1, 3, 0, 4)]
    with pytest.raises(ValueError):
        sched(5, 4, sizes=[2, 2])
