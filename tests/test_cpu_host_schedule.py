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
