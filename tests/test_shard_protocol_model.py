"""The two completion-signal protocols of the row-sharded GEMV loop, as a small state machine explored
exhaustively on the CPU: how many y buffers a loop needs so that a rank never reads a buffer another
rank may already be overwriting.  (The GPU tests run the real kernels; this pins the argument.)

Deferred signal (pdk_q4k_gemv_shard_lagged): launch s of a rank starts by posting "my step s - 1 is in
place" to every rank, stores its band of step s into buffer s % R of every rank while it runs, and can only
end once every rank has posted step s - 1.  The reader of step s - 1 sits between launch s and launch s + 1.

Serial signal (pdk_q4k_gemv_shard_sync + pdk_peer_flags_wait): launch s stores into buffer s % R and posts
step s when it ends; a wait passes once every rank has posted step s; the reader of step s follows the wait."""
from collections import deque


def explore(n_ranks, n_steps, n_bufs, program):
    """Breadth-first over every interleaving of the ranks' event sequences.  program(rank state) yields the
    rank's events in order; an event is (kind, step).  Returns the first violation found, or None."""
    events = program(n_steps)
    start = (tuple([0] * n_ranks), tuple([0] * n_ranks), tuple([0] * n_ranks))   # next event index, posted, started
    seen = {start}
    todo = deque([start])
    while todo:
        pc, posted, started = todo.popleft()
        for r in range(n_ranks):
            if pc[r] == len(events):
                continue
            kind, s = events[pc[r]]
            posted2, started2 = list(posted), list(started)
            if kind == "start":                  # the launch begins: from now on its stores may have landed anywhere
                started2[r] = s
            elif kind == "post":
                posted2[r] = s
            elif kind == "need":                 # blocks until every rank has posted step s
                if any(p < s for p in posted):
                    continue
            elif kind == "read":                 # step s of every rank must be in buffer s % R of this rank, untouched since
                if any(p < s for p in posted):
                    return ("not arrived", r, s, posted)
                for q in range(n_ranks):
                    t = started[q]
                    if t > s and any(u % n_bufs == s % n_bufs for u in range(s + 1, t + 1)):
                        return ("overwritten", r, s, q, t)
            pc2 = list(pc)
            pc2[r] += 1
            state = (tuple(pc2), tuple(posted2), tuple(started2))
            if state not in seen:
                seen.add(state)
                todo.append(state)
    return None


def deferred(n_steps):
    ev = []
    for s in range(1, n_steps + 1):
        ev += [("post", s - 1), ("start", s), ("need", s - 1)]   # launch s: post s - 1 when it starts, end only when all have
        if s >= 2:
            ev.append(("read", s - 1))                            # between launch s and launch s + 1
    return ev


def serial(n_steps):
    ev = []
    for s in range(1, n_steps + 1):
        ev += [("start", s), ("post", s), ("need", s), ("read", s)]
    return ev


def test_deferred_signal_needs_three_buffers():
    assert explore(2, 6, 2, deferred) is not None          # a peer one launch ahead stores step s + 1 over step s - 1
    assert explore(2, 7, 3, deferred) is None
    assert explore(3, 5, 3, deferred) is None
    assert explore(2, 7, 4, deferred) is None


def test_deferred_signal_read_is_never_early():
    v = explore(2, 6, 2, deferred)
    assert v[0] == "overwritten"                            # the arrival check itself holds with any buffer count


def test_serial_signal_needs_two_buffers():
    assert explore(2, 5, 1, serial) is not None
    assert explore(2, 6, 2, serial) is None
    assert explore(3, 4, 2, serial) is None


def grouped(group, n_steps):
    """The captured end-to-end loop: launches in groups; the copy-out of step u - 1 is enqueued behind launch
    u on another stream and only known to be done when the next group's first kernel starts - the latest
    it can be, which is where the model puts it."""
    def program(_):
        ev = []
        for g0 in range(1, n_steps + 1, group):
            steps = list(range(g0, min(g0 + group, n_steps + 1)))
            for s in steps:
                ev += [("post", s - 1), ("start", s), ("need", s - 1)]
            ev += [("read", s - 1) for s in steps if s >= 2]
        return ev
    return program


def test_grouped_capture_needs_group_plus_two_buffers():
    for group in (2, 3, 4):
        assert explore(2, 4 * group, group + 2, grouped(group, 4 * group)) is None
        assert explore(2, 4 * group, group + 1, grouped(group, 4 * group)) is not None
