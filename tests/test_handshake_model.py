"""The cross-rank handshake as a small model, checked over EVERY interleaving of its steps.

The kernels that write peers' windows (the exchange, the fused QKV scatter, the fp8 exchange)
all run the same protocol (csrc/kernels/handshake.cuh): monotonic per-sender flags in the
receiver's control block, raised with a release and polled with an acquire, and a phase counter
that advances by two per call.

    opening   every rank raises its flag at every peer to base + 1: "I have finished reading my
              window"; a sender waits for the flag of the ONE peer it is about to write to
    payload   stores into the peers' windows
    closing   every rank raises its flags to base + 2: "all my writes have landed", waits for
              everyone's, and only then reads its own window

This file states that protocol as a program per rank made of atomic steps and explores all
interleavings (a depth-first search over the reachable states) for two and three ranks over two
consecutive calls. Three properties must hold in every reachable state:

  * a rank that reads its window finds, from every sender, the payload of THIS call;
  * a sender never overwrites a payload its owner has not read yet;
  * the buffer a sender writes to is the one its owner chose for THIS call (the choice travels as
    a byte stored just before the opening flag is raised, FuCtrl::slot_of: the output pool).

Two negative controls show that the search can find what it looks for: without the opening wait
the second property breaks, and with the completion announced before the payload (the kernels'
FU_A2A_EARLY_PUBLISH test flag) the first one does. No GPU, no process group. The reference checks
the same ordering on hardware with its armed/clean controls (test/distributed/ce_ordering.py,
window_race.py); this is the exhaustive counterpart on paper.
"""

import pytest

CALLS = 2


def program(world, me, *, opening_wait=True, early_publish=False):
    """The steps of one rank for CALLS consecutive calls: (kind, peer, call)."""
    steps = []
    for call in range(1, CALLS + 1):
        steps += [("announce_open", p, call) for p in range(world)]
        if early_publish:
            steps += [("announce_close", p, call) for p in range(world)]
        for p in range(world):
            if opening_wait:
                steps.append(("wait_open", p, call))
            steps.append(("write", p, call))
        if not early_publish:
            steps += [("announce_close", p, call) for p in range(world)]
        steps.append(("wait_close", None, call))
        steps.append(("read", None, call))
    return steps


def explore(world, **variant):
    """Depth-first search over all interleavings. Returns the first violated property, or None."""
    programs = [program(world, r, **variant) for r in range(world)]
    opening_waits = variant.get("opening_wait", True)
    # state: program counters, flags[receiver][sender], window[receiver][sender] = call whose payload
    # lies there, consumed[rank] = last call whose window that rank has read, choice[sender][owner] =
    # the buffer `owner` last told `sender` to use (modelled as the number of the call it was chosen for)
    zeros = tuple(tuple([0] * world) for _ in range(world))
    start = (tuple([0] * world), zeros, zeros, tuple([0] * world), zeros)
    seen, stack = {start}, [start]
    finished = False
    while stack:
        pcs, flags, window, consumed, choice = stack.pop()
        if all(pcs[r] == len(programs[r]) for r in range(world)):
            finished = True
            continue
        progressed = False
        for r in range(world):
            if pcs[r] == len(programs[r]):
                continue
            kind, p, call = programs[r][pcs[r]]
            base = 2 * (call - 1)  # the phase counter of this rank's window before this call
            f = [list(row) for row in flags]
            w = [list(row) for row in window]
            c = list(consumed)
            ch = [list(row) for row in choice]
            if kind == "announce_open":
                ch[p][r] = call  # the byte is stored first, by the same thread, then the flag is raised
                f[p][r] = max(f[p][r], base + 1)
            elif kind == "announce_close":
                f[p][r] = max(f[p][r], base + 2)
            elif kind == "wait_open":
                if flags[r][p] < base + 1:
                    continue  # blocked
            elif kind == "wait_close":
                if any(flags[r][q] < base + 2 for q in range(world)):
                    continue
            elif kind == "write":
                if consumed[p] < call - 1:
                    return f"rank {r} overwrites in rank {p}'s window a payload of call {window[p][r]} that rank {p} has not read"
                if opening_waits and choice[r][p] != call:
                    return f"rank {r} writes call {call} into the buffer rank {p} chose for call {choice[r][p]}"
                w[p][r] = call
            elif kind == "read":
                for q in range(world):
                    if window[r][q] != call:
                        return f"rank {r} reads its window in call {call} and finds rank {q}'s payload of call {window[r][q]}"
                c[r] = call
            progressed = True
            nxt = (tuple(pcs[i] + (1 if i == r else 0) for i in range(world)), tuple(map(tuple, f)),
                   tuple(map(tuple, w)), tuple(c), tuple(map(tuple, ch)))
            if nxt not in seen:
                seen.add(nxt)
                stack.append(nxt)
        if not progressed:
            return f"deadlock at program counters {pcs}"
    assert finished, "the search never reached the end of the programs"
    return None


@pytest.mark.parametrize("world", [1, 2, 3])
def test_protocol_holds_in_every_interleaving(world):
    assert explore(world) is None


@pytest.mark.parametrize("world", [2, 3])
def test_without_the_opening_wait_a_payload_is_overwritten_unread(world):
    found = explore(world, opening_wait=False)
    assert found is not None and "overwrites" in found


@pytest.mark.parametrize("world", [2, 3])
def test_with_completion_announced_before_the_payload_a_reader_sees_stale_data(world):
    found = explore(world, early_publish=True)
    assert found is not None and "finds rank" in found


# ---- the pull direction ------------------------------------------------------------------------------
# The output projection and the gradient pull READ peers' memory: the owner produces its buffer in
# stream order before the kernel, the opening says "my buffer is complete", a reader loads from a peer
# once THAT peer has said so, the closing says "I have finished reading everybody's", and only after
# everyone's closing may the owner's next step overwrite its buffer.
def pull_program(world, *, closing_wait=True):
    steps = []
    for call in range(1, CALLS + 1):
        steps.append(("produce", None, call))
        steps += [("announce_open", p, call) for p in range(world)]
        for p in range(world):
            steps += [("wait_open", p, call), ("load", p, call)]
        steps += [("announce_close", p, call) for p in range(world)]
        if closing_wait:
            steps.append(("wait_close", None, call))
    return steps


def explore_pull(world, **variant):
    programs = [pull_program(world, **variant) for _ in range(world)]
    zeros = tuple(tuple([0] * world) for _ in range(world))
    # state: program counters, flags[receiver][sender], holds[owner] = call whose data the owner's
    # buffer holds, loaded[reader][owner] = last call of `owner` that `reader` has loaded
    start = (tuple([0] * world), zeros, tuple([0] * world), zeros)
    seen, stack = {start}, [start]
    while stack:
        pcs, flags, holds, loaded = stack.pop()
        if all(pcs[r] == len(programs[r]) for r in range(world)):
            continue
        progressed = False
        for r in range(world):
            if pcs[r] == len(programs[r]):
                continue
            kind, p, call = programs[r][pcs[r]]
            base = 2 * (call - 1)
            f = [list(row) for row in flags]
            h = list(holds)
            ld = [list(row) for row in loaded]
            if kind == "produce":
                late = [q for q in range(world) if loaded[q][r] < call - 1]
                if late:
                    return f"rank {r} overwrites its buffer while rank {late[0]} has yet to load call {call - 1}"
                h[r] = call
            elif kind == "announce_open":
                f[p][r] = max(f[p][r], base + 1)
            elif kind == "announce_close":
                f[p][r] = max(f[p][r], base + 2)
            elif kind == "wait_open":
                if flags[r][p] < base + 1:
                    continue
            elif kind == "wait_close":
                if any(flags[r][q] < base + 2 for q in range(world)):
                    continue
            elif kind == "load":
                if holds[p] != call:
                    return f"rank {r} loads rank {p}'s buffer in call {call} and finds call {holds[p]}"
                ld[r][p] = call
            progressed = True
            nxt = (tuple(pcs[i] + (1 if i == r else 0) for i in range(world)), tuple(map(tuple, f)), tuple(h),
                   tuple(map(tuple, ld)))
            if nxt not in seen:
                seen.add(nxt)
                stack.append(nxt)
        if not progressed:
            return f"deadlock at program counters {pcs}"
    return None


@pytest.mark.parametrize("world", [1, 2, 3])
def test_pull_protocol_holds_in_every_interleaving(world):
    assert explore_pull(world) is None


@pytest.mark.parametrize("world", [2, 3])
def test_pull_without_the_closing_wait_overwrites_what_a_peer_still_reads(world):
    found = explore_pull(world, closing_wait=False)
    assert found is not None and "overwrites its buffer" in found
