"""The GEMM core's mbarrier pipeline as a model, checked over every interleaving of its roles.

`fu::gemm::run` (csrc/kernels/gemm_sm100.cuh) has three roles that never share a program counter:
a TMA producer filling a ring of STAGES operand buffers, one MMA thread consuming them into one of
two tensor-memory accumulators, and epilogue warps draining a finished accumulator while the next
tile's main loop already runs. They meet only in mbarriers, and which PHASE PARITY each side waits
for is the part that is easy to get wrong:

    producer   waits  empty[s]           with parity ((it / STAGES) & 1) ^ 1    then fills stage s
    MMA        waits  tmem_empty[acc]    with parity ((tile >> 1) & 1) ^ 1      once per tile
               waits  full[s]            with parity  (it / STAGES) & 1         then reads stage s
               its commit arrives on empty[s]; after the last K-block, on tmem_full[acc]
    epilogue   waits  tmem_full[acc]     with parity  (tile >> 1) & 1           then reads the accumulator
               every epilogue warp arrives on tmem_empty[acc] (count = number of warps)

An mbarrier is modelled as (current phase parity, arrivals still missing); a wait with parity P
passes when the barrier's current phase parity differs from P (the phase with parity P has
completed), which is also why the very first wait on an `empty` barrier, with parity 1, passes at
once. The search explores every interleaving of the role steps for a ring that the K-loop length
does not divide and an odd number of tiles, and checks in every reachable state that

  * the producer never refills a stage the MMA has not read,
  * the MMA reads stage contents in order, and never writes into an accumulator that an epilogue
    warp has yet to drain,
  * the epilogue reads the accumulator of ITS tile, complete,
  * nobody waits for ever.

Negative controls: the same search with the producer's parity un-flipped, and with the accumulator
barrier counting one warp too few, must each find a violation. The CTA-pair kernel (`run_pair`) has
the same structure with the `tmem_empty` count doubled (both CTAs' epilogue warps arrive on the even
CTA's barrier); `warps` below stands for that count.
"""

import pytest


class Bar:
    """mbarrier: phase parity and the arrivals still missing in the current phase."""

    @staticmethod
    def new(count):
        return (0, count, count)

    @staticmethod
    def arrive(b):
        parity, missing, count = b
        return (parity ^ 1, count, count) if missing == 1 else (parity, missing - 1, count)

    @staticmethod
    def passes(b, parity):
        return b[0] != parity


def explore(stages=3, kblocks=2, tiles=3, warps=2, producer_flip=1, empty_count=None):
    empty_count = warps if empty_count is None else empty_count
    total = tiles * kblocks
    # state: producer it, mma (tile, kb, waiting_acc), epilogue per-warp tile index,
    #        barriers, stage contents, stage consumed marks, accumulator contents and drain marks
    init = (0, (0, 0, True), tuple([0] * warps),
            tuple(Bar.new(1) for _ in range(stages)), tuple(Bar.new(1) for _ in range(stages)),
            (Bar.new(1), Bar.new(1)), (Bar.new(empty_count), Bar.new(empty_count)),
            tuple([-1] * stages), tuple([True] * stages),  # stage holds item, stage has been read
            ((-1, 0), (-1, 0)), ((True,) * warps, (True,) * warps))  # acc = (tile, K-blocks added); drained by warp
    seen, stack = {init}, [init]
    while stack:
        st = stack.pop()
        p_it, (m_tile, m_kb, m_wait), e_tiles, full, empty, tfull, tempty, holds, read, acc, drained = st
        done = p_it == total and m_tile == tiles and all(t == tiles for t in e_tiles)
        if done:
            continue
        nxt_states = []
        # ---- producer
        if p_it < total:
            s = p_it % stages
            if Bar.passes(empty[s], ((p_it // stages) & 1) ^ producer_flip):
                if not read[s]:
                    return f"producer refills stage {s} (item {holds[s]}) before the MMA has read it"
                h, r, f = list(holds), list(read), list(full)
                h[s], r[s] = p_it, False
                f[s] = Bar.arrive(f[s])
                nxt_states.append((p_it + 1, (m_tile, m_kb, m_wait), e_tiles, tuple(f), empty, tfull, tempty,
                                   tuple(h), tuple(r), acc, drained))
        # ---- MMA thread
        if m_tile < tiles:
            a = m_tile & 1
            if m_wait:
                if Bar.passes(tempty[a], ((m_tile >> 1) & 1) ^ 1):
                    if not all(drained[a]):
                        return f"MMA starts tile {m_tile} in accumulator {a} before every epilogue warp has drained tile {acc[a][0]}"
                    ac = list(acc)
                    ac[a] = (m_tile, 0)
                    nxt_states.append((p_it, (m_tile, 0, False), e_tiles, full, empty, tfull, tempty, holds, read,
                                       tuple(ac), drained))
            else:
                it = m_tile * kblocks + m_kb
                s = it % stages
                if Bar.passes(full[s], (it // stages) & 1):
                    if holds[s] != it:
                        return f"MMA expects item {it} in stage {s} and finds item {holds[s]}"
                    r, e, ac, tf, dr = list(read), list(empty), list(acc), list(tfull), list(drained)
                    r[s] = True
                    e[s] = Bar.arrive(e[s])  # the commit
                    ac[a] = (m_tile, acc[a][1] + 1)
                    if m_kb + 1 == kblocks:
                        tf[a] = Bar.arrive(tf[a])
                        dr[a] = (False,) * warps
                        nxt_states.append((p_it, (m_tile + 1, 0, True), e_tiles, full, tuple(e), tuple(tf), tempty,
                                           holds, tuple(r), tuple(ac), tuple(dr)))
                    else:
                        nxt_states.append((p_it, (m_tile, m_kb + 1, False), e_tiles, full, tuple(e), tfull, tempty,
                                           holds, tuple(r), tuple(ac), drained))
        # ---- epilogue warps
        for w in range(warps):
            t = e_tiles[w]
            if t == tiles:
                continue
            a = t & 1
            if Bar.passes(tfull[a], (t >> 1) & 1):
                if acc[a] != (t, kblocks):
                    return f"epilogue warp {w} reads accumulator {a} for tile {t} and finds {acc[a]}"
                et, te, dr = list(e_tiles), list(tempty), list(drained)
                et[w] = t + 1
                te[a] = Bar.arrive(te[a])
                d = list(dr[a])
                d[w] = True
                dr[a] = tuple(d)
                nxt_states.append((p_it, (m_tile, m_kb, m_wait), tuple(et), full, empty, tfull, tuple(te), holds, read,
                                   acc, tuple(dr)))
        if not nxt_states:
            return f"deadlock: producer at {p_it}, MMA at {(m_tile, m_kb)}, epilogue at {e_tiles}"
        for n in nxt_states:
            if n not in seen:
                seen.add(n)
                stack.append(n)
    return None


@pytest.mark.parametrize("stages,kblocks,tiles,warps", [(4, 3, 3, 2), (3, 2, 5, 2), (4, 1, 5, 2), (2, 5, 3, 4), (4, 6, 2, 4)])
def test_pipeline_parities_hold_in_every_interleaving(stages, kblocks, tiles, warps):
    assert explore(stages, kblocks, tiles, warps) is None


def test_a_producer_waiting_for_the_wrong_parity_is_found():
    found = explore(3, 2, 3, 2, producer_flip=0)
    assert found is not None and ("deadlock" in found or "refills" in found)


def test_an_accumulator_barrier_that_counts_one_warp_too_few_is_found():
    found = explore(3, 2, 5, 2, empty_count=1)
    assert found is not None and ("before every epilogue warp" in found or "finds" in found or "deadlock" in found)
