"""Host model of the K/V ring bookkeeping of the attention pipeline
(megaattention_b200/csrc/fused_prefill.cu: the TMA producer's load sequence and the two MMA
issuers' ``my_slot`` walk), for both stage layouts: shared stages (two heads of a task share
a kv head: one K and one V tile per key block, both issuers consume every slot) and separate
stages (heads share no kv head: per key block the K tiles of the task's heads, then their V
tiles; each issuer consumes only its own).  The two sides are written independently, as in
the kernel: the producer as one linear sequence of loads, the issuers as per-issuer position
arithmetic.  Over random task sequences every slot an issuer waits for must hold exactly
the tile the producer put there in that ring pass, every slot must be released by exactly
the number of arrivals its barrier was initialised with, and the issuers must stay in step."""
import random

KV_SLOTS = 5


def producer_sequence(tasks, sep):
    """[(slot, pass, task, block, which, tile)] in load order."""
    out, slot, rpass = [], 0, 0
    for t, (nt, nblk) in enumerate(tasks):
        nld = nt if sep else 1
        for jj in range(nblk):
            for ld in range(2 * nld):
                which = int(ld >= nld)               # 0 = K, 1 = V
                tile = ld - nld if which else ld     # head of the task (separate stages)
                out.append((slot, rpass, t, jj, which, tile if sep else None))
                slot += 1
                if slot == KV_SLOTS:
                    slot, rpass = 0, rpass + 1
    return out


def issuer_walk(tasks, sep, mi):
    """[(slot, pass, task, block, which)] this issuer waits for and releases; also the
    final ring position, which both issuers must agree on."""
    slot, rpass, out = 0, 0, []

    def my_slot(nt):
        nonlocal slot, rpass
        s, p = slot + (mi if sep else 0), rpass
        if s >= KV_SLOTS:
            s, p = s - KV_SLOTS, p + 1
        slot += nt if sep else 1
        if slot >= KV_SLOTS:
            slot, rpass = slot - KV_SLOTS, rpass + 1
        return s, p

    for t, (nt, nblk) in enumerate(tasks):
        act = mi < nt
        walk = act or not sep
        s, p = my_slot(nt)                            # K of the first block
        if walk:
            out.append((s, p, t, 0, 0))
        for jj in range(nblk):
            s, p = my_slot(nt)                        # V of block jj
            if walk:
                out.append((s, p, t, jj, 1))
            if jj + 1 < nblk:
                s, p = my_slot(nt)                    # K of block jj + 1
                if walk:
                    out.append((s, p, t, jj + 1, 0))
    return out, (slot, rpass)


def check(tasks, sep):
    loads = {(s, p): (t, jj, which, tile) for s, p, t, jj, which, tile in producer_sequence(tasks, sep)}
    assert len(loads) == sum((nt if sep else 1) * 2 * nblk for nt, nblk in tasks)
    releases = {}
    ends = []
    for mi in (0, 1):
        walk, end = issuer_walk(tasks, sep, mi)
        ends.append(end)
        for s, p, t, jj, which in walk:
            lt, ljj, lwhich, ltile = loads[(s, p)]
            assert (lt, ljj, lwhich) == (t, jj, which), (sep, mi, s, p)
            if sep:
                assert ltile == mi                    # its own head's tile, nobody else's
            releases[(s, p)] = releases.get((s, p), 0) + 1
    assert ends[0] == ends[1]
    want = 1 if sep else 2                            # kv_empty's arrival count
    assert set(releases) == set(loads) and all(v == want for v in releases.values())


def test_shared_and_separate_stage_rings_stay_consistent():
    rng = random.Random(7)
    for _ in range(200):
        n = rng.randint(1, 12)
        # shared stages: always two heads per task; separate: the odd head runs alone
        check([(2, rng.randint(1, 9)) for _ in range(n)], sep=False)
        check([(rng.choice((1, 2, 2)), rng.randint(1, 9)) for _ in range(n)], sep=True)
    check([(1, 1)], sep=True)
    check([(1, 3), (1, 2), (1, 7)], sep=False)        # a single head per rank: issuer 1 only keeps count
    check([(2, 1), (1, 1), (2, 3)], sep=True)
