"""Row-sharded weights between optimizer steps (--use_fsdp with the fused data-parallel step):
ownership boundaries, packing order and the freshness bookkeeping, all on the CPU."""
import torch

from pfeife_b200.parallel.dp_fused import ALIGN, row_ends, shard_bounds
from pfeife_b200.runtime.params import RankParams, StateEntry, gather_deferrable


def test_bounds_fall_between_rows_of_the_matrix_they_cut():
    # two matrices of 1000 x 520 and a tail of small parameters
    mats = [(0, 520, 1000), (520000, 520, 1000)]
    n = 2 * 520000 + 4096
    for world in (2, 3, 4, 8):
        b = shard_bounds(n, world, mats)
        assert b[0] == 0 and b[-1] == n and all(x <= y for x, y in zip(b, b[1:]))
        for off, cols, rows in mats:
            for x in b[1:-1]:
                if off < x < off + rows * cols:
                    assert (x - off) % cols == 0
            ends = row_ends(off, cols, rows, b)
            assert ends[-1] == rows and all(x <= y for x, y in zip(ends, ends[1:]))
            # every row's flat range lies inside its owner's range
            start = 0
            for r, e in enumerate(ends):
                if e > start:
                    assert b[r] <= off + start * cols and off + e * cols <= max(b[r + 1], off + e * cols)
                    assert off + e * cols <= b[r + 1] or r == world - 1
                start = e
        # shards stay vector-aligned for the kernel
        assert all(x % 4 == 0 for x in b)


def test_even_split_without_matrices():
    b = shard_bounds(10 * ALIGN + 5, 4)
    assert b[0] == 0 and b[-1] == 10 * ALIGN + 5
    assert all((x % ALIGN == 0) for x in b[:-1])


def test_deferrable_matrices_are_packed_first_within_a_group():
    big = torch.zeros(512, 512)
    entries = [StateEntry(0, "bias", "param", torch.zeros(512), True, 0),
               StateEntry(1, "w1", "param", big.clone(), True, 0),
               StateEntry(2, "ln", "param", torch.zeros(512), True, 0),
               StateEntry(3, "w2", "param", big.clone(), True, 1),
               StateEntry(4, "small", "param", torch.zeros(8, 8), True, 1)]
    assert gather_deferrable(big) and not gather_deferrable(torch.zeros(8, 8))
    p = RankParams(entries, torch.device("cpu"), torch.bfloat16, "adamw", [{}, {}], native=True,
                   defer_gather=True)
    assert p.slots[1].deferred and p.slots[3].deferred and not p.slots[0].deferred
    assert p.slots[1].offset == 0                        # the matrix leads its group
    assert p.deferred_below[0] == 512 * 512
    g1_lo = [lo for g, lo, hi in p.group_ranges if g == 1][0]
    assert p.slots[3].offset == g1_lo and p.deferred_below[1] == g1_lo + 512 * 512
    # without the flag the order is the placeholder order
    q = RankParams(entries, torch.device("cpu"), torch.bfloat16, "adamw", [{}, {}], native=True)
    assert q.slots[0].offset == 0 and not q.slots[1].deferred


def test_weights_read_through_their_shadow_precede_the_fp32_read_tail():
    """The fused data-parallel step pushes fp32 masters to the replicas only from
    ``master_from`` on: weights that every op reads through the 16-bit shadow are packed before
    what some op reads in fp32; a group with a parameter nobody analysed is pushed whole."""
    big = torch.zeros(512, 512)
    mk = lambda lp: [StateEntry(0, "bias", "param", torch.zeros(512), True, 0, lp_only=False),
                     StateEntry(1, "w1", "param", big.clone(), True, 0, lp_only=True),
                     StateEntry(2, "pos", "param", torch.zeros(1, 4, 512), True, 0, lp_only=False),
                     StateEntry(3, "conv", "param", torch.zeros(8, 4, 3, 3), True, 0, lp_only=True),
                     StateEntry(4, "w2", "param", big.clone(), True, 1, lp_only=lp)]
    p = RankParams(mk(True), torch.device("cpu"), torch.bfloat16, "adamw", [{}, {}], native=True)
    order = sorted((s.offset, s.entry.qualname) for s in p.packed_slots())
    assert [n for _, n in order] == ["w1", "conv", "bias", "pos", "w2"]
    assert p.master_from[0] == p.slots[0].offset         # the tail starts at the first fp32 read
    g1 = [(lo, hi) for g, lo, hi in p.group_ranges if g == 1][0]
    assert p.master_from[1] == g1[1]                     # nothing of group 1 is read in fp32
    q = RankParams(mk(None), torch.device("cpu"), torch.bfloat16, "adamw", [{}, {}], native=True)
    g1 = [(lo, hi) for g, lo, hi in q.group_ranges if g == 1][0]
    assert q.master_from[1] == g1[0]                     # not analysed: pushed as a whole
    # deferral (row-sharded weights) never applies to a weight that some op reads in fp32
    e = mk(True)
    e[1].lp_only = False
    r = RankParams(e, torch.device("cpu"), torch.bfloat16, "adamw", [{}, {}], native=True,
                   defer_gather=True)
    assert not r.slots[1].deferred and r.slots[4].deferred
    # without a shadow every master is read directly
    f = RankParams(mk(True), torch.device("cpu"), None, "adamw", [{}, {}], native=True)
    assert f.master_from[0] == 0


def test_torch_optimizer_groups_keep_their_own_hyper_parameters():
    """A pipeline rank that holds only parameters of the user's SECOND group must step them
    with that group's learning rate."""
    entries = [StateEntry(0, "w", "param", torch.ones(4), True, 1)]
    hyper = [{"lr": 1.0}, {"lr": 0.25}]
    p = RankParams(entries, torch.device("cpu"), None, "sgd", hyper, native=False)
    p.slots[0].grad.fill_(1.0)
    p.step()
    assert torch.allclose(p.slots[0].master, torch.full((4,), 0.75))
    hyper[1]["lr"] = 0.5
    p.set_hyper(hyper)
    p.slots[0].grad.fill_(1.0)
    p.step()
    assert torch.allclose(p.slots[0].master, torch.full((4,), 0.25))


def test_weights_are_gathered_once_per_gather_session():
    from pfeife_b200.ops import functional as Fn
    w = torch.zeros(256, 1024)
    lp = w.to(torch.bfloat16)
    Fn.register_param(w, lp, None)
    try:
        slot = Fn._slot(w)
        assert Fn._slot(lp) is slot and not Fn._stale(slot)
        Fn.set_gather(w, Fn.GatherInfo(None, (128, 256), 2, 0, torch.zeros(2, dtype=torch.int32)))
        assert not Fn._stale(slot)            # outside a session weights count as complete
        Fn.gather_session(True)
        assert Fn._stale(slot)
        slot.gathered_in = Fn._session_tls.id  # what the gathering op records
        assert not Fn._stale(slot)            # a second use in the same forward does not gather
        Fn.gather_session(False)
        assert not Fn._stale(slot)
        Fn.gather_session(True)               # the next optimizer step's first forward
        assert Fn._stale(slot)
        Fn.gather_session(False)
    finally:
        Fn.unregister_params()
