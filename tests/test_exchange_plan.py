"""The host-side planner of the exchange kernel (allgather, broadcast,
alltoall), replayed on the CPU: the plans of all ranks are executed on numpy
arrays with the kernel's semantics (stage my blocks into a region, then copy
what I want out of the region that holds it) and the outputs compared with the
collective's definition. Covers pulling and pushing, messages that need
several rounds (slices), per-receiver layouts of pushed alltoall blocks, empty
blocks, and that all ranks agree on the rounds.
"""
import numpy as np
import pytest

IN, OUT = 1 << 40, 1 << 41  # two fake address spaces


def _plan(blocks_for, world, region, push, ctas=4, chunk=65536):
    from horovod_b200 import _C
    plans = []
    for me in range(world):
        bl = [(s, d, IN + so if so is not None else 0, OUT + do if do is not None else 0, n)
              for (s, d, so, do, n) in blocks_for(me)]
        plans.append(_C.testing.plan_exchange(bl, me, world, region, push, ctas, chunk))
    rounds = len(plans[0])
    assert all(len(p) == rounds for p in plans)
    for k in range(rounds):  # every rank derives the same epochs for a round
        assert len({plans[me][k][3] for me in range(world)}) == 1
    return plans, rounds


def _replay(plans, rounds, world, inputs, out_sizes, region):
    outs = [np.zeros(n, np.uint8) for n in out_sizes]
    regions = [np.zeros(region, np.uint8) for _ in range(world)]
    for k in range(rounds):
        for me in range(world):
            for (src, self_dst, off, n, dst) in plans[me][k][0]:
                data = inputs[me][src - IN: src - IN + n]
                assert len(data) == n
                if self_dst:
                    outs[me][self_dst - OUT: self_dst - OUT + n] = data
                if off >= 0:
                    targets = [me] if dst == -2 else [dst] if dst >= 0 else \
                        [p for p in range(world) if p != me]
                    for t in targets:
                        assert off % 256 == 0 and off + n <= region
                        regions[t][off:off + n] = data
        for me in range(world):
            for (dst, off, n, src_rank, sig_rank, before) in plans[me][k][1]:
                assert before >= 0
                outs[me][dst - OUT: dst - OUT + n] = regions[src_rank][off:off + n]
    return outs


@pytest.mark.parametrize("world", [2, 3, 8])
@pytest.mark.parametrize("push", [False, True])
def test_allgather_plans(world, push):
    rng = np.random.default_rng(world)
    sizes = [(r + 1) * 148000 + r for r in range(world)]  # uneven, odd byte counts
    inputs = [rng.integers(1, 255, n, dtype=np.uint8) for n in sizes]
    total = sum(sizes)

    def blocks(me):
        out, disp = [], 0
        for r in range(world):
            out.append((r, -1, 0 if r == me else None, disp, sizes[r]))
            disp += sizes[r]
        return out

    for region in (1 << 18, 1 << 24):  # several rounds / one round
        plans, rounds = _plan(blocks, world, region, push)
        assert (rounds > 1) == (region == 1 << 18)
        outs = _replay(plans, rounds, world, inputs, [total] * world, region)
        want = np.concatenate(inputs)
        assert all((o == want).all() for o in outs)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("push", [False, True])
def test_alltoall_plans_and_per_receiver_layout(world, push):
    rng = np.random.default_rng(10 + world)
    row = 4096 + 12
    splits = [[(r + 2 * p) % 4 for p in range(world)] for r in range(world)]
    inputs = [rng.integers(1, 255, sum(splits[r]) * row, dtype=np.uint8) for r in range(world)]
    out_sizes = [sum(splits[r][me] for r in range(world)) * row for me in range(world)]

    def blocks(me):
        send_off = np.concatenate([[0], np.cumsum([s * row for s in splits[me]])])
        recv_off = np.concatenate([[0], np.cumsum([splits[r][me] * row for r in range(world)])])
        out = []
        for r in range(world):
            for j in range(1, world + 1):
                p = (r + j) % world
                out.append((r, p, int(send_off[p]) if r == me else None,
                            int(recv_off[r]) if p == me else None, splits[r][p] * row))
        return out

    region = 1 << 20
    plans, rounds = _plan(blocks, world, region, push)
    outs = _replay(plans, rounds, world, inputs, out_sizes, region)
    for me in range(world):
        pieces = []
        for r in range(world):
            off = sum(splits[r][:me]) * row
            pieces.append(inputs[r][off: off + splits[r][me] * row])
        assert (outs[me] == np.concatenate(pieces)).all()
    if push:
        # A pushed block takes room in its receiver's region only: what one
        # rank receives fits one round although all blocks together would not.
        big = 300000
        def even(me):
            return [(r, p, (p * big if r == me else None), (r * big if p == me else None), big)
                    for r in range(world) for p in range(world)]
        cap = 256 * ((world * big + 255) // 256 + world)
        _, rounds = _plan(even, world, cap, True)
        assert rounds == 1


def test_broadcast_plan_rounds_slice_by_slice():
    world, n, region = 4, 1000001, 1 << 18
    rng = np.random.default_rng(3)
    src = rng.integers(1, 255, n, dtype=np.uint8)
    inputs = [src if r == 2 else np.zeros(0, np.uint8) for r in range(world)]

    def blocks(me):
        return [(2, -1, 0 if me == 2 else None, None if me == 2 else 0, n)]

    for push in (False, True):
        plans, rounds = _plan(blocks, world, region, push)
        assert rounds == 4  # ceil((n + padding) / region)
        outs = _replay(plans, rounds, world, inputs, [0 if r == 2 else n for r in range(world)],
                       region)
        for r in range(world):
            if r != 2:
                assert (outs[r] == src).all()
