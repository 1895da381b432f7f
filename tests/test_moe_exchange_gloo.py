"""Host-side logic of the expert-parallel MoE exchange, run as two gloo ranks on
CPU: the split plan derived from the gathered per-(rank, expert) counts, the
dispatch all-to-all, the arrival order assumed by the grouped FFN (source-rank
major, local expert minor) and the return all-to-all that restores each rank's
slot order.
"""
import os

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fe2o3_b200.moe import pair_plan, split_plan

EXPERTS, WIDTH = 4, 3


def _rank_main(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(100 + rank)
        per = EXPERTS // world
        counts_local = rng.integers(0, 6, EXPERTS).astype(np.int32)
        if rank == 0:
            counts_local[1] = 0  # an empty segment
        gathered = [torch.zeros(EXPERTS, dtype=torch.int32) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(counts_local))
        counts = np.stack([g.numpy() for g in gathered])
        send_rows, recv_rows, group_offsets = split_plan(counts, rank, world)
        # local compact rows are expert-major; row payload = (source rank, expert, index within the segment)
        rows = [(rank, e, i) for e in range(EXPERTS) for i in range(counts_local[e])]
        compact = torch.tensor(rows, dtype=torch.float32).reshape(-1, WIDTH)
        assert sum(send_rows) == len(rows)
        recv = torch.zeros(sum(recv_rows), WIDTH)
        dist.all_to_all_single(recv, compact, [r for r in recv_rows], [r for r in send_rows])
        # arrival order: group g = (source s, local expert le) occupies rows [offsets[g], offsets[g+1])
        for s in range(world):
            for le in range(per):
                g = s * per + le
                seg = recv[group_offsets[g]:group_offsets[g + 1]].numpy()
                want = [(s, rank * per + le, i) for i in range(counts[s, rank * per + le])]
                assert seg.tolist() == [list(map(float, w)) for w in want], (rank, g)
        assert group_offsets[-1] == sum(recv_rows)
        # "FFN": tag every row, then return it; each rank must get its own slot order back
        processed = recv + 1000.0
        back = torch.zeros(len(rows), WIDTH)
        dist.all_to_all_single(back, processed, [r for r in send_rows], [r for r in recv_rows])
        assert torch.equal(back, compact + 1000.0)
        results[rank] = 1
    finally:
        dist.destroy_process_group()


def test_exchange_plan_two_ranks():
    world = 2
    port = 29500 + (os.getpid() % 2000)
    with mp.Manager() as m:
        results = m.dict()
        mp.spawn(_rank_main, args=(world, port, results), nprocs=world, join=True)
        assert dict(results) == {0: 1, 1: 1}


def test_split_plan_single_rank_is_identity():
    counts = np.array([[3, 0, 2, 5]])
    send, recv, off = split_plan(counts, 0, 1)
    assert send == [10] and recv == [10] and off.tolist() == [0, 3, 3, 5, 10]


def test_split_plan_uses_admitted_rows_when_capacity_drops():
    """With a capacity below demand the senders' compact buffers hold admitted rows only, so the plan
    must be fed the admitted counts: the send sizes then add up to each sender's compact row count and
    every receiver's segments tile its receive buffer."""
    requested = np.array([[9, 2, 7, 4], [1, 8, 3, 6]])
    capacity = 5
    admitted = np.minimum(requested, capacity)
    world = 2
    plans = [split_plan(admitted, r, world) for r in range(world)]
    for r, (send, recv, off) in enumerate(plans):
        assert sum(send) == admitted[r].sum()
        assert off[-1] == sum(recv) and (np.diff(off.astype(np.int64)) >= 0).all()
    for src in range(world):
        for dst in range(world):
            assert plans[src][0][dst] == plans[dst][1][src]   # what one sends the other expects


def test_pair_plan_layout():
    """Row layout of the peer exchange: on its owner every expert's rows are one contiguous segment made
    of one run per source rank, and the runs of all (owner, expert, source) triples tile the owners'
    buffers without gaps or overlaps."""
    rng = np.random.default_rng(7)
    world, experts = 4, 8
    per = experts // world
    counts = rng.integers(0, 9, (world, experts))
    counts[2, 3] = 0
    covered = [np.zeros(int(counts[:, d * per:(d + 1) * per].sum()), np.int32) for d in range(world)]
    for r in range(world):
        pairs, bases = pair_plan(counts, r, world)
        assert pairs[0] == 0 and pairs[-1] == counts[:, r * per:(r + 1) * per].sum()
        for le in range(per):
            for k in range(world):   # run k of a segment holds the rows of source (owner + k) % world
                assert pairs[le * world + k + 1] - pairs[le * world + k] == counts[(r + k) % world, r * per + le]
        assert bases[r * per] == 0   # own rows of the first local expert: placed without knowing any other rank's counts
        for e in range(experts):
            d = e // per
            covered[d][bases[e]:bases[e] + counts[r, e]] += 1
            # the sender's base agrees with the owner's pair table
            owner_pairs, _ = pair_plan(counts, d, world)
            assert bases[e] == owner_pairs[(e % per) * world + (r - d) % world]
    assert all((c == 1).all() for c in covered)
