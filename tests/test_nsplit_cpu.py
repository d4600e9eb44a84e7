"""Host-side logic of the N-split (column-wise) sharding, on CPU: shard boundaries fall on row groups, shards are
contiguous byte slices of the tensor, the checker's result for a shard equals the matching slice of the full result, and
two gloo ranks exchanging handles see each other's in rank order."""
import multiprocessing as mp
import os

import numpy as np
import pytest

from nntrainer_b200 import nsplit
from oracle import oracle as O


def test_shard_rows_are_whole_row_groups():
    for world in (1, 2, 4, 8):
        spans = [nsplit.shard_rows(4096, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == 4096
        for (lo, hi), (lo2, _) in zip(spans, spans[1:] + [(4096, 0)]):
            assert lo % 8 == 0 and hi % 8 == 0 and hi == lo2
    with pytest.raises(ValueError):
        nsplit.shard_rows(4100, 8, 0)  # 4100 rows do not split into 8 shards of whole row groups
    assert nsplit.shard_rows(151936, 8, 7, "q6_K") == (132944, 151936)  # lm_head: 18992 rows per rank


@pytest.mark.parametrize("q,gen", [("q4_K", O.random_q4_Kx8), ("q4_0", O.random_q4_0x8), ("q6_K", O.random_q6_K)])
def test_a_shard_is_a_byte_slice_and_gives_the_matching_output_slice(port, q, gen):
    rng = np.random.default_rng(4)
    N, K, world = 64, 512, 4
    B = gen(rng, N, K)
    x = rng.standard_normal((1, K)).astype(np.float32)
    full = port.gemm(q, x, B, N)[0]
    for r in range(world):
        b0, b1 = nsplit.shard_bytes(q, N, K, world, r)
        lo, hi = nsplit.shard_rows(N, world, r, q)
        part = port.gemm(q, x, np.ascontiguousarray(B[b0:b1]), hi - lo)[0]
        assert np.array_equal(part.view(np.uint32), full[lo:hi].view(np.uint32))


def test_sequence_numbers_are_consecutive_across_passes():
    # 48 launches per pass: the last launch of pass 2 and the first of pass 3 are consecutive,
    # so a launch always waits for "its number minus one" whatever its position
    assert nsplit.sequence_number(1, 48, 0) == 1
    assert nsplit.sequence_number(2, 48, 47) + 1 == nsplit.sequence_number(3, 48, 0)
    assert [nsplit.sequence_number(1, 3, i) for i in range(3)] + [nsplit.sequence_number(2, 3, 0)] == [1, 2, 3, 4]


def _rank_main(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mine = [f"handle-{rank}-{i}".encode() for i in range(3)]  # what NSplitGroup exports: two buffers + a counter
        allh = [None] * world
        dist.all_gather_object(allh, mine)
        ok = all(allh[r][i] == f"handle-{r}-{i}".encode() for r in range(world) for i in range(3))
        lo, hi = nsplit.shard_rows(4096 * world, world, rank)
        q.put((rank, ok, lo, hi))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_exchange_handles_in_rank_order():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 200
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res == [(0, True, 0, 4096), (1, True, 4096, 8192)]


def test_odd_launch_count_per_pass_is_rejected():
    """Two gathered buffers alternate per launch: with an odd number of launches per pass consecutive launches across a
    pass boundary would write the same buffer. The group refuses such a sequence before touching any device."""
    with pytest.raises(ValueError):
        nsplit.NSplitGroup(512, 3)
    with pytest.raises(ValueError):
        nsplit.NSplitGroup(512, 6, ring=4)  # six launches per pass do not continue a rotation of four buffers
    # consecutive launch numbers alternate parity across a pass boundary exactly when the count is even
    for L in (2, 4, 48):
        seq = [nsplit.sequence_number(e, L, l) for e in (1, 2, 3) for l in range(L)]
        assert all((a + 1) == b for a, b in zip(seq, seq[1:]))
        assert all((nsplit.sequence_number(e, L, l) % 2) == ((l + 1) % 2) for e in (1, 2, 3) for l in range(L))


def test_ring_of_four_takes_launches_of_one_size_only():
    """The per-CTA "done reading" slots of the ring-of-four exchange assume every launch runs the same CTAs; two
    buffers take any sequence of sizes."""
    from nntrainer_b200.nsplit import check_ring_rows
    assert check_ring_rows(4, None, 4096) == 4096
    assert check_ring_rows(4, 4096, 4096) == 4096
    with pytest.raises(ValueError):
        check_ring_rows(4, 4096, 320)
    assert check_ring_rows(2, 4096, 320) == 4096
