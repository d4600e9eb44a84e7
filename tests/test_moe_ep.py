"""Expert-parallel MoE: ownership helper on CPU; on two or more GPUs the expert-parallel forward must equal the
single-GPU forward bit for bit on every rank (same routing, same expert kernels, same combine order)."""
import os

import numpy as np
import pytest

from nntrainer_b200 import nsplit


def test_expert_ranges_partition_the_experts():
    for E, world in ((128, 8), (32, 8), (128, 2), (16, 1)):
        spans = [nsplit.expert_range(E, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == E
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    with pytest.raises(ValueError):
        nsplit.expert_range(30, 8, 0)



def _make_layer_weights(rng, form, H, I, E, torch, O):
    """(router, gate, up, down, kwargs) of a Qwen-form layer with Q4_K experts or a GPT-OSS-form layer with Q4_0 experts
    and biases."""
    router = torch.from_numpy((rng.standard_normal((H, E)) * 0.02).astype(np.float32)).cuda()
    if form == "qwen_q4_K":
        mk = lambda n, k: torch.from_numpy(O.random_q4_Kx8(rng, n, k)).cuda()
        kw = {}
    else:
        mk = lambda n, k: torch.from_numpy(O.random_q4_0x8(rng, n, k)).cuda()
        vec = lambda n, s: torch.from_numpy((rng.standard_normal(n) * s).astype(np.float32)).cuda()
        kw = dict(qtype="q4_0", kind=1, router_bias=vec(E, 0.01), gate_b=[vec(I, 0.1) for _ in range(E)],
                  up_b=[vec(I, 0.1) for _ in range(E)], down_b=[vec(H, 0.1) for _ in range(E)], alpha=1.702)
    gate = [mk(I, H) for _ in range(E)]
    up = [mk(I, H) for _ in range(E)]
    down = [mk(H, I) for _ in range(E)]
    return router, gate, up, down, kw


def _rank_main(rank, world, port, q):
    import torch
    import torch.distributed as dist
    from nntrainer_b200 import backend as be, build
    from oracle import oracle as O
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        build.build()
        be.init(rank)
        ok = True
        for form, (H, I, E, k) in (("qwen_q4_K", (512, 256, 16, 4)), ("gpt_oss_q4_0", (352, 352, 8, 4))):
            rng = np.random.default_rng(5)  # the same layer on every rank
            router, gate, up, down, kw = _make_layer_weights(rng, form, H, I, E, torch, O)
            full = be.MoeLayer(router, gate, up, down, k, **kw)
            lo, hi = nsplit.expert_range(E, world, rank)
            own = lambda ws: [w if lo <= e < hi else None for e, w in enumerate(ws)]
            for T in (1, 5):
                part = be.MoeLayer(router, own(gate), own(up), own(down), k, **kw).enable_expert_parallel(
                    T, layers_per_epoch=3)
                for call in range(7):  # several passes: buffer alternation and call numbering across passes
                    x = torch.from_numpy(rng.standard_normal((T, H)).astype(np.float32)).cuda()
                    want = full.forward(x)
                    got = part.forward_ep(x, layer=call % 3, bump_epoch=(call % 3 == 0))
                    torch.cuda.synchronize()
                    ok = ok and bool(torch.equal(got.view(torch.int32), want.view(torch.int32)))
                be.device_status()
                part._ep_buf.close()
        q.put((rank, ok))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.parametrize("form,H,I,E,k", [("qwen_q4_K", 512, 256, 8, 2), ("gpt_oss_q4_0", 352, 352, 8, 4)])
def test_expert_parallel_path_with_one_rank_equals_plain_forward(form, H, I, E, k):
    """One rank owning every expert: the publishing down projection and the waiting combine against the plain path,
    over several passes (two alternating buffers, call numbers that keep growing); Q4_K experts in the Qwen form and
    Q4_0 experts with biases in the GPT-OSS form."""
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from nntrainer_b200 import backend as be, build
    from oracle import oracle as O
    build.build()
    be.init(0)
    rng = np.random.default_rng(9)
    router, gate, up, down, kw = _make_layer_weights(rng, form, H, I, E, torch, O)
    full = be.MoeLayer(router, gate, up, down, k, **kw)
    for T in (1, 3):
        part = be.MoeLayer(router, gate, up, down, k, **kw).enable_expert_parallel(T, layers_per_epoch=2)
        for call in range(5):
            x = torch.from_numpy(rng.standard_normal((T, H)).astype(np.float32)).cuda()
            want = full.forward(x)
            got = part.forward_ep(x, layer=call % 2, bump_epoch=(call % 2 == 0))
            torch.cuda.synchronize()
            assert torch.equal(got.view(torch.int32), want.view(torch.int32))
        be.device_status()
        part._ep_buf.close()


@pytest.mark.gpu
def test_expert_parallel_forward_equals_single_gpu_forward_on_every_rank():
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + os.getpid() % 200
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=240) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res == [(r, True) for r in range(world)]
