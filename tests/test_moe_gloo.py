"""Expert parallelism of the mixture-of-experts block, the exchange on the host: two gloo ranks hold half of the experts each, compute the
results of the (token, expert) pairs they own with the oracle's pieces (zero bits elsewhere), add the buffers as 32-bit integers with an
all-reduce - one share of every value is not zero, so the sum is that share bit for bit - and combine. Every rank must get the oracle's
whole block. (The device blocks do the same through quintrit_b200_moe_forward_partial / _pairs / _finish: tests/test_moe_gpu.py.)"""
import os
import socket
import sys

import numpy as np
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

H, I, E, K, B = 256, 64, 8, 3, 4


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _block():
    import oracle

    rng = np.random.default_rng(31)
    router = oracle.f32_to_bf16_bits((rng.standard_normal(E * H) * 0.05).astype(np.float32))
    gu = [oracle.pack_planar(rng.integers(-1, 2, 2 * I * H).astype(np.int8), 2 * I, H) for _ in range(E)]
    dn = [oracle.pack_planar(rng.integers(-1, 2, H * I).astype(np.int8), H, I) for _ in range(E)]
    scales = rng.uniform(0.5, 2.0, (E, 3)).astype(np.float32)
    scales[3, 2] = -scales[3, 2]  # a negative weight scale: its zero results are -0.0, which an addition of floats would lose
    x = rng.standard_normal((B, H)).astype(np.float32)
    x[1, :] = 0.0
    x[1, 0] = 1.0  # few non-zero activations: many exactly zero sums
    return router, gu, dn, scales, x


def _rank_main(rank: int, world: int, port: int, out_dir: str) -> None:
    import torch
    import torch.distributed as dist

    from oracle import moe as omoe

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        router, gu, dn, scales, x = _block()
        per = E // world
        lo, hi = rank * per, (rank + 1) * per
        for b in range(B):
            probs = omoe.router_probs(x[b], router, E)
            chosen, w = omoe.select(probs, K)
            pairs = np.zeros((K, H), np.float32)
            for i, e in enumerate(chosen):
                if lo <= e < hi:
                    pairs[i] = omoe.expert(x[b], gu[e], dn[e], H, I, *scales[e])
            t = torch.from_numpy(pairs.view(np.int32))
            dist.all_reduce(t)
            got = omoe.combine(t.numpy().view(np.float32), w)
            want, want_ids, want_w = omoe.forward(x[b], router, gu, dn, scales, H, I, K)
            assert list(chosen) == list(want_ids) and np.array_equal(got.view(np.uint32), want.view(np.uint32)), (rank, b)
        with open(os.path.join(out_dir, f"rank{rank}.ok"), "w") as f:
            f.write("ok")
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_exchange_the_pairs_exactly(tmp_path):
    port = _free_port()
    mp.start_processes(_rank_main, args=(2, port, str(tmp_path)), nprocs=2, join=True, start_method="spawn")
    assert (tmp_path / "rank0.ok").exists() and (tmp_path / "rank1.ok").exists()
