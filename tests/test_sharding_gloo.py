"""The N > 1 path of the benchmark on CPU: two `gloo` ranks shard the output rows of each projection exactly as
`bench.py --gpus N` does (whole 32-row tiles, no data-path collective), compute their rows with the CPU oracle, and the
gathered slices must equal the unsharded GEMV bit for bit. The barrier + MAX-over-ranks timing reduction of the
benchmark is exercised too. Row sharding of the reference: quintrit-core/src/simd/avx512.rs:1141-1169 (threads take whole
tiles); quintrit-cuda/src/gemv.rs:191-226 computes rows independently, so any row split gives the same integers."""
from __future__ import annotations

import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SHAPES = [(96, 320), (100, 161), (33, 3072), (1, 160), (257, 640)]  # (rows, cols): awkward row counts on purpose


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, out_dir: str) -> None:
    import bench  # the benchmark's own sharding function
    import oracle
    from quintrit_b200 import synth

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        for idx, (rows, cols) in enumerate(SHAPES):
            seed = synth.seed_for(7, idx, 0, 0)
            trits = synth.trits(seed, rows * cols).reshape(rows, cols)
            act = synth.quantize_int8_np(synth.normal_f32(synth.seed_for(7, idx, 0, 2), cols))[0]
            r0, r1 = bench.shard_rows(rows, rank, world)
            mine = oracle.gemv_bruteforce(trits[r0:r1].reshape(-1), r1 - r0, cols, act) if r1 > r0 else np.zeros(0, np.int32)
            # gather (this is the checker's exchange, not part of the data path: every rank keeps only its rows)
            padded = torch.zeros(rows, dtype=torch.int32)
            padded[: r1 - r0] = torch.from_numpy(np.ascontiguousarray(mine, dtype=np.int32))
            gathered = [torch.zeros(rows, dtype=torch.int32) for _ in range(world)]
            dist.all_gather(gathered, padded)
            bounds = [bench.shard_rows(rows, r, world) for r in range(world)]
            full = torch.cat([gathered[r][: b[1] - b[0]] for r, b in enumerate(bounds)]).numpy()
            want = oracle.gemv_bruteforce(trits.reshape(-1), rows, cols, act)
            assert full.shape == want.shape and np.array_equal(full, want), (rank, rows, cols)
        # the timing reduction of the benchmark: barrier, then the maximum over ranks
        dist.barrier()
        t = torch.tensor([1.0 + rank], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        assert t.item() == float(world)
        ok = torch.tensor([1], dtype=torch.int32)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        assert ok.item() == 1
        with open(os.path.join(out_dir, f"rank{rank}.ok"), "w") as f:
            f.write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_two_gloo_ranks_reproduce_the_unsharded_gemv(tmp_path, world):
    port = _free_port()
    mp.start_processes(_rank_main, args=(world, port, str(tmp_path)), nprocs=world, join=True, start_method="spawn")
    for r in range(world):
        assert (tmp_path / f"rank{r}.ok").exists()


@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("rows", [1, 31, 32, 33, 1024, 3072, 23040, 131072 + 5])
def test_shards_partition_the_rows_in_whole_tiles(rows, world):
    import bench

    bounds = [bench.shard_rows(rows, r, world) for r in range(world)]
    assert bounds[0][0] == 0 and bounds[-1][1] == rows
    for (a0, a1), (b0, b1) in zip(bounds, bounds[1:]):
        assert a1 == b0 and a0 <= a1
    for r0, r1 in bounds[:-1]:
        assert r0 % 32 == 0 and r1 % 32 == 0  # only the last shard may end inside a tile
    sizes = [(b[1] - b[0] + 31) // 32 for b in bounds]
    assert max(sizes) - min(sizes) <= 1  # tiles are balanced to within one


@pytest.mark.parametrize("layers,world", [(40, 1), (40, 2), (40, 4), (40, 8), (12, 8), (7, 2)])
def test_shard_plan_covers_every_weight_once(layers, world):
    """Whole layers per rank when they divide evenly (equal shares, full-height matrices), rows otherwise; either way every weight exactly once."""
    import bench

    seen = {}
    totals = []
    for r in range(world):
        units, rule = bench.shard_plan(layers, r, world)
        assert rule == (f"layers/{world}" if world > 1 and layers % world == 0 else f"rows/{world}")
        totals.append(sum((r1 - r0) * k for _, _, r0, r1, k in units))
        for (l, p, r0, r1, k) in units:
            for a, b in seen.get((l, p), []):
                assert r1 <= a or r0 >= b  # row ranges of one projection never overlap
            seen.setdefault((l, p), []).append((r0, r1))
    for (l, p, n, k) in bench.sweep_shapes(layers):
        assert sum(b - a for a, b in seen[(l, p)]) == n
    assert max(totals) <= min(totals) * 1.02 + 32 * 23040  # balanced to a tile row of the widest matrix
