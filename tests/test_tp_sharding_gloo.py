"""Host logic of the tensor-parallel split on CPU: two `gloo` ranks take their shares of a model (synth.shard_spec), compute
the integer GEMV of their rows with the CPU oracle, and the gathered results must equal the whole projection - the
property the device relies on when it lets every rank write its rows into every rank's vector. The split itself (heads of
q/k/v, row ranges of o/gate/up/down and of the output head) is checked against the whole model's arrays."""
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


def _spec():
    from quintrit_b200 import synth

    return synth.make_model(0, False, 256, 512, 2, 4, 2, 64, 384, 256, 500000.0, 1e-5, config=31, random_norms=True)


def _shapes(spec):
    H, I, hd = spec["hidden"], spec["inter"], spec["head_dim"]
    qd, kvd = spec["q_heads"] * hd, spec["kv_heads"] * hd
    return [(qd, H), (kvd, H), (kvd, H), (H, qd), (I, H), (I, H), (H, I)]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, out_dir: str) -> None:
    import oracle
    from quintrit_b200 import synth

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        spec = _spec()
        mine = synth.shard_spec(spec, rank, world)
        assert mine["tp_rank"] == rank and mine["tp_world"] == world and mine["hidden"] == spec["hidden"]
        for i, (rows, cols) in enumerate(_shapes(spec) * spec["layers"]):
            act = synth.quantize_int8_np(synth.normal_f32(synth.seed_for(31, i, 0, 2), cols))[0]
            n = rows // world
            part = oracle.gemv_planar(mine["weights"][i], n, cols, act)
            gathered = [torch.zeros(n, dtype=torch.int32) for _ in range(world)]
            dist.all_gather(gathered, torch.from_numpy(np.ascontiguousarray(part, dtype=np.int32)))
            whole = oracle.gemv_planar(spec["weights"][i], rows, cols, act)
            assert np.array_equal(torch.cat(gathered).numpy(), whole), (rank, i)
        # the partial maxima every rank contributes give the maximum of the whole vector (the SwiGLU scale exchange)
        x = synth.normal_f32(77, spec["inter"])
        n = spec["inter"] // world
        t = torch.tensor([float(np.abs(x[rank * n:(rank + 1) * n]).max())], dtype=torch.float32)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        assert np.float32(t.item()) == np.abs(x).max()
        with open(os.path.join(out_dir, f"rank{rank}.ok"), "w") as f:
            f.write("ok")
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_cover_every_projection(tmp_path):
    port = _free_port()
    mp.start_processes(_rank_main, args=(2, port, str(tmp_path)), nprocs=2, join=True, start_method="spawn")
    assert (tmp_path / "rank0.ok").exists() and (tmp_path / "rank1.ok").exists()


@pytest.mark.parametrize("world", [1, 2])
def test_shards_are_the_row_ranges_of_the_whole_model(world):
    import quintrit_b200 as q
    from quintrit_b200 import synth

    spec = _spec()
    shards = [synth.shard_spec(spec, r, world) for r in range(world)]
    for i, (rows, cols) in enumerate(_shapes(spec) * spec["layers"]):
        rb = q.row_bytes(cols)
        whole = np.asarray(spec["weights"][i], np.uint8).reshape(rows, rb)
        again = np.concatenate([np.asarray(s["weights"][i], np.uint8).reshape(rows // world, rb) for s in shards])
        assert np.array_equal(again, whole)
    head = np.concatenate([np.asarray(s["lm_head"], np.uint16) for s in shards])
    assert np.array_equal(head, np.asarray(spec["lm_head"], np.uint16))
    assert all(np.array_equal(s["embed"], spec["embed"]) for s in shards)  # the embedding stays whole on every rank
    # 2 KV heads do not split over 4 ranks: q, k and v stay whole on every rank (attention is replicated), the rest is split by rows
    four = [synth.shard_spec(spec, r, 4) for r in range(4)]
    for i, (rows, cols) in enumerate(_shapes(spec) * spec["layers"]):
        rb = q.row_bytes(cols)
        whole = np.asarray(spec["weights"][i], np.uint8).reshape(rows, rb)
        if i % 7 < 3:
            assert all(np.array_equal(np.asarray(s["weights"][i], np.uint8).reshape(rows, rb), whole) for s in four)
        else:
            assert np.array_equal(np.concatenate([np.asarray(s["weights"][i], np.uint8).reshape(rows // 4, rb) for s in four]), whole)
