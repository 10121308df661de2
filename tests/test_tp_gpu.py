"""Tensor-parallel decode over 2 GPUs (one process per GPU, exchange through NVLink peer stores inside the token kernel)
against the CPU oracle of the whole model: every rank's logits slice bit for bit, the same greedy tokens on every rank.
The reference's GPU decoder runs on one GPU; the split is the one quintrit's north star names (rows of q/k/v/gate/up and of
o/down per GPU), and because every exchanged value is an exact integer sum, a maximum or a copied float, the result is
the one-GPU result. Skipped unless two GPUs are visible."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, out_dir: str, geometry) -> None:
    import torch.distributed as dist

    import oracle
    import quintrit_b200 as q
    from quintrit_b200 import synth

    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        f32_values, q_heads, kv_heads, head_dim, hidden, inter = geometry
        spec = synth.make_model(q.ARCH_LLAMA, f32_values, hidden, inter, 3, q_heads, kv_heads, head_dim, 512, 768, 500000.0, 1e-5, config=21,
                                random_norms=True)
        dec = q.Decoder(synth.shard_spec(spec, rank, world), device=rank)
        handles = [None] * world
        dist.all_gather_object(handles, dec.tp_handle())
        dec.tp_attach(handles)
        dist.barrier()
        ref = oracle.Model(spec)
        v = spec["vocab"] // world
        tokens = synth.prompt_tokens(5, 300 if head_dim == 64 else 20, spec["vocab"])
        for pos, tok in enumerate(tokens):
            want = ref.forward(int(tok), pos)
            check = pos < 8 or pos % 37 == 0 or pos == len(tokens) - 1
            got, greedy = dec.forward(int(tok), pos, want_logits=check)
            if check:
                assert np.array_equal(got.view(np.uint32), want[rank * v:(rank + 1) * v].view(np.uint32)), (rank, pos)
            assert greedy == oracle.argmax(want), (rank, pos)
        out = dec.generate(tokens[:5], 6)
        ref2 = oracle.Model(spec)
        for pos, tok in enumerate(tokens[:5]):
            last = ref2.forward(int(tok), pos)
        want_tokens = []
        for i in range(6):
            t = oracle.argmax(last)
            want_tokens.append(t)
            last = ref2.forward(t, 5 + i)
        assert list(out) == want_tokens, (rank, list(out), want_tokens)
        dist.barrier()
        dec.free()
        with open(os.path.join(out_dir, f"rank{rank}.ok"), "w") as f:
            f.write("ok")
    finally:
        dist.destroy_process_group()


# the third geometry has three KV heads: two ranks do not divide them, so attention is replicated on both and only o, the FFN and the head are split
@pytest.mark.parametrize("geometry", [(False, 4, 2, 64, 256, 512), (True, 4, 2, 128, 512, 1024), (False, 6, 3, 64, 384, 512)])
def test_two_ranks_decode_like_one_cpu_model(tmp_path, geometry):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    port = _free_port()
    mp.start_processes(_rank_main, args=(2, port, str(tmp_path), geometry), nprocs=2, join=True, start_method="spawn")
    assert (tmp_path / "rank0.ok").exists() and (tmp_path / "rank1.ok").exists()


def test_a_silent_rank_ends_in_an_error_not_in_a_hang(monkeypatch):
    """Failure detection without a GPU fault: rank 0 of a two-rank group decodes alone (its peer exists but never launches), so
    the pairs it waits for never arrive. The wait is bounded (QUINTRIT_B200_TP_WAIT_MS, here 200 ms): the kernel gives up, sets
    its status, every CTA leaves through the grid barrier, and the call returns QUINTRIT_ERR_DEVICE. The context stays usable.
    Only one kernel runs at any time, so nothing on the GPU waits on another launch."""
    import oracle
    import quintrit_b200 as q
    from quintrit_b200 import synth

    monkeypatch.setenv("QUINTRIT_B200_TP_WAIT_MS", "200")
    spec = synth.make_model(q.ARCH_LLAMA, False, 256, 512, 2, 4, 2, 64, 512, 256, 500000.0, 1e-5, config=22, random_norms=True)
    group = [q.Decoder(synth.shard_spec(spec, r, 2), device=0) for r in range(2)]
    for d in group:
        d.tp_attach_local(group)
    import time

    group[1].info()  # nothing of rank 1 ever launches
    t0 = time.perf_counter()
    with pytest.raises(q.QuintritError) as e:
        group[0].forward(1, 0)
    elapsed = time.perf_counter() - t0
    assert e.value.code == 15 and "another rank" in str(e.value)
    # the patience runs out ONCE: after the first wait gave up, every later exchange of the launch returns at once
    assert elapsed < 0.6, f"the kernel took {elapsed:.2f} s to give up with 0.2 s of patience"
    for d in group:
        d.free()
    # the device still works: a decoder of the whole model gives the oracle's logits
    whole = q.Decoder(spec)
    want = oracle.Model(spec).forward(1, 0)
    got, _ = whole.forward(1, 0)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    whole.free()
    # set-up errors of the in-process attach
    lone = q.Decoder(spec)
    with pytest.raises(q.QuintritError) as e:
        lone.tp_attach_local([lone])
    assert e.value.code == 2
    lone.free()


def test_a_grid_barrier_that_cannot_complete_gives_up():
    """The barrier's give-up path, made to run out without a fault or a hang: four resident CTAs wait for a fifth arrival
    with 5000 polls of patience. Status 2 comes back as QUINTRIT_ERR_DEVICE, every CTA was released by the failure bit and
    saw it again at its next barrier, and the device keeps working."""
    import quintrit_b200 as q

    with pytest.raises(q.QuintritError) as e:
        q.selftest_barrier(0, ctas=4, spin_limit=5000)
    assert e.value.code == 15 and "grid barrier" in str(e.value)
    assert q.last_selftest_released() == 4
    m = q.Matrix(np.full(32 * 32, 125, np.uint8), 32, 160)
    assert not m.gemv_i32(np.ones(160, np.int8)).any()
