"""The GEMV entry point that allocates nothing gives the integers of the regular device entry point.

Collected last on purpose (file name): it shares one static device array with every other call of its kind in the
process, so a failure here must not hide the results of the other tests. It is written to pass in a fresh process and
after the rest of the suite alike: the first call performs the per-device set-up whichever test ran before.
"""
import numpy as np
import pytest
import torch

import quintrit_b200 as q

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,cols", [(3072, 3072), (1000, 23040), (40, 161)])
def test_noalloc_entry_matches_the_regular_entry_twice_in_a_row(rows, cols):
    rng = np.random.default_rng(rows + cols)
    trits = rng.choice([-1, 1, 0], rows * cols, p=[0.3, 0.3, 0.4]).astype(np.int8)
    m = q.Matrix.from_trits(trits, rows, cols)
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):  # the second call reuses the array with the first call's contents still in it
        act = torch.from_numpy(rng.integers(-128, 128, cols).astype(np.int8)).cuda()
        want = torch.full((rows,), 12345, dtype=torch.int32, device="cuda")
        got = torch.full((rows,), -777, dtype=torch.int32, device="cuda")
        m.gemv_i32_device(act.data_ptr(), want.data_ptr(), stream)
        m.gemv_i32_noalloc(act.data_ptr(), got.data_ptr(), stream)
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"call {call}"  # integers: the tolerance is zero
        assert torch.equal(want.cpu(), torch.from_numpy(m.gemv_i32(act.cpu().numpy())))
    m.free()


def test_noalloc_entry_rejects_bad_arguments():
    m = q.Matrix.from_trits(np.zeros(32 * 160, np.int8), 32, 160)
    with pytest.raises(q.QuintritError) as e:
        m.gemv_i32_noalloc(0, 0)
    assert e.value.code == 1
    m.free()
    with pytest.raises(q.QuintritError) as e:
        m.gemv_i32_noalloc(16, 16)
    assert e.value.code == 14


def test_noalloc_entry_takes_the_widest_matrix_the_library_accepts():
    """The static array holds 4096 work items. A matrix needs fewer than (CTA slots + block pairs) of them, and the library
    accepts at most 131072 columns = 410 block pairs, so no matrix that can be created reaches the INVALID_SHAPE answer
    of this entry; the widest one is the case nearest to it and has to give the integers of the regular entry."""
    rows, cols = 40, 131072
    with pytest.raises(q.QuintritError) as e:
        q.Matrix.from_trits(np.zeros(8 * (cols + 160), np.int8), 8, cols + 160)
    assert e.value.code == 3  # QUINTRIT_ERR_INVALID_SHAPE at creation, before any GEMV entry sees it
    rng = np.random.default_rng(11)
    m = q.Matrix.from_trits(rng.integers(-1, 2, rows * cols).astype(np.int8), rows, cols)
    act = torch.from_numpy(rng.integers(-128, 128, cols).astype(np.int8)).cuda()
    got = torch.full((rows,), -777, dtype=torch.int32, device="cuda")
    want = torch.full((rows,), 12345, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    m.gemv_i32_noalloc(act.data_ptr(), got.data_ptr(), stream)
    m.gemv_i32_device(act.data_ptr(), want.data_ptr(), stream)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    m.free()


def test_noalloc_entry_inside_a_stream_capture():
    """The first call (outside a capture) does the per-device set-up; a later call is recorded into a CUDA graph, and
    each replay of the graph gives the integers of the regular entry for the activations then in the buffer."""
    rows, cols = 2048, 8192
    rng = np.random.default_rng(7)
    m = q.Matrix.from_trits(rng.integers(-1, 2, rows * cols).astype(np.int8), rows, cols)
    act = torch.from_numpy(rng.integers(-128, 128, cols).astype(np.int8)).cuda()
    got = torch.zeros(rows, dtype=torch.int32, device="cuda")
    want = torch.zeros(rows, dtype=torch.int32, device="cuda")
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        m.gemv_i32_noalloc(act.data_ptr(), got.data_ptr(), side.cuda_stream)
    side.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        m.gemv_i32_noalloc(act.data_ptr(), got.data_ptr(), torch.cuda.current_stream().cuda_stream)
    for replay in range(3):
        act.copy_(torch.from_numpy(rng.integers(-128, 128, cols).astype(np.int8)))
        got.fill_(-777)
        torch.cuda.synchronize()
        graph.replay()
        m.gemv_i32_device(act.data_ptr(), want.data_ptr(), torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"replay {replay}"
    del graph
    m.free()
