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
