"""The seeded generator: numpy definition == torch implementation, and the stated distributions hold."""
import numpy as np
import torch

from quintrit_b200 import synth


def test_splitmix_known_answer():
    # SplitMix64 with seed 0: the first output of the published generator is 0xE220A8397B1DCDAF
    with np.errstate(over="ignore"):
        z = np.uint64(0) + np.uint64(1) * np.uint64(synth.GAMMA)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(synth.M1)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(synth.M2)
        z = z ^ (z >> np.uint64(31))
    assert int(z) == 0xE220A8397B1DCDAF
    assert int(synth.splitmix_u32(0, 0, 1)[0]) == 0xE220A839


def test_torch_and_numpy_agree(oracle):
    seed = synth.seed_for(0, 3, 4, 0)
    a = synth.splitmix_u32(seed, 1000, 5000)
    b = synth.torch_splitmix_u32(seed, 1000, 5000, "cpu").numpy().astype(np.uint32)
    assert np.array_equal(a, b)
    for rows, cols in [(5, 161), (40, 320), (3, 3072)]:
        planar = synth.torch_planar(seed, rows, cols, "cpu", chunk_rows=2).numpy()
        assert np.array_equal(planar, oracle.pack_planar(synth.trits(seed, rows * cols), rows, cols))


def test_distributions():
    t = synth.trits(synth.seed_for(0, 0, 0, 0), 200000)
    frac = [(t == v).mean() for v in (-1, 1, 0)]
    assert abs(frac[0] - 0.3) < 0.01 and abs(frac[1] - 0.3) < 0.01 and abs(frac[2] - 0.4) < 0.01
    s = [float(synth.weight_scale(synth.seed_for(0, l, 0, 1))) for l in range(64)]
    assert min(s) >= 0.5 and max(s) < 2.0
    x = synth.normal_f32(synth.seed_for(0, 0, 0, 2), 100000)
    assert abs(x.mean()) < 0.02 and abs(x.std() - 1.0) < 0.02 and np.isfinite(x).all()
    assert len({synth.seed_for(0, l, p, s) for l in range(40) for p in range(7) for s in range(3)}) == 840


def test_the_oracle_generator_equals_the_numpy_definition(oracle):
    for seed, rows, cols, row0 in [(synth.seed_for(2, 3, 4, 0), 33, 161, 0), (synth.seed_for(0, 0, 6, 0), 7, 3072, 5), (1, 2, 23040, 1)]:
        want = oracle.pack_planar(synth.trits(seed, rows * cols, start=row0 * cols), rows, cols)
        assert np.array_equal(oracle.synth_planar(seed, rows, cols, row0), want)


def test_portable_tables_and_block_scales():
    a = synth.table_bits_np(123, 4096, False)
    assert np.array_equal(a, synth.torch_table_bits(123, 4096, False, "cpu"))
    x = a.view(np.float16).astype(np.float32)
    assert abs(x.std() - 0.02) < 0.002 and abs(x.mean()) < 0.002
    b = synth.table_bits_np(123, 100, True, start=50)
    assert np.array_equal(b, synth.torch_table_bits(123, 150, True, "cpu")[50:])
    s = synth.block_scales_np(9, 1000)
    assert np.array_equal(s, synth.torch_block_scales(9, 1000, "cpu"))
    assert s.min() >= 0.5 and s.max() <= 2.0 and np.array_equal(s.astype(np.float16).astype(np.float32), s)


def test_the_oracle_table_generators_equal_the_numpy_definitions(oracle):
    for bf16 in (False, True):
        assert np.array_equal(oracle.synth_table(77, 5000, bf16, start=3), synth.table_bits_np(77, 5000, bf16, start=3))
    assert np.array_equal(oracle.synth_block_scales(78, 3000, start=11), synth.block_scales_np(78, 3000, start=11))
    assert oracle.stream_read_gbs(1 << 24, reps=3) > 0.1
