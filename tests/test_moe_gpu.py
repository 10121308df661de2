"""The mixture-of-experts block on the GPU (quintrit_b200_moe_*) against its composition from the reference's pieces in oracle/moe.py: the
chosen experts, their weights and the output, bit for bit, token by token. The reference has no softmax-routed block with ternary SwiGLU
experts to run (its Moe is Nemotron-H's), so the oracle is pinned piecewise only: every piece it calls is pinned by the other tests."""
import numpy as np
import pytest

import oracle
import quintrit_b200 as q
from oracle import moe as omoe

pytestmark = pytest.mark.gpu


def _block(seed, hidden, inter, n_experts):
    rng = np.random.default_rng(seed)
    router = oracle.f32_to_bf16_bits((rng.standard_normal(n_experts * hidden) * 0.05).astype(np.float32))
    gu = [oracle.pack_planar(rng.choice([-1, 1, 0], 2 * inter * hidden, p=[0.3, 0.3, 0.4]).astype(np.int8), 2 * inter, hidden) for _ in range(n_experts)]
    dn = [oracle.pack_planar(rng.choice([-1, 1, 0], hidden * inter, p=[0.3, 0.3, 0.4]).astype(np.int8), hidden, inter) for _ in range(n_experts)]
    scales = rng.uniform(0.5, 2.0, (n_experts, 3)).astype(np.float32)
    return rng, router, gu, dn, scales


@pytest.mark.parametrize("hidden,inter,n_experts,top_k,batch", [(256, 128, 16, 4, 5), (384, 208, 24, 8, 16), (2048, 768, 12, 8, 3)])
def test_block_equals_its_composition_from_the_reference_pieces(hidden, inter, n_experts, top_k, batch):
    rng, router, gu, dn, scales = _block(hidden + inter, hidden, inter, n_experts)
    block = q.Moe(hidden, inter, top_k, router, gu, dn, scales, max_batch=16)
    for call in range(2):  # the second call reuses every buffer
        x = (rng.standard_normal((batch, hidden)) * (1.0 + call)).astype(np.float32)
        out, ids, w = block.forward(x)
        for b in range(batch):
            want, want_ids, want_w = omoe.forward(x[b], router, gu, dn, scales, hidden, inter, top_k)
            assert list(ids[b]) == list(want_ids), (call, b)
            assert np.array_equal(w[b].view(np.uint32), want_w.view(np.uint32)), (call, b)
            assert np.array_equal(out[b].view(np.uint32), want.view(np.uint32)), (call, b)
    # a zero token: every expert is equally probable (std::sort decides which are chosen), the activation scale is 0 and the experts give
    # zeros (layer.rs:148-150)
    out, ids, w = block.forward(np.zeros((1, hidden), np.float32))
    assert not out.any() and len(set(int(i) for i in ids[0])) == top_k and np.all(w[0] == w[0][0])
    assert block.time_ms(1, 3) > 0  # (timed on the batch of the last forward: the zero token)
    block.free()


def test_equal_probabilities_are_ordered_as_std_sort_orders_them():
    """Two experts with the same router row have exactly the same probability. The device flags the token and the host's std::sort decides;
    whatever it decides, both of the tied experts are among the chosen when they rank above the cut, and the weights still sum to one."""
    hidden, inter, n_experts, top_k = 256, 64, 8, 3
    rng, router, gu, dn, scales = _block(5, hidden, inter, n_experts)
    r = np.asarray(router, np.uint16).reshape(n_experts, hidden).copy()
    x = rng.standard_normal((1, hidden)).astype(np.float32)
    probs = omoe.router_probs(x[0], r, n_experts)
    top = int(np.argmax(probs))
    twin = (top + 1) % n_experts
    r[twin] = r[top]
    block = q.Moe(hidden, inter, top_k, r, gu, dn, scales, max_batch=4)
    out, ids, w = block.forward(x)
    assert {top, twin} <= set(int(i) for i in ids[0]) and abs(float(w[0].sum()) - 1.0) < 1e-6
    assert w[0][0] == w[0][1]  # the two equal probabilities lead
    block.free()


def test_arguments():
    rng, router, gu, dn, scales = _block(9, 256, 64, 4)
    with pytest.raises(q.QuintritError) as e:
        q.Moe(200, 64, 2, router[:800], gu, dn, scales)  # hidden not a multiple of 128 (and the matrices do not fit it)
    assert e.value.code in (3, 6)
    with pytest.raises(q.QuintritError) as e:
        q.Moe(256, 64, 5, router, gu, dn, scales)  # more experts chosen than there are
    assert e.value.code == 2
    block = q.Moe(256, 64, 2, router, gu, dn, scales, max_batch=2)
    with pytest.raises(q.QuintritError) as e:
        block.forward(np.zeros((3, 256), np.float32))
    assert e.value.code == 2
    block.free()


def test_expert_parallel_shares_add_up_to_the_one_gpu_block():
    """Two blocks that hold half of the experts each (here on one GPU; on several GPUs the addition is an all-reduce): every share routes all
    tokens alike, runs its own pairs, and the pairs' buffers added as integers give the one-GPU result bit for bit."""
    hidden, inter, n_experts, top_k, batch = 256, 128, 16, 4, 7
    rng, router, gu, dn, scales = _block(77, hidden, inter, n_experts)
    x = rng.standard_normal((batch, hidden)).astype(np.float32)
    whole = q.Moe(hidden, inter, top_k, router, gu, dn, scales)
    want, want_ids, want_w = whole.forward(x)
    half = n_experts // 2
    shares = [q.Moe(hidden, inter, top_k, router, gu[r * half:(r + 1) * half], dn[r * half:(r + 1) * half], scales[r * half:(r + 1) * half], n_experts=n_experts, expert_first=r * half)
              for r in range(2)]
    with pytest.raises(q.QuintritError) as e:
        shares[0].forward(x)  # a share alone cannot finish
    assert e.value.code == 2
    for sh in shares:
        sh.forward_partial(x)
    a, b = shares[0].pairs_tensor(), shares[1].pairs_tensor()
    assert a.numel() == batch * top_k * hidden
    nonzero_a, nonzero_b = (a != 0), (b != 0)
    assert not bool((nonzero_a & nonzero_b).any())  # every value has one owner
    total = a + b
    a.copy_(total)
    b.copy_(total)
    import torch

    torch.cuda.synchronize()
    for sh in shares:
        out, ids, w = sh.finish()
        assert np.array_equal(ids, want_ids) and np.array_equal(w.view(np.uint32), want_w.view(np.uint32))
        assert np.array_equal(out.view(np.uint32), want.view(np.uint32))
    for blk in shares + [whole]:
        blk.free()
