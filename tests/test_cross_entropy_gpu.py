"""lm_head + cross-entropy / accuracy fused into the head GEMM's epilogue (xaxb_lm_head_cross_entropy) against the
CPU restatement of chunked_cross_entropy_loss / chunked_cross_entropy_acc (xax/arch/llm.py:718-887): float32
logits from bf16 hidden states and a bf16 head, log-softmax in float32, masked means."""

import numpy as np
import pytest
import torch

from helpers import bf16, to_numpy, to_torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,V,H", [(1, 8, 64), (7, 1000, 128), (130, 4104, 256), (300, 32000, 512), (64, 128256, 256)])
def test_fused_loss_and_accuracy_match_the_restatement(T, V, H):
    from oracle import llm as ollm
    from xax_b200 import _lib, ops

    rng = np.random.default_rng(T + V)
    hidden = rng.standard_normal((T, H)).astype(np.float32).astype(bf16)
    weight = (rng.standard_normal((V, H)) * 0.08).astype(np.float32).astype(bf16)
    targets = rng.integers(0, V, T).astype(np.int32)
    # make a good share of the positions "correct", ties and edge columns included
    logits = hidden.astype(np.float32) @ weight.astype(np.float32).T
    am = logits.argmax(axis=-1)
    pick = rng.random(T) < 0.5
    targets[pick] = am[pick]
    targets[0] = V - 1
    mask = rng.random(T) < 0.8
    mask[0] = True

    for use_mask in (False, True):
        mk = mask if use_mask else None
        want_loss, want_acc = ollm.chunked_cross_entropy(hidden, targets, weight, mk)
        res, row_loss, row_pred = ops.lm_head_cross_entropy(to_torch(hidden), to_torch(weight), torch.tensor(targets),
                                                            None if mk is None else torch.tensor(mk))
        _lib.device_status()
        res = to_numpy(res)
        assert abs(res[0] - want_loss) <= 2e-5 * max(1.0, abs(want_loss)), (res[0], want_loss)
        assert abs(res[1] - want_acc) < 1e-6, (res[1], want_acc)
        assert res[2] == (mask.sum() if use_mask else T)
    # per-row values: arg-max equal to NumPy's (first index), loss equal to float32 accuracy
    assert np.array_equal(to_numpy(row_pred), am.astype(np.int32))
    m = logits.max(axis=-1)
    lse = m + np.log(np.exp(logits - m[:, None]).sum(axis=-1))
    want_rows = lse - logits[np.arange(T), targets]
    assert np.allclose(to_numpy(row_loss), want_rows, rtol=2e-5, atol=2e-5)


def test_module_level_functions_and_edge_cases():
    import xax_b200 as xax
    from xax_b200 import _lib
    from xax_b200.arch.attention import Linear

    g = torch.Generator(device="cuda").manual_seed(0)
    T, V, H = 20, 512, 128
    hidden = torch.randn((T, H), generator=g, device="cuda").to(torch.bfloat16)
    head = Linear(H, V, use_bias=False, weight=(torch.randn((V, H), generator=g, device="cuda") * 0.1).to(torch.bfloat16))
    targets = torch.randint(0, V, (T,), generator=g, device="cuda")
    loss = xax.chunked_cross_entropy_loss(hidden, targets, head, chunk_size=8)
    acc = xax.chunked_cross_entropy_acc(hidden, targets, head)
    logits = (hidden.float() @ head.weight.float().t())
    want = torch.nn.functional.cross_entropy(logits, targets.long())
    assert abs(float(loss) - float(want)) < 2e-5 * max(1.0, float(want))
    assert abs(float(acc) - float((logits.argmax(-1) == targets).float().mean())) < 1e-6
    none = torch.zeros((T,), dtype=torch.bool, device="cuda")
    assert float(xax.chunked_cross_entropy_loss(hidden, targets, head, none)) == 0.0  # :788: no valid position
    assert float(xax.chunked_cross_entropy_acc(hidden, targets, head, none)) == 0.0
    with pytest.raises(ValueError):
        xax.chunked_cross_entropy_loss(hidden, targets, lambda h: h)
    with pytest.raises(ValueError):
        xax.chunked_cross_entropy_loss(hidden[0], targets, head)
    _lib.device_status()
