"""The fused attention kernel through its raw C-ABI entry point (odla_b200_attention) against float64 numpy:
softmax(scale * Q K^T) V for heads of 128 positions x 64 channels, fp16 and bf16, both output layouts, one head up to
more heads than the grid has CTAs (every CTA then walks several heads through the same shared and tensor memory)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
S, D = 128, 64


def reference(q, k, v, scale):
    s = np.einsum("bhid,bhjd->bhij", q.astype(np.float64), k.astype(np.float64)) * scale
    s -= s.max(axis=-1, keepdims=True)
    p = np.exp(s)
    p /= p.sum(axis=-1, keepdims=True)
    return np.einsum("bhij,bhjd->bhid", p, v.astype(np.float64))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("batch,heads,merge", [(1, 1, 0), (2, 12, 1), (3, 5, 0), (40, 12, 1)])
def test_attention_matches_numpy(gpu_lib, dtype, batch, heads, merge):
    g = torch.Generator().manual_seed(batch * 100 + heads)
    q, k, v = (torch.randn((batch, heads, S, D), generator=g).to(dtype) for _ in range(3))
    q = q * 1.5   # scores of a few units: a soft-max that is neither flat nor one-hot
    scale = 1.0 / 8.0
    want = reference(q.float().numpy(), k.float().numpy(), v.float().numpy(), scale)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    shape = (batch, S, heads, D) if merge else (batch, heads, S, D)
    y = torch.full(shape, float("nan"), dtype=dtype, device="cuda")
    rc = gpu_lib.b200_attention(0 if dtype == torch.float16 else 1, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), y.data_ptr(), batch, heads, S, D,
                                scale, merge, None)
    assert rc == 0
    got = y.float().cpu().numpy()
    if merge:
        got = got.transpose(0, 2, 1, 3)
    assert np.isfinite(got).all()
    # probabilities and the result are each rounded once to the two-byte type: a few units in the last place of the largest terms
    ulp = 2.0 ** -10 if dtype == torch.float16 else 2.0 ** -7
    err = np.abs(got - want)
    assert err.max() <= 4 * ulp * max(1.0, np.abs(want).max()), err.max()
    assert err.mean() <= ulp * 0.5


def test_attention_rejects_other_shapes(gpu_lib):
    x = torch.zeros((1, 1, 64, 64), dtype=torch.float16, device="cuda")
    assert gpu_lib.b200_attention(0, x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), 1, 1, 64, 64, 1.0, 0, None) == -1
    assert gpu_lib.b200_attention(2, x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), 1, 1, 128, 64, 1.0, 0, None) == -1
