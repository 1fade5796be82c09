"""The pointwise kernels of blocks and mixers beyond the pre-norm block, and the per-head products, each against
plain PyTorch in float32: aligned sizes (16-byte forms) and odd ones (element forms), operands that are column
ranges of wider rows."""

import pytest
import torch

from miniserve_b200 import ops

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda")
DTYPES = [torch.float32, torch.bfloat16]


def _tol(dtype):
    return dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


@pytest.fixture(autouse=True)
def _seeded():
    torch.manual_seed(99)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("t, h, k, n", [(7, 3, 12, 20), (33, 4, 64, 48), (1, 5, 40, 8), (130, 2, 16, 128)])
def test_per_head_products(dtype, t, h, k, n):
    wide = torch.randn(t, h * k + 24, device=DEV).to(dtype)  # x is a column range of wider rows
    x = wide[:, 8:8 + h * k].unflatten(1, (h, k))
    w = (torch.randn(h, n, k, device=DEV) * k ** -0.5).to(dtype)
    out = torch.full((t, h, n), float("nan"), device=DEV, dtype=dtype)
    ops.linear_heads(x, w, out)
    want = torch.einsum("thk,hnk->thn", x.float(), w.float())
    assert torch.allclose(out.float(), want, **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("t, nq, d_pad, dv, inter", [(9, 4, 32, 16, 72), (5, 3, 48, 40, 52), (17, 2, 16, 12, 36), (64, 8, 128, 128, 256)])
def test_gate_and_squared_relu_in_one_launch_and_each_alone(dtype, t, nq, d_pad, dv, inter):
    attn = torch.randn(t, nq, d_pad, device=DEV).to(dtype)
    proj = torch.randn(t, nq * dv + inter + 16, device=DEV).to(dtype)
    gate, up = proj[:, 8:8 + nq * dv], proj[:, 8 + nq * dv:8 + nq * dv + inter]
    row = torch.zeros(t, nq * dv + inter + 8, device=DEV, dtype=dtype)
    ops.gate_relu_squared(row[:, :nq * dv + inter], attn, gate, dv, up)
    want_a = (attn[..., :dv].float() * torch.sigmoid(gate.float()).unflatten(1, (nq, dv))).flatten(1)
    want_b = torch.relu(up.float()) ** 2
    assert torch.allclose(row[:, :nq * dv].float(), want_a, **_tol(dtype))
    assert torch.allclose(row[:, nq * dv:nq * dv + inter].float(), want_b, **_tol(dtype))
    assert (row[:, nq * dv + inter:] == 0).all()  # nothing beyond the features is touched
    alone = torch.zeros_like(row)
    ops.channel_gate(alone[:, :nq * dv], attn, gate, dv, 0.5)
    ops.relu_squared(alone[:, nq * dv:nq * dv + inter], up)
    assert torch.allclose(alone[:, :nq * dv].float(), 0.5 * want_a, **_tol(dtype))
    assert torch.allclose(alone[:, nq * dv:nq * dv + inter].float(), want_b, **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [40, 36, 1032])
def test_stream_concat_and_row_vector(dtype, hidden):
    t, vocab = 6, 19
    res, delta = torch.randn(t, hidden, device=DEV), torch.randn(t, hidden, device=DEV).to(dtype)
    table = torch.randn(vocab, hidden, device=DEV).to(dtype)
    ids = torch.tensor([3, 18, 0, 7, 7, 11], dtype=torch.int32, device=DEV)
    out = torch.full((t, 2 * hidden), float("nan"), device=DEV, dtype=dtype)
    ops.stream_concat(out, res, delta, 0.25, table, ids)
    assert torch.allclose(out[:, :hidden].float(), res + 0.25 * delta.float(), **_tol(dtype))
    assert torch.equal(out[:, hidden:], table[ids.long()])
    keep = out.clone()
    ops.stream_concat(out, res, None, 1.0, table, ids, first=True, second=False)  # the second half stays as it is
    assert torch.equal(out[:, hidden:], keep[:, hidden:]) and torch.allclose(out[:, :hidden].float(), res, **_tol(dtype))
    x, vec = torch.randn(t, hidden, device=DEV), torch.randn(hidden, device=DEV)
    want = x + vec
    ops.add_row_vector(x, vec)
    assert torch.allclose(x, want, atol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rank, d_pad, page", [(40, 48, 8), (128, 128, 16), (10, 16, 4)])
def test_latent_into_pages(dtype, rank, d_pad, page):
    from tests.kernel_util import PagedBatch

    rows = [(5, 9), (0, 3)]
    pb = PagedBatch(rows, page, 1, d_pad, dtype, seed=4)
    proj = torch.randn(pb.num_tokens, rank + 24, device=DEV).to(dtype) * 3
    w = torch.rand(rank, device=DEV) + 0.5
    ops.latent_prepare(pb.k_pool, proj[:, 16:16 + rank], w, 1e-5, pb.positions, pb.row_of_token, pb.page_indptr, pb.page_indices, page,
                       pb.status)
    assert pb.status.item() == 0
    x = proj[:, 16:16 + rank].float()
    want = x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * w
    at = 0
    for r, (start, n) in enumerate(rows):
        got = pb.read(r, pb.k_pool, start + n)[start:, 0].float()
        assert torch.allclose(got[:, :rank], want[at:at + n], **_tol(dtype))
        assert (got[:, rank:] == 0).all()
        at += n
