"""add + ReLU (with gradient) and 3x3/s2/p1 max pooling against torch on the same inputs.

Shapes follow the reference's tests (tests/torch/test_add_relu.py:32-64,
tests/torch/test_npu_max_pool2d.py:31-40), with the largest ones scaled down along the batch
dimension. Both operators are exact: results must be bit-identical to torch's.
"""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.float16, torch.bfloat16]


def _inputs(shape, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = (torch.rand(shape, generator=g) * 4 - 2).to(dtype)
    y = (torch.rand(shape, generator=g) * 4 - 2).to(dtype)
    return x.cuda(), y.cuda()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(1, 100, 3), (18,), (3, 256, 232, 100), (5, 7, 11), (1,),
                                   (2, 3, 1000003)])
def test_add_relu_matches_torch(shape, dtype):
    import mx_driving
    x, y = _inputs(shape, dtype, 1)
    want = F.relu(x + y)
    got = mx_driving.npu_add_relu(x.clone(), y)
    assert got.dtype == dtype and got.shape == want.shape
    assert torch.equal(got, want)


def test_add_relu_overwrites_large_x_and_leaves_small_x_alone():
    """The reference's observable contract (mx_driving/ops/npu_add_relu.py:22-25): x is
    overwritten from 2,000,000 elements up, below that the result is a new tensor. Both on
    views that start 4 bytes past a 16-byte boundary."""
    import mx_driving
    base_x, base_y = _inputs((2000001,), torch.float32, 2)
    x, y = base_x[1:], base_y[1:]
    want = F.relu(x + y)
    got = mx_driving.npu_add_relu(x, y)
    assert got.data_ptr() == x.data_ptr()
    assert torch.equal(x, want)

    base_x, base_y = _inputs((4099,), torch.float32, 2)
    x, y = base_x[1:], base_y[1:]
    keep = x.clone()
    got = mx_driving.npu_add_relu(x, y)
    assert got.data_ptr() != x.data_ptr()
    assert torch.equal(x, keep) and torch.equal(got, F.relu(keep + y))


def test_add_relu_never_overwrites_non_contiguous_x():
    import mx_driving
    x, y = _inputs((1500, 1500), torch.float32, 4)
    xt, keep = x.t(), x.t().clone()
    got = mx_driving.npu_add_relu(xt, y)
    assert torch.equal(xt, keep) and torch.equal(got, F.relu(keep + y))


def test_add_relu_propagates_nan_like_torch():
    import mx_driving
    x = torch.tensor([float("nan"), 1.0, -1.0, float("inf"), -float("inf")] * 5, device="cuda")
    y = torch.zeros_like(x)
    want = F.relu(x + y)
    got = mx_driving.npu_add_relu(x.clone(), y)
    assert torch.equal(torch.isnan(got), torch.isnan(want))
    assert torch.equal(got[~torch.isnan(got)], want[~torch.isnan(want)])


@pytest.mark.parametrize("dtype", DTYPES)
def test_add_relu_backward(dtype):
    import mx_driving
    x, y = _inputs((2, 64, 58, 100), dtype, 3)
    xr, yr = x.clone().requires_grad_(), y.clone().requires_grad_()
    F.relu(xr + yr).backward(torch.ones_like(x) * 0.5)
    # leaves that require grad are copied, intermediates are overwritten
    xa, ya = x.clone().requires_grad_(), y.clone().requires_grad_()
    out = mx_driving.npu_add_relu(xa * 1, ya)
    out.backward(torch.ones_like(x) * 0.5)
    assert torch.equal(xa.grad, xr.grad) and torch.equal(ya.grad, yr.grad)
    xb = x.clone().requires_grad_()
    out = mx_driving.npu_add_relu(xb, y)
    assert torch.equal(xb.detach(), x)  # the leaf was not overwritten
    out.sum().backward()
    assert torch.equal(xb.grad, (out > 0).to(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(2, 64, 464, 800), (1, 32, 4640, 18), (2, 16, 42, 2479),
                                   (1, 16, 3, 3), (1, 8, 100, 100), (1, 1, 1, 1), (3, 5, 7, 9),
                                   (1, 2, 1, 17), (1, 2, 17, 1)])
def test_max_pool2d_matches_torch(shape, dtype):
    import mx_driving
    g = torch.Generator().manual_seed(123)
    x = (torch.rand(shape, generator=g) - 0.5).to(dtype).cuda()
    want = F.max_pool2d(x.float(), 3, 2, 1).to(dtype)
    got = mx_driving.npu_max_pool2d(x, 3, 2, 1)
    assert got.shape == want.shape and got.dtype == dtype
    assert torch.equal(got, want)


def test_max_pool2d_nan_and_argument_checks():
    import mx_driving
    x = torch.zeros(1, 1, 6, 6, device="cuda")
    x[0, 0, 2, 2] = float("nan")
    x[0, 0, 5, 5] = -float("inf")
    want = F.max_pool2d(x, 3, 2, 1)
    got = mx_driving.npu_max_pool2d(x, 3, 2, 1)
    assert torch.equal(torch.isnan(got), torch.isnan(want))
    assert torch.equal(got[~torch.isnan(got)], want[~torch.isnan(want)])
    for bad in [(2, 2, 1), (3, 1, 1), (3, 2, 0)]:
        with pytest.raises(RuntimeError):
            mx_driving.npu_max_pool2d(x, *bad)
    with pytest.raises(RuntimeError):
        mx_driving.npu_max_pool2d(x[0], 3, 2, 1)
