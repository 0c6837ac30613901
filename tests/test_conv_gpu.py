"""GPU parity of the Conv2d entry points (patch extraction + tensor-core products) against the
oracle: the reference's own known answers (test/convnodes.cu.cpp:38-109), then seeded shapes with
several channels, filters, strides and batches in fp32 and Half, values and both gradients, with
the gradients accumulated onto non-zero tensors as Conv2dNode::backward_ does (`+=`)."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from ginn_b200 import binding as B
from helpers import check, randn

pytestmark = pytest.mark.gpu


def test_known_answers(gpu, kat):
    for case in kat["conv2d"]["cases"]:
        x = np.asarray(case["x"], np.float32)[None, :, :, None]
        f = np.asarray(case["f"], np.float32)[None, None]
        want = np.asarray(case["y"], np.float32)
        y = B.colmajor_nd((1,) + want.shape + (1,), torch.float32, fill=0.0)
        gpu.conv2d_forward(B.from_host_nd(x), B.from_host_nd(f), y, *case["strides"])
        torch.cuda.synchronize()
        np.testing.assert_allclose(B.to_host(y)[0, :, :, 0], want, rtol=1e-6)


@pytest.mark.parametrize("dt", [np.float32, np.float16])
@pytest.mark.parametrize("shape", [
    (1, 28, 28, 16, 8, 5, 5, 1, 1),      # the first layer of examples/mnist-conv.cu.cpp, scaled down
    (8, 14, 14, 4, 16, 3, 3, 1, 1),
    (3, 9, 11, 2, 5, 3, 2, 2, 1),
    (4, 8, 7, 3, 6, 2, 3, 2, 3),
    (16, 6, 6, 2, 32, 1, 1, 1, 1),       # 1 x 1 filters: a plain product
])
def test_forward_and_gradients(gpu, dt, shape):
    C, R, W, Bn, F, KR, KC, sr, sc = shape
    rng = np.random.default_rng(31)
    x, k = randn(rng, (C, R, W, Bn), dt), randn(rng, (F, C, KR, KC), dt, 0.2)
    ref_y = orc.conv2d_forward(x, k, sr, sc)
    dy = randn(rng, ref_y.shape, dt)
    tdt = torch.float32 if dt == np.float32 else torch.float16
    xd, kd, dyd = B.from_host_nd(x), B.from_host_nd(k), B.from_host_nd(dy)
    y = B.colmajor_nd(ref_y.shape, tdt, fill=0.0)
    ws = torch.empty(gpu.conv2d_workspace_bytes(xd, kd, sr, sc), dtype=torch.uint8, device="cuda")
    for workspace in (ws, None):          # caller's workspace, then the library's own
        y.zero_()
        gpu.conv2d_forward(xd, kd, y, sr, sc, workspace)
        dx, dk = B.colmajor_nd(x.shape, tdt, fill=0.5), B.colmajor_nd(k.shape, tdt, fill=0.25)
        gpu.conv2d_backward(xd, kd, dyd, dx, dk, sr, sc, workspace)
        torch.cuda.synchronize()
        check(B.to_host(y), ref_y, dt, "value")
        rdx, rdk = orc.conv2d_backward(x, k, dy, sr, sc)
        check(B.to_host(dx), 0.5 + rdx.astype(np.float64), dt, "dx +=")
        check(B.to_host(dk), 0.25 + rdk.astype(np.float64), dt, "dk +=")
    only_dk = B.colmajor_nd(k.shape, tdt, fill=0.0)
    gpu.conv2d_backward(xd, kd, dyd, None, only_dk, sr, sc)     # input without a gradient
    torch.cuda.synchronize()
    check(B.to_host(only_dk), orc.conv2d_backward(x, k, dy, sr, sc)[1], dt, "dk alone")


def test_argument_errors(gpu):
    x = B.colmajor_nd((2, 4, 4, 1), torch.float32, fill=0.0)
    k = B.colmajor_nd((3, 2, 3, 3), torch.float32, fill=0.0)
    y = B.colmajor_nd((3, 4, 4, 1), torch.float32, fill=0.0)
    with pytest.raises(gpu.GinnB200Error):
        gpu.conv2d_forward(x, k, y, 0, 1)                       # zero stride
    lib = gpu.lib()
    assert lib.ginn_b200_conv2d_workspace(0, 2, 4, 4, 1, 3, 3, 3, 1, 1) == 2 * 9 * 16 * 4 + (256 - (2 * 9 * 16 * 4) % 256) % 256
    assert lib.ginn_b200_conv2d_workspace(0, 0, 4, 4, 1, 3, 3, 3, 1, 1) == 0
