"""Back-to-back product `(f(A @ B)) @ C` against two fp32 matrix products with `f` between them: the
shapes of the reference's own test of its fused template (monkeypatch/template/fused_bmm.py:437-449,
inputs make_tensor's U[-9, 9)) and N(0,1) cases with every pointwise function."""
import pytest
import torch

import flashlight_b200
from flashlight_b200.monkeypatch.template.fused_bmm import fused_bmm
from oracle import attention_oracle as ao

pytestmark = pytest.mark.gpu


def close(out, ref):
    """rtol 1.6e-2 as torch.testing.assert_close takes for bf16, on top of 1 % of the result's RMS (a
    sum of hundreds of products has no meaningful absolute scale of its own)."""
    flashlight_b200.check_status()
    o, r = out.float(), ref.float()
    assert o.shape == r.shape and out.dtype == torch.bfloat16
    band = 1.6e-2 * r.abs() + 1e-2 * r.pow(2).mean().sqrt()
    assert bool(((o - r).abs() <= band).all()), ((o - r).abs() / band).max().item()


def uniform(shape, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.rand(*shape, generator=g, device="cuda") * 18 - 9).to(torch.bfloat16)


def normal(shape, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(*shape, generator=g, device="cuda").to(torch.bfloat16)


@pytest.mark.parametrize("batch,n_ctx,head_dim", [(2, 1024, 128), (1, 2048, 64), (4, 512, 256), (2, 64, 32)])
def test_reference_test_shapes(batch, n_ctx, head_dim):
    q, k, v = uniform((batch, n_ctx, head_dim), 1), uniform((batch, head_dim, n_ctx), 2), uniform((batch, n_ctx, head_dim), 3)
    close(fused_bmm(q, k, v), ao.product_chain(q, k, v))


def test_widths_above_256_have_no_kernel():
    q, k, v = uniform((1, 256, 264), 1), uniform((1, 264, 256), 2), uniform((1, 256, 264), 3)
    with pytest.raises(NotImplementedError):
        fused_bmm(q, k, v)


@pytest.mark.parametrize("pointwise", ["identity", "relu", "tanh", "sigmoid"])
@pytest.mark.parametrize("M,N,O,P", [(300, 128, 520, 128), (128, 64, 128, 64), (1000, 32, 77, 32), (257, 96, 640, 48),
                                     (300, 200, 333, 256)])
def test_pointwise_middles_and_odd_shapes(pointwise, M, N, O, P):
    a, b, c = normal((3, M, N), 4), normal((3, N, O), 5), normal((3, O, P), 6)
    scale = N ** -0.5
    close(fused_bmm(a, b, c, pointwise=pointwise, scale=scale), ao.product_chain(a, b, c, pointwise, scale))


def test_b_as_a_transposed_view_and_leading_dims():
    a, bt, c = normal((2, 3, 200, 64), 7), normal((2, 3, 333, 64), 8), normal((2, 3, 333, 64), 9)
    b = bt.transpose(-1, -2)                                  # [.., 64, 333] with the feature axis contiguous
    out = fused_bmm(a, b, c, pointwise="relu", scale=0.125)
    assert out.shape == (2, 3, 200, 64)
    close(out, ao.product_chain(a, b, c, "relu", 0.125))


def test_torch_compile_wraps_the_op():
    a, b, c = normal((2, 256, 64), 10), normal((2, 64, 256), 11), normal((2, 256, 64), 12)
    fn = torch.compile(fused_bmm, dynamic=False)
    close(fn(a, b, c), ao.product_chain(a, b, c))
