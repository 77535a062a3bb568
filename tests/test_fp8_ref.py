"""Block-scaled fp8 reference arithmetic (CPU): quantise/dequantise round trip and the linear path through it."""
import torch

from mcore_bridge_b200.ops import fp8
from mcore_bridge_b200.ops.linear import LinearSpec, linear
from mcore_bridge_b200.utils.dequantizer import Fp8Dequantizer


def test_quantisers_agree_with_checkpoint_dequantiser():
    torch.manual_seed(0)
    w = torch.randn(300, 256) * 0.1
    w8, s = fp8.quantize_128x128_ref(w)
    back = Fp8Dequantizer().convert(w8, s)
    assert back.shape == w.shape
    assert ((back.float() - w).abs() <= w.abs() * 0.07 + 2e-3).all()
    x = torch.randn(5, 384)
    x8, sx = fp8.quantize_1x128_ref(x)
    assert sx.shape == (3, 5)
    deq = x8.float().view(5, 3, 128) * sx.t()[..., None]
    assert ((deq.view(5, 384) - x).abs() <= x.abs() * 0.07 + 2e-2).all()


def test_fp8_linear_cpu_path_matches_dequantised_product():
    torch.manual_seed(1)
    x = torch.randn(64, 256, dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(128, 256) * 0.05).to(torch.bfloat16).requires_grad_()
    y = linear(x, w, None, LinearSpec(fp8=True))
    y.sum().backward()
    ref = x.detach().float() @ w.detach().float().t()
    assert ((y.float() - ref).norm() / ref.norm()).item() < 6e-2
    assert x.grad is not None and w.grad is not None
