"""cake_linear (the reference's PyTorch binding, python/cake.py + src/linear.cpp) on CUDA tensors:
forward and backward against torch's own float64 linear layer."""
import pytest

pytestmark = pytest.mark.gpu


def test_cake_linear_forward_backward(cake):
    import torch
    from cake_on_cpu_b200.cake import cake_linear
    torch.manual_seed(0)
    for (batch, fin, fout, bias) in [(64, 300, 200, True), (1000, 512, 1024, True), (7, 33, 5, False)]:
        layer = cake_linear(fin, fout, bias=bias).cuda()
        x = (torch.rand((batch, fin), device="cuda") * 2 - 1).requires_grad_(True)
        y = layer(x)
        loss_w = torch.rand_like(y)
        (y * loss_w).sum().backward()
        x64 = x.detach().double().requires_grad_(True)
        w64 = layer.weight.detach().double().requires_grad_(True)
        b64 = layer.bias.detach().double().requires_grad_(True) if bias else None
        y64 = torch.nn.functional.linear(x64, w64, b64)
        (y64 * loss_w.double()).sum().backward()
        scale = fin ** 0.5
        assert (y.double() - y64).abs().max().item() <= 1e-5 * scale
        assert (x.grad.double() - x64.grad).abs().max().item() <= 1e-5 * fout ** 0.5
        assert (layer.weight.grad.double() - w64.grad).abs().max().item() <= 1e-5 * batch ** 0.5 * 4
        if bias:
            assert (layer.bias.grad.double() - b64.grad).abs().max().item() <= 1e-4
