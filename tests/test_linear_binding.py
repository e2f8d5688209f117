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


def _ext(cake):
    from cake_on_cpu_b200 import build
    from cake_on_cpu_b200.cake import linear_cpp
    build.build_linear_ext()
    ext = linear_cpp()
    assert ext is not None
    return ext


def test_linear_cpp_extension_both_call_forms(cake):
    """The compiled extension (csrc/linear.cpp): forward / backward with and without the leading cache-size
    tensor of the reference's C++ signature (src/linear.cpp:12,52), on CUDA tensors (device pointers straight
    through) and on CPU tensors (host pointers through cake_sgemm, as the reference's extension does)."""
    import torch
    ext = _ext(cake)
    torch.manual_seed(1)
    cache_sz = torch.tensor([2097152, 110100480], dtype=torch.int32)
    for device in ("cuda", "cpu"):
        for (batch, fin, fout) in [(640, 384, 512), (33, 70, 9)]:
            x = torch.rand((batch, fin), device=device) * 2 - 1
            w = torch.rand((fout, fin), device=device) * 0.2 - 0.1
            b = torch.rand((fout,), device=device)
            dy = torch.rand((batch, fout), device=device) * 2 - 1
            want = torch.nn.functional.linear(x.double(), w.double(), b.double())
            for y in (ext.forward(x, w, b), ext.forward(cache_sz, x, w, b)):
                assert y.device.type == device
                assert (y.double() - want).abs().max().item() <= 1e-5 * fin ** 0.5
            y_nobias = ext.forward(x, w, None)
            assert (y_nobias.double() - (want - b.double())).abs().max().item() <= 1e-5 * fin ** 0.5
            y_nobias = ext.forward(cache_sz, x, w)  # three tensors, the first 1-D: cache sizes, no bias
            assert (y_nobias.double() - (want - b.double())).abs().max().item() <= 1e-5 * fin ** 0.5
            for gi, gw, gb in (ext.backward(dy, x, w, b), ext.backward(cache_sz, dy, x, w, b)):
                assert (gi.double() - dy.double() @ w.double()).abs().max().item() <= 1e-5 * fout ** 0.5
                assert (gw.double() - dy.double().t() @ x.double()).abs().max().item() <= 1e-5 * batch ** 0.5 * 4
                assert (gb.double() - dy.double().sum(0)).abs().max().item() <= 1e-4 * batch ** 0.5


def test_cake_linear_module_uses_the_extension(cake):
    """python/cake.py's module on top of the extension: same numbers as the ctypes routines."""
    import torch
    from cake_on_cpu_b200 import cake as binding
    _ext(cake)
    torch.manual_seed(2)
    layer = binding.cake_linear(300, 200).cuda()
    x = (torch.rand((128, 300), device="cuda") * 2 - 1).requires_grad_(True)
    y = layer(x)
    y.sum().backward()
    want = binding.linear_forward(x.detach(), layer.weight.detach(), layer.bias.detach())
    assert torch.equal(y.detach(), want)
    gi, gw, gb = binding.linear_backward(torch.ones_like(y), x.detach(), layer.weight.detach(), layer.bias.detach())
    assert torch.equal(x.grad, gi) and torch.equal(layer.weight.grad, gw) and torch.allclose(layer.bias.grad, gb)
