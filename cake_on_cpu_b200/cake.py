"""``cake_linear`` on CUDA tensors.

Mirrors the reference's PyTorch binding: the autograd function and module of
python/cake.py:18-49 and the three products of src/linear.cpp (forward
y = x W^T + b at :12-49; backward dX = dY W and dW = dY^T X at :52-102), each
product being one cake_sgemm call.  Tensors stay on the GPU: the library is
handed device pointers, transposed operands are read where they lie (the weight
of the forward product and dY of the weight gradient; the reference makes
contiguous transposed copies at src/linear.cpp:22 and :76-80) and the bias is
added in the product's epilogue instead of a second pass (:44-46).
"""
import os

import torch
from torch import nn
from torch.nn import Parameter

from . import api


def linear_cpp():
    """The compiled extension `linear_cpp` (csrc/linear.cpp, the counterpart of the reference's
    src/linear.cpp built by python/setup.py); None when it has not been built
    (`python -m cake_on_cpu_b200.build --linear`)."""
    if not os.path.exists(os.path.join(os.path.dirname(os.path.abspath(__file__)), "linear_cpp.so")):
        return None
    api.lib()
    from . import linear_cpp as ext
    return ext



def _rows(t):
    """A 2-D view whose rows are contiguous (copies only if they are not)."""
    return t if t.stride(-1) == 1 or t.shape[-1] == 1 else t.contiguous()


def linear_forward(input, weight, bias=None):
    """y = input @ weight.T (+ bias), as linear_forward in src/linear.cpp:12-49."""
    x = _rows(input.reshape(-1, input.shape[-1]))
    out = api.cake_sgemm_ex(x, _rows(weight), trans_b=True, bias=None if bias is None else bias.contiguous())
    return out.reshape(*input.shape[:-1], weight.shape[0])


def linear_backward(grad_output, input, weight, bias=None):
    """(grad_input, grad_weight, grad_bias), as linear_backward in src/linear.cpp:52-102."""
    dy = _rows(grad_output.reshape(-1, grad_output.shape[-1]))
    x = _rows(input.reshape(-1, input.shape[-1]))
    grad_input = api.cake_sgemm_ex(dy, _rows(weight)).reshape(input.shape)
    grad_weight = api.cake_sgemm_ex(dy, x, trans_a=True)
    grad_bias = dy.sum(0) if bias is not None else None
    return grad_input, grad_weight, grad_bias


class cake_linear_function(torch.autograd.Function):
    """The autograd function of python/cake.py:18-31.  With the compiled extension present the three
    products go through `linear_cpp.forward / backward` exactly as there; without it the ctypes
    routines above compute the same products through the same C-ABI entry point."""

    @staticmethod
    def forward(ctx, data, weight, bias=None):
        ext = linear_cpp()
        if ext is not None and data.dim() == 2:
            output = ext.forward(data, weight, bias)
        else:
            output = linear_forward(data, weight, bias)
        ctx.save_for_backward(data, weight, bias)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        data, weight, bias = ctx.saved_tensors
        ext = linear_cpp()
        if ext is not None and data.dim() == 2:
            gi, gw, gb = ext.backward(grad_output.contiguous(), data, weight, bias)
            return gi, gw, (gb if bias is not None else None)
        return linear_backward(grad_output, data, weight, bias)


class cake_linear(nn.Module):
    """Drop-in for the reference's ``cake_linear`` module (python/cake.py:33-49)."""

    def __init__(self, input_features, output_features, bias=True):
        super().__init__()
        self.input_features = input_features
        self.output_features = output_features
        self.weight = Parameter(torch.empty(output_features, input_features))
        if bias:
            self.bias = Parameter(torch.empty(output_features))
        else:
            self.register_parameter("bias", None)
        self.weight.data.uniform_(-0.1, 0.1)
        if bias:
            self.bias.data.uniform_(-0.1, 0.1)

    def forward(self, data):
        return cake_linear_function.apply(data, self.weight, self.bias)
