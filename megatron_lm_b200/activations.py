"""Activation functions selectable by name or passed as callables in ``TransformerConfig.activation_func``
(reference: megatron/core/activations.py:8 squared_relu, :14 quick_gelu, :20 fast_gelu).  GELU, SwiGLU and the
bias-fused variants run as CUDA kernels through ``ops``; the ones here are elementwise expressions."""
import torch
import torch.nn.functional as F


def squared_relu(x: torch.Tensor) -> torch.Tensor:
    return F.relu(x).square()


def quick_gelu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(1.702 * x)


def fast_gelu(x: torch.Tensor) -> torch.Tensor:
    # tanh form; 0.7978845608 = sqrt(2 / pi)
    return 0.5 * x * (1.0 + torch.tanh(0.7978845608 * x * (1.0 + 0.044715 * x * x)))


def openai_gelu(x: torch.Tensor) -> torch.Tensor:
    """The tanh approximation of GELU (``--openai-gelu``; reference: megatron/legacy/model/utils.py:52)."""
    return F.gelu(x, approximate="tanh")


BY_NAME = {"openai_gelu": openai_gelu, "squared_relu": squared_relu, "quick_gelu": quick_gelu, "fast_gelu": fast_gelu, "relu": torch.relu,
           "silu": F.silu, "gelu": F.gelu}
