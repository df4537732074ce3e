"""Functional ops: each dispatches CUDA tensors to the native sm_100a kernels and CPU tensors to
the PyTorch reference formula."""
from .gemm import gemm, linear, linear_nt, gelu_tanh_ref, dgelu_tanh_ref  # noqa: F401
from .nn import (LAYERNORM, RMSNORM, activation, cross_entropy, cross_entropy_ref, embedding, gelu, layer_norm, norm,  # noqa: F401
                 norm_ref, rms_norm)
from .attention import attention, attention_ref  # noqa: F401
