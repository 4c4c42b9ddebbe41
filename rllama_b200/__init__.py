"""rllama_b200: a B200 (sm_100a) backend for rllama's decode / prefill hot path.

``Transformer`` / ``TransformerCaches`` / ``DataSettings`` / ``TokenSampler`` mirror the
reference's types; ``Cuda`` / ``CudaTensor`` mirror its OpenCL tensor backend. All arithmetic
runs in hand-written CUDA kernels behind the C ABI of ``include/rllama_b200.h``.
"""
from ._ffi import F16, F32, RllamaError  # noqa: F401
from .data_source import DataSource, ModelParams  # noqa: F401
from .tensor import Cuda, CudaTensor  # noqa: F401
from .token_sampler import NativeTokenSampler, TokenSampler  # noqa: F401
from .tokenizer import Tokenizer  # noqa: F401
from .transformer import DataSettings, Transformer, TransformerCaches  # noqa: F401
