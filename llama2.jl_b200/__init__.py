"""llama2.jl_b200: the per-token decode path of cafaxo/Llama2.jl as a B200 (sm_100a) CUDA library behind a C ABI,
with a host-side mirror of the reference's interface (src/Llama2.jl:12-14)."""
from ._lib import L2BError, lib  # noqa: F401
from .load_gguf import load_gguf_model  # noqa: F401
from .load_karpathy import load_karpathy_model  # noqa: F401
from .model import (BatchRunState, LanguageModel, ModelConfig, QuantMatrix, RunState, TransformerLayerWeights, TransformerWeights,  # noqa: F401
                    dequantize, generate, matmul_, prefill, sample, transformer_)
from .tokenizer import BPETokenizer, CharTokenizer, encode  # noqa: F401

__all__ = ["ModelConfig", "CharTokenizer", "LanguageModel", "load_gguf_model", "load_karpathy_model", "encode", "sample"]
