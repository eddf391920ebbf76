"""nfai_b200: the Llama-3 forward path of NFAI on B200 (sm_100a) behind a C ABI.

`nfai_b200.api` mirrors the reference's model interface (ModelOptions, LlamaModelFactory, LlamaModel) over
libnfai_cuda.so; `nfai_b200.synth` makes the seeded synthetic models; `nfai_b200.gguf_io` reads and writes GGUF;
`nfai_b200.tokenizer` mirrors the reference's Tokenizer over the native byte-pair encoder.
"""
from .api import (CudaContext, LlamaModel, LlamaModelFactory, ModelOptions, NfaiError,  # noqa: F401
                  create_synthetic_model, synthetic_tensors)
from .gguf_io import ComputeCollection, Parser  # noqa: F401
from .tokenizer import Tokenizer  # noqa: F401

__all__ = ["CudaContext", "LlamaModel", "LlamaModelFactory", "ModelOptions", "NfaiError", "ComputeCollection",
           "Parser", "Tokenizer", "create_synthetic_model", "synthetic_tensors"]
