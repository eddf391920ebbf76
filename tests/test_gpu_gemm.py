"""The tensor-core GEMM of the batched prompt path against a float64 product of the same float16 operands."""
import numpy as np
import pytest

from .gpu_util import call, dev, host, ptr, rel_err

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 32, 128), (1, 32, 64), (17, 96, 256), (128, 3072, 2048),
                                   (200, 2048, 2048), (512, 16384, 2048), (300, 2048, 8192), (64, 520, 72),
                                   (1024, 4096, 4096), (33, 77, 512), (8, 2048, 8192),
                                   (1000, 3000, 2048), (2048, 8192, 3072), (1024, 16384, 256), (1024, 16384, 128), (2048, 2048, 512)])
def test_gemm_f16(cuda_ctx, M, N, K):
    rng = np.random.default_rng(M * 131 + N * 7 + K)
    A = (rng.standard_normal((M, K)) * 0.5).astype(np.float16)
    W = (rng.standard_normal((N, K)) * 0.05).astype(np.float16)
    dA, dW = dev(A), dev(W)
    C = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    call(cuda_ctx, "nfai_op_gemm_f16", ptr(dA), ptr(dW), M, N, K, ptr(C))
    want = A.astype(np.float64) @ W.astype(np.float64).T
    got = host(C)
    assert np.isfinite(got).all()
    assert rel_err(got, want) < 1e-4


def test_split_k_equals_single_pass(cuda_ctx, monkeypatch):
    """A short chunk splits K over the SMs and adds the partial tiles in a second kernel: same product."""
    M, N, K = 128, 3072, 2048
    rng = np.random.default_rng(9)
    A = (rng.standard_normal((M, K)) * 0.5).astype(np.float16)
    W = (rng.standard_normal((N, K)) * 0.05).astype(np.float16)
    dA, dW = dev(A), dev(W)
    out = {}
    for split in ("1", "0"):
        monkeypatch.setenv("NFAI_GEMM_SPLIT", split)
        C = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
        call(cuda_ctx, "nfai_op_gemm_f16", ptr(dA), ptr(dW), M, N, K, ptr(C))
        out[split] = host(C)
    assert rel_err(out["1"], out["0"]) < 1e-5
