"""tcgen05 GEMM vs a plain fp32 PyTorch matmul of the same bf16 operands."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 256), (300, 520, 192), (64, 264, 72),
                                   (1024, 2048, 5120), (4096, 1024, 1024)])
def test_gemm_bf16_matches_fp32_reference(M, N, K):
    from hipengine_b200.ops import gemm as G
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    x = (torch.randn(M, K, generator=g, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(N, K, generator=g, device="cuda") * 0.05).bfloat16()
    out = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
    G.gemm_bf16(x, w, out)
    torch.cuda.synchronize()
    G.check_status()
    ref = x.float() @ w.float().t()
    err = (out.float() - ref).abs().max().item()
    assert torch.isfinite(out.float()).all()
    assert err < 0.02 * ref.abs().max().item() + 1e-3, err
    out32 = torch.zeros(M, N, device="cuda")
    G.gemm_bf16(x, w, out32)
    assert torch.allclose(out32, ref, atol=1e-3 * max(1.0, ref.abs().max().item()), rtol=1e-3)
    G.gemm_bf16(x, w, out32, epi=2)
    torch.cuda.synchronize()
    G.check_status()
    assert torch.allclose(out32, 2 * ref, atol=2e-3 * max(1.0, ref.abs().max().item()), rtol=1e-3)


def test_gemm_strided_output_and_quant_weight():
    from hipengine_b200.ops import gemm as G
    from hipengine_b200.ops import kernels as K
    from hipengine_b200.quant import ggml as Q
    from hipengine_b200.models.executor import _Scratch
    M, N, Kd = 200, 512, 512
    x = (torch.randn(M, Kd, device="cuda") * 0.5).bfloat16()
    w = torch.randn(N, Kd, device="cuda") * 0.05
    raw = Q.quantize(w, Q.GGMLType.Q4_K)
    deq = Q.dequantize_torch(raw, Q.GGMLType.Q4_K, N, Kd)
    dw = K.to_device_weight(raw, Q.GGMLType.Q4_K, N, Kd)
    big = torch.zeros(M, 2 * N, device="cuda", dtype=torch.bfloat16)
    G.gemm_quant(x, dw, big[:, N:], _Scratch(torch.device("cuda")))
    torch.cuda.synchronize()
    G.check_status()
    ref = x.float() @ deq.bfloat16().float().t()
    assert (big[:, :N] == 0).all()
    assert torch.allclose(big[:, N:].float(), ref, atol=0.02 * ref.abs().max().item(), rtol=2e-2)


@pytest.mark.parametrize("M,N,K", [(16, 512, 2048), (100, 5120, 6144), (9, 768, 17408)])
def test_splitk_accumulates_into_fp32(M, N, K):
    from hipengine_b200.ops import gemm as G
    g = torch.Generator(device="cuda").manual_seed(M)
    x = (torch.randn(M, K, device="cuda", generator=g) * 0.5).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).bfloat16()
    acc = torch.randn(M, N, device="cuda", generator=g)
    want = acc + x.float() @ w.float().t()
    G.gemm_bf16_splitk_add(x, w, acc)
    G.check_status()
    torch.testing.assert_close(acc, want, atol=2e-2, rtol=2e-2)
    acc2 = torch.zeros(M, N, device="cuda")
    G.gemm_bf16_splitk_add(x, w, acc2, k_splits=3)
    G.check_status()
    torch.testing.assert_close(acc2, x.float() @ w.float().t(), atol=2e-2, rtol=2e-2)
    # deterministic variant: same numbers, bit-identical across runs, strided output rows
    from hipengine_b200.models.executor import _Scratch
    sc = _Scratch(torch.device("cuda"))
    wide = torch.zeros(M, 2 * N, device="cuda")
    a = G.gemm_bf16_splitk_det(x, w, wide[:, N:], sc).clone()
    b = G.gemm_bf16_splitk_det(x, w, wide[:, N:], sc).clone()
    G.check_status()
    assert torch.equal(a, b)
    torch.testing.assert_close(a, x.float() @ w.float().t(), atol=2e-2, rtol=2e-2)
    h = acc2.clone()
    G.gemm_bf16_splitk_det(x, w, h, sc, add=True)
    torch.testing.assert_close(h, 2 * (x.float() @ w.float().t()), atol=4e-2, rtol=2e-2)
