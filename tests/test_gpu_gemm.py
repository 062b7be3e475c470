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


def _quant_case(t, N, Kd, seed=0, std=0.05):
    from hipengine_b200.ops import kernels as K
    from hipengine_b200.quant import ggml as Q
    g = torch.Generator(device="cuda").manual_seed(seed)
    w = torch.randn(N, Kd, device="cuda", generator=g) * std
    raw = Q.quantize(w, t)
    deq = Q.dequantize_torch(raw, t, N, Kd)
    return K.to_device_weight(raw, t, N, Kd), deq


@pytest.mark.parametrize("qt", ["Q4_K", "Q6_K", "Q8_0"])
@pytest.mark.parametrize("M,N,K", [(128, 256, 256), (200, 520, 768), (1024, 1536, 5120), (4096, 512, 2304)])
def test_gemm_quant_in_pipeline_matches_fp32_dequant_matmul(qt, M, N, K):
    """The tensor-core GEMM that reads raw quantised blocks against fp32 matmul with the exactly dequantised weight:
    the only differences allowed are the bf16 roundings of the expanded weight (scale, offset, product)."""
    from hipengine_b200.models.executor import _Scratch
    from hipengine_b200.ops import gemm as G
    from hipengine_b200.quant import ggml as Q
    t = getattr(Q.GGMLType, qt)
    dw, deq = _quant_case(t, N, K, seed=M + N)
    g = torch.Generator(device="cuda").manual_seed(7)
    x = (torch.randn(M, K, generator=g, device="cuda") * 0.5).bfloat16()
    sc = _Scratch(torch.device("cuda"))
    out = torch.full((M, N), float("nan"), device="cuda")
    G.gemm_quant(x, dw, out, sc)
    torch.cuda.synchronize()
    G.check_status()
    ref = x.float() @ deq.t()
    assert torch.isfinite(out).all()
    rel = (out - ref).norm() / ref.norm()
    assert rel < 6e-3, rel                       # bf16 weight rounding alone gives ~2e-3
    assert (out - ref).abs().max() < 0.03 * ref.abs().max()
    # bf16 output, a row slice of the weight, and accumulation into fp32
    out_b = torch.zeros(M, 2 * N, device="cuda", dtype=torch.bfloat16)
    G.gemm_quant(x, dw, out_b[:, N:], sc)
    assert (out_b[:, :N] == 0).all()
    assert (out_b[:, N:].float() - ref).abs().max() < 0.03 * ref.abs().max()
    if N >= 512:
        part = torch.zeros(M, 256, device="cuda")
        G.gemm_quant(x, dw, part, sc, row0=256, rows=256)
        assert (part - ref[:, 256:512]).norm() / ref[:, 256:512].norm() < 6e-3
    acc = ref.clone()
    G.gemm_quant(x, dw, acc, sc, epi=2)
    torch.cuda.synchronize()
    G.check_status()
    assert (acc - 2 * ref).norm() / (2 * ref).norm() < 6e-3


@pytest.mark.parametrize("qt", ["Q4_K", "Q6_K", "Q8_0"])
@pytest.mark.parametrize("M,N,K", [(16, 512, 2048), (100, 5120, 6144), (9, 768, 17408), (128, 1024, 1280)])
def test_gemm_quant_splitk_is_deterministic_and_accurate(qt, M, N, K):
    from hipengine_b200.models.executor import _Scratch
    from hipengine_b200.ops import gemm as G
    from hipengine_b200.quant import ggml as Q
    t = getattr(Q.GGMLType, qt)
    dw, deq = _quant_case(t, N, K, seed=M)
    x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    ref = x.float() @ deq.t()
    sc = _Scratch(torch.device("cuda"))
    wide = torch.zeros(M, 2 * N, device="cuda")
    a = G.gemm_quant_splitk(x, dw, wide[:, N:], sc).clone()
    b = G.gemm_quant_splitk(x, dw, wide[:, N:], sc).clone()
    torch.cuda.synchronize()
    G.check_status()
    assert torch.equal(a, b)
    assert (a - ref).norm() / ref.norm() < 6e-3
    h = ref.clone()
    G.gemm_quant_splitk(x, dw, h, sc, add=True)
    G.check_status()
    assert (h - 2 * ref).norm() / (2 * ref).norm() < 6e-3


@pytest.mark.parametrize("qt", ["Q4_K", "Q8_0"])
def test_gemm_quant_grouped_experts_and_padded_k(qt):
    """Grouped form (MoE experts, tiles carrying their expert id, -1 tiles skipped) and activations narrower than the
    weight's zero-padded K."""
    from hipengine_b200.models.executor import _Scratch
    from hipengine_b200.ops import gemm as G
    from hipengine_b200.quant import ggml as Q
    t = getattr(Q.GGMLType, qt)
    E, Nn, Kd = 5, 320, 768
    dw, deq = _quant_case(t, E * Nn, Kd, seed=3)
    tiles = torch.tensor([2, -1, 0, 4, 4, 1], device="cuda", dtype=torch.int32)
    M = tiles.numel() * 128
    a = (torch.randn(M, Kd, device="cuda") * 0.5).bfloat16()
    out = torch.zeros(M, Nn, device="cuda")
    G.gemm_quant_grouped(a, dw, out, E, tiles)
    torch.cuda.synchronize()
    G.check_status()
    for tm, e in enumerate(tiles.tolist()):
        rows = slice(tm * 128, tm * 128 + 128)
        if e < 0:
            assert (out[rows] == 0).all()
            continue
        ref = a[rows].float() @ deq[e * Nn:(e + 1) * Nn].t()
        assert (out[rows] - ref).norm() / ref.norm() < 6e-3
    # K padded: the weight has 768 columns of which the last 64 are zero blocks; activations carry 704 columns
    if qt == "Q8_0":
        w = torch.randn(256, 768, device="cuda") * 0.05
        w[:, 704:] = 0
        raw = Q.quantize(w, t)
        deq2 = Q.dequantize_torch(raw, t, 256, 768)
        from hipengine_b200.ops import kernels as K
        dw2 = K.to_device_weight(raw, t, 256, 768)
        x = (torch.randn(300, 704, device="cuda") * 0.5).bfloat16()
        o = torch.zeros(300, 256, device="cuda")
        G.gemm_quant(x, dw2, o, _Scratch(torch.device("cuda")))
        G.check_status()
        ref = x.float() @ deq2[:, :704].t()
        assert (o - ref).norm() / ref.norm() < 6e-3


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
