"""Each sm_100a kernel against a plain PyTorch fp32 reference of the same op (small and odd shapes)."""
import math

import pytest
import torch

from hipengine_b200.quant import ggml as Q
from hipengine_b200.ref import ops as R

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from hipengine_b200.ops import kernels
    return kernels


def _qweight(K, t, n, k, seed=0, std=0.02):
    g = torch.Generator(device="cuda").manual_seed(seed)
    w = torch.randn(n, k, generator=g, device="cuda") * std
    raw = Q.quantize(w, t)
    deq = Q.dequantize_torch(raw, t, n, k)
    return K.to_device_weight(raw, t, n, k), deq, raw


@pytest.mark.parametrize("t", [Q.GGMLType.Q4_K, Q.GGMLType.Q6_K, Q.GGMLType.Q8_0, Q.GGMLType.F32, Q.GGMLType.BF16])
@pytest.mark.parametrize("rows", [1, 3, 8])
def test_gemv_matches_dequant_matmul(K, t, rows):
    n, k = 515, 768
    dw, deq, _ = _qweight(K, t, n, k)
    x = torch.randn(rows, k, device="cuda")
    out = torch.zeros(rows, n, device="cuda")
    K.gemv(x, [K.GemvSegment(dw, out)])
    ref = x @ deq.t()
    # int8 activation quantisation bounds the error at ~1% of |x||w| per 32-block
    err = (out - ref).abs().max() / ref.abs().max()
    assert err < 2e-2, err
    xq, dx = R.q8_1_quantize(x)
    xr = (xq.float().reshape(rows, k // 32, 32) * dx[..., None]).reshape(rows, k)
    ref_q = xr @ deq.t()
    if t in (Q.GGMLType.Q4_K, Q.GGMLType.Q6_K, Q.GGMLType.Q8_0):
        assert torch.allclose(out, ref_q, atol=2e-4 * ref.abs().max().item() + 1e-5, rtol=2e-3)


@pytest.mark.parametrize("t", [Q.GGMLType.Q4_K, Q.GGMLType.Q6_K, Q.GGMLType.Q8_0])
@pytest.mark.parametrize("n,k", [(9600, 5120), (4736, 5120), (1027, 1280)], ids=["rg8", "rg4", "rg2"])
def test_gemv_multi_row_pair_lanes_at_every_rows_per_item(K, t, n, k):
    """Batches of 2+ rows run with two weight rows per lane; the three shapes make the launcher pick 8, 4 and 2 weight
    rows per work item (the lane map differs for each).  Checked against the same int8-activation reference as the
    single-row kernel, with the fused norm, an odd row count at the end and the accumulate epilogue."""
    rows = 4
    dw, deq, _ = _qweight(K, t, n, k, seed=7)
    x = torch.randn(rows, k, device="cuda")
    nw = torch.rand(k, device="cuda") + 0.5
    out = torch.zeros(rows, n, device="cuda")
    K.gemv(x, [K.GemvSegment(dw, out)], norm_w=nw)
    xn = R.rmsnorm(x, nw)
    xq, dx = R.q8_1_quantize(xn)
    xr = (xq.float().reshape(rows, k // 32, 32) * dx[..., None]).reshape(rows, k)
    ref_q = xr @ deq.t()
    tol = 5e-4 * ref_q.abs().max().item() + 1e-5      # an activation on a rounding boundary may quantise either way
    assert torch.allclose(out, ref_q, atol=tol, rtol=2e-3), (out - ref_q).abs().max()
    one = torch.zeros(1, n, device="cuda")
    K.gemv(x[2:3], [K.GemvSegment(dw, one)], norm_w=nw)                      # the single-row kernel on row 2
    assert torch.allclose(out[2:3], one, atol=tol, rtol=2e-3)
    acc = torch.ones(rows, n, device="cuda")
    K.gemv(x, [K.GemvSegment(dw, acc, K.EPI_ADD_F32)], norm_w=nw)
    assert torch.allclose(acc, ref_q + 1.0, atol=tol, rtol=2e-3)


@pytest.mark.parametrize("rows", [2, 5])
def test_gemv_multi_row_gate_up_pair_and_mixed_segments(K, rows):
    """Gate/up pair segment of one block type (both rows of a pair sit in one lane) beside a plain segment of another
    type and a float segment in the same launch."""
    k, f, n1, n2 = 1024, 1030, 520, 24
    wg, dg, _ = _qweight(K, Q.GGMLType.Q4_K, f, k, 3, std=0.2)
    wu, du, _ = _qweight(K, Q.GGMLType.Q4_K, f, k, 4, std=0.2)
    w1, d1, _ = _qweight(K, Q.GGMLType.Q6_K, n1, k, 5)
    w2, d2, _ = _qweight(K, Q.GGMLType.F32, n2, k, 6)
    h = torch.randn(rows, k, device="cuda") * 2
    nw = torch.rand(k, device="cuda") + 0.5
    act = torch.zeros(rows, f, device="cuda", dtype=torch.bfloat16)
    o1 = torch.zeros(rows, n1, device="cuda")
    o2 = torch.zeros(rows, n2, device="cuda")
    K.gemv(h, [K.GemvSegment(wg, act, K.EPI_SILU_MUL, wu), K.GemvSegment(w1, o1), K.GemvSegment(w2, o2)], norm_w=nw)
    xn = R.rmsnorm(h, nw)
    xq, dx = R.q8_1_quantize(xn)
    xr = (xq.float().reshape(rows, k // 32, 32) * dx[..., None]).reshape(rows, k)
    ref = R.swiglu(xr @ dg.t(), xr @ du.t())
    assert (act.float() - ref).abs().max() < 0.01 * ref.abs().max() + 0.02
    r1 = xr @ d1.t()
    assert torch.allclose(o1, r1, atol=2e-4 * r1.abs().max().item() + 1e-5, rtol=2e-3)
    assert torch.allclose(o2, xn @ d2.t(), atol=1e-3, rtol=1e-3)


def test_gemv_norm_prologue_multi_segment_and_epilogues(K):
    k, n1, n2, f = 512, 256, 40, 384
    w1, d1, _ = _qweight(K, Q.GGMLType.Q4_K, n1, k, 1)
    w2, d2, _ = _qweight(K, Q.GGMLType.F32, n2, k, 2)
    wg, dg, _ = _qweight(K, Q.GGMLType.Q4_K, f, k, 3, std=0.2)
    wu, du, _ = _qweight(K, Q.GGMLType.Q6_K, f, k, 4, std=0.2)
    h = torch.randn(2, k, device="cuda") * 3
    nw = torch.rand(k, device="cuda") + 0.5
    o1 = torch.zeros(2, n1, device="cuda")
    o2 = torch.zeros(2, n2, device="cuda")
    K.gemv(h, [K.GemvSegment(w1, o1), K.GemvSegment(w2, o2)], norm_w=nw, eps=1e-6)
    xn = R.rmsnorm(h, nw)
    assert torch.allclose(o1, xn @ d1.t(), atol=3e-2 * (xn @ d1.t()).abs().max().item())
    assert torch.allclose(o2, xn @ d2.t(), atol=1e-3, rtol=1e-3)
    act = torch.zeros(2, f, device="cuda", dtype=torch.bfloat16)
    K.gemv(h, [K.GemvSegment(wg, act, K.EPI_SILU_MUL, wu)], norm_w=nw)
    ref = R.swiglu(xn @ dg.t(), xn @ du.t())
    assert (act.float() - ref).abs().max() < 0.03 * ref.abs().max() + 0.02
    res = torch.randn(2, n1, device="cuda")
    res0 = res.clone()
    K.gemv(h.bfloat16(), [K.GemvSegment(w1, res, K.EPI_ADD_F32)])
    ref = res0 + h.bfloat16().float() @ d1.t()
    assert torch.allclose(res, ref, atol=3e-2 * ref.abs().max().item())


@pytest.mark.parametrize("t", [Q.GGMLType.Q6_K, Q.GGMLType.Q8_0])
def test_repack_round_trip_is_lossless(K, t):
    dw, _, raw = _qweight(K, t, 37, 512)
    assert torch.equal(K.unpack_device_weight(dw).reshape(-1), raw.reshape(-1))


@pytest.mark.parametrize("t", [Q.GGMLType.Q4_K, Q.GGMLType.Q6_K, Q.GGMLType.Q8_0, Q.GGMLType.F32])
def test_dequant_bf16_is_exact_rounding(K, t):
    dw, deq, _ = _qweight(K, t, 33, 512)
    out = K.dequant_bf16(dw, row0=5, rows=20)
    assert torch.equal(out, deq[5:25].to(torch.bfloat16))


def test_embed_rows(K):
    dw, deq, _ = _qweight(K, Q.GGMLType.Q4_K, 100, 256)
    ids = torch.tensor([3, 99, 0, 3], device="cuda")
    out = torch.empty(4, 256, device="cuda")
    K.embed(dw, ids, out, 2.0)
    assert torch.equal(out, deq[ids] * 2.0)


def test_rmsnorm_and_act_mul(K):
    x = torch.randn(5, 1024, device="cuda") * 2
    w = torch.rand(1024, device="cuda")
    out = torch.empty(5, 1024, device="cuda", dtype=torch.bfloat16)
    K.rmsnorm_rows(x, w, out)
    assert torch.allclose(out.float(), R.rmsnorm(x, w), atol=2e-2, rtol=1e-2)
    gu = torch.randn(5, 2 * 264, device="cuda").bfloat16()
    o = torch.empty(5, 264, device="cuda", dtype=torch.bfloat16)
    K.act_mul(gu, o, "silu")
    ref = R.swiglu(gu[:, :264].float(), gu[:, 264:].float())
    assert torch.allclose(o.float(), ref, atol=2e-2, rtol=2e-2)


def _paged_setup(T, Hkv, D, n_slots=2, max_ctx=256):
    mp = (max_ctx + 15) // 16
    n_pages = n_slots * mp + 1
    cache = torch.zeros(n_pages, 2, Hkv, 16, D, device="cuda", dtype=torch.bfloat16)
    perm = torch.randperm(n_pages - 1, device="cuda").int() + 1
    bt = perm.reshape(n_slots, mp).contiguous()
    return cache, bt


@pytest.mark.parametrize("D,H,Hkv", [(256, 6, 1), (256, 4, 2), (128, 8, 1), (64, 4, 4)])
def test_qkv_post_and_paged_decode_attention(K, D, H, Hkv):
    T = 37
    cache, bt = _paged_setup(T, Hkv, D)
    g = torch.Generator(device="cuda").manual_seed(0)
    qf = torch.randn(T, H * 2 * D, generator=g, device="cuda")
    kf = torch.randn(T, Hkv * D, generator=g, device="cuda")
    vf = torch.randn(T, Hkv * D, generator=g, device="cuda")
    qn = torch.rand(D, device="cuda") + 0.5
    kn = torch.rand(D, device="cuda") + 0.5
    slot = torch.full((T,), 1, device="cuda", dtype=torch.int32)
    pos = torch.arange(T, device="cuda", dtype=torch.int32)
    q_out = torch.empty(T, H, D, device="cuda", dtype=torch.bfloat16)
    gate = torch.empty(T, H, D, device="cuda", dtype=torch.bfloat16)
    rope_dim, theta = 64, 1e7
    K.qkv_post(qf, kf, vf, qn, kn, q_out, gate, cache, bt, slot, pos, H, Hkv, D, 16, True, rope_dim, theta, 1e-6)
    qg = qf.reshape(T, H, 2, D)
    q_ref = R.rope_neox(R.rmsnorm(qg[:, :, 0], qn), pos, theta, rope_dim)
    k_ref = R.rope_neox(R.rmsnorm(kf.reshape(T, Hkv, D), kn), pos, theta, rope_dim)
    assert torch.allclose(q_out.float(), q_ref, atol=3e-2, rtol=2e-2)
    assert torch.allclose(gate.float(), qg[:, :, 1], atol=2e-2, rtol=1e-2)
    # gather the cache back through the block table
    pages = bt[1, (pos // 16).long()].long()
    k_back = cache[pages, 0, :, (pos % 16).long()]
    v_back = cache[pages, 1, :, (pos % 16).long()]
    assert torch.allclose(k_back.float(), k_ref, atol=3e-2, rtol=2e-2)
    assert torch.allclose(v_back.float(), vf.reshape(T, Hkv, D), atol=2e-2, rtol=1e-2)
    # attention for every row with its causal context (decode kernel used row-wise)
    out = torch.empty(T, H * D, device="cuda", dtype=torch.bfloat16)
    split_len, max_splits = 16, 3
    part = torch.empty(K.attn_decode_scratch_floats(T, H, max_splits, D), device="cuda")
    scale = D ** -0.5
    K.attn_decode(q_out, gate, cache, bt, slot, pos + 1, part, out, H, Hkv, D, 16, split_len, max_splits, scale)
    o_ref = R.causal_gqa_attention(q_out.float(), k_back.float(), v_back.float(), pos, scale)
    o_ref = R.bf16_round(o_ref) * torch.sigmoid(gate.float())
    assert torch.allclose(out.float().reshape(T, H, D), o_ref, atol=2e-2, rtol=2e-2)


def test_sliding_window_decode_attention(K):
    T, H, Hkv, D, win = 50, 2, 1, 64, 16
    cache, bt = _paged_setup(T, Hkv, D)
    q = torch.randn(T, H, D, device="cuda").bfloat16()
    kf = torch.randn(T, Hkv * D, device="cuda")
    vf = torch.randn(T, Hkv * D, device="cuda")
    slot = torch.zeros(T, device="cuda", dtype=torch.int32)
    pos = torch.arange(T, device="cuda", dtype=torch.int32)
    dummy_q = torch.empty(T, H, D, device="cuda", dtype=torch.bfloat16)
    K.qkv_post(torch.zeros(T, H * D, device="cuda"), kf, vf, None, None, dummy_q, None, cache, bt, slot, pos, H, Hkv,
               D, 16, False, 0, 1e6, 1e-6)
    out = torch.empty(T, H * D, device="cuda", dtype=torch.bfloat16)
    part = torch.empty(K.attn_decode_scratch_floats(T, H, 2, D), device="cuda")
    K.attn_decode(q, None, cache, bt, slot, pos + 1, part, out, H, Hkv, D, 16, 8, 2, 1.0, window=win)
    kb = kf.reshape(T, Hkv, D).bfloat16().float()
    vb = vf.reshape(T, Hkv, D).bfloat16().float()
    ref = R.causal_gqa_attention(q.float(), kb, vb, pos, 1.0, window=win)
    assert torch.allclose(out.float().reshape(T, H, D), ref, atol=2e-2, rtol=2e-2)


def test_conv1d_segments_and_state(K):
    C, KW = 96, 4
    segs = [(0, 5), (2, 1), (1, 2)]  # (slot, length)
    T = sum(n for _, n in segs)
    x = torch.randn(T, C, device="cuda")
    w = torch.randn(C, KW, device="cuda") * 0.5
    state = torch.randn(3, C, KW - 1, device="cuda")
    state0 = state.clone()
    seg_start = torch.tensor([0, 5, 6, 8], device="cuda", dtype=torch.int32)
    seg_slot = torch.tensor([s for s, _ in segs], device="cuda", dtype=torch.int32)
    tok_seg = torch.tensor([0] * 5 + [1] + [2] * 2, device="cuda", dtype=torch.int32)
    out = torch.empty(T, C, device="cuda")
    K.conv1d(x, w, state, seg_start, seg_slot, tok_seg, out, C)
    t0 = 0
    for s, n in segs:
        ref, ns = R.causal_conv1d_silu(x[t0:t0 + n], w, state0[s])
        assert torch.allclose(out[t0:t0 + n], ref, atol=1e-5, rtol=1e-5)
        assert torch.allclose(state[s], ns, atol=0, rtol=0)
        t0 += n


@pytest.mark.parametrize("segs", [[(0, 1), (1, 1)], [(1, 40)], [(0, 3), (1, 17)]])
def test_gdn_prepare_and_scan(K, segs):
    G, Hv, S = 2, 4, 128
    C = 2 * G * S + Hv * S
    T = sum(n for _, n in segs)
    g = torch.Generator(device="cuda").manual_seed(0)
    conv = torch.randn(T, C, generator=g, device="cuda")
    a = torch.randn(T, Hv, generator=g, device="cuda")
    b = torch.randn(T, Hv, generator=g, device="cuda")
    ssm_a = -(torch.rand(Hv, generator=g, device="cuda") * 4 + 0.5)
    dtb = torch.randn(Hv, generator=g, device="cuda") * 0.5
    state = torch.randn(2, Hv, S, S, generator=g, device="cuda") * 0.1
    state0 = state.clone()
    decay = torch.empty(T, Hv, device="cuda")
    beta = torch.empty(T, Hv, device="cuda")
    conv_k = conv.clone()
    K.gdn_prepare(conv_k, a, b, ssm_a, dtb, decay, beta, G, Hv, S)
    dref, bref = R.gdn_gates(a, b, ssm_a, dtb)
    assert torch.allclose(decay, dref, atol=1e-5, rtol=1e-4) and torch.allclose(beta, bref, atol=1e-6, rtol=1e-5)
    q = R.l2norm(conv[:, :G * S].reshape(T, G, S)) * S ** -0.5
    k = R.l2norm(conv[:, G * S:2 * G * S].reshape(T, G, S))
    v = conv[:, 2 * G * S:].reshape(T, Hv, S)
    assert torch.allclose(conv_k[:, :G * S].reshape(T, G, S), q, atol=1e-5, rtol=1e-4)
    seg_start = torch.tensor([0] + list(torch.tensor([n for _, n in segs]).cumsum(0)), device="cuda", dtype=torch.int32)
    seg_slot = torch.tensor([s for s, _ in segs], device="cuda", dtype=torch.int32)
    out = torch.empty(T, Hv, S, device="cuda")
    journal = torch.empty(T, Hv, S, S, device="cuda")
    K.gdn_scan(conv_k, decay, beta, state, seg_start, seg_slot, out, G, Hv, journal=journal)
    idx = torch.arange(Hv, device="cuda") % G
    t0 = 0
    for s, n in segs:
        o_ref, s_ref = R.gdn_recurrent(q[t0:t0 + n][:, idx], k[t0:t0 + n][:, idx], v[t0:t0 + n], dref[t0:t0 + n],
                                       bref[t0:t0 + n], state0[s])
        assert torch.allclose(out[t0:t0 + n], o_ref, atol=2e-4, rtol=1e-3)
        assert torch.allclose(state[s], s_ref, atol=2e-4, rtol=1e-3)
        assert torch.allclose(journal[t0 + n - 1], s_ref, atol=2e-4, rtol=1e-3)
        t0 += n
    # gated output norm
    z = torch.randn(T, Hv * S, device="cuda")
    nw = torch.rand(S, device="cuda") + 0.5
    og = torch.empty(T, Hv * S, device="cuda", dtype=torch.bfloat16)
    K.gdn_gated_norm(out, z, nw, og, Hv, S, 1e-6)
    ref = R.gated_rmsnorm(out, nw, z.reshape(T, Hv, S)).reshape(T, Hv * S)
    assert torch.allclose(og.float(), ref, atol=3e-2, rtol=2e-2)
    # speculative commit copies the chosen journal row into the slot
    st2 = torch.zeros_like(state)
    commit = torch.tensor([0] * len(segs), device="cuda", dtype=torch.int32)
    K.state_commit(st2, journal, seg_slot, commit, Hv * S * S)
    assert torch.equal(st2[seg_slot[0].item()], journal[0])


def test_argmax_ties_and_sampler(K):
    V = 5000
    lg = torch.randn(3, V, device="cuda")
    lg[0, 77] = 9.0
    lg[0, 4000] = 9.0
    lg[1, 4999] = 12.0
    pv = torch.empty(3 * 64, device="cuda")
    pi = torch.empty(3 * 64, device="cuda", dtype=torch.int32)
    ids = torch.empty(3, device="cuda", dtype=torch.int64)
    K.argmax_rows(lg, pv, pi, ids)
    assert ids.tolist()[:2] == [77, 4999] and ids[2].item() == int(lg[2].argmax())
    # greedy via sampler, top-k=1 via sampler, and distribution check for top-k=3
    params = K.pack_sample_params([(0.0, 0, 1.0, 0.0, 1, 0), (1.0, 1, 1.0, 0.0, 1, 0), (1.0, 0, 1.0, 0.0, 1, 0)], "cuda")
    K.sample_rows(lg, params, ids)
    assert ids[0].item() == 77 and ids[1].item() == 4999
    lg2 = torch.full((1, V), -30.0, device="cuda")
    lg2[0, [5, 50, 500, 4500]] = torch.tensor([2.0, 1.0, 0.0, -1.0], device="cuda")
    counts = {}
    one = torch.empty(1, device="cuda", dtype=torch.int64)
    for c in range(400):
        p = K.pack_sample_params([(1.0, 3, 1.0, 0.0, 1234, c)], "cuda")
        K.sample_rows(lg2, p, one)
        counts[one.item()] = counts.get(one.item(), 0) + 1
    assert set(counts) <= {5, 50, 500}
    probs = torch.softmax(torch.tensor([2.0, 1.0, 0.0]), 0)
    for tok, pr in zip((5, 50, 500), probs.tolist()):
        assert abs(counts.get(tok, 0) / 400 - pr) < 0.08
    # top-p keeps the smallest prefix reaching the mass
    for c in range(50):
        p = K.pack_sample_params([(1.0, 0, 0.6, 0.0, 99, c)], "cuda")
        K.sample_rows(lg2, p, one)
        assert one.item() == 5            # p(5) = 0.64 >= 0.6
    ids_n, lps, clp = K.topn_logprobs(lg2, 3, 1.0, torch.tensor([50], device="cuda"))
    assert ids_n[0].tolist() == [5, 50, 500]
    ref_lp = torch.log_softmax(lg2[0], 0)
    assert torch.allclose(lps[0], ref_lp[[5, 50, 500]], atol=1e-4)
    assert abs(clp.item() - ref_lp[50].item()) < 1e-4


def test_small_gemm_f32(K):
    x = torch.randn(70, 200, device="cuda").bfloat16()
    w = torch.randn(50, 200, device="cuda")
    out = torch.empty(70, 50, device="cuda")
    K.small_gemm_f32(x, w, out)
    assert torch.allclose(out, x.float() @ w.t(), atol=1e-3, rtol=1e-3)


@pytest.mark.parametrize("D,H,Hkv,T,pos0", [(256, 6, 1, 200, 0), (256, 4, 2, 70, 37), (128, 8, 2, 129, 0), (64, 4, 4, 33, 5)])
def test_flash_prefill_matches_reference(K, D, H, Hkv, T, pos0):
    from hipengine_b200.ops import attention as A
    S = pos0 + T
    cache, bt = _paged_setup(S, Hkv, D, n_slots=2, max_ctx=320)
    g = torch.Generator(device="cuda").manual_seed(1)
    kf = torch.randn(S, Hkv * D, generator=g, device="cuda")
    vf = torch.randn(S, Hkv * D, generator=g, device="cuda")
    slot = torch.full((S,), 1, device="cuda", dtype=torch.int32)
    pos = torch.arange(S, device="cuda", dtype=torch.int32)
    dummy = torch.empty(S, H, D, device="cuda", dtype=torch.bfloat16)
    K.qkv_post(torch.zeros(S, H * D, device="cuda"), kf, vf, None, None, dummy, None, cache, bt, slot, pos, H, Hkv, D,
               16, False, 0, 1e6, 1e-6)
    q = (torch.randn(T, H, D, generator=g, device="cuda") * 0.5).bfloat16()
    gate = torch.randn(T, H, D, generator=g, device="cuda").bfloat16()
    out = torch.empty(T, H * D, device="cuda", dtype=torch.bfloat16)
    scale = D ** -0.5
    A.flash_prefill(q, gate, cache, bt, 1, pos0, out, H, Hkv, D, 16, scale)
    kb = kf.reshape(S, Hkv, D).bfloat16().float()
    vb = vf.reshape(S, Hkv, D).bfloat16().float()
    qpos = torch.arange(pos0, pos0 + T, device="cuda")
    ref = R.causal_gqa_attention(q.float(), kb, vb, qpos, scale)
    ref = R.bf16_round(ref) * torch.sigmoid(gate.float())
    assert torch.allclose(out.float().reshape(T, H, D), ref, atol=2e-2, rtol=2e-2)
    # sliding window, no gate
    A.flash_prefill(q, None, cache, bt, 1, pos0, out, H, Hkv, D, 16, scale, window=48)
    ref = R.causal_gqa_attention(q.float(), kb, vb, qpos, scale, window=48)
    assert torch.allclose(out.float().reshape(T, H, D), ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("lens", [[64], [200], [37, 150, 16]], ids=["one_chunked", "ragged_tail", "three_segments"])
def test_gdn_chunked_scan_matches_reference(lens):
    """Chunked (WY, TF32 tensor-core) scan against the fp32 recurrence: outputs and final states."""
    from hipengine_b200.ops import kernels as K
    from hipengine_b200.ref import ops as R
    G, Hv, S = 2, 4, 128
    C = 2 * G * S + Hv * S
    T = sum(lens)
    g = torch.Generator().manual_seed(T)
    q = R.l2norm(torch.randn(T, G, S, generator=g)) * S ** -0.5
    k = R.l2norm(torch.randn(T, G, S, generator=g))
    v = torch.randn(T, Hv, S, generator=g) * 0.5
    decay = torch.rand(T, Hv, generator=g) * 0.5 + 0.5
    decay[3] = 1e-9                                        # a near-total reset must not produce inf / nan
    beta = torch.rand(T, Hv, generator=g)
    state0 = torch.randn(len(lens), Hv, S, S, generator=g) * 0.1
    qkv = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], 1).contiguous()
    idx = torch.arange(Hv) % G
    want_o, want_s = [], []
    t0 = 0
    for si, n in enumerate(lens):
        o, s = R.gdn_recurrent(q[t0:t0 + n][:, idx], k[t0:t0 + n][:, idx], v[t0:t0 + n], decay[t0:t0 + n],
                               beta[t0:t0 + n], state0[si].clone())
        want_o.append(o)
        want_s.append(s)
        t0 += n
    want_o, want_s = torch.cat(want_o), torch.stack(want_s)
    seg_start = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    seg_slot = torch.arange(len(lens), dtype=torch.int32, device="cuda")
    state = state0.cuda().clone()
    out = torch.zeros(T, Hv, S, device="cuda")
    K.gdn_scan_chunked(qkv.cuda(), decay.cuda(), beta.cuda(), state, seg_start, seg_slot, out, G, Hv)
    torch.cuda.synchronize()
    assert torch.isfinite(out).all() and torch.isfinite(state).all()
    scale_o, scale_s = want_o.abs().max(), want_s.abs().max()
    assert (out.cpu() - want_o).abs().max() / scale_o < 2e-2
    assert (state.cpu() - want_s).abs().max() / scale_s < 2e-2


@pytest.mark.parametrize("D,H,Hkv,rows,ctxs,window", [
    (256, 24, 4, 3, (1, 333, 1100), 0),          # 27B geometry: 6 query heads per KV head
    (256, 8, 1, 2, (64, 2049), 0),               # 8 heads in one group, span ends on / just past a tile edge
    (128, 8, 2, 4, (17, 500, 31, 4097), 0),
    (512, 8, 2, 2, (700, 90), 0),                # head_dim 512 (Gemma 4 global layers)
    (256, 8, 2, 2, (900, 300), 256),             # sliding window
])
def test_tensor_core_decode_attention_matches_fp32(K, D, H, Hkv, rows, ctxs, window):
    """Split-K decode attention on mma.sync tiles (whole pages streamed by bulk copies) against fp32 PyTorch, with
    the split sizes the engine would pick for one row and for a wide batch."""
    page = 16
    g = torch.Generator(device="cuda").manual_seed(D + H + rows)
    max_ctx = max(ctxs)
    mp = (max_ctx + page - 1) // page
    cache = (torch.randn(rows * mp + 1, 2, Hkv, page, D, device="cuda", generator=g) * 0.5).bfloat16()
    bt = (torch.randperm(rows * mp, device="cuda", generator=g).int() + 1).reshape(rows, mp).contiguous()
    slot = torch.arange(rows, device="cuda", dtype=torch.int32)
    ctx_len = torch.tensor(ctxs, device="cuda", dtype=torch.int32)
    q = torch.randn(rows, H, D, device="cuda", generator=g).bfloat16()
    gate = torch.randn(rows, H, D, device="cuda", generator=g).bfloat16()
    scale = D ** -0.5
    # fp32 reference per row
    ref = torch.empty(rows, H, D, device="cuda")
    G = H // Hkv
    for r in range(rows):
        n = ctxs[r]
        pages = bt[r, : (n + page - 1) // page].long()
        kk = cache[pages, 0].permute(1, 0, 2, 3).reshape(Hkv, -1, D)[:, :n].float()
        vv = cache[pages, 1].permute(1, 0, 2, 3).reshape(Hkv, -1, D)[:, :n].float()
        if window > 0 and n > window:
            kk, vv = kk[:, n - window:], vv[:, n - window:]
        for h in range(H):
            s = (kk[h // G] @ q[r, h].float()) * scale
            p = torch.softmax(s, -1)
            ref[r, h] = p @ vv[h // G]
    ref = R.bf16_round(ref) * torch.sigmoid(gate.float())
    span = min(max_ctx, window) if window > 0 else max_ctx
    for batch_rows in (1, 64):                    # split sizes of a single row and of a wide batch
        split_len, max_splits = K.attn_decode_split(span, batch_rows, Hkv)
        max_splits += 1 if window > 0 else 0
        part = torch.full((K.attn_decode_scratch_floats(rows, H, max_splits, D),), float("nan"), device="cuda")
        out = torch.empty(rows, H * D, device="cuda", dtype=torch.bfloat16)
        K.attn_decode(q, gate, cache, bt, slot, ctx_len, part, out, H, Hkv, D, page, split_len, max_splits, scale,
                      window=window)
        torch.cuda.synchronize()
        K.check_status()
        got = out.float().reshape(rows, H, D)
        assert torch.isfinite(got).all()
        assert torch.allclose(got, ref, atol=2e-2, rtol=2e-2), (split_len, (got - ref).abs().max())
