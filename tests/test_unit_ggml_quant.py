"""GGML block formats: numpy oracle vs torch twin bit-exactness, quantizer round trips, hand fixtures."""
import numpy as np
import pytest
import torch

from hipengine_b200.quant import ggml as Q


def _rand_blocks(t, rows, cols, seed=0):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(rows, cols, generator=g) * 0.02
    return w, Q.quantize(w, t)


@pytest.mark.parametrize("t", [Q.GGMLType.Q4_K, Q.GGMLType.Q6_K, Q.GGMLType.Q8_0])
def test_numpy_and_torch_dequant_are_bit_identical(t):
    w, raw = _rand_blocks(t, 7, 512)
    a = Q.dequantize_np(raw.numpy(), t, 7, 512)
    b = Q.dequantize_torch(raw, t, 7, 512).numpy()
    assert a.dtype == np.float32 and b.dtype == np.float32
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


@pytest.mark.parametrize("t,tol", [(Q.GGMLType.Q4_K, 0.09), (Q.GGMLType.Q6_K, 0.025), (Q.GGMLType.Q8_0, 0.006)])
def test_quantizer_error_is_bounded(t, tol):
    w, raw = _rand_blocks(t, 16, 1024, seed=3)
    d = Q.dequantize_torch(raw, t, 16, 1024)
    rel = (d - w).norm() / w.norm()
    assert rel < tol, rel


def test_q4_k_hand_fixture():
    blk = np.zeros(144, np.uint8)
    blk[0:2] = np.array([2.0], np.float16).view(np.uint8)      # d
    blk[2:4] = np.array([0.5], np.float16).view(np.uint8)      # dmin
    sc = [1, 2, 3, 4, 33, 34, 35, 36]
    mn = [5, 6, 7, 8, 41, 42, 43, 44]
    for j in range(4):
        blk[4 + j] = (sc[j] & 63) | ((sc[j + 4] >> 4) << 6)
        blk[8 + j] = (mn[j] & 63) | ((mn[j + 4] >> 4) << 6)
        blk[12 + j] = (sc[j + 4] & 15) | ((mn[j + 4] & 15) << 4)
    q = (np.arange(256) % 16).astype(np.uint8).reshape(4, 2, 32)
    blk[16:144] = (q[:, 0] | (q[:, 1] << 4)).reshape(-1)
    y = Q.dequant_q4_k_np(blk[None])[0]
    for e in (0, 31, 32, 100, 255):
        sb = e // 32
        expect = np.float32(np.float32(2.0 * sc[sb]) * np.float32(e % 16)) - np.float32(0.5 * mn[sb])
        assert y[e] == expect


def test_q6_k_hand_fixture():
    rng = np.random.default_rng(0)
    q = rng.integers(0, 64, size=256)
    sc = rng.integers(-20, 20, size=16).astype(np.int8)
    blk = np.zeros(210, np.uint8)
    qq = q.reshape(2, 4, 32)
    for n in range(2):
        for l in range(32):
            blk[n * 64 + l] = (qq[n, 0, l] & 15) | ((qq[n, 2, l] & 15) << 4)
            blk[n * 64 + 32 + l] = (qq[n, 1, l] & 15) | ((qq[n, 3, l] & 15) << 4)
            blk[128 + n * 32 + l] = (qq[n, 0, l] >> 4) | ((qq[n, 1, l] >> 4) << 2) | ((qq[n, 2, l] >> 4) << 4) | ((qq[n, 3, l] >> 4) << 6)
    blk[192:208] = sc.view(np.uint8)
    blk[208:210] = np.array([0.25], np.float16).view(np.uint8)
    y = Q.dequant_q6_k_np(blk[None])[0]
    for e in (0, 15, 16, 33, 127, 128, 200, 255):
        expect = np.float32(np.float32(0.25) * np.float32(sc[e // 16])) * np.float32(int(q[e]) - 32)
        assert y[e] == expect


def test_q8_0_round_trip_exact_on_grid():
    d = np.float16(0.125)
    q = np.arange(-16, 16, dtype=np.int8)
    blk = np.concatenate([np.array([d]).view(np.uint8), q.view(np.uint8)])
    y = Q.dequant_q8_0_np(blk[None])[0]
    assert np.array_equal(y, q.astype(np.float32) * np.float32(d))


def test_legacy_formats_decode():
    rng = np.random.default_rng(1)
    for t, fn in [(Q.GGMLType.Q4_0, Q.dequant_q4_0_np), (Q.GGMLType.Q4_1, Q.dequant_q4_1_np),
                  (Q.GGMLType.Q5_0, Q.dequant_q5_0_np), (Q.GGMLType.Q5_1, Q.dequant_q5_1_np),
                  (Q.GGMLType.Q5_K, Q.dequant_q5_k_np)]:
        lay = Q.layout_of(t)
        blk = rng.integers(0, 256, size=(3, lay.block_bytes)).astype(np.uint8)
        blk[:, 0:2] = np.array([0.5], np.float16).view(np.uint8)
        blk[:, 2:4] = np.array([0.25], np.float16).view(np.uint8)
        y = fn(blk)
        assert y.shape == (3, lay.block_elems) and np.isfinite(y).all()


def test_row_bytes_and_errors():
    assert Q.row_bytes(Q.GGMLType.Q4_K, 5120) == 20 * 144
    assert Q.row_bytes(Q.GGMLType.Q6_K, 256) == 210
    assert Q.row_bytes(Q.GGMLType.Q8_0, 64) == 68
    with pytest.raises(ValueError):
        Q.row_bytes(Q.GGMLType.Q4_K, 100)
