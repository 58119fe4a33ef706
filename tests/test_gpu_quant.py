"""GPU parity of quant_mx / dequant_mx / transform_sf against the oracle: byte-exact codes,
UE8M0 bytes and packed words (the expectations of deepgemm/tests/e2e_gpu.rs:80-117, 582-624),
through the C ABI."""
import numpy as np
import pytest
import torch

import oracle as o
from deepgemm import Dtype, SfGran, SfTensor, dequant_mx, quant_mx, transform_sf
from helpers import dev, randn

pytestmark = pytest.mark.gpu

CASES = [  # (m, k, dtype, gran)
    (128, 512, "fp8", 128), (128, 512, "fp8", 32), (128, 512, "fp4", 32),
    (33, 256, "fp8", 32),       # m not a multiple of 4 or 32
    (257, 7168, "fp8", 128),    # 56 groups, ragged m
    (5, 384, "fp8", 128),       # 3 groups: partial SF word
    (70, 224, "fp8", 32),       # 7 groups: partial SF word
    (70, 224, "fp4", 32),
    (1, 32, "fp4", 32), (1, 128, "fp8", 128),
    (1000, 4096, "fp4", 32), (1000, 4096, "fp8", 32),
]


def _special(m, k, seed):
    """N(0,1) data with the edge values of the format mixed in."""
    x = randn((m, k), seed)
    flat = x.reshape(-1)
    rng = np.random.default_rng(seed + 1)
    idx = rng.choice(flat.size, size=min(flat.size // 4, 4000), replace=False)
    specials = np.array([0.0, -0.0, 1e-38, -1e-38, 1e-30, 448.0, -448.0, 464.0, 6.0, -6.0, 3.5, 2.5, 0.25, 1.75,
                         5.0, 7.0, 1e30, -1e30, 2.0 ** -9, 3 * 2.0 ** -10, 0.0625, 500.0, np.nan, -np.nan],
                        dtype=np.float32)
    flat[idx] = specials[rng.integers(0, specials.size, idx.size)]
    if m > 2:
        x[1, :] = 0.0                         # an all-zero row: amax floor
        x[2, : k // 2] *= 1e-20               # tiny block
    return x


@pytest.mark.parametrize("m,k,kind,gran", CASES)
def test_quant_mx_bytes_equal_oracle(m, k, kind, gran):
    x = _special(m, k, 1234 + m + k)
    dt, odt = (Dtype.Fp4, o.FP4) if kind == "fp4" else (Dtype.Fp8, o.FP8)
    want_data, want_sf = o.quant_mx_host(x, odt, gran)
    data, sf = quant_mx(dev(x), m, k, dt, gran)
    torch.cuda.synchronize()
    assert (sf.rows, sf.cols) == want_sf.shape
    got_sf = sf.buf.cpu().numpy().view(np.uint32)
    got_data = data.cpu().numpy()
    assert np.array_equal(got_sf, want_sf), f"SF words differ at {np.argwhere(got_sf != want_sf)[:4]}"
    bad = np.argwhere(got_data != want_data)
    assert bad.size == 0, f"{len(bad)} code bytes differ, first {bad[:4]}"


def test_quant_mx_host_entry_matches_device_entry():
    m, k = 300, 1024
    x = _special(m, k, 7)
    d1, s1 = quant_mx(x, m, k, Dtype.Fp8, 128)          # host slice, like the reference API
    d2, s2 = quant_mx(dev(x), m, k, Dtype.Fp8, 128)
    torch.cuda.synchronize()
    assert torch.equal(d1, d2) and torch.equal(s1.buf, s2.buf)


def test_quant_outputs_need_no_clearing():
    """Every SF word, padding included, is written: poison the outputs first."""
    from deepgemm import _lib
    import ctypes as C
    m, k = 33, 224
    x = _special(m, k, 3)
    want_data, want_sf = o.quant_mx_host(x, o.FP8, 32)
    data = torch.full((m, k), 0xAB, dtype=torch.uint8, device="cuda")
    sf = torch.full(want_sf.shape, -1, dtype=torch.int32, device="cuda")
    xd = dev(x)
    st = _lib.load().dg_quant_mx(xd.data_ptr(), m, k, 0, 32, data.data_ptr(), sf.data_ptr(),
                                 C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == 0
    torch.cuda.synchronize()
    assert np.array_equal(sf.cpu().numpy().view(np.uint32), want_sf)
    assert np.array_equal(data.cpu().numpy(), want_data)


@pytest.mark.parametrize("m,k,kind,gran", CASES[:8])
def test_dequant_mx_equals_oracle(m, k, kind, gran):
    x = _special(m, k, 99 + m)
    odt, dt = (o.FP4, Dtype.Fp4) if kind == "fp4" else (o.FP8, Dtype.Fp8)
    data, sf = o.quant_mx_host(x, odt, gran)
    if k % 8:
        pytest.skip("dequant kernel walks 8 elements per thread")
    want = o.dequant_mx_host(data, sf, m, k, odt, gran)
    sft = SfTensor(sf.shape[0], sf.shape[1], SfGran(gran), dev(sf.view(np.int32)))
    got = dequant_mx(dev(data), sft, m, k, dt).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_dequant_all_codes_and_scale_extremes():
    """All 256 E4M3 bytes (NaN codes included) under scale bytes 0, 1, 127, 254."""
    m, k = 4, 256
    data = np.tile(np.arange(256, dtype=np.uint8), (m, 1))
    sf = np.zeros((1, 4), dtype=np.uint32)
    for r, e in enumerate([0, 1, 127, 254]):
        sf[0, r] = e * 0x01010101
    sf = np.repeat(sf, 2, axis=0)  # k/32 = 8 groups -> 2 word rows
    want = o.dequant_mx_host(data, sf, m, k, o.FP8, 32)
    got = dequant_mx(dev(data), SfTensor(2, 4, SfGran.G32, dev(sf.view(np.int32))), m, k, Dtype.Fp8).cpu().numpy()
    assert np.array_equal(np.isnan(got), np.isnan(want))
    ok = ~np.isnan(want)
    assert np.array_equal(got[ok].view(np.uint32), want[ok].view(np.uint32))


@pytest.mark.parametrize("mn,sf_k", [(33, 7), (64, 16), (128, 4), (257, 32), (24576, 12), (4100, 224), (1, 1)])
def test_transform_sf_words_equal_oracle(mn, sf_k):
    rng = np.random.default_rng(mn * 1000 + sf_k)
    sf = (2.0 ** rng.integers(-40, 40, size=(mn, sf_k))).astype(np.float32)
    want = o.transform_sf_host(sf, mn)
    got = transform_sf(dev(sf), mn, SfGran.G32)
    assert (got.rows, got.cols) == want.shape
    assert np.array_equal(got.buf.cpu().numpy().view(np.uint32), want)
    got_h = transform_sf(sf, mn, SfGran.G32)              # host slice, like the reference API
    assert np.array_equal(got_h.buf.cpu().numpy().view(np.uint32), want)


def test_quant_then_dequant_round_trip_at_full_size():
    """Size-independent property at a bandwidth-benchmark shape: dequant(quant(x)) is within
    half a grid step of x, and quantising the dequantised tensor reproduces the codes."""
    m, k = 4096, 7168
    x = torch.randn((m, k), device="cuda", generator=torch.Generator("cuda").manual_seed(0))
    data, sf = quant_mx(x, m, k, Dtype.Fp8, 128)
    back = dequant_mx(data, sf, m, k, Dtype.Fp8)
    amax = x.view(m, k // 128, 128).abs().amax(dim=2, keepdim=True)
    err = (back - x).view(m, k // 128, 128).abs()
    assert bool((err <= amax * (2.0 ** -4) + 1e-30).all())
    data2, sf2 = quant_mx(back, m, k, Dtype.Fp8, 128)
    # requantising can only keep or lower a block's scale; where the scale is kept the codes repeat
    same = (sf2.buf == sf.buf).all()
    if bool(same):
        assert torch.equal(data, data2)
