"""GPU parity of mqa_logits against the oracle's mqa_logits_ref (deepgemm/src/golden.rs:469-501),
through the C ABI.  Tolerance: calc_diff <= 1e-3 (the FP8 bound of the stated contract) plus an
element-wise bound; columns outside [ks, ke) must stay untouched."""
import numpy as np
import pytest
import torch

import oracle as o
from deepgemm import Dtype, Operand, mqa_logits, mqa_logits_f32, poll_device_status
from helpers import dev, randn, sf_tensor

pytestmark = pytest.mark.gpu
E4M3 = o.e4m3_table()


def _inputs_f32(T, S, H, D, seed):
    q8 = o.quant_e4m3_array(randn((T, H, D), seed))
    kvf = randn((S, D), seed + 1)
    scale = (np.abs(kvf).max(axis=1) / 448.0).astype(np.float32)
    kv8 = o.quant_e4m3_array(kvf / scale[:, None])
    w = randn((T, H), seed + 2)
    return q8, kv8, scale, w


def _check(got, ref, ks, ke, S, fill):
    T = got.shape[0]
    for t in range(T):
        n = max(0, min(int(ke[t]), S) - int(ks[t]))
        assert (got[t, n:] == fill).all(), f"row {t}: columns beyond the span were written"
        if n:
            want = ref[t, ks[t]:ks[t] + n]
            assert np.isfinite(got[t, :n]).all()
    gv = np.concatenate([got[t, :max(0, min(int(ke[t]), S) - int(ks[t]))] for t in range(T)])
    rv = np.concatenate([ref[t, ks[t]:min(int(ke[t]), S)] if ke[t] > ks[t] else ref[t, :0] for t in range(T)])
    assert o.calc_diff(gv, rv) <= 1e-3
    rms = np.sqrt(np.mean(rv.astype(np.float64) ** 2)) + 1e-30
    assert np.abs(gv - rv).max() / rms <= 0.05


@pytest.mark.parametrize("T,S,H,D,mode", [
    (8, 256, 64, 128, "full"), (64, 1024, 64, 128, "causal"), (37, 700, 64, 128, "ragged"),
    (16, 384, 32, 128, "ragged"), (10, 300, 128, 128, "ragged"), (12, 512, 64, 64, "causal"),
    (12, 512, 64, 32, "ragged"), (600, 2048, 64, 128, "causal"),
])
def test_mqa_logits_f32_contract(T, S, H, D, mode):
    q8, kv8, scale, w = _inputs_f32(T, S, H, D, T + S)
    rng = np.random.default_rng(T * S)
    if mode == "full":
        ks, ke = np.zeros(T, np.uint32), np.full(T, S, np.uint32)
    elif mode == "causal":                       # ke_i = S - T + i + 1, ks = 0
        ks, ke = np.zeros(T, np.uint32), (S - T + np.arange(T) + 1).astype(np.uint32)
    else:                                        # arbitrary windows, some empty, some past the end
        ks = rng.integers(0, S, T).astype(np.uint32)
        ke = (ks + rng.integers(0, S, T)).astype(np.uint32)
        ke[::5] = ks[::5]
        ke[1::7] = S + 50
    ref = o.mqa_logits_ref(E4M3[q8], E4M3[kv8] * scale[:, None], w, ks, ke)
    stride = S + 3
    fill = -777.0
    logits = torch.full((T, stride), fill, dtype=torch.float32, device="cuda")
    mqa_logits_f32(dev(q8), dev(kv8), dev(scale), dev(w), dev(ks.view(np.int32)), dev(ke.view(np.int32)),
                   T, S, H, D, logits, stride)
    poll_device_status()
    _check(logits.cpu().numpy(), ref, ks, ke, S, fill)


@pytest.mark.parametrize("T,S,H,D", [(8, 256, 64, 128), (50, 900, 64, 128), (24, 512, 32, 128), (12, 384, 64, 64)])
def test_mqa_logits_ue8m0_contract(T, S, H, D):
    """The reference SM100 flavour: UE8M0 per-32 scales on q and kv, bf16 weights and output."""
    qf, kvf = randn((T * H, D), 3), randn((S, D), 4) * 3.0
    q8, qsf = o.quant_mx_host(qf, o.FP8, 32)
    kv8, kvsf = o.quant_mx_host(kvf, o.FP8, 32)
    wb = torch.from_numpy(randn((T, H), 5)).to(torch.bfloat16)
    rng = np.random.default_rng(T)
    ks = rng.integers(0, S // 2, T).astype(np.uint32)
    ke = (ks + rng.integers(1, S, T)).astype(np.uint32)
    qd = o.dequant_mx_host(q8, qsf, T * H, D, o.FP8, 32).reshape(T, H, D)
    kvd = o.dequant_mx_host(kv8, kvsf, S, D, o.FP8, 32)
    ref = o.mqa_logits_ref(qd, kvd, wb.float().numpy(), ks, ke)
    qop = Operand.k_major(Dtype.Fp8, T * H, D, D, sf_tensor(qsf, 32), dev(q8))
    kvop = Operand.k_major(Dtype.Fp8, S, D, D, sf_tensor(kvsf, 32), dev(kv8))
    fill = -9.0
    logits = torch.full((T, S), fill, dtype=torch.bfloat16, device="cuda")
    mqa_logits(qop, kvop, wb.cuda(), dev(ks.view(np.int32)), dev(ke.view(np.int32)), T, S, H, D, logits, S)
    poll_device_status()
    got = logits.float().cpu().numpy()
    _check(got, o.bf16_bits_to_f32(o.f32_to_bf16_bits_np(ref)), ks, ke, S, fill)
