"""Seeded synthetic inputs for the benchmark and the full-size tests (device side, torch only
as tensor plumbing).  The distributions and shapes are those of the benchmark configurations:
N(0,1) values, E4M3 with UE8M0 scales at granularity 128 (1x128 on activations through
quant_mx, 128x128 blocks on weights), uniform-random distinct top-k routing."""
import torch

from .api import quant_mx
from .types import Dtype, Operand, SfGran, SfTensor


def block128_quant_fp8(x):
    """x f32 [n, k] (device), n % 128 == 0, k % 512 == 0 -> (codes u8 [n, k], packed SF words
    i32 [k/512, n]).  One UE8M0 exponent per 128x128 block with the exponent rule of
    deepgemm/src/golden.rs:211-224, written as the per-row G128 layout (byte replicated on the
    block's 128 rows).  Checked against the oracle's block quantiser in the GPU tests."""
    n, k = x.shape
    assert n % 128 == 0 and k % 512 == 0
    xb = x.view(n // 128, 128, k // 128, 128)
    amax = xb.abs().amax(dim=(1, 3)).clamp_min(1e-30)                          # [n/128, k/128]
    bits = amax.view(torch.int32)
    e = torch.clamp((bits + 0x7FFFFF - 0x600000) >> 23, min=113) - 8             # biased exponent
    inv = ((254 - e) << 23).view(torch.float32)
    codes = (xb * inv[:, None, :, None]).to(torch.float8_e4m3fn).view(torch.uint8).reshape(n, k)
    e4 = e.view(n // 128, k // 512, 4)
    words = e4[..., 0] | (e4[..., 1] << 8) | (e4[..., 2] << 16) | (e4[..., 3] << 24)   # [n/128, k/512]
    sf = words.t().contiguous().repeat_interleave(128, dim=1).contiguous()                # [k/512, n]
    return codes, sf.to(torch.int32)


def expert_seed(seed, expert):
    """Seed of one expert's weight matrix: experts are generated independently, so that any one of them
    can be regenerated alone (a parity check on one GPU can rebuild an expert that lives on another)."""
    return seed * 1000003 + expert


def expert_weight(seed, expert, n, k, device):
    """(codes u8 [n, k], packed SF words i32 [k/512, n]) of expert `expert` of the stack seeded `seed`."""
    g = torch.Generator(device=device).manual_seed(expert_seed(seed, expert))
    return block128_quant_fp8(torch.randn((n, k), device=device, generator=g))


def random_expert_weights(num_local_experts, n, k, seed, device):
    """Stacked FP8 weights [E*n, k] + SF of the stacked matrix, generated and quantised expert
    by expert so that no f32 tensor of the whole stack is ever held."""
    codes = torch.empty((num_local_experts * n, k), dtype=torch.uint8, device=device)
    sf = torch.empty((k // 512, num_local_experts * n), dtype=torch.int32, device=device)
    for e in range(num_local_experts):
        c, s = expert_weight(seed, e, n, k, device)
        codes[e * n:(e + 1) * n] = c
        sf[:, e * n:(e + 1) * n] = s
    op = Operand.k_major(Dtype.Fp8, n, k, k, SfTensor(k // 512, num_local_experts * n, SfGran.G128, sf), codes)
    return op


def random_topk_routing(tokens, num_experts, topk, seed, device):
    """Uniform-random distinct top-k experts per token and positive weights that sum to 1."""
    g = torch.Generator(device=device).manual_seed(seed)
    idx = torch.rand((tokens, num_experts), device=device, generator=g).topk(topk, dim=1).indices.to(torch.int32)
    w = torch.rand((tokens, topk), device=device, generator=g) + 0.1
    return idx, (w / w.sum(1, keepdim=True)).contiguous()


def quantised_tokens(x, gran=128):
    """f32 [T, K] device tokens -> (codes, SfTensor) through the library's quant_mx."""
    t, k = x.shape
    return quant_mx(x, t, k, Dtype.Fp8, gran)
