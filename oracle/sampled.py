"""Sampled parity checks of full-size GPU results against the oracle (test infrastructure only).

A benchmark-size GEMM has far too many outputs for gemm_ref (f64, one MAC at a time) to recompute, but any
sub-rectangle of D depends only on the sampled rows of A and of B over the full K.  The helpers here pull
those rows (codes and packed scale-factor columns) from device tensors, rebuild compact GoldenOperands and
compare the corresponding outputs: calc_diff (the contract's measure) plus the largest element error in
units of the reference's RMS, which exposes a single wrong tile that calc_diff would average away.
Device tensors are torch tensors; torch is imported by the caller, not here.
"""
import numpy as np

from . import oracle as o


def pick(total, count, seed, must=()):
    """`count` sorted distinct indices below `total`: the given ones (tile edges, first / last) plus random ones."""
    rng = np.random.default_rng(seed)
    base = [i for i in must if 0 <= i < total]
    need = max(0, min(count, total) - len(set(base)))
    rest = rng.choice(total, size=min(total, need + len(base)), replace=False)
    out = list(dict.fromkeys(base + [int(r) for r in rest]))[:min(count, total)]
    return np.array(sorted(out), dtype=np.int64)


def edges(total, tile):
    """Indices around the first few and the last tile boundaries."""
    e = [0, 1, total - 1, total - 2]
    for t in (tile, 2 * tile, (total // tile) * tile, (total // tile - 1) * tile):
        e += [t - 1, t, t + 1]
    return [i for i in e if 0 <= i < total]


def golden_rows(codes, sf_words, rows, dtype, gran, k, row_offset=0):
    """GoldenOperand of the sampled `rows` (indices into the stacked operand, already including any group offset)
    of a device operand: codes [R, k or k/2] uint8, sf_words [sf_rows, cols] int32 (columns = rows of the operand)."""
    import torch
    idx = torch.as_tensor(np.asarray(rows) + row_offset, device=codes.device, dtype=torch.long)
    c = codes.index_select(0, idx).cpu().numpy()
    w = sf_words.index_select(1, idx).cpu().numpy().view(np.uint32)
    pad = (-w.shape[1]) % 4
    if pad:
        w = np.concatenate([w, np.zeros((w.shape[0], pad), dtype=np.uint32)], axis=1)
    return o.GoldenOperand(c, np.ascontiguousarray(w), dtype, gran, k)


def compare(got, ref, out_is_bf16=True):
    """(calc_diff, max element error / rms of the reference) of a sampled block; got / ref f32 arrays."""
    got = np.asarray(got, dtype=np.float32)
    ref = np.asarray(ref, dtype=np.float32)
    if out_is_bf16:
        ref = o.bf16_bits_to_f32(o.f32_to_bf16_bits_np(ref))
    if not np.isfinite(got).all():
        return float("inf"), float("inf")
    rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2))) + 1e-30
    return o.calc_diff(got, ref), float(np.abs(got - ref).max() / rms)


def check_gemm_sample(a_codes, a_sf, b_codes, b_sf, out, rows, cols, a_dtype, a_gran, b_dtype, b_gran, k,
                      b_row_offset=0, out_rows=None):
    """Compares out[out_rows or rows][:, cols] with gemm_ref over the sampled rows of A and rows (b_row_offset + cols)
    of B.  Returns {"calc_diff", "max_err"}."""
    import torch
    ga = golden_rows(a_codes, a_sf, rows, a_dtype, a_gran, k)
    gb = golden_rows(b_codes, b_sf, cols, b_dtype, b_gran, k, row_offset=b_row_offset)
    ref = o.gemm_ref(ga, gb, m=len(rows), n=len(cols))
    r = torch.as_tensor(np.asarray(out_rows if out_rows is not None else rows), device=out.device, dtype=torch.long)
    c = torch.as_tensor(np.asarray(cols), device=out.device, dtype=torch.long)
    got = out.index_select(0, r).index_select(1, c).float().cpu().numpy()
    d, e = compare(got, ref, out_is_bf16=out.dtype != torch.float32)
    return {"calc_diff": d, "max_err": e}
