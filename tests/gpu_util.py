"""Helpers shared by the GPU parity tests."""
import torch

ATOL_BF16, RTOL_BF16 = 2e-2, 1e-2      # attention outputs, bf16 KV
ATOL_FP8, RTOL_FP8 = 5e-2, 1e-2        # attention outputs, e4m3 KV


def assert_close(got, want, atol, rtol, what=""):
    got, want = got.float().cpu(), want.float().cpu()
    assert got.shape == want.shape, (got.shape, want.shape)
    assert torch.isfinite(got).all(), f"{what}: non-finite output"
    err = (got - want).abs()
    bound = atol + rtol * want.abs()
    bad = err > bound
    if bad.any():
        idx = torch.nonzero(bad)[0].tolist()
        raise AssertionError(f"{what}: {int(bad.sum())} of {bad.numel()} elements out of tolerance; "
                             f"max err {err.max():.4g}; first at {idx}: got {got[tuple(idx)]:.5g} want {want[tuple(idx)]:.5g}")


def bits_equal(a, b):
    return torch.equal(a.contiguous().view(torch.uint8).cpu(), b.contiguous().view(torch.uint8).cpu())


def to_dev(w, device="cuda"):
    """Copies of a workload's tensors on the GPU (the CPU originals stay for the oracle)."""
    return dict(q=w.q.to(device), k=w.k.to(device), v=w.v.to(device), k_cache=w.k_cache.to(device),
                v_cache=w.v_cache.to(device), slot_mapping=w.slot_mapping.to(device),
                context_lens=w.context_lens_tensor().to(device), block_tables=w.block_tables_tensor().to(device))
