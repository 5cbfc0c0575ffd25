"""Shared pieces of the parity tests."""
import torch

# Tolerance of the parity gate: fp32 accumulation, fp16/bf16 outputs (element-wise), plus the
# reference test-suite's own criterion (tests/test_decoding_attn.py:94, :128).
ATOL, RTOL = 2e-3, 1e-2
REF_MEAN_ABS = 5e-3


def assert_close(out, expect, what=""):
    out32, exp32 = out.float().cpu(), expect.float().cpu()
    assert out32.shape == exp32.shape, f"{what}: shape {out32.shape} vs {exp32.shape}"
    assert torch.isfinite(out32).all(), f"{what}: non-finite output"
    err = (out32 - exp32).abs()
    bound = ATOL + RTOL * exp32.abs()
    worst = (err - bound).max().item()
    assert worst <= 0, f"{what}: max |err| {err.max().item():.3e} exceeds atol {ATOL} + rtol {RTOL} by {worst:.3e}"
    assert err.mean().item() <= REF_MEAN_ABS, f"{what}: mean |err| {err.mean().item():.3e} > {REF_MEAN_ABS}"
    return err.max().item()


def merge_reference(part_o, part_lse):
    """fp64 LSE merge of partials [parts, rows, dv] / [parts, rows] (the checker for merge tests)."""
    lse = part_lse.double()
    m = lse.max(dim=0).values
    m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    w = torch.exp(lse - m_safe)
    tot = w.sum(dim=0)
    o = (w.unsqueeze(-1) * part_o.double()).sum(dim=0) / torch.where(tot == 0, torch.ones_like(tot), tot).unsqueeze(-1)
    return o, m_safe + torch.log(tot)
