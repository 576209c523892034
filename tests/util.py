"""Comparison helpers shared by the parity tests."""
import torch

# Tolerances of the parity contract: routing integers bit-exact; values within rtol 1e-5 for
# fp32 and 1e-2 for bf16.  The absolute term is scaled to the tensor's RMS: a bf16 result carries
# the rounding of bf16 intermediates (activations, expert outputs), which is relative to the
# magnitude of the row it was accumulated from, not to each element.
RTOL = {torch.float32: 1e-5, torch.bfloat16: 1e-2}


def assert_close(actual, expected, dtype, what="", scale=1.0):
    a = actual.detach().float().cpu()
    e = expected.detach().float().cpu()
    assert a.shape == e.shape, f"{what}: shape {tuple(a.shape)} != {tuple(e.shape)}"
    assert torch.isfinite(a).all(), f"{what}: non-finite values"
    rtol = RTOL[dtype] * scale
    # absolute term per row (last dimension): rows of one tensor differ in scale by orders of
    # magnitude (gate weights, expert loads), and an element near zero inherits the rounding of
    # the row it was accumulated from
    rms = e.pow(2).mean(dim=-1, keepdim=True).sqrt() if e.dim() > 1 else e.pow(2).mean().sqrt()
    atol = rtol * rms.clamp_min(1e-30) * (10.0 if dtype == torch.float32 else 1.0)
    err = (a - e).abs()
    bound = atol + rtol * e.abs()
    bad = err > bound
    if bad.any():
        i = torch.argmax((err - bound).flatten())
        raise AssertionError(
            f"{what}: {int(bad.sum())}/{bad.numel()} elements outside rtol={rtol:g} (+ rtol x row rms); "
            f"worst actual={a.flatten()[i].item():.6g} expected={e.flatten()[i].item():.6g} "
            f"(rms of expected {e.pow(2).mean().sqrt().item():.4g})")


def rel_fro(actual, expected):
    a = actual.detach().double().cpu()
    e = expected.detach().double().cpu()
    return ((a - e).norm() / e.norm().clamp_min(1e-30)).item()
