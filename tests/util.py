"""Helpers shared by the tests: raw-bit views between numpy (oracle side) and torch (device side),
and the tolerance rules the parity tests apply."""
import numpy as np
import torch

import oracle as O

TORCH_OF = {O.FP32: torch.float32, O.FP16: torch.float16, O.BF16: torch.bfloat16,
            O.E4M3: torch.float8_e4m3fn, O.E5M2: torch.float8_e5m2}
FWD_DTS = [O.FP32, O.FP16, O.BF16, O.E4M3, O.E5M2]
BWD_DTS = [O.FP32, O.FP16, O.BF16]
PAIRS = [(O.FP32, O.FP32), (O.FP16, O.FP16), (O.BF16, O.BF16), (O.E4M3, O.FP16), (O.E4M3, O.BF16), (O.E5M2, O.FP16), (O.E5M2, O.BF16)]
DT_NAME = {O.FP32: "fp32", O.FP16: "fp16", O.BF16: "bf16", O.E4M3: "fp8e4m3", O.E5M2: "fp8e5m2"}
# one unit in the last place, relative, of each type (used to scale tolerances)
ULP_REL = {O.FP32: 2.0 ** -23, O.FP16: 2.0 ** -10, O.BF16: 2.0 ** -7, O.E4M3: 2.0 ** -3, O.E5M2: 2.0 ** -2}


def to_dev(a: np.ndarray, dt: int, device="cuda") -> torch.Tensor:
    """numpy raw-bit array (oracle convention) -> torch tensor of the matching dtype on `device`."""
    if dt == O.FP32:
        return torch.from_numpy(np.ascontiguousarray(a)).to(device)
    if dt in (O.FP16, O.BF16):
        return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).to(device).view(TORCH_OF[dt])
    return torch.from_numpy(np.ascontiguousarray(a)).to(device).view(TORCH_OF[dt])


def to_host(t: torch.Tensor, dt: int) -> np.ndarray:
    """torch tensor -> numpy raw-bit array (oracle convention)."""
    t = t.detach().contiguous().cpu()
    if dt == O.FP32:
        return t.numpy()
    if dt in (O.FP16, O.BF16):
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.view(torch.uint8).numpy()


def f32(a: np.ndarray, dt: int) -> np.ndarray:
    return O.to_f32(np.ascontiguousarray(a), dt)


def check_lowp(got_bits, ref_bits, dt, what, rel=1e-2, scale=None, max_ulps=None):
    """The low-precision output rule: |got - ref| <= rel * max(|ref|, scale), where `scale` defaults to
    the RMS of the reference tensor (an absolute floor for elements that cancel to ~0). fp32 tensors use
    rel = 1e-5 unless told otherwise. Returns the fraction of bit-identical elements."""
    got, ref = f32(got_bits, dt).astype(np.float64), f32(ref_bits, dt).astype(np.float64)
    assert got.shape == ref.shape, what
    finite = np.isfinite(ref)
    assert np.array_equal(np.isfinite(got), finite), f"{what}: non-finite pattern differs"
    if scale is None:
        scale = float(np.sqrt(np.mean(ref[finite] ** 2))) if finite.any() else 0.0
    tol = rel * np.maximum(np.abs(ref), scale)
    err = np.abs(got - ref)
    bad = finite & (err > tol)
    if bad.any():
        i = np.unravel_index(np.argmax(np.where(finite, err - tol, -np.inf)), err.shape)
        raise AssertionError(f"{what}: {int(bad.sum())}/{bad.size} elements outside {rel:g} rel "
                             f"(worst at {i}: got {got[i]!r}, ref {ref[i]!r}, scale {scale:g})")
    return float(np.mean(np.asarray(got_bits) == np.asarray(ref_bits)))


def check_f32(got, ref, what, rel=1e-5, scale=None):
    """fp32 statistics rule: |got - ref| <= rel * max(|ref|, scale)."""
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    s = 0.0 if scale is None else scale
    tol = rel * np.maximum(np.abs(ref), s)
    err = np.abs(got - ref)
    if (err > tol).any():
        i = int(np.argmax(err - tol))
        raise AssertionError(f"{what}: {int((err > tol).sum())}/{err.size} outside {rel:g} rel (worst idx {i}: got {got.flat[i]!r}, ref {ref.flat[i]!r})")
