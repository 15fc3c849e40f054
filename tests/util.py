"""Helpers shared by the tests: the package loader and NumPy <-> torch moves
that keep bf16 / uint32 bit patterns intact."""
import os
import sys

import ml_dtypes
import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from __graft_entry__ import load_package  # noqa: E402

bf16 = ml_dtypes.bfloat16


def pkg():
    return load_package()


def dev(a, device="cuda"):
    """NumPy array -> torch tensor on the device, bit for bit."""
    import torch
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint32:
        return torch.from_numpy(a.view(np.int32)).to(device)
    if a.dtype == bf16:
        return torch.from_numpy(a.view(np.int16)).to(device).view(torch.bfloat16)
    return torch.from_numpy(a).to(device)


def host(t):
    """torch tensor -> NumPy, bf16 kept as ml_dtypes.bfloat16."""
    import torch
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(bf16)
    return t.numpy()


def dev_params(params, device="cuda"):
    """The oracle's NumPy decoder pytree moved to the device."""
    def mv(v):
        return {k: dev(x, device) for k, x in v.items()} if isinstance(v, dict) else dev(v, device)
    out = {k: mv(v) for k, v in params.items() if k != "layers"}
    out["layers"] = [{k: mv(v) for k, v in lp.items()} for lp in params["layers"]]
    return out


def rel_rms_err(got, want):
    got = np.asarray(got).astype(np.float64)
    want = np.asarray(want).astype(np.float64)
    rms = np.sqrt(np.mean(want * want))
    return float(np.max(np.abs(got - want)) / max(rms, 1e-30))
