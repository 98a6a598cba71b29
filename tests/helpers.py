"""Shared helpers for the test-suite (fixture decoding, error metrics)."""
import numpy as np
import torch

GOLDEN_FN_CASES = ["v2_tiny", "v3_tiny", "v3_alltaps_d8", "v3_d64", "v2_hd80", "v2_fp32"]
GOLDEN_MODULE_CASES = ["la43", "la45"]


def bf16_from_bits(a):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def load_case(golden, name):
    """Decode one golden case into torch tensors.  Inputs are fp32 (bf16-valued when the
    reference was fed bf16); `bf16` tells which."""
    bf16 = bool(int(golden[f"{name}/bf16_inputs"]))
    case = {"bf16": bf16, "offsets": [int(x) for x in golden[f"{name}/offsets"]],
            "shape": tuple(int(x) for x in golden[f"{name}/shape"])}
    for key in golden.files:
        if not key.startswith(name + "/"):
            continue
        nm = key.split("/", 1)[1]
        if nm in ("shape", "offsets", "bf16_inputs"):
            continue
        arr = golden[key]
        if bf16 and nm in ("q", "k", "v", "dout"):
            case[nm] = bf16_from_bits(arr).float()
        else:
            case[nm] = torch.from_numpy(arr.copy())
    return case


def rel_inf(x, ref):
    """||x - ref||_inf / ||ref||_inf, the per-tensor relative error used for the fp32 gate."""
    x, ref = x.double(), ref.double()
    return ((x - ref).abs().max() / ref.abs().max().clamp_min(1e-30)).item()


def max_abs(x, ref):
    return (x.double() - ref.double()).abs().max().item()
