"""Helpers to load the golden FLCE vectors (see tests/golden/make_golden.py)."""

import ast
import glob
import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _all_names():
    return sorted(os.path.splitext(os.path.basename(p))[0] for p in glob.glob(os.path.join(GOLDEN_DIR, "*.npz")))


_PREFIXES = ("xent_", "jsd_", "sce_")


def golden_names():
    """Fused linear cross-entropy cases."""
    return [n for n in _all_names() if not n.startswith(_PREFIXES)]


def jsd_golden_names():
    """Fused linear JSD cases."""
    return [n for n in _all_names() if n.startswith("jsd_")]


def sce_golden_names():
    """Fused linear scaled cross-entropy cases."""
    return [n for n in _all_names() if n.startswith("sce_")]


def ce_golden_names():
    """Stand-alone cross-entropy cases (logits given)."""
    return [n for n in _all_names() if n.startswith("xent_")]


def load_golden(name):
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"), allow_pickle=False)
    rec = {k: z[k] for k in z.files if k != "meta"}
    meta = ast.literal_eval(str(z["meta"]))
    return rec, meta


def golden_kwargs(rec, meta):
    """Keyword arguments of the FLCE call that a golden record describes."""
    return dict(
        bias=None if "bias" not in rec else torch.from_numpy(rec["bias"]),
        ce_weight=None if "ce_weight" not in rec else torch.from_numpy(rec["ce_weight"]),
        ignore_index=meta["ignore_index"],
        lse_square_scale=meta.get("lse_square_scale", 0.0),
        label_smoothing=meta.get("label_smoothing", 0.0),
        reduction=meta.get("reduction", "mean"),
        softcap=meta.get("softcap"),
        use_token_scaling=meta.get("use_token_scaling", False),
    )


def golden_grad_output(rec, meta):
    if "token_grad" in rec:
        return torch.from_numpy(rec["token_grad"])
    if meta.get("grad_output") is not None:
        return torch.tensor(float(meta["grad_output"]))
    return None
