"""Communicator factory for the tensor-parallel decoder."""
from __future__ import annotations

import torch

from .group import TPComm


def make_comm(kind: str, device: torch.device):
    """``"nccl"``: library collectives (baseline).  ``"fused"``: in-kernel NVLink exchange over symmetric memory."""
    if kind == "fused":
        try:
            from .symm import FusedComm
        except ImportError:
            return TPComm()
        return FusedComm(device)
    return TPComm()
