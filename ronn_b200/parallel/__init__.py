"""Tensor-parallel plumbing: process groups, symmetric memory, fused compute+collective ops."""
from .group import TPComm, init_distributed


def make_comm(kind: str, device):
    """Communicator of the tensor-parallel runners.  ``"nccl"``: library collectives (the baseline).  ``"fused"``:
    in-kernel NVLink exchange over symmetric memory; raises when the symmetric-memory communicator cannot be built
    (a caller that asked for the fused kernels must not silently measure the library path)."""
    if kind == "nccl":
        return TPComm()
    if kind != "fused":
        raise ValueError(f"unknown communicator kind '{kind}' (expected 'fused' or 'nccl')")
    from ..api.errors import ProviderError
    try:
        from .symm import FusedComm
    except ImportError as e:
        raise ProviderError(f"the fused tensor-parallel communicator is unavailable: {e}") from e
    return FusedComm(device)
