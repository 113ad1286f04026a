"""Tensor-parallel plumbing: process groups, symmetric memory, fused compute+collective ops."""
from .group import TPComm, init_distributed
