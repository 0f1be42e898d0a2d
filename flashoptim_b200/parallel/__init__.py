"""NVLink peer-memory data path: symmetric buffers, flag protocol, and the DDP /
FSDP2 integrations whose collectives are fused into the optimizer kernels."""

from .ddp import FusedDDPState, fuse_ddp_allreduce
from .fsdp import FusedFSDPState, enable_fused_fsdp, tuned_options
from .symm import CommTimeoutError, PeerGradients, PeerGroup, SymmBuffer

__all__ = [
    "PeerGroup", "SymmBuffer", "PeerGradients", "CommTimeoutError", "fuse_ddp_allreduce", "FusedDDPState",
    "enable_fused_fsdp", "FusedFSDPState", "tuned_options",
]
