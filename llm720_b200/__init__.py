"""B200-native (sm_100a) PEER forward: a drop-in for the PEER layer of
wrmedford/llm720 backed by hand-written CUDA kernels behind a C ABI."""
from .peer import PEER, PeerOp  # noqa: F401
from .functional import peer_forward, peer_forward_cutlass  # noqa: F401

__all__ = ["PEER", "PeerOp", "peer_forward", "peer_forward_cutlass"]
