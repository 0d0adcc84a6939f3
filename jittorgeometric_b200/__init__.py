"""jittorgeometric_b200: B200-native (sm_100a) message-passing operators behind the
``jittor_geometric.ops`` API.  Importing this package does not load the CUDA
library; the first operator call does, and raises if it has not been built."""
from .data import CSC, CSR  # noqa: F401
from .ops import *  # noqa: F401,F403
from . import dist, nn, ops, partition, sampling, synth  # noqa: F401
from .sampling import csctocsr, from_nodes, getweight, gpuinitco, sampleprocessing, to_nodes  # noqa: F401
from .dist import DistSpmm  # noqa: F401

__version__ = "0.1.0"
