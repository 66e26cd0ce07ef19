from .CommSplits import CommSplits  # noqa: F401
from .CommBuffer import CommBuffer, CommBufferForQuantization  # noqa: F401
from .DistributedGraph import DistributedGraph, DistributedGraphForPre  # noqa: F401
from .graph_builder import build_distributed_graph, partition_edges  # noqa: F401
