from .CommSplits import CommSplits  # noqa: F401
from .CommBuffer import CommBuffer, CommBufferForQuantization  # noqa: F401
from .DistributedGraph import DistributedGraph, DistributedGraphForPre  # noqa: F401
from .graph_builder import build_distributed_graph, order_nodes_by_degree, partition_edges  # noqa: F401
from .pre_post import build_distributed_graph_pre_post, decide_pre_or_post_aggr, min_vertex_cover  # noqa: F401
from .DataLoader import load_data, save_partition  # noqa: F401
