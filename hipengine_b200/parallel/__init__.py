"""Multi-GPU execution: one process per GPU, ``torch.distributed`` for the plumbing, own kernels over peer
memory for the latency-critical reductions (``csrc/comm.cu``)."""
from .groups import DistContext, init_distributed, max_over_ranks  # noqa: F401
from .sharding import TPPlan, shard_weights  # noqa: F401
