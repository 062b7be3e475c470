"""Speculative decoding: contracts, transaction stages, the exact sampling law, planner, serving admission and the
NextN/MTP chain cycle on the GPU executor."""
from .contracts import SpecCycleResult, SpeculativeCapability  # noqa: F401
from .policy import plan_draft_depth  # noqa: F401
from .sampling import (acceptance_probability, residual_distribution,  # noqa: F401
                       sampled_accept_from_distributions)
from .serving import MTPServingDecision, resolve_mtp_serving_plan  # noqa: F401
from .transaction import SpecTransaction, Stage, TransactionError  # noqa: F401
