from speculators_b200.proposals.base import TokenProposalConfig
from speculators_b200.proposals.greedy import GreedyTokenProposalConfig

__all__ = ["GreedyTokenProposalConfig", "TokenProposalConfig"]
