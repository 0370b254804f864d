"""Greedy chain proposal: the draft emits ``speculative_tokens`` tokens in one
chain; a token is accepted if it is within the verifier's top
``verifier_accept_k`` (and within ``accept_tolerance`` log-likelihood of the
top-1 when k > 1).  Parity: src/speculators/proposals/greedy.py:24-73 (field
names, defaults 5 / 1 / 0.0 and lower bounds are what vLLM reads back)."""

from typing import Literal

from pydantic import Field

from speculators_b200.proposals.base import TokenProposalConfig

__all__ = ["GreedyTokenProposalConfig"]


@TokenProposalConfig.register("greedy")
class GreedyTokenProposalConfig(TokenProposalConfig):
    proposal_type: Literal["greedy"] = "greedy"
    speculative_tokens: int = Field(default=5, ge=1)
    verifier_accept_k: int = Field(default=1, ge=1)
    accept_tolerance: float = Field(default=0.0, ge=0.0)
