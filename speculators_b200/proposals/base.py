"""Base config of a token-proposal method (how draft tokens are produced and
accepted at serving time).  Parity: src/speculators/proposals/base.py:32-39."""

from typing import ClassVar

from pydantic import Field

from speculators_b200.utils import PydanticClassRegistryMixin

__all__ = ["TokenProposalConfig"]


class TokenProposalConfig(PydanticClassRegistryMixin):
    schema_discriminator: ClassVar[str] = "proposal_type"

    proposal_type: str = Field(description="registered name of the proposal method")
