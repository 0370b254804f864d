from speculators_b200.verifier.model import RandomVerifier, write_random_verifier_stub
from speculators_b200.verifier.tp import TensorParallelVerifier

__all__ = ["RandomVerifier", "TensorParallelVerifier", "write_random_verifier_stub"]
