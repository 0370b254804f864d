from speculators_b200.verifier.model import RandomVerifier, write_random_verifier_stub

__all__ = ["RandomVerifier", "write_random_verifier_stub"]
