from speculators_b200.convert.mtp.converter import MTP_EXACT_REMAP, MTP_PREFIX_REMAP, MTPConverter

__all__ = ["MTP_EXACT_REMAP", "MTP_PREFIX_REMAP", "MTPConverter"]
