from speculators_b200.convert.dflash.converter import DFlashConverter

__all__ = ["DFlashConverter"]
