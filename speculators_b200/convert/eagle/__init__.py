from speculators_b200.convert.eagle.eagle3_converter import Eagle3Converter

__all__ = ["Eagle3Converter"]
