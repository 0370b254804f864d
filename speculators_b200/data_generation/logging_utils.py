"""Console logger for the data pipeline: section banners, aligned config dumps and
status glyphs over the standard ``logging`` module (colour only on a TTY).

Reference surface: src/speculators/data_generation/logging_utils.py:11 (PipelineLogger).
"""

from __future__ import annotations

import logging
import sys
from typing import Any

__all__ = ["PipelineLogger"]

_RESET = "\033[0m"
_STYLES = {"banner": "\033[1;34m", "bold": "\033[1m", "dim": "\033[2m", "ok": "\033[92m", "warn": "\033[93m", "err": "\033[91m"}


class PipelineLogger:
    def __init__(self, name: str = ""):
        self.logger = logging.getLogger(name)
        self.use_colors = sys.stdout.isatty()

    def _paint(self, text: str, style: str) -> str:
        return f"{_STYLES[style]}{text}{_RESET}" if self.use_colors else text

    def section(self, title: str) -> None:
        rule = self._paint("━" * (len(title) + 4), "banner")
        for line in (rule, self._paint(f"  {title}", "banner"), rule):
            self.logger.info("%s", line)

    def subsection(self, title: str) -> None:
        self.logger.info("\n%s", self._paint(f"▸ {title}", "bold"))

    def config(self, config_dict: dict[str, Any]) -> None:
        if not config_dict:
            return
        width = max(len(str(k)) for k in config_dict)
        for key, value in config_dict.items():
            self.logger.info("  %s │ %s", self._paint(str(key).ljust(width), "dim"), value)

    def info(self, message: str) -> None:
        self.logger.info("  %s", message)

    def success(self, message: str) -> None:
        self.logger.info("  %s %s", self._paint("✓", "ok"), message)

    def warning(self, message: str) -> None:
        self.logger.warning("  %s %s", self._paint("⚠", "warn"), message)

    def error(self, message: str) -> None:
        self.logger.error("  %s %s", self._paint("✗", "err"), message)

    def debug(self, message: str) -> None:
        self.logger.debug("%s", self._paint(f"  {message}", "dim"))
