"""``Precision`` (iron/common/declare/precision.py:9-24)."""

from iron_b200.lm.config import Precision  # noqa: F401
