"""``suffix_scan_pullbacks``: K interface Jacobian transposes [B, K, R, R] -> the K + 1 suffix products [B, K + 1, R, R]
(reference cuda/interface/__init__.py:33-39)."""
from ...ops import suffix_scan_pullbacks

__all__ = ["suffix_scan_pullbacks"]
