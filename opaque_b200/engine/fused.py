"""Placeholder replaced below by the fused engine."""
_ACTIVE = None


def current_capture():
    return _ACTIVE
