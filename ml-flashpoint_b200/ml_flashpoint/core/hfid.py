"""Human-friendly unique ids: ``<prefix>_<32 hex digits>`` (reference: core/hfid.py:19-39)."""

import uuid

_ALLOWED = frozenset("abcdefghijklmnopqrstuvwxyz0123456789")


def generate_hfid(prefix: str) -> str:
    if not prefix:
        raise ValueError("Prefix cannot be empty.")
    if not set(prefix) <= _ALLOWED:
        raise ValueError("Prefix must contain only lowercase alphanumeric characters.")
    return f"{prefix}_{uuid.uuid4().hex}"
