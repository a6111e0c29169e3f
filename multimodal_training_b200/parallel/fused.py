"""Fused compute+collective paths over peer memory (attached to the trainers when available)."""
from __future__ import annotations


def try_create(mesh, config):
    """Returns ``(heap, fused)`` or ``(None, None)`` when peer memory cannot be set up."""
    return None, None
