"""Ring (context-parallel) execution of the VSA path."""
from __future__ import annotations


def ring_attention(q, k, v, gate, layout, *, scale=None):
    raise NotImplementedError("ring execution is being built")
