"""Fused gradient-bucket engine: all-reduce + 1/N scale (+ AdamW) in one sm_100a kernel.

Filled in by `attach_if_possible`; see `BucketEngine`.
"""
from __future__ import annotations


def attach_if_possible(reducer) -> bool:
    """Attach the fused bucket engine to `reducer` when its group can use it."""
    return False
