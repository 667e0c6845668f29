"""Reference arm of bench.py: runs the unmodified reference package installed under baseline/_ref."""
from __future__ import annotations


def run(args) -> dict:
    return {"impl": "reference", "unavailable": "reference arm not wired up yet"}
