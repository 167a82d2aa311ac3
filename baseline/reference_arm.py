"""Reference arm of the benchmark: runs the unmodified reference package installed under ``baseline/_ref``."""

from __future__ import annotations


def run_reference(cli, spec: dict, repo_root: str):
    return {"impl": "reference", "unavailable": "reference arm is not wired up yet"}
