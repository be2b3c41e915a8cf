"""`pack_solution_from_files` of the stand-in: a solution is the text of its files (kbench packs
inside a temporary directory that is gone before the benchmark runs, kbench/flashinfer.py:112-113)."""
from __future__ import annotations

from pathlib import Path

from . import Solution


def pack_solution_from_files(path, spec, name, definition, author):
    root = Path(path)
    files = {str(p.relative_to(root)): p.read_text() for p in sorted(root.rglob("*")) if p.is_file()}
    if spec.entry_point.split("::")[0] not in files:
        raise FileNotFoundError(f"entry file {spec.entry_point} is not among the packed sources")
    return Solution(name=name, definition=definition, author=author, spec=spec, files=files)
