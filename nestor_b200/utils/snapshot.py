"""Source snapshot of a run: the code that produced a checkpoint, zipped beside it.

``snapshot_sources(root, out)`` writes ``out`` (``.zip``) with every file under ``root`` that is source rather than
data or build output. What counts as "not source" is a list of directory names pruned during the walk and of file
name patterns skipped one by one; both can be replaced. Kernels' build products (``_C``, ``*.o``, ``*.so``) stay out:
they are rebuilt from the ``.cu`` files, which are in. Behaviour follows the reference's run-directory snapshot
(``nestor/utils/repo_snapshot.py:68-110``, enabled per experiment by ``save_source_snapshot``).
"""

from __future__ import annotations

import fnmatch
import zipfile
from pathlib import Path

PRUNED_DIRS = frozenset({
    ".git", ".cursor", ".claude", "__pycache__", ".venv", "venv", ".mypy_cache", ".ruff_cache", ".pytest_cache",
    ".hypothesis", "data", "logs", "tmp", "outputs", "checkpoints", "wandb", "_C", "_ref", "build",
})
SKIPPED_FILES = ("*.pyc", "*.pyo", "*.pt", "*.pth", "*.ckpt", "*.zip", "*.tar", "*.tar.gz", "*.h5", "*.hdf5", "*.bin",
                 "*.o", "*.so", "*.a", "*.ncu-rep", ".env", ".DS_Store")


def _scratch_dirs(root: Path) -> set[str]:
    """Top-level directories that the repository's own ignore file lists: scratch output is not source."""

    ignore = root / ".gitignore"
    if not ignore.is_file():
        return set()
    return {line.strip().strip("/") for line in ignore.read_text().splitlines()
            if line.strip().endswith("/") and "*" not in line and not line.startswith("#")}


def source_files(root: Path, pruned_dirs=PRUNED_DIRS, skipped_files=SKIPPED_FILES) -> list[Path]:
    """Relative paths of the files a snapshot of ``root`` contains, sorted (the walk never enters a pruned directory)."""

    root = Path(root)
    pruned_dirs = set(pruned_dirs) | _scratch_dirs(root)
    out: list[Path] = []
    stack = [root]
    while stack:
        here = stack.pop()
        try:
            entries = sorted(here.iterdir())
        except OSError:
            continue
        for e in entries:
            if e.is_symlink():
                continue
            if e.is_dir():
                if e.name not in pruned_dirs and not e.name.endswith(".egg-info"):
                    stack.append(e)
            elif not any(fnmatch.fnmatch(e.name, pat) for pat in skipped_files):
                out.append(e.relative_to(root))
    return sorted(out)


def snapshot_sources(root: Path, out: Path, pruned_dirs=PRUNED_DIRS, skipped_files=SKIPPED_FILES,
                     max_file_bytes: int = 8 << 20) -> Path:
    """Zip the sources under ``root`` into ``out`` (suffix forced to ``.zip``); returns the path written.

    Files larger than ``max_file_bytes`` are left out (a stray dump in the tree must not bloat every run directory).
    """

    root, out = Path(root), Path(out).with_suffix(".zip")
    out.parent.mkdir(parents=True, exist_ok=True)
    with zipfile.ZipFile(out, "w", zipfile.ZIP_DEFLATED) as zf:
        for rel in source_files(root, pruned_dirs, skipped_files):
            f = root / rel
            try:
                if f.stat().st_size <= max_file_bytes:
                    zf.write(f, rel.as_posix())
            except OSError:
                pass
    return out
