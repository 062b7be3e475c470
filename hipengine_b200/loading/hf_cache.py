"""Local-only resolution of Hugging Face style model ids to GGUF files.  Never downloads.

``resolve_model_path("org/name")`` looks, in order, at: the string as a filesystem path; ``$HE_MODEL_DIR/org/name``
and ``$HE_MODEL_DIR/name``; the Hugging Face hub cache layout (``$HF_HOME/hub`` or ``~/.cache/huggingface/hub``):
``models--org--name/snapshots/<rev>/`` taking the revision named by ``refs/main`` when present, else the newest
snapshot.  A directory resolves to its GGUF files (multi-part ``-00001-of-0000N`` sets are kept in order).
Same policy as the reference (``hipengine/loading/hf_cache.py``; its API docs state models are resolved from local
caches only and nothing is fetched).
"""
from __future__ import annotations

import os
from pathlib import Path
from typing import List, Optional


class ModelNotFound(FileNotFoundError):
    pass


def _hub_dirs() -> List[Path]:
    out = []
    if os.environ.get("HF_HUB_CACHE"):
        out.append(Path(os.environ["HF_HUB_CACHE"]))
    if os.environ.get("HF_HOME"):
        out.append(Path(os.environ["HF_HOME"]) / "hub")
    out.append(Path.home() / ".cache" / "huggingface" / "hub")
    return out


def _snapshot_dir(repo_dir: Path, revision: Optional[str]) -> Optional[Path]:
    snaps = repo_dir / "snapshots"
    if not snaps.is_dir():
        return None
    if revision and (snaps / revision).is_dir():
        return snaps / revision
    ref = repo_dir / "refs" / (revision or "main")
    if ref.is_file():
        rev = ref.read_text().strip()
        if (snaps / rev).is_dir():
            return snaps / rev
    cands = [d for d in snaps.iterdir() if d.is_dir()]
    return max(cands, key=lambda d: d.stat().st_mtime) if cands else None


def gguf_files(path: Path, quant_hint: Optional[str] = None) -> List[Path]:
    if path.is_file():
        return [path]
    files = sorted(p for p in path.rglob("*.gguf") if "mmproj" not in p.name.lower())
    if quant_hint:
        hit = [p for p in files if quant_hint.lower() in p.name.lower()]
        files = hit or files
    if not files:
        return []
    # keep one multi-part set (or the single file) -- the first in name order
    stem = files[0].name.split("-00001-of-")[0] if "-of-" in files[0].name else None
    return [p for p in files if stem and p.name.startswith(stem)] if stem else [files[0]]


def resolve_model_path(model: str, revision: Optional[str] = None, quant_hint: Optional[str] = None) -> List[Path]:
    """GGUF file(s) for ``model`` found locally; raises ``ModelNotFound`` (never reaches for the network)."""
    p = Path(model).expanduser()
    if p.exists():
        files = gguf_files(p, quant_hint)
        if files:
            return files
        raise ModelNotFound(f"{model}: no GGUF file inside")
    roots = [Path(os.environ["HE_MODEL_DIR"])] if os.environ.get("HE_MODEL_DIR") else []
    for root in roots:
        for cand in (root / model, root / model.split("/")[-1]):
            if cand.exists():
                files = gguf_files(cand, quant_hint)
                if files:
                    return files
    if "/" in model:
        repo = "models--" + model.replace("/", "--")
        for hub in _hub_dirs():
            snap = _snapshot_dir(hub / repo, revision)
            if snap is not None:
                files = gguf_files(snap, quant_hint)
                if files:
                    return files
    raise ModelNotFound(f"{model}: not found locally (checked the path, HE_MODEL_DIR and the Hugging Face hub cache); "
                        f"models are never downloaded")
