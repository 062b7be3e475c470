"""In-tree build of the sm_100a kernel library and the native host runtime.

Every ``csrc/*.cu`` / ``csrc/*.cpp`` file is compiled with ``nvcc -gencode
arch=compute_100a,code=sm_100a -lineinfo`` into an object file and linked into
one shared library next to the package (``hipengine_b200/_native/libhe_b200.so``).
Objects are rebuilt only when the sha256 of (source bytes + included headers +
flags + compiler version) changes -- the same content-hash idea as the
reference's JIT cache (``hipengine/core/build.py:29-66,212-420``), except the
artefacts stay in-tree so a snapshot of the repository carries them, and no
compiler is ever invoked implicitly at import time on a GPU box.
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import Dict, List, Optional, Sequence

PKG_ROOT = Path(__file__).resolve().parent.parent
CSRC = PKG_ROOT / "csrc"
OUT_DIR = PKG_ROOT / "_native"
LIB_NAME = "libhe_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def nvcc_path() -> Optional[str]:
    for cand in (os.environ.get("HE_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    return None


def _compiler_version(nvcc: str) -> str:
    try:
        return subprocess.run([nvcc, "--version"], capture_output=True, text=True, check=True).stdout.strip()
    except Exception:
        return "unknown"


def sources() -> List[Path]:
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cpp")))


def _headers() -> List[Path]:
    return sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")))


def _key(src: Path, flags: Sequence[str], cver: str) -> str:
    h = hashlib.sha256()
    h.update(src.read_bytes())
    for hd in _headers():
        h.update(hd.name.encode())
        h.update(hd.read_bytes())
    h.update(" ".join(flags).encode())
    h.update(cver.encode())
    return h.hexdigest()


def variant() -> str:
    """Name of the library variant in use: '' (the product) or e.g. 'checked' (``HE_NATIVE_VARIANT``)."""
    return os.environ.get("HE_NATIVE_VARIANT", "").strip()


# extra compiler flags of the named variants
VARIANT_FLAGS = {
    # every index taken from device data is range-checked; a violation records a code in the bounds word
    # (he_bounds_status) and skips the access instead of performing it
    "checked": ["-DHE_BOUNDS_CHECK=1"],
    # role cycle counters in the quantised GEMM (he_gemm_q_debug_counters)
    "prof": ["-DHE_WQ_PROFILE=1"],
}


def lib_path(name: Optional[str] = None) -> Path:
    v = variant() if name is None else name
    return OUT_DIR / (LIB_NAME if not v else LIB_NAME.replace(".so", f"_{v}.so"))


def build_plan(extra_flags: Sequence[str] = ()) -> Dict[str, object]:
    """Dry-run description of what ``build`` would compile (used by tests)."""
    nvcc = nvcc_path()
    flags = list(NVCC_FLAGS) + list(extra_flags)
    return {"nvcc": nvcc, "flags": flags, "sources": [str(s) for s in sources()], "output": str(lib_path())}


def build(verbose: bool = False, force: bool = False, extra_flags: Sequence[str] = (), jobs: int = 0,
          name: str = "") -> Path:
    """Compile every source for sm_100a and link ``libhe_b200.so`` (or the variant ``libhe_b200_<name>.so`` with the
    variant's flags plus ``extra_flags``).  Returns the library path."""
    nvcc = nvcc_path()
    if nvcc is None:
        raise RuntimeError("nvcc not found; set HE_NVCC or install the CUDA toolkit")
    OUT_DIR.mkdir(parents=True, exist_ok=True)
    obj_dir = OUT_DIR / ("obj" if not name else f"obj_{name}")
    obj_dir.mkdir(exist_ok=True)
    flags = list(NVCC_FLAGS) + list(VARIANT_FLAGS.get(name, [])) + list(extra_flags)
    cver = _compiler_version(nvcc)
    manifest_path = OUT_DIR / ("manifest.json" if not name else f"manifest_{name}.json")
    try:
        manifest = json.loads(manifest_path.read_text())
    except Exception:
        manifest = {}
    srcs = sources()
    todo = []
    objs = []
    for s in srcs:
        obj = obj_dir / (s.name + ".o")
        objs.append(obj)
        k = _key(s, flags, cver)
        if force or manifest.get(s.name) != k or not obj.exists():
            todo.append((s, obj, k))

    def compile_one(item):
        s, obj, k = item
        cmd = [nvcc] + flags + ["-I", str(CSRC), "-c", str(s), "-o", str(obj)]
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {s.name}:\n{r.stdout}\n{r.stderr}")
        return s.name, k

    if todo:
        with ThreadPoolExecutor(max_workers=jobs or min(8, os.cpu_count() or 4)) as ex:
            for src_name, k in ex.map(compile_one, todo):
                manifest[src_name] = k
    lib = lib_path(name)
    link_key = hashlib.sha256(("".join(manifest.get(s.name, "") for s in srcs)).encode()).hexdigest()
    if todo or not lib.exists() or manifest.get("__link__") != link_key:
        cmd = [nvcc, "-shared", "-o", str(lib)] + [str(o) for o in objs] + ["-Xcompiler", "-fPIC"]
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        manifest["__link__"] = link_key
    manifest_path.write_text(json.dumps(manifest, indent=1, sort_keys=True))
    return lib


if __name__ == "__main__":
    names = [a.split("=", 1)[1] for a in sys.argv if a.startswith("--variant=")]
    p = build(verbose="-v" in sys.argv, force="--force" in sys.argv, name=names[0] if names else "")
    print(p)
