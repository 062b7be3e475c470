"""The user documentation names real things: every `--flag` in docs/API.md and docs/SERVING.md exists in a parser,
every `LLM` method listed exists, every file path mentioned in the docs and profiles exists, and the examples run."""
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _read(rel):
    with open(os.path.join(ROOT, rel), encoding="utf-8") as f:
        return f.read()


def _all_flags():
    from hipengine_b200.server.__main__ import build_parser
    flags = set()
    for a in build_parser()._actions:
        flags.update(a.option_strings)
    src = _read("hipengine_b200/server/router.py") + _read("hipengine_b200/benchmark/serving_load.py") + \
        _read("hipengine_b200/chat_cli.py") + _read("bench.py") + _read("hipengine_b200/core/build.py") + \
        _read("hipengine_b200/benchmark/micro.py") + _read("hipengine_b200/parallel/selftest.py")
    flags.update(re.findall(r'"(--[a-z][a-z0-9-]*)"', src))
    flags.update(re.findall(r"(--variant)=", src))
    return flags


def test_flags_named_in_the_docs_exist():
    flags = _all_flags()
    external = {"--nnodes", "--nproc-per-node", "--master-addr", "--master-port", "--no-build-isolation", "--suite",
                "--help", "--set", "--clock-control", "--metrics-only"}
    for doc in ("docs/API.md", "docs/SERVING.md", "docs/TESTING.md", "docs/KERNELS.md", "README.md"):
        named = set(re.findall(r"(?<![\w-])(--[a-z][a-z0-9-]+)", _read(doc)))
        missing = sorted(f for f in named if f not in flags and f not in external)
        assert not missing, (doc, missing)


def test_llm_methods_named_in_the_api_guide_exist():
    from hipengine_b200.llm import LLM
    text = _read("docs/API.md")
    block = text[text.index("`LLM` methods:"):text.index("Every output carries")]
    names = re.findall(r"`([a-z_]+)`", block)
    assert len(names) >= 20
    missing = [n for n in names if not hasattr(LLM, n)]
    assert not missing, missing


def test_paths_named_in_docs_and_profiles_exist():
    docs = ["README.md"] + [os.path.join("docs", f) for f in os.listdir(os.path.join(ROOT, "docs")) if f.endswith(".md")]
    docs += [os.path.join("profiles", f) for f in os.listdir(os.path.join(ROOT, "profiles")) if f.endswith(".md")]
    pat = re.compile(r"`((?:hipengine_b200|tests|docs|profiles|csrc|server|models|generation|speculative|kvcache|loading|"
                     r"parallel|ops|ref|quant|core|utils|benchmark)/[A-Za-z0-9_./-]+\.(?:py|cuh|cu|cpp|h|md|sh))(?![A-Za-z0-9_])")
    missing = []
    for d in docs:
        for rel in set(pat.findall(_read(d))):
            cands = [rel, os.path.join("hipengine_b200", rel), os.path.join("hipengine_b200", "csrc", os.path.basename(rel))]
            if not any(os.path.exists(os.path.join(ROOT, c)) for c in cands):
                missing.append((d, rel))
    assert not missing, missing


@pytest.mark.parametrize("script", ["docs/examples/offline_generate.py"])
def test_examples_run(script):
    env = dict(os.environ, PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, os.path.join(ROOT, script)], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "prompt tokens" in r.stdout and "max_new_tokens" in r.stdout
