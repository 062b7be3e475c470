"""The range-checked library variant (-DHE_BOUNDS_CHECK=1): indices taken from device data are tested against their
limits; a violation is recorded in a status word and the access is clamped or skipped, never performed out of range.
Run in a child process, because a process loads one variant of the library."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

CHILD = r"""
import json, sys, torch
sys.path.insert(0, %r)
from hipengine_b200.core import native as N
from hipengine_b200.loading.synth import build_random_model
from hipengine_b200.models.config import TINY_HYBRID
from hipengine_b200.models.executor import HybridExecutor
from hipengine_b200.ops import kernels as K
out = {"variant_is_checked": N.bounds_status() is not None}
w = build_random_model(TINY_HYBRID, seed=0, device="cpu", std=0.05).to("cuda")
ex = HybridExecutor(w, device="cuda", max_slots=2, max_context=256)
prompt = torch.randint(0, TINY_HYBRID.vocab, (40,), generator=torch.Generator().manual_seed(1)).tolist()
lg = ex.prefill(0, prompt)
toks = [int(lg.argmax(-1))]
for i in range(4):
    lg = ex.forward_logits(0, [toks[-1]], len(prompt) + i)
    toks.append(int(lg.argmax(-1)))
torch.cuda.synchronize()
out["tokens"] = toks
out["clean_after_normal_run"] = N.bounds_status()
# a token id past the vocabulary: recorded, and the row is the embedding of id 0 instead of an out-of-range read
ids = torch.tensor([3, TINY_HYBRID.vocab + 7, 5], dtype=torch.int64, device="cuda")
e = torch.empty(3, TINY_HYBRID.hidden, device="cuda")
K.embed(ex.dw["token_embd.weight"], ids, e, 1.0)
e0 = torch.empty(1, TINY_HYBRID.hidden, device="cuda")
K.embed(ex.dw["token_embd.weight"], torch.zeros(1, dtype=torch.int64, device="cuda"), e0, 1.0)
torch.cuda.synchronize()
out["after_bad_token"] = N.bounds_status()
out["bad_row_is_row0"] = bool(torch.equal(e[1], e0[0]))
out["clean_after_reset"] = N.bounds_status()
print("RESULT " + json.dumps(out))
"""


def _run(variant):
    env = dict(os.environ)
    if variant:
        env["HE_NATIVE_VARIANT"] = variant
    else:
        env.pop("HE_NATIVE_VARIANT", None)
    r = subprocess.run([sys.executable, "-c", CHILD % str(ROOT)], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1]
    return json.loads(line[len("RESULT "):])


def test_checked_variant_records_out_of_range_indices_and_matches_product_build():
    from hipengine_b200.core import build as B
    if not B.lib_path("checked").exists():
        pytest.skip("checked variant not built (python -m hipengine_b200.core.build --variant=checked)")
    chk = _run("checked")
    assert chk["variant_is_checked"] is True
    assert chk["clean_after_normal_run"] == [0, 0, 0, 0]
    code, site, index, limit = chk["after_bad_token"]
    assert (code, site) == (2, 1) and limit == 2048 and index == 2048 + 7      # HE_ERR_BOUNDS at the embedding
    assert chk["bad_row_is_row0"] is True
    assert chk["clean_after_reset"] == [0, 0, 0, 0]
    prod = _run("")
    assert prod["variant_is_checked"] is False and prod["after_bad_token"] is None
    assert prod["tokens"] == chk["tokens"]
