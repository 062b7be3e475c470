"""Poison probe: every scratch buffer (activations, split-K partials, attention partials, argmax scratch) is filled
with 0xFF bytes -- NaN as a float, -1 as an integer -- between two runs of the same work; a kernel that reads scratch
it did not write this call would change the result or make it non-finite.  The check the reference makes with its
poison probe (``tests/_poison_probe.py:1-22``), used here in place of an initcheck tool."""
import pytest
import torch

from hipengine_b200.loading.synth import build_random_model
from hipengine_b200.models.config import TINY_DENSE, TINY_GEMMA4, TINY_HYBRID, TINY_HYBRID_MOE

pytestmark = pytest.mark.gpu


def _poison(ex) -> int:
    n = 0
    for t in list(ex.scratch.bufs.values()) + list(ex.scratch.retired):
        t.view(torch.uint8).fill_(0xFF)
        n += t.numel() * t.element_size()
    for name in ("am_v", "am_i"):
        t = getattr(ex, name, None)
        if isinstance(t, torch.Tensor):
            t.view(torch.uint8).fill_(0xFF)
    return n


def _run(ex, prompt, rows):
    """Prefill (tensor-core path), a few decode steps (GEMV path) and one packed step of `rows` rows (split-K path)."""
    from hipengine_b200.models.executor import make_batch
    out = []
    for s in range(ex.max_slots):
        ex.reset_slot(s)
    out.append(ex.prefill(0, prompt).clone())
    tok = int(out[-1].argmax(-1))
    for i in range(3):
        lg = ex.forward_logits(0, [tok], len(prompt) + i)
        out.append(lg.clone())
        tok = int(lg.argmax(-1))
    ex.prefill(1, prompt[: len(prompt) // 2])
    b = make_batch([(1, len(prompt) // 2, prompt[:rows])], ex.device)
    h = ex.forward(b)
    out.append(h.clone())
    return out


@pytest.mark.parametrize("cfg", [TINY_HYBRID, TINY_DENSE, TINY_HYBRID_MOE, TINY_GEMMA4], ids=["hybrid", "dense", "moe", "gemma4"])
def test_outputs_do_not_depend_on_scratch_contents(cfg):
    from hipengine_b200.models import make_executor
    from hipengine_b200.ops import kernels as K
    w = build_random_model(cfg, seed=2, std=0.05).to("cuda")
    ex = make_executor(w, device="cuda", max_slots=2, max_context=512)
    ex.scratch.canaries = True                 # canary words behind every scratch buffer, checked at the end
    prompt = torch.randint(0, cfg.vocab, (200,), generator=torch.Generator().manual_seed(4)).tolist()
    first = _run(ex, prompt, rows=24)
    torch.cuda.synchronize()
    assert _poison(ex) > 0
    second = _run(ex, prompt, rows=24)
    torch.cuda.synchronize()
    K.check_status()
    for a, b in zip(first, second):
        assert torch.isfinite(b).all()
        assert torch.equal(a, b)
    assert len(ex.scratch._raw) > 5 and ex.scratch.check_canaries() == []      # nothing wrote past its extent
