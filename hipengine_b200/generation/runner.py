"""Model runners: the scheduler-facing adapters over a model executor.

The engine loop talks to a runner through a small protocol (the role of the reference's
``EngineLoopRunner``, ``hipengine/generation/engine_loop.py:420-488``, implemented there by
``Qwen35GGUFResidentModelRunner``, ``hipengine/generation/qwen35_gguf.py:7133-13320``):
``admit`` (slot + KV pages + prefix-cache match), ``prefill`` (chunked, packed), ``decode`` (one step for all
resident rows), ``release``.  Two runners exist: ``CpuReferenceRunner`` (fp32 reference forward; the
"cpu_reference backend" used for correctness runs and host-only tests) and ``GpuRunner`` (sm_100a executor,
decode graphs, paged pool, radix prefix cache with recurrent-state snapshots).
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from ..config import EngineConfig
from ..kvcache.pool import PagePool, PoolExhausted
from ..kvcache.radix import PrefixCompatibilityKey, RadixCache
from . import sampling as S
from .scheduler import GenerationAdmissionRejected, RequestState
from .types import TokenLogprob


class ExecutionFailure(RuntimeError):
    """A contained failure: only ``request_ids`` are affected; the engine keeps serving the others.

    ``mutation`` says how far device state for those requests got: none | partial | committed | unknown
    (``hipengine/generation/engine_loop.py:301-340``).
    """

    def __init__(self, request_ids: Sequence[int], phase: str, message: str, mutation: str = "unknown"):
        super().__init__(message)
        self.request_ids = list(request_ids)
        self.phase = phase
        self.mutation = mutation


class BaseRunner:
    eos_token_id: Optional[int] = None
    vocab: int = 0
    max_slots: int = 1
    max_context: int = 0
    supports_mtp: bool = False

    # -- sampling shared by both runners ------------------------------------------------------------
    def _row_processors(self, rs: RequestState) -> Dict[str, Any]:
        req = rs.req
        suppress = list(req.suppress_token_ids)
        eos = req.eos_token_id if req.eos_token_id is not None else self.eos_token_id
        if eos is not None and (len(rs.generated) < req.min_tokens or (rs.thinking and rs.thinking.suppress_eos())
                                or req.ignore_eos and False):
            suppress.append(eos)
        bias = list(req.logit_bias)
        if rs.thinking is not None:
            b = rs.thinking.close_bias()
            if b > 0 and rs.thinking.close_ids:
                bias.append((rs.thinking.close_ids[0], b))
        mask = None
        if rs.grammar is not None and not rs.grammar.dead() and not (rs.thinking is not None and rs.thinking.thinking):
            mask = rs.grammar.allowed_mask()
            if mask.shape[0] != self.vocab:       # tokenizer and model vocabularies may differ in padding
                full = torch.zeros(self.vocab, dtype=torch.bool)
                full[:min(self.vocab, mask.shape[0])] = mask[:self.vocab]
                mask = full
        return dict(logit_bias=bias, history=rs.generated, prompt=req.prompt_token_ids,
                    repetition_penalty=req.repetition_penalty, presence_penalty=req.presence_penalty,
                    frequency_penalty=req.frequency_penalty, suppress=suppress, allowed_mask=mask)

    def _needs_processing(self, rs: RequestState) -> bool:
        req = rs.req
        return bool(req.logit_bias or req.suppress_token_ids or req.repetition_penalty != 1.0
                    or req.presence_penalty != 0.0 or req.frequency_penalty != 0.0
                    or len(rs.generated) < req.min_tokens or rs.grammar is not None
                    or (rs.thinking is not None and (rs.thinking.suppress_eos() or rs.thinking.close_bias() > 0)))

    def sample_host(self, rs: RequestState, logits: torch.Tensor) -> Tuple[int, Optional[TokenLogprob]]:
        """Full host sampler law on one logits row (CPU tensor or CUDA tensor)."""
        req = rs.req
        if rs.forced:
            tok = rs.forced.pop()
            lp = None
            if req.logprobs:
                lp = TokenLogprob(tok, S.token_logprob(logits, tok, req.temperature or 1.0),
                                  tuple(S.top_logprobs(logits, req.top_logprobs, req.temperature or 1.0)))
            return tok, lp
        lg = S.apply_processors(logits, **self._row_processors(rs)) if self._needs_processing(rs) else logits
        tok, _ = S.sample_token(lg, req.temperature, req.top_k, req.top_p, req.min_p, rs.seed, rs.sample_counter)
        lp = None
        if req.logprobs:
            t = req.temperature if req.temperature > 0 else 1.0
            lp = TokenLogprob(tok, S.token_logprob(lg, tok, t), tuple(S.top_logprobs(lg, req.top_logprobs, t)))
        return tok, lp

    # -- protocol defaults ---------------------------------------------------------------------------
    def capacity(self) -> Dict[str, Any]:
        return {"max_slots": self.max_slots, "max_context": self.max_context}

    def snapshot(self) -> Dict[str, Any]:
        return {}

    def reset(self) -> None:
        pass

    def close(self) -> None:
        pass


class CpuReferenceRunner(BaseRunner):
    """fp32 reference forward on the host.  One ``RefState`` per admitted request."""

    def __init__(self, weights, config: EngineConfig, eos_token_id: Optional[int] = None):
        from ..ref.model import RefModel
        # the host backend keeps K/V exact unless INT8 storage was asked for (then every stored row goes through the
        # per-token-and-head INT8 format, the oracle of that storage mode)
        self.model = RefModel(weights, kv_storage="int8" if config.kv.storage == "int8" else "fp32")
        self.cfg = weights.config
        self.vocab = self.cfg.vocab
        self.eos_token_id = eos_token_id
        self.max_slots = config.scheduler.max_active_requests
        self.max_context = min(config.max_sequence_length, self.cfg.max_context)
        self.states: Dict[int, Any] = {}
        self.last_logits: Dict[int, torch.Tensor] = {}
        # NextN (MTP) speculative decoding on the host: the oracle of the GPU cycle (``speculative/mtp.py``).  Per
        # request: the draft block's own KV state and the post-norm hidden of the row that produced the last token.
        self.config = config
        self.spec_depth = 0
        if (config.speculative.mode == "mtp" and self.cfg.nextn_layers > 0
                and f"blk.{self.cfg.n_layers}.nextn.eh_proj.weight" in self.model.w):
            self.spec_depth = max(1, int(config.speculative.draft_depth))
        # Gemma 4: the assistant head (a separate artifact, ``config.speculative.draft_model``) drafts from the raw
        # hidden of the row that produced the last token against the backbone's own KV (``ref/gemma4.py``)
        self.assistant = None
        dm = config.speculative.draft_model
        if (config.speculative.mode in ("mtp", "gemma4_mtp") and self.cfg.arch == "gemma4"
                and dm not in (None, "", "off")):
            from ..loading.weights import ModelWeights
            from ..ref.gemma4 import AssistantRef
            if isinstance(dm, ModelWeights):
                head_w = dm
            elif dm == "random":
                from ..loading.gemma4 import build_random_assistant
                from ..models.config import NAMED_ASSISTANTS
                acfg = next(a for a in NAMED_ASSISTANTS.values()
                            if a.backbone_hidden == self.cfg.hidden and a.vocab == self.cfg.vocab)
                head_w = build_random_assistant(acfg, self.cfg, seed=0)
            else:
                from ..loading.gemma4 import load_assistant_gguf
                head_w = load_assistant_gguf(dm, self.cfg)
            self.assistant = AssistantRef(head_w, self.model._gemma)
            self.spec_depth = max(1, int(config.speculative.draft_depth))
        # host drafters over the token history (no draft network): the same classes the GPU provider uses
        self.lookup = None
        if config.speculative.mode in ("prompt_lookup", "ngram"):
            from ..speculative.providers import NGramCacheDrafter, PromptLookupDrafter
            self.lookup = PromptLookupDrafter() if config.speculative.mode == "prompt_lookup" else NGramCacheDrafter()
            self.spec_depth = max(1, int(config.speculative.draft_depth))
        self.supports_mtp = self.spec_depth > 0
        self.draft_states: Dict[int, Any] = {}
        self.h_prev: Dict[int, torch.Tensor] = {}
        self.spec_stats = {"cycles": 0, "drafted": 0, "accepted": 0}

    def _rows(self, toks, st):
        """(seed rows, logits) of a forward over ``toks``: the seed of a draft is the post-norm hidden for the NextN
        block and the raw hidden (before the output norm) for the assistant head."""
        from ..ref import ops as R
        t = torch.tensor(list(toks), dtype=torch.long)
        if self.assistant is not None:
            raw = self.model._gemma.forward_raw(t, st)
            hid = R.rmsnorm(raw, self.model.w["output_norm.weight"], self.cfg.rms_eps)
            return raw, self.model.logits_from_hidden(hid)
        hid = self.model.forward_hidden(t, st)
        return hid, self.model.logits_from_hidden(hid)

    def admit(self, rs: RequestState) -> bool:
        if rs.total_budget_tokens > self.max_context:
            raise GenerationAdmissionRejected(
                f"context_overflow: prompt {rs.prompt_len} + max_tokens {rs.req.max_tokens} exceeds {self.max_context}")
        if len(self.states) >= self.max_slots:
            return False
        self.states[rs.rid] = self.model.new_state()
        if self.supports_mtp:
            if self.assistant is None and self.lookup is None:
                self.draft_states[rs.rid] = self.model.new_state()
            self.h_prev[rs.rid] = torch.zeros(self.cfg.hidden)
        rs.slot = len(self.states) - 1
        return True

    @torch.no_grad()
    def prefill(self, work: List[Tuple[RequestState, int]]) -> Dict[int, Tuple[int, Optional[TokenLogprob]]]:
        out: Dict[int, Tuple[int, Optional[TokenLogprob]]] = {}
        for rs, n in work:
            toks = rs.req.prompt_token_ids[rs.prefilled:rs.prefilled + n]
            if self.supports_mtp:
                # the draft block sees every prompt row: token j with the hidden of position j - 1
                st = self.states[rs.rid]
                pos0 = st.pos
                hid, logits = self._rows(toks, st)
                if self.assistant is None and self.lookup is None:
                    for j, t in enumerate(toks):
                        self.model.nextn_step(int(t), self.h_prev[rs.rid] if j == 0 else hid[j - 1], pos0 + j,
                                              self.draft_states[rs.rid])
                self.h_prev[rs.rid] = hid[-1].clone()
            else:
                logits, _ = self.model.forward(torch.tensor(toks, dtype=torch.long), self.states[rs.rid])
            if rs.prefilled + n >= rs.prompt_len:
                out[rs.rid] = self.sample_host(rs, logits[-1])
        return out

    @torch.no_grad()
    def decode(self, rows: List[RequestState]) -> List[Tuple[int, Optional[TokenLogprob]]]:
        res = []
        for rs in rows:
            if self.supports_mtp:
                # keep the draft block in step on plain steps too (a request may alternate between the two paths)
                st = self.states[rs.rid]
                pos = st.pos
                hid, logits = self._rows([rs.last_token], st)
                if self.assistant is None and self.lookup is None:
                    self._truncate_draft(rs.rid, pos)
                    self.model.nextn_step(int(rs.last_token), self.h_prev[rs.rid], pos, self.draft_states[rs.rid])
                self.h_prev[rs.rid] = hid[-1].clone()
            else:
                logits, _ = self.model.forward(torch.tensor([rs.last_token], dtype=torch.long), self.states[rs.rid])
            res.append(self.sample_host(rs, logits[-1]))
        return res

    # ------------------------------------------------------------------ NextN speculative cycles (greedy)
    def speculative_eligible(self, rs: RequestState) -> bool:
        from ..speculative.serving import resolve_mtp_serving_plan
        d = resolve_mtp_serving_plan("on", self.supports_mtp, rs.req.temperature, self._needs_processing(rs),
                                     bool(rs.forced), bool(rs.req.logprobs), depth=self.spec_depth)
        return d.use_mtp and d.sampling_mode == "greedy"

    def _truncate_draft(self, rid: int, n_rows: int) -> None:
        """Positions rewind: the draft block's KV keeps the rows below ``n_rows`` only."""
        ds = self.draft_states[rid]
        for i in list(ds.k):
            ds.k[i], ds.v[i] = ds.k[i][:n_rows], ds.v[i][:n_rows]

    @torch.no_grad()
    def speculative_cycle(self, rows: List[RequestState]):
        """Draft K tokens with the NextN block, verify them with one target forward on a copy of the state, accept
        the longest matching prefix, commit by running the accepted tokens through the live state.  The same cycle
        as ``speculative/mtp.py::MTPCycle`` (seed = hidden of the row that produced the last token; the draft
        block's KV below the cycle's first position is kept, the rest is rewritten by the next cycle)."""
        from ..speculative.contracts import SpecCycleResult
        from ..speculative.policy import plan_draft_depth
        from ..speculative.sampling import greedy_accept
        out = []
        for rs in rows:
            depth = plan_draft_depth(self.spec_depth, rs.remaining(), rs.total_budget_tokens - rs.position,
                                     rs.telemetry.speculative_drafted, rs.telemetry.speculative_accepted,
                                     adaptive=self.config.speculative.adaptive_depth)
            if depth < 1:
                tok, _ = self.decode([rs])[0]
                out.append(SpecCycleResult([tok], 0, 0))
                continue
            st, rid = self.states[rs.rid], rs.rid
            p = st.pos                                       # position of the last committed (not yet fed) token
            if self.lookup is not None:
                history = list(rs.req.prompt_token_ids) + rs.generated
                drafts = [int(t) for t in self.lookup.propose(history, depth)]
                if not drafts:                               # nothing repeats: a plain step is cheaper than a verify
                    tok, _ = self.decode([rs])[0]
                    self.lookup.observe(history + [tok])
                    out.append(SpecCycleResult([tok], 0, 0))
                    continue
                depth = len(drafts)
            elif self.assistant is not None:
                # every step of a draft at the same position, against the backbone's KV as it stands
                drafts = self.assistant.draft(int(rs.last_token), self.h_prev[rid], st, depth)
            else:
                self._truncate_draft(rid, p)
                cur, hp, drafts = int(rs.last_token), self.h_prev[rid], []
                for j in range(depth):
                    lg, hp = self.model.nextn_step(cur, hp, p + j, self.draft_states[rid])
                    cur = int(lg.argmax())
                    drafts.append(cur)
            chain = [int(rs.last_token)] + drafts
            target = self._rows(chain, st.clone())[1].argmax(-1).tolist()
            n, emitted = greedy_accept(drafts, target)
            hid, _ = self._rows(chain[:n + 1], st)                      # commit: the live state advances by n + 1
            self.h_prev[rid] = hid[n].clone()
            if self.lookup is not None:
                self.lookup.observe(list(rs.req.prompt_token_ids) + rs.generated + [int(t) for t in emitted])
            out.append(SpecCycleResult([int(t) for t in emitted], depth, n))
            self.spec_stats["cycles"] += 1
            self.spec_stats["drafted"] += depth
            self.spec_stats["accepted"] += n
        return out

    def release(self, rs: RequestState) -> None:
        self.states.pop(rs.rid, None)
        self.draft_states.pop(rs.rid, None)
        self.h_prev.pop(rs.rid, None)

    def reset(self) -> None:
        self.states.clear()
        self.draft_states.clear()
        self.h_prev.clear()

    def capacity(self) -> Dict[str, Any]:
        return {"backend": "cpu_reference", "max_slots": self.max_slots, "max_context": self.max_context,
                "active": len(self.states)}
