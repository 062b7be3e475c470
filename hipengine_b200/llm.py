"""Public Python API: ``LLM`` and ``SamplingParams``.

Surface parity with the reference (``hipengine/llm.py:196-343`` for the sampling
dataclass, ``:365-394`` for constructor kwargs, ``:538-1578`` for methods):
``generate``, ``generate_detailed``, ``stream``, ``stream_detailed``, ``chat``,
``tokenize/detokenize/count_tokens``, ``prepare``, ``reset``, ``close``,
``resident_capacity_estimate``, ``engine_service_health``, ``live_loop_snapshot``.
Construction resolves model metadata -> weights -> executor -> engine service;
one driver thread owns the device (``hipengine/generation/engine_service.py:207-297``).
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass, field, replace
from pathlib import Path
from typing import Any, Dict, Iterator, List, Mapping, Optional, Sequence, Tuple, Union

import torch

from .config import EngineConfig, ExecutionProfile, KVConfig, SchedulerConfig, SpeculativeConfig
from .generation.types import (FinishDetails, GenerationOutput, GenerationRequest, GenerationStreamChunk,
                               normalize_logit_bias, normalize_stop_sequences)


class ResidentPreparationError(RuntimeError):
    """Raised when the engine cannot become resident (weights / KV / scratch do not fit, or no device)."""


class UnsupportedModalityError(NotImplementedError):
    """Raised by the entry points of modalities this engine does not serve (it is a text-generation engine)."""


@dataclass(frozen=True)
class SamplingParams:
    """Every sampler / finish / constraint knob of a request (``hipengine/llm.py:196-343``)."""
    max_tokens: int = 16
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    logit_bias: Any = ()
    suppress_token_ids: Tuple[int, ...] = ()
    min_tokens: int = 0
    eos_token_id: Optional[int] = None
    stop_token_ids: Tuple[int, ...] = ()
    stop_token_sequences: Tuple[Tuple[int, ...], ...] = ()
    forced_tokens_pending: Tuple[int, ...] = ()
    json_object_close_forcing: bool = False
    tool_call_constraint: Any = None
    grammar: Optional[Mapping[str, Any]] = None
    thinking_close_token_ids: Tuple[int, ...] = ()
    thinking_hard_token_cap: Optional[int] = None
    thinking_soft_close_window: int = 0
    ignore_eos: bool = False
    kv_storage: str = "auto"
    seed: Optional[int] = None
    row_seeds: Tuple[int, ...] = ()
    deadline_at: Optional[float] = None
    cancellation_token: Any = field(default=None, compare=False, repr=False)
    resident_session_key: Optional[str] = field(default=None, compare=False, repr=False)
    speculative_mtp: bool = False
    logprobs: bool = False
    top_logprobs: int = 0

    def __post_init__(self) -> None:
        s = object.__setattr__
        s(self, "max_tokens", int(self.max_tokens))
        s(self, "temperature", float(self.temperature))
        s(self, "top_p", float(self.top_p))
        s(self, "top_k", int(self.top_k))
        s(self, "min_p", float(self.min_p))
        s(self, "logit_bias", normalize_logit_bias(self.logit_bias))
        s(self, "suppress_token_ids", tuple(int(t) for t in self.suppress_token_ids))
        s(self, "stop_token_ids", tuple(int(t) for t in self.stop_token_ids))
        s(self, "stop_token_sequences", normalize_stop_sequences(self.stop_token_sequences))
        s(self, "forced_tokens_pending", tuple(int(t) for t in self.forced_tokens_pending))
        s(self, "row_seeds", tuple(int(t) for t in self.row_seeds))
        s(self, "top_logprobs", int(self.top_logprobs))
        if self.max_tokens < 0:
            raise ValueError("max_tokens must be >= 0")
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError("top_p must be in (0, 1]")
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")
        if not (0.0 <= self.min_p <= 1.0):
            raise ValueError("min_p must be in [0, 1]")
        if self.repetition_penalty <= 0:
            raise ValueError("repetition_penalty must be > 0")
        if not (0 <= self.top_logprobs <= 20):
            raise ValueError("top_logprobs must be in [0, 20]")
        if self.grammar is not None:
            raise ValueError("user-supplied grammars are rejected before generation")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0


PromptLike = Union[str, Sequence[int]]


class LLM:
    """Load a model and generate.

    ``model`` may be a GGUF path / directory, a ``ModelWeights`` object, or the name of a built-in
    random-init geometry (``"tiny-hybrid"``, ``"qwen35-27b"``, ...; see ``models.config.NAMED_CONFIGS``).
    """

    def __init__(self, model: Any, *, backend: str = "auto", quant: Optional[str] = None,
                 execution_profile: Any = None, max_active_requests: int = 8,
                 max_sequence_length: Optional[int] = None, prefix_cache: str = "radix",
                 speculative_mtp_serving: str = "off", speculative_candidate_budget: int = 3,
                 speculative_provider: str = "mtp", mtp_hot_vocab: Any = None, draft_model: Any = None,
                 kv_cold_tier_bytes: int = 0,
                 kv_cold_tier_dir: Optional[str] = None,
                 kv_storage: str = "bf16", tensor_parallel: int = 1, expert_parallel: int = 1,
                 engine_command_timeout_seconds: float = 300.0, seed: int = 0, tokenizer: Any = None,
                 engine_config: Optional[EngineConfig] = None, device: Optional[str] = None,
                 weights_recipe: str = "q4_k_m", expected_quant: Optional[str] = None):
        self.model = model
        self._expected_quant = expected_quant
        self.backend = self._resolve_backend(backend, device)
        self.profile = ExecutionProfile.parse(execution_profile)
        if kv_storage in ("auto", None):
            kv_storage = "bf16"
        if kv_storage not in ("bf16", "int8"):
            raise ValueError(f"kv_storage={kv_storage!r} is unknown (bf16 | int8)")
        if kv_storage == "int8" and self.backend != "cpu_reference":
            # the GPU writer and both attention readers exist for bf16 pages only (the INT8 format is defined and
            # served by the host reference backend): refuse instead of silently storing bf16
            raise ValueError("kv_storage='int8' is not supported by the cuda_sm100a backend of this build (bf16 only)")
        base = engine_config or EngineConfig.from_env()
        self.config = replace(
            base,
            max_sequence_length=int(max_sequence_length or base.max_sequence_length),
            profile=self.profile,
            scheduler=replace(base.scheduler, max_active_requests=int(max_active_requests)),
            kv=replace(base.kv, storage=kv_storage, prefix_cache=prefix_cache,
                       cold_tier_bytes=int(kv_cold_tier_bytes or base.kv.cold_tier_bytes),
                       cold_tier_dir=kv_cold_tier_dir or base.kv.cold_tier_dir),
            speculative=replace(base.speculative,
                                mode=speculative_provider if speculative_mtp_serving not in ("off", None) else "off",
                                draft_depth=int(speculative_candidate_budget),
                                hot_vocab=str(mtp_hot_vocab) if mtp_hot_vocab is not None
                                else base.speculative.hot_vocab,
                                draft_model=draft_model if draft_model is not None
                                else base.speculative.draft_model),
            parallel=replace(base.parallel, tp=int(tensor_parallel), ep=int(expert_parallel)),
            command_timeout_seconds=float(engine_command_timeout_seconds),
        )
        self._seed = seed
        self._weights_recipe = weights_recipe
        self._tokenizer = tokenizer
        self._engine = None
        self._lock = threading.Lock()
        self._closed = False
        self._weights = None

    @classmethod
    def from_executor(cls, executor, tokenizer: Any = None, max_active_requests: Optional[int] = None,
                      engine_config: Optional[EngineConfig] = None, **kw) -> "LLM":
        """Wrap an already-resident GPU executor (weights stay where they are) in the public API."""
        from .generation.engine_service import engine_from_runner
        from .generation.gpu_runner import GpuRunner
        from .tokenization.gguf_tokenizer import ByteTokenizer
        self = cls.__new__(cls)
        self.model = executor
        self.backend = "cuda_sm100a"
        self.profile = ExecutionProfile.PRODUCTION
        base = engine_config or EngineConfig.from_env()
        n = int(max_active_requests or executor.max_slots)
        self.config = replace(base, max_sequence_length=executor.max_context,
                              scheduler=replace(base.scheduler, max_active_requests=n),
                              kv=replace(base.kv, prefix_cache=kw.get("prefix_cache", "off"),
                                         pool_pages=executor.n_pages))
        self._seed = 0
        self._weights_recipe = "q4_k_m"
        self._tokenizer = tokenizer or ByteTokenizer(executor.cfg.vocab)
        self._lock = threading.Lock()
        self._closed = False
        self._weights = None
        runner = GpuRunner(None, self.config, getattr(self._tokenizer, "eos_token_id", None), executor=executor)
        self._engine = engine_from_runner(runner, self.config, self._tokenizer)
        return self

    # ------------------------------------------------------------------ construction
    @staticmethod
    def _resolve_backend(backend: str, device: Optional[str]) -> str:
        if backend in ("auto", None):
            return "cuda_sm100a" if torch.cuda.is_available() else "cpu_reference"
        if backend not in ("cuda_sm100a", "cpu_reference"):
            raise ValueError(f"unknown backend {backend!r}; expected cuda_sm100a or cpu_reference")
        if backend == "cuda_sm100a" and not torch.cuda.is_available():
            raise ResidentPreparationError("backend cuda_sm100a requested but no CUDA device is visible")
        return backend

    def _load_weights(self):
        if self._weights is not None:
            return self._weights
        from .loading.weights import ModelWeights
        m = self.model
        dev = "cuda" if self.backend == "cuda_sm100a" else "cpu"
        if isinstance(m, ModelWeights):
            self._weights = m
        elif isinstance(m, (str, Path)) and Path(str(m)).exists():
            from .loading.model_loader import load_gguf_model
            self._weights = load_gguf_model(m, device=dev, pin=(dev == "cuda"))
        elif isinstance(m, str):
            from .loading.synth import build_random_model
            from .models.config import NAMED_CONFIGS
            if m not in NAMED_CONFIGS:
                raise FileNotFoundError(f"model {m!r} is neither a local GGUF path nor a built-in geometry "
                                        f"({sorted(NAMED_CONFIGS)}); nothing is ever downloaded")
            self._weights = build_random_model(NAMED_CONFIGS[m], seed=self._seed, device=dev,
                                               recipe=self._weights_recipe)
        else:
            raise TypeError(f"unsupported model argument {type(m)}")
        return self._weights

    @property
    def startup(self) -> Dict[str, Any]:
        """Record of how the engine came up: stages in order with their durations, checks, device memory (the
        start-up block of the server's readiness document; ``LOAD_TIMING`` in the reference's logs)."""
        st = self.__dict__.get("_startup")
        if st is None:
            st = self.__dict__["_startup"] = {"model_loaded": False, "warmup_complete": False, "eager_load": False,
                                              "stages": [], "timings_s": {}, "checks": {}, "memory": {}, "error": None}
        return st

    def _stage(self, name: str, fn):
        st = self.startup
        t0 = time.time()
        try:
            out = fn()
        except Exception as exc:
            st["stages"].append({"name": name, "seconds": round(time.time() - t0, 3), "ok": False})
            st["error"] = f"{name}: {type(exc).__name__}: {exc}"
            raise
        dt = round(time.time() - t0, 3)
        st["stages"].append({"name": name, "seconds": dt, "ok": True})
        st["timings_s"][name] = dt
        return out

    def _admit(self, weights) -> None:
        """Plan contract + memory preflight before the engine (KV pool, state slots, scratch) is built; the report
        goes into the start-up record, a rejection raises with every reason listed."""
        from .loading.admission import admit
        free = None
        if self.backend == "cuda_sm100a":
            try:
                import torch
                f, _total = torch.cuda.mem_get_info()
                on_dev = any(t.raw.is_cuda for t in list(weights.tensors.values())[:1])
                free = int(f) + (int(weights.nbytes()) if on_dev else 0)
            except Exception:
                free = None
        rep = admit(weights, self.config, free_bytes=free, strict=True,
                    expected_quant=getattr(self, "_expected_quant", None))
        self.startup["checks"]["admission"] = {k: rep[k] for k in ("admitted", "plan_complete", "plan_digest",
                                                                   "planned_weights", "widened_to_bf16", "memory")}

    def _get_engine(self):
        if self._closed:
            raise RuntimeError("LLM is closed")
        if self._engine is None:
            with self._lock:
                if self._engine is None:
                    from .generation.engine_service import build_engine
                    w = self._stage("load_weights", self._load_weights)
                    self._stage("admission", lambda: self._admit(w))
                    tok = self._stage("tokenizer", self._get_tokenizer)
                    self._engine = self._stage("build_engine",
                                               lambda: build_engine(w, self.backend, self.config, tok))
                    st = self.startup
                    st["model_loaded"] = True
                    st["checks"]["native_library"] = "loaded" if self.backend == "cuda_sm100a" else "not_needed"
                    if self.backend == "cuda_sm100a":
                        try:
                            import torch
                            free, total = torch.cuda.mem_get_info()
                            st["memory"] = {"device_total_bytes": int(total), "device_free_bytes": int(free),
                                            "torch_allocated_bytes": int(torch.cuda.memory_allocated())}
                        except Exception:
                            pass
        return self._engine

    def _get_tokenizer(self):
        if self._tokenizer is None:
            from .tokenization.gguf_tokenizer import tokenizer_from_metadata
            w = self._load_weights()
            self._tokenizer = tokenizer_from_metadata(w.metadata, w.config.vocab)
        return self._tokenizer

    @property
    def vocab_size(self) -> int:
        cfg = getattr(self.model, "cfg", None)
        return int(cfg.vocab) if cfg is not None else int(self._load_weights().config.vocab)

    def prepare(self) -> Dict[str, Any]:
        """Make the engine resident now (weights uploaded, KV pool and scratch reserved)."""
        t0 = time.time()
        self.startup["eager_load"] = True
        eng = self._get_engine()
        info = eng.capacity()
        info["prepare_seconds"] = time.time() - t0
        return info

    def mark_warm(self) -> None:
        """Called after a start-up smoke request went through: graphs are captured and scratch is sized."""
        self.startup["warmup_complete"] = True

    def follow(self) -> None:
        """Ranks other than 0 of a tensor/expert-parallel serving group: make the engine resident and execute the
        command batches rank 0 publishes until it says stop (rank 0 owns HTTP, the scheduler and the sampler)."""
        eng = self._get_engine()
        if eng.coord is None or eng.coord.is_leader:
            raise RuntimeError("follow() is for the non-zero ranks of a parallel serving group")
        eng.thread.join()

    # ------------------------------------------------------------------ requests
    def _request(self, prompt: PromptLike, sp: SamplingParams, index: int) -> GenerationRequest:
        if isinstance(prompt, str):
            ids = self.tokenize(prompt)
            text = prompt
        else:
            ids = [int(t) for t in prompt]
            text = None
        # token ids index the embedding table on the device: an id outside the vocabulary must never get there
        if not ids:
            raise ValueError("the prompt is empty")
        vocab = self.vocab_size
        lo, hi = min(ids), max(ids)
        if lo < 0 or hi >= vocab:
            raise ValueError(f"prompt token id {lo if lo < 0 else hi} is outside the vocabulary [0, {vocab})")
        # the same for every other field whose ids are fed back to the model or index a logits row
        for field_name, values in (("forced_tokens_pending", sp.forced_tokens_pending),
                                   ("suppress_token_ids", sp.suppress_token_ids),
                                   ("logit_bias", [t for t, _ in (sp.logit_bias or ())])):
            bad = [int(t) for t in values if not 0 <= int(t) < vocab]
            if bad:
                raise ValueError(f"{field_name}: token id {bad[0]} is outside the vocabulary [0, {vocab})")
        return GenerationRequest.from_sampling(ids, sp, prompt_text=text, row_index=index)

    def generate_detailed(self, prompts: Union[PromptLike, Sequence[PromptLike]],
                          sampling_params: Optional[Union[SamplingParams, Sequence[SamplingParams]]] = None
                          ) -> List[GenerationOutput]:
        single = isinstance(prompts, str) or (len(prompts) > 0 and isinstance(prompts[0], int))
        plist = [prompts] if single else list(prompts)
        if sampling_params is None:
            sps = [SamplingParams()] * len(plist)
        elif isinstance(sampling_params, SamplingParams):
            sps = [sampling_params] * len(plist)
        else:
            sps = list(sampling_params)
            if len(sps) != len(plist):
                raise ValueError("one SamplingParams per prompt expected")
        reqs = [self._request(p, sp, i) for i, (p, sp) in enumerate(zip(plist, sps))]
        outs = self._get_engine().generate(reqs)
        tok = self._get_tokenizer()
        for o in outs:
            if o.text is None:
                o.text = tok.decode(o.token_ids)
        return outs

    def generate(self, prompts, sampling_params=None) -> List[str]:
        return [o.text for o in self.generate_detailed(prompts, sampling_params)]

    def generate_token_ids(self, prompts, sampling_params=None) -> List[List[int]]:
        return [o.token_ids for o in self.generate_detailed(prompts, sampling_params)]

    def stream_detailed(self, prompt: PromptLike, sampling_params: Optional[SamplingParams] = None
                        ) -> Iterator[GenerationStreamChunk]:
        req = self._request(prompt, sampling_params or SamplingParams(), 0)
        tok = self._get_tokenizer()
        dec = tok.stream_decoder()
        for ch in self._get_engine().stream(req):
            if ch.text is None:
                ch.text = dec.feed(ch.token_ids) + (dec.flush() if ch.finished else "")
            yield ch

    def stream(self, prompt: PromptLike, sampling_params: Optional[SamplingParams] = None) -> Iterator[str]:
        for ch in self.stream_detailed(prompt, sampling_params):
            if ch.text:
                yield ch.text

    def stream_many_detailed(self, prompts: Sequence[PromptLike], sampling_params=None):
        """Concurrent streams: yields (index, chunk) as chunks arrive."""
        sps = sampling_params if isinstance(sampling_params, (list, tuple)) else [sampling_params or SamplingParams()] * len(prompts)
        reqs = [self._request(p, sp, i) for i, (p, sp) in enumerate(zip(prompts, sps))]
        yield from self._get_engine().stream_many(reqs)

    def chat(self, messages: Sequence[Mapping[str, Any]], sampling_params: Optional[SamplingParams] = None,
             tools: Optional[Sequence[Mapping[str, Any]]] = None, enable_thinking: bool = True) -> GenerationOutput:
        from .chat.templates import render_chat
        prompt = render_chat(messages, tools=tools, enable_thinking=enable_thinking,
                             arch=self._load_weights().config.arch)
        return self.generate_detailed(prompt, sampling_params or SamplingParams(max_tokens=256))[0]

    def generate_speculative_mtp_detailed(self, prompts, sampling_params=None) -> List[GenerationOutput]:
        sps = sampling_params or SamplingParams()
        if isinstance(sps, SamplingParams):
            sps = replace(sps, speculative_mtp=True)
        return self.generate_detailed(prompts, sps)

    def stream_speculative_mtp_detailed(self, prompt: PromptLike, sampling_params: Optional[SamplingParams] = None
                                        ) -> Iterator[GenerationStreamChunk]:
        """Stream one request through the speculative path: a chunk carries the 1 .. depth + 1 tokens a cycle
        committed (``hipengine/llm.py:859`` of the reference)."""
        yield from self.stream_detailed(prompt, replace(sampling_params or SamplingParams(), speculative_mtp=True))

    def generate_speculative_detailed(self, prompts, sampling_params=None) -> List[GenerationOutput]:
        """Speculative decoding with whichever provider the engine was built with (NextN block, assistant head,
        prompt lookup, n-gram table); an engine without one raises instead of silently decoding step by step."""
        if self.config.speculative.mode in ("off", "", None):
            raise ValueError("this engine was built without a speculative provider "
                             "(speculative_mtp_serving / speculative_provider)")
        return self.generate_speculative_mtp_detailed(prompts, sampling_params)

    def resolve_speculative_mtp_serving_plan(self, sampling_params: Optional[SamplingParams] = None,
                                             breaker_open: bool = False):
        """Would a request with these parameters take the speculative path, and if not, why
        (``hipengine/llm.py:1041``; rules in ``speculative/serving.py``)."""
        from .speculative.serving import resolve_mtp_serving_plan
        sp = sampling_params or SamplingParams()
        mode = self.config.speculative.mode
        eng = self._get_engine()
        runner = getattr(getattr(eng, "loop", None), "runner", None)
        # the runner's rule (``generation/runner.py::_needs_processing``) as far as it can be read off the parameters
        processed = bool(sp.logit_bias or sp.suppress_token_ids or sp.repetition_penalty != 1.0
                         or sp.presence_penalty != 0.0 or sp.frequency_penalty != 0.0 or sp.min_tokens
                         or sp.grammar is not None or sp.tool_call_constraint is not None)
        return resolve_mtp_serving_plan("off" if mode in ("off", "", None) else "on",
                                        bool(getattr(runner, "supports_mtp", False)), float(sp.temperature or 0.0),
                                        processed, bool(sp.forced_tokens_pending), bool(sp.logprobs),
                                        breaker_open=breaker_open, depth=self.config.speculative.draft_depth,
                                        requested=True)

    # ------------------------------------------------------------------ modalities that are not served
    def _no_modality(self, what: str, ref: str):
        raise UnsupportedModalityError(
            f"{what} is not served by this engine: it runs text decoders (Qwen3.5 hybrid dense / MoE, Gemma 4, "
            f"Qwen3 / Llama-shaped dense and MoE) and has no encoder, codec or diffusion stack (reference: {ref})")

    def generate_multimodal_detailed(self, *args, **kwargs):
        """Image / video + text generation (reference ``hipengine/llm.py:611``): not served; raises."""
        self._no_modality("multimodal generation", "hipengine/llm.py:611")

    def transcribe(self, *args, **kwargs):
        """Speech to text (reference ``hipengine/llm.py:632``): not served; raises."""
        self._no_modality("speech transcription", "hipengine/llm.py:632")

    def synthesize(self, *args, **kwargs):
        """Text to speech (reference ``hipengine/llm.py:645``): not served; raises."""
        self._no_modality("speech synthesis", "hipengine/llm.py:645")

    def generate_song(self, *args, **kwargs):
        """Lyrics + style to audio (reference ``hipengine/llm.py:664``): not served; raises."""
        self._no_modality("song generation", "hipengine/llm.py:664")

    def submit_independent_batches_detailed(self, batches: Sequence[Sequence[PromptLike]], sampling_params=None
                                            ) -> List[List[GenerationOutput]]:
        """Several caller-side batches admitted together: the engine batches continuously across all of them, the
        outputs come back grouped as they were submitted (``hipengine/llm.py:577``)."""
        flat = [p for b in batches for p in b]
        if isinstance(sampling_params, (list, tuple)):
            if len(sampling_params) != len(batches):
                raise ValueError("one SamplingParams per batch (or a single one for all) is expected")
            sps = [sp or SamplingParams() for b, sp in zip(batches, sampling_params) for _ in b]
        else:
            sps = [sampling_params or SamplingParams()] * len(flat)
        outs = self.generate_detailed(flat, sps) if flat else []
        grouped, i = [], 0
        for b in batches:
            grouped.append(outs[i:i + len(b)])
            i += len(b)
        return grouped

    def fit_context(self, prompt: PromptLike, max_tokens: Optional[int] = None) -> Dict[str, Any]:
        """Does ``prompt`` (text or token ids) fit the served context, and how many tokens may follow it."""
        n = len(self.tokenize(prompt)) if isinstance(prompt, str) else len(list(prompt))
        mx = getattr(self, "_served_context", None)
        if mx is None:
            # fixed once the engine is built; asked once, because the answer comes from the driver thread between two
            # ticks and a route handler must not wait for a tick on every request
            mx = int(self.resident_capacity_estimate().get("max_context") or self.config.max_sequence_length)
            self._served_context = mx
        room = max(0, mx - n)
        out = {"prompt_tokens": n, "max_context": mx, "max_new_tokens": room, "fits": n < mx}
        if max_tokens is not None:
            out["fits_with_max_tokens"] = n + int(max_tokens) <= mx
        return out

    # ------------------------------------------------------------------ tokenizer helpers
    def tokenize(self, text: str) -> List[int]:
        return self._get_tokenizer().encode(text)

    def detokenize(self, ids: Sequence[int]) -> str:
        return self._get_tokenizer().decode(list(ids))

    def count_tokens(self, text: str) -> int:
        return len(self.tokenize(text))

    # ------------------------------------------------------------------ introspection / lifecycle
    def resident_capacity_estimate(self) -> Dict[str, Any]:
        return self._get_engine().capacity()

    def engine_service_health(self) -> Dict[str, Any]:
        if self._engine is None:
            return {"state": "not_started", "healthy": True}
        return self._engine.health()

    def live_loop_snapshot(self) -> Dict[str, Any]:
        if self._engine is None:
            return {}
        return self._engine.snapshot()

    def reset(self) -> None:
        if self._engine is not None:
            self._engine.reset()

    def close(self) -> None:
        self._closed = True
        if self._engine is not None:
            self._engine.close()
            self._engine = None

    def __enter__(self) -> "LLM":
        return self

    def __exit__(self, *exc) -> None:
        self.close()
