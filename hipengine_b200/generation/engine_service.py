"""Engine service: one driver thread owns the model; front-end threads talk to it through a command queue.

Same ownership rule as the reference (``hipengine/generation/engine_service.py:207-297,937-1025``): callers
enqueue commands (submit / cancel / control) on a bounded queue and wait on per-request collectors; the
driver loop drains commands, runs one engine tick, routes events and finishes requests.  A fatal failure
records an ``unhealthy`` cause, fails every request and stops the loop (``:354-398``); a command that is not
served within ``command_timeout_seconds`` raises ``EngineCommandTimeout`` (``:44,65-77``).
"""
from __future__ import annotations

import queue
import threading
import time
import traceback
from dataclasses import dataclass, field
from typing import Any, Dict, Iterator, List, Optional, Sequence, Tuple

from ..config import EngineConfig
from .engine_loop import EngineLoop
from .scheduler import FINISHED, GenerationAdmissionRejected, RequestState
from .types import FinishDetails, GenerationOutput, GenerationRequest, GenerationStreamChunk

COMMAND_QUEUE_DEPTH = 1024


class EngineCommandTimeout(TimeoutError):
    pass


class EngineUnavailable(RuntimeError):
    """The service is closed or unhealthy (HTTP 503, retryable)."""


class OutputCollector:
    """Per-request mailbox: stream chunks (bounded) and the final output."""

    def __init__(self, mailbox: int = 64, stream: bool = False):
        self.stream = stream
        self.chunks: "queue.Queue[GenerationStreamChunk]" = queue.Queue(maxsize=mailbox if stream else 0)
        self.done = threading.Event()
        self.output: Optional[GenerationOutput] = None
        self.rid: Optional[int] = None

    def put_chunk(self, ch: GenerationStreamChunk) -> None:
        if self.stream:
            try:
                self.chunks.put(ch, timeout=30.0)
            except queue.Full:
                pass

    def finish(self, out: GenerationOutput) -> None:
        self.output = out
        self.done.set()


@dataclass
class _Command:
    kind: str
    payload: Any = None
    reply: "queue.Queue" = field(default_factory=lambda: queue.Queue(maxsize=1))


class EngineService:
    def __init__(self, loop: EngineLoop, config: EngineConfig, name: str = "he-engine-service", coordinator=None):
        self.loop = loop
        self.config = config
        # parallel group: rank 0 publishes every tick's command batch, all ranks apply it (parallel/serving.py)
        self.coord = coordinator
        self.orphans: Dict[int, GenerationOutput] = {}      # follower: outputs finished before their caller arrived
        if coordinator is not None:
            self.loop.external_lifetimes = True
        self.commands: "queue.Queue[_Command]" = queue.Queue(maxsize=COMMAND_QUEUE_DEPTH)
        self.collectors: Dict[int, OutputCollector] = {}
        self.unhealthy: Optional[Dict[str, Any]] = None
        self.closed = False
        # bounded ring of recent engine events (submits, finishes, errors): attached to the unhealthy report and to
        # snapshot(), so a failed server can say what it was doing
        from ..utils.tracing import FlightRecorder
        self.recorder = FlightRecorder(capacity=256)
        self._wake = threading.Event()
        self.loop.on_event = self._on_event
        self.thread = threading.Thread(target=self._drive, name=name, daemon=True)
        self.started_at = time.time()
        self.thread.start()

    # ------------------------------------------------------------------ front-end API (any thread)
    def _call(self, kind: str, payload: Any = None, wait: bool = True) -> Any:
        if self.closed:
            raise EngineUnavailable("engine service is closed")
        if self.unhealthy is not None:
            raise EngineUnavailable(f"engine service is unhealthy: {self.unhealthy.get('exception_type')}: "
                                    f"{self.unhealthy.get('message')}")
        cmd = _Command(kind, payload)
        try:
            self.commands.put(cmd, timeout=self.config.command_timeout_seconds)
        except queue.Full:
            raise EngineCommandTimeout("engine command queue is full") from None
        self._wake.set()
        if not wait:
            return None
        try:
            ok, val = cmd.reply.get(timeout=self.config.command_timeout_seconds)
        except queue.Empty:
            raise EngineCommandTimeout(f"engine did not serve {kind!r} within "
                                       f"{self.config.command_timeout_seconds}s") from None
        if not ok:
            raise val
        return val

    def submit(self, req: GenerationRequest, stream: bool = False) -> OutputCollector:
        col = OutputCollector(self.config.scheduler.stream_mailbox, stream)
        col.rid = req.request_id
        self.recorder.record("submit", rid=req.request_id, prompt_tokens=len(req.prompt_token_ids),
                             max_tokens=req.max_tokens, stream=bool(stream))
        self._call("submit", (req, col))
        return col

    def generate(self, reqs: Sequence[GenerationRequest]) -> List[GenerationOutput]:
        cols = [self.submit(r) for r in reqs]
        outs = []
        for c in cols:
            self._wait(c)
            outs.append(c.output)
        return outs

    def _wait(self, col: OutputCollector) -> None:
        while not col.done.wait(timeout=0.5):
            if self.unhealthy is not None or self.closed:
                if not col.done.is_set():
                    raise EngineUnavailable("engine stopped while the request was in flight")

    def stream(self, req: GenerationRequest) -> Iterator[GenerationStreamChunk]:
        col = self.submit(req, stream=True)
        try:
            while True:
                try:
                    ch = col.chunks.get(timeout=0.5)
                except queue.Empty:
                    if col.done.is_set() and col.chunks.empty():
                        return
                    if self.unhealthy is not None or self.closed:
                        raise EngineUnavailable("engine stopped while streaming")
                    continue
                yield ch
                if ch.finished:
                    return
        finally:
            if not col.done.is_set():
                self.cancel(req.request_id)

    def stream_many(self, reqs: Sequence[GenerationRequest]) -> Iterator[Tuple[int, GenerationStreamChunk]]:
        cols = [self.submit(r, stream=True) for r in reqs]
        live = set(range(len(cols)))
        while live:
            progressed = False
            for i in list(live):
                try:
                    ch = cols[i].chunks.get_nowait()
                except queue.Empty:
                    continue
                progressed = True
                yield i, ch
                if ch.finished:
                    live.discard(i)
            if not progressed:
                if self.unhealthy is not None or self.closed:
                    raise EngineUnavailable("engine stopped while streaming")
                time.sleep(0.001)

    def cancel(self, rid: int, reason: str = "cancelled", wait: bool = True) -> bool:
        """Cancel a request.  With ``wait=False`` the command is only posted (the driver serves it before its next
        tick) and the answer is True: for callers that must not wait for a tick, such as an event loop."""
        try:
            if not wait:
                self._call("cancel", (rid, reason), wait=False)
                return True
            return bool(self._call("cancel", (rid, reason)))
        except EngineUnavailable:
            return False

    def snapshot(self) -> Dict[str, Any]:
        snap = self._call("snapshot")
        if isinstance(snap, dict):
            snap["recent_events"] = self.recorder.dump(last=16)
        return snap

    def capacity(self) -> Dict[str, Any]:
        return self._call("capacity")

    def reset(self) -> None:
        self._call("reset")

    def health(self) -> Dict[str, Any]:
        return {"healthy": self.unhealthy is None and not self.closed, "closed": self.closed,
                "unhealthy": self.unhealthy, "uptime_seconds": time.time() - self.started_at,
                "driver_alive": self.thread.is_alive(), "queued_commands": self.commands.qsize()}

    def close(self) -> None:
        if self.closed:
            return
        try:
            if self.coord is not None and not self.coord.is_leader:
                # a follower's engine is stopped by rank 0's stop batch; wait for it instead of asking
                self.thread.join(timeout=self.config.command_timeout_seconds)
            elif self.thread.is_alive():
                self._call("close")
        except Exception:
            pass
        self.closed = True
        self._wake.set()
        self.thread.join(timeout=10.0)
        try:
            self.loop.runner.close()      # drops captured graphs (they may hold library collectives)
        except Exception:
            pass

    # ------------------------------------------------------------------ driver thread
    def _on_event(self, rs: RequestState) -> None:
        col = self.collectors.get(rs.rid)
        if col is None:
            return
        toks = self.loop.sched.take_stream_tokens(rs)
        finished = rs.status == FINISHED
        if col.stream and (toks or finished):
            lps = None
            if rs.req.logprobs and rs.logprobs:
                lps = rs.logprobs[rs.emitted - len(toks):rs.emitted]
            col.put_chunk(GenerationStreamChunk(rs.rid, toks, None, finished, rs.finish if finished else None, lps,
                                                rs.telemetry if finished else None, rs.error))
        if finished:
            self.recorder.record("finish", rid=rs.rid, reason=getattr(rs.finish, "reason", None), tokens=rs.emitted,
                                 error=rs.error)
            col.finish(self.loop.sched.make_output(rs))
            self.collectors.pop(rs.rid, None)
            self.loop.sched.pop_finished(rs.rid)

    def _on_event_follower(self, rs: RequestState) -> None:
        """Follower ranks: deliver to a caller of the same request on this rank if there is one (SPMD use of the Python
        API), otherwise keep the finished output for a short while in case the caller registers late."""
        if rs.rid in self.collectors:
            self._on_event(rs)
            return
        self.loop.sched.take_stream_tokens(rs)
        if rs.status == FINISHED:
            self.orphans[rs.rid] = self.loop.sched.make_output(rs)
            self.loop.sched.pop_finished(rs.rid)
            while len(self.orphans) > 256:
                self.orphans.pop(next(iter(self.orphans)))

    def _serve(self, cmd: _Command) -> bool:
        """Returns False when the loop should stop."""
        try:
            if cmd.kind == "submit":
                req, col = cmd.payload
                self.collectors[req.request_id] = col
                try:
                    self.loop.submit(req)
                except GenerationAdmissionRejected as exc:
                    self.collectors.pop(req.request_id, None)
                    out = GenerationOutput(req.request_id, list(req.prompt_token_ids), [], None,
                                           FinishDetails("error", message=str(exc)), None, error=str(exc))
                    col.put_chunk(GenerationStreamChunk(req.request_id, [], None, True, out.finish, None, None,
                                                        str(exc)))
                    col.finish(out)
                cmd.reply.put((True, None))
            elif cmd.kind == "cancel":
                rid, reason = cmd.payload
                cmd.reply.put((True, self.loop.cancel(rid, reason)))
            elif cmd.kind == "snapshot":
                cmd.reply.put((True, self.loop.snapshot()))
            elif cmd.kind == "capacity":
                cmd.reply.put((True, self.loop.runner.capacity()))
            elif cmd.kind == "reset":
                self.loop.fail_all("engine reset")
                self.loop.runner.reset()
                cmd.reply.put((True, None))
            elif cmd.kind == "close":
                self.loop.fail_all("engine closed")
                self.loop.runner.close()
                cmd.reply.put((True, None))
                return False
            else:
                cmd.reply.put((False, ValueError(f"unknown command {cmd.kind}")))
        except Exception as exc:  # a failing control command must not kill the driver
            try:
                cmd.reply.put_nowait((False, exc))
            except queue.Full:
                pass
        return True

    def _drive(self) -> None:
        # The CUDA "current device" is per thread and starts at device 0: bind this thread to the runner's
        # device before it launches anything (on rank r > 0 the model lives on another GPU).
        try:
            dev = getattr(self.loop.runner, "device", None)
            if dev is not None and getattr(dev, "type", "cpu") == "cuda" and dev.index is not None:
                import torch
                torch.cuda.set_device(dev)
            if self.coord is not None:
                if self.coord.is_leader:
                    self._drive_leader()
                else:
                    self._drive_follower()
                return
            while True:
                drained = 0
                while drained < 64:
                    try:
                        cmd = self.commands.get_nowait()
                    except queue.Empty:
                        break
                    drained += 1
                    if not self._serve(cmd):
                        return
                if self.loop.idle():
                    self._wake.wait(timeout=0.05)
                    self._wake.clear()
                    continue
                self.loop.tick()
        except BaseException as exc:  # fatal: record, fail everything, stop
            if self.coord is not None and self.coord.is_leader:
                try:
                    self.coord.publish({"cmds": [], "tick": False, "stop": True})   # never blocks on a follower
                except Exception:
                    pass
            tb = traceback.extract_tb(exc.__traceback__)
            loc = f"{tb[-1].filename}:{tb[-1].lineno}" if tb else "?"
            self.unhealthy = {"exception_type": type(exc).__name__, "message": str(exc), "location": loc,
                              "cause_type": type(exc.__cause__).__name__ if exc.__cause__ else None,
                              "request_ids": list(self.loop.sched.active), "at": time.time()}
            self.recorder.record("fatal", exception=type(exc).__name__, message=str(exc), location=loc)
            self.unhealthy["recent_events"] = self.recorder.dump(last=32)
            try:
                self.loop.fail_all(f"engine_unavailable: {type(exc).__name__}: {exc}")
            except Exception:
                pass
            for col in list(self.collectors.values()):
                if not col.done.is_set():
                    out = GenerationOutput(col.rid or 0, [], [], None, FinishDetails("error", message=str(exc)),
                                           None, error=f"engine_unavailable: {exc}")
                    col.put_chunk(GenerationStreamChunk(col.rid or 0, [], None, True, out.finish, None, None,
                                                        out.error))
                    col.finish(out)
            self.collectors.clear()


    # ------------------------------------------------------------------ parallel group: leader / follower loops
    _REPLICATED = ("submit", "cancel", "reset", "close")

    def _apply_replicated(self, kind: str, payload) -> Any:
        """The part of a command that every rank performs (device / scheduler state); returns its result."""
        if kind == "submit":
            return self.loop.submit(payload)
        if kind == "cancel":
            return self.loop.cancel(payload[0], payload[1])
        if kind == "reset":
            self.loop.fail_all("engine reset")
            self.loop.runner.reset()
            return None
        if kind == "close":
            self.loop.fail_all("engine closed")
            self.loop.runner.close()
            return None
        raise ValueError(kind)

    def _drive_leader(self) -> None:
        from ..parallel.serving import portable_request
        last_beat = time.time()
        while True:
            local: List[_Command] = []
            while len(local) < 64:
                try:
                    local.append(self.commands.get_nowait())
                except queue.Empty:
                    break
            wire: List[Tuple[str, Any]] = []
            todo: List[Tuple[_Command, Any]] = []
            for cmd in local:
                if cmd.kind not in self._REPLICATED:
                    self._serve(cmd)                      # snapshot / capacity: answered from rank 0's own state
                elif cmd.kind == "submit":
                    req, col = cmd.payload
                    self.collectors[req.request_id] = col
                    wire.append(("submit", portable_request(req)))
                    todo.append((cmd, req))
                else:
                    wire.append((cmd.kind, cmd.payload))
                    todo.append((cmd, cmd.payload))
            expired = self.loop.expired()
            for rid, reason in expired:
                wire.append(("cancel", (rid, reason)))
            self.coord.check_followers()      # a lost rank is found here, on the host, before the next launch
            idle = self.loop.idle() and not wire
            if idle:
                if time.time() - last_beat > 1.0:          # heartbeat: followers learn that rank 0 is alive
                    self.coord.publish({"cmds": [], "tick": False, "stop": False})
                    last_beat = time.time()
                self._wake.wait(timeout=0.05)
                self._wake.clear()
                continue
            stop = any(k == "close" for k, _ in wire)
            self.coord.publish({"cmds": wire, "tick": not stop, "stop": stop})
            last_beat = time.time()
            for cmd, payload in todo:
                try:
                    if cmd.kind == "submit":
                        try:
                            self.loop.submit(payload)
                        except GenerationAdmissionRejected as exc:
                            col = self.collectors.pop(payload.request_id, None)
                            out = GenerationOutput(payload.request_id, list(payload.prompt_token_ids), [], None,
                                                   FinishDetails("error", message=str(exc)), None, error=str(exc))
                            if col is not None:
                                col.put_chunk(GenerationStreamChunk(payload.request_id, [], None, True, out.finish,
                                                                    None, None, str(exc)))
                                col.finish(out)
                        cmd.reply.put((True, None))
                    else:
                        cmd.reply.put((True, self._apply_replicated(cmd.kind, payload)))
                except Exception as exc:
                    try:
                        cmd.reply.put_nowait((False, exc))
                    except queue.Full:
                        pass
            for rid, reason in expired:
                self.loop.cancel(rid, reason)
            if stop:
                return
            self.loop.tick()

    def _drive_follower(self) -> None:
        self.loop.on_event = self._on_event_follower
        while True:
            # callers on this rank (SPMD use of the API) only register their collectors; rank 0's batch drives
            while True:
                try:
                    cmd = self.commands.get_nowait()
                except queue.Empty:
                    break
                if cmd.kind == "submit":
                    req, col = cmd.payload
                    done = self.orphans.pop(req.request_id, None)
                    if done is not None:
                        col.put_chunk(GenerationStreamChunk(req.request_id, list(done.token_ids), None, True,
                                                            done.finish, None, done.telemetry, done.error))
                        col.finish(done)
                    else:
                        self.collectors[req.request_id] = col
                    cmd.reply.put((True, None))
                elif cmd.kind in ("snapshot", "capacity"):
                    self._serve(cmd)
                else:
                    cmd.reply.put((True, None))          # cancel / reset / close: decided by rank 0
            batch = self.coord.receive()
            for kind, payload in batch.get("cmds", []):
                try:
                    self._apply_replicated(kind, payload)
                except GenerationAdmissionRejected:
                    pass                                  # rank 0 rejected it too and told its caller
            if batch.get("stop"):
                # answer whatever this rank's own callers queued meanwhile (their close() waits for a reply)
                while True:
                    try:
                        cmd = self.commands.get_nowait()
                    except queue.Empty:
                        break
                    try:
                        cmd.reply.put_nowait((True, None))
                    except queue.Full:
                        pass
                self.stopped_by_leader = True
                return
            if batch.get("tick"):
                self.loop.tick()


def build_engine(weights, backend: str, config: EngineConfig, tokenizer=None) -> EngineService:
    """weights + backend -> runner -> loop -> service."""
    eos = getattr(tokenizer, "eos_token_id", None)
    if backend == "cpu_reference":
        from .runner import CpuReferenceRunner
        runner = CpuReferenceRunner(weights, config, eos)
    elif config.parallel.tp > 1 or config.parallel.ep > 1:
        # SPMD serving: this process is one rank of a torchrun job; every rank builds the same engine over its own
        # weight shard and must be driven with identical requests (the collectives inside the executor keep the
        # ranks in step).  Prefix caching is per rank and deterministic, so the ranks make the same decisions.
        from ..parallel.groups import init_distributed
        from ..parallel.tp import TPHybridExecutor
        from .gpu_runner import GpuRunner
        ctx = init_distributed()
        want = max(config.parallel.tp, config.parallel.ep)
        if ctx.world != want:
            raise RuntimeError(f"tensor/expert parallel size {want} needs a {want}-process job "
                               f"(python -m torch.distributed.run --nproc-per-node {want} ...); this job has "
                               f"{ctx.world} process(es)")
        n_snap = config.kv.max_snapshots if (config.kv.prefix_cache != "off" and weights.config.is_hybrid) else 0
        max_ctx = min(config.max_sequence_length, weights.config.max_context)
        pages_per_slot = (max_ctx + config.kv.page_tokens - 1) // config.kv.page_tokens
        n_slots = config.scheduler.max_active_requests
        from ..config import resolve_pool_pages
        n_pages = resolve_pool_pages(config.kv, weights.config.kv_bytes_per_token(), n_slots, pages_per_slot)
        ex = TPHybridExecutor(weights.to(ctx.device), ctx, max_slots=n_slots + n_snap, max_context=max_ctx,
                              n_pages=n_pages)
        runner = GpuRunner(None, config, eos, executor=ex)
        coord = None
        if ctx.world > 1:
            from ..parallel.serving import GroupCoordinator
            coord = GroupCoordinator(ctx.rank, ctx.world)
        return EngineService(EngineLoop(runner, config, tokenizer), config, coordinator=coord)
    else:
        from .gpu_runner import GpuRunner
        runner = GpuRunner(weights, config, eos)
    return EngineService(EngineLoop(runner, config, tokenizer), config)


def engine_from_runner(runner, config: EngineConfig, tokenizer=None, coordinator=None) -> EngineService:
    return EngineService(EngineLoop(runner, config, tokenizer), config, coordinator=coordinator)
