"""Artifact admission: decide BEFORE anything is uploaded whether a checkpoint can be served, and say why not.

Three checks, each a plain function over the scanned tensors and the geometry:

* role manifest   - which GGML block types each tensor role of the checkpoint uses;
* plan contract   - for every (role, block type) whether the decode GEMV, the tensor-core GEMM and the embedding
                    lookup read it in place, widen it once to bf16 at load (costs memory, listed), or cannot run it;
                    missing tensors of the geometry and shapes that the kernels' alignment rules exclude are listed as
                    unsupported operations; a digest of the planned weights identifies the plan;
* memory preflight - resident weight bytes (device layouts, widened tensors counted at 2 bytes per element) + KV pool
                    + recurrent-state slots + a scratch estimate against the free device memory.

``admit`` runs all three and raises ``ArtifactRejected`` with the full list of reasons.  This is the role of the
reference's GGUF admission (``hipengine/loading/qwen35_gguf_admission.py``: role manifest ``:686-766``, operation
coverage and plan contract ``:858-1830``) reduced to one backend and one kernel per operation.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from ..quant.ggml import GGMLType

# block types the kernels read in place (ops/kernels.py::_KERNEL_QTYPES); everything else GGML defines and
# quant/ggml.py can dequantise is widened to bf16 once at load
IN_PLACE = {GGMLType.Q4_K, GGMLType.Q6_K, GGMLType.Q8_0, GGMLType.F32, GGMLType.F16, GGMLType.BF16}
WIDENED = {GGMLType.Q4_0, GGMLType.Q4_1, GGMLType.Q5_0, GGMLType.Q5_1, GGMLType.Q5_K}


class ArtifactRejected(RuntimeError):
    def __init__(self, reasons: List[str], report: Dict[str, Any]):
        super().__init__("checkpoint not admitted: " + "; ".join(reasons))
        self.reasons, self.report = reasons, report


def role_of(name: str) -> str:
    """Tensor role: the name without its layer index (``blk.7.ffn_down.weight`` -> ``ffn_down``)."""
    parts = name.split(".")
    if parts[0] == "blk" and len(parts) > 2:
        parts = parts[2:]
    if parts and parts[-1] in ("weight", "bias"):
        suffix = "" if parts[-1] == "weight" else ".bias"
        parts = parts[:-1]
        return ".".join(parts) + suffix
    return ".".join(parts)


def build_role_manifest(weights) -> Dict[str, Dict[str, int]]:
    """role -> {block type name: tensor count}."""
    out: Dict[str, Dict[str, int]] = {}
    for name, t in weights.tensors.items():
        d = out.setdefault(role_of(name), {})
        key = GGMLType(t.ggml_type).name
        d[key] = d.get(key, 0) + 1
    return out


@dataclass(frozen=True)
class UnsupportedOperation:
    slot: str
    qtype: str
    operation: str
    reason: str

    def as_dict(self) -> Dict[str, str]:
        return {"slot": self.slot, "qtype": self.qtype, "operation": self.operation, "reason": self.reason}


@dataclass
class PlanContract:
    records: List[str] = field(default_factory=list)            # one line per planned weight
    unsupported: List[UnsupportedOperation] = field(default_factory=list)
    widened: List[str] = field(default_factory=list)            # tensors widened to bf16 at load
    resident_bytes: int = 0

    @property
    def is_complete(self) -> bool:
        return not self.unsupported

    @property
    def digest(self) -> str:
        h = hashlib.sha256()
        for r in sorted(self.records):
            h.update(r.encode())
            h.update(b"\n")
        return h.hexdigest()[:16]


def _required_tensors(cfg) -> List[str]:
    need = ["token_embd.weight", "output_norm.weight"]
    for i in range(cfg.n_layers):
        need.append(f"blk.{i}.attn_norm.weight")
        if cfg.arch.startswith("qwen35") and not cfg.is_full_attention_layer(i):
            need += [f"blk.{i}.attn_qkv.weight", f"blk.{i}.ssm_out.weight", f"blk.{i}.ssm_conv1d.weight"]
        elif cfg.arch != "gemma4":
            need += [f"blk.{i}.attn_q.weight", f"blk.{i}.attn_k.weight", f"blk.{i}.attn_v.weight",
                     f"blk.{i}.attn_output.weight"]
    return need


def plan_contract(weights) -> PlanContract:
    cfg = weights.config
    pc = PlanContract()
    have = weights.tensors
    for name in _required_tensors(cfg):
        if name not in have:
            pc.unsupported.append(UnsupportedOperation(name, "-", "load", "tensor missing from the checkpoint"))
    for name, t in have.items():
        qt = GGMLType(t.ggml_type)
        matrix = len(t.shape) >= 2
        rows = 1
        for d in t.shape[:-1]:
            rows *= int(d)
        cols = int(t.shape[-1])
        if qt in IN_PLACE:
            mode = "in_place"
            nbytes = int(t.raw.numel())
            if qt == GGMLType.Q6_K:
                nbytes = nbytes // 210 * 224            # device blocks are padded to 224 bytes
        elif qt in WIDENED:
            mode = "widened_bf16"
            nbytes = rows * cols * 2
            pc.widened.append(name)
        else:
            pc.unsupported.append(UnsupportedOperation(name, qt.name, "dequantise", "block type without a reader"))
            continue
        if matrix and qt in (GGMLType.Q4_K, GGMLType.Q6_K) and cols % 256 != 0:
            pc.unsupported.append(UnsupportedOperation(name, qt.name, "gemv/gemm",
                                                       f"row length {cols} is not a whole number of 256-wide blocks"))
        if matrix and qt == GGMLType.Q8_0 and cols % 32 != 0:
            pc.unsupported.append(UnsupportedOperation(name, qt.name, "gemv/gemm",
                                                       f"row length {cols} is not a whole number of 32-wide blocks"))
        pc.resident_bytes += nbytes
        pc.records.append(f"{name}|{qt.name}|{'x'.join(str(int(d)) for d in t.shape)}|{mode}")
    return pc


def memory_preflight(weights, engine_config, free_bytes: Optional[int], contract: Optional[PlanContract] = None
                     ) -> Dict[str, Any]:
    cfg = weights.config
    pc = contract or plan_contract(weights)
    kvc, sched = engine_config.kv, engine_config.scheduler
    max_ctx = min(engine_config.max_sequence_length, cfg.max_context)
    pages_per_slot = -(-max_ctx // kvc.page_tokens)
    n_slots = sched.max_active_requests
    from ..config import resolve_pool_pages
    n_pages = resolve_pool_pages(kvc, cfg.kv_bytes_per_token(), n_slots, pages_per_slot)
    kv_bytes = n_pages * kvc.page_tokens * cfg.kv_bytes_per_token()
    n_snap = kvc.max_snapshots if (kvc.prefix_cache != "off" and cfg.is_hybrid) else 0
    state_bytes = (n_slots + n_snap) * cfg.recurrent_state_bytes()
    # scratch of one 4096-row prefill chunk: a dozen [rows, widest projection] bf16/fp32 buffers + logits rows
    widest = max(cfg.hidden, 2 * getattr(cfg, "ffn", cfg.hidden), getattr(cfg, "linear_qkv_width", 0) or 0)
    scratch_bytes = 4096 * widest * 2 * 6 + 4096 * cfg.hidden * 4 * 4 + 64 * cfg.vocab * 4
    reserve_bytes = int(getattr(kvc, "memory_reserve_mib", 0)) << 20    # what has to stay free after everything
    need = pc.resident_bytes + kv_bytes + state_bytes + scratch_bytes
    fits = free_bytes is None or need + reserve_bytes <= free_bytes
    return {"weight_bytes": pc.resident_bytes, "kv_pool_bytes": int(kv_bytes), "kv_pool_pages": int(n_pages),
            "recurrent_state_bytes": int(state_bytes), "scratch_estimate_bytes": int(scratch_bytes),
            "required_bytes": int(need), "reserve_bytes": reserve_bytes, "free_bytes": free_bytes, "fits": bool(fits)}


def dominant_block_type(weights) -> str:
    """Block type holding most of the checkpoint's bytes among its matrices (what ``--quant`` is checked against)."""
    by: Dict[str, int] = {}
    for t in weights.tensors.values():
        if len(t.shape) >= 2:
            k = GGMLType(t.ggml_type).name
            by[k] = by.get(k, 0) + int(t.raw.numel())
    return max(by, key=by.get) if by else "-"


def admit(weights, engine_config, free_bytes: Optional[int] = None, strict: bool = True,
          expected_quant: Optional[str] = None) -> Dict[str, Any]:
    """Full admission report; raises ``ArtifactRejected`` (when ``strict``) if the plan is incomplete or does not fit."""
    pc = plan_contract(weights)
    mem = memory_preflight(weights, engine_config, free_bytes, pc)
    report = {"arch": weights.config.arch, "plan_complete": pc.is_complete, "plan_digest": pc.digest,
              "planned_weights": len(pc.records), "widened_to_bf16": len(pc.widened),
              "unsupported": [u.as_dict() for u in pc.unsupported[:32]], "memory": mem,
              "role_manifest": build_role_manifest(weights)}
    reasons = [f"{u.slot} ({u.qtype}): {u.operation}: {u.reason}" for u in pc.unsupported[:8]]
    report["dominant_block_type"] = dominant_block_type(weights)
    if expected_quant and expected_quant.upper().replace("_M", "").replace("_S", "") != report["dominant_block_type"]:
        reasons.append(f"expected {expected_quant} weights, the checkpoint is mostly {report['dominant_block_type']}")
    if not mem["fits"]:
        reasons.append(f"needs {mem['required_bytes'] / 2**30:.1f} GiB (weights {mem['weight_bytes'] / 2**30:.1f}, KV "
                       f"{mem['kv_pool_bytes'] / 2**30:.1f}, state {mem['recurrent_state_bytes'] / 2**30:.1f}), "
                       f"{mem['reserve_bytes'] / 2**30:.1f} to stay free, {(free_bytes or 0) / 2**30:.1f} GiB free")
    report["admitted"] = not reasons
    if reasons and strict:
        raise ArtifactRejected(reasons, report)
    return report
