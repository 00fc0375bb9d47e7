"""Pipeline parallelism over the text-layer axis: stage plans, boundary hand-off, stage walks.

The reference implements the pipeline as a same-process stage walk whose boundary hidden states travel through a
checksummed file (`--stage-layers SPEC --stage-handoff DIR`, src/core/stage_plan.h:66-160,
src/targets/qwen3_6/impl/runtime/text_context_impl.h:1720-1830): a correctness harness for the layer split.  Here the
same plan grammar drives

* `stage_walk_reference`: that same-process walk on the oracle model (file hand-off with FNV-1a check and the
  negative-control "cut"), and
* `PipelineStage`: one process per GPU, each holding a contiguous layer range; the residual stream [T, hidden] bf16
  moves to the next rank with NCCL point-to-point over NVLink, the last stage selects the tokens and broadcasts them.
"""
from __future__ import annotations

import os
import struct
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

MAX_STAGES = 64
MAX_LAYER = 4096
_MAGIC = b"NFBSTAGE"


class StagePlanError(ValueError):
    pass


@dataclass(frozen=True)
class StagePlan:
    """Contiguous ascending layer ranges covering [0, n_layers); ranges are half-open here, inclusive in the SPEC."""
    stages: Tuple[Tuple[int, int], ...]

    @property
    def world(self) -> int:
        return len(self.stages)

    @property
    def is_identity(self) -> bool:
        return len(self.stages) == 1

    @property
    def uniform(self) -> bool:
        return len({b - a for a, b in self.stages}) == 1

    def spec(self) -> str:
        return ",".join(f"{a}-{b - 1}" for a, b in self.stages)

    @staticmethod
    def parse(spec: str, n_layers: int) -> "StagePlan":
        """SPEC = `first-last[,first-last...]` with inclusive bounds, e.g. `0-31,32-63`.  Strict: a typo is refused."""
        if not spec:
            raise StagePlanError("refused-stage-layers: empty SPEC")
        out: List[Tuple[int, int]] = []
        for part in spec.split(","):
            a, sep, b = part.partition("-")
            if not sep or not a.isdigit() or not b.isdigit():
                raise StagePlanError(f"refused-stage-layers: '{part}' is not first-last")
            lo, hi = int(a), int(b)
            if lo > hi or hi > MAX_LAYER:
                raise StagePlanError(f"refused-stage-layers: '{part}' is not an ascending range below {MAX_LAYER}")
            out.append((lo, hi + 1))
        if len(out) > MAX_STAGES:
            raise StagePlanError(f"refused-stage-layers: more than {MAX_STAGES} stages")
        want = 0
        for lo, hi in out:
            if lo != want:
                raise StagePlanError(f"refused-stage-layers-partition: stage starting at {lo} does not continue layer {want}")
            want = hi
        if want != n_layers:
            raise StagePlanError(f"refused-stage-layers-partition: stages cover {want} layers, the model has {n_layers}")
        return StagePlan(tuple(out))

    @staticmethod
    def balanced(n_layers: int, n_stages: int, interval: int = 1) -> "StagePlan":
        """Even split; boundaries fall on multiples of `interval` (4 keeps every stage the same GDN / attention mix)."""
        if n_stages < 1 or n_stages > min(MAX_STAGES, n_layers):
            raise StagePlanError(f"refused-stage-layers-axis: cannot split {n_layers} layers into {n_stages} stages")
        units = n_layers // interval
        if units < n_stages:
            interval, units = 1, n_layers
        cuts = [round(i * units / n_stages) * interval for i in range(n_stages)] + [n_layers]
        return StagePlan(tuple((cuts[i], cuts[i + 1]) for i in range(n_stages)))


# ---------------------------------------------------------------------------------------- file hand-off
def fnv1a64(data: bytes) -> int:
    h = 0xCBF29CE484222325
    for chunk_start in range(0, len(data), 1 << 16):
        for b in data[chunk_start:chunk_start + (1 << 16)]:
            h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


def handoff_path(directory: str, boundary: int) -> str:
    return os.path.join(directory, f"stage_{boundary}.bin")


def write_handoff(directory: str, boundary: int, hidden: torch.Tensor) -> None:
    """Residual stream after stage `boundary` -> stage_<boundary>.bin (bf16 payload, FNV-1a 64 checked)."""
    os.makedirs(directory, exist_ok=True)
    t = hidden.detach().to(torch.bfloat16).cpu().contiguous()
    payload = t.view(torch.uint8).numpy().tobytes()
    head = _MAGIC + struct.pack("<IIQ", t.shape[0], t.shape[1], fnv1a64(payload))
    tmp = handoff_path(directory, boundary) + ".tmp"
    with open(tmp, "wb") as f:
        f.write(head + payload)
    os.replace(tmp, handoff_path(directory, boundary))


def read_handoff(directory: str, boundary: int, T: int, hidden: int) -> torch.Tensor:
    path = handoff_path(directory, boundary)
    try:
        with open(path, "rb") as f:
            blob = f.read()
    except OSError as e:
        raise StagePlanError(f"refused-stage-handoff: {path}: {e}") from e
    if len(blob) < 24 or blob[:8] != _MAGIC:
        raise StagePlanError(f"refused-stage-handoff: {path} is not a stage hand-off file")
    t, h, check = struct.unpack("<IIQ", blob[8:24])
    payload = blob[24:]
    if (t, h) != (T, hidden) or len(payload) != T * hidden * 2:
        raise StagePlanError(f"refused-stage-handoff: {path} holds [{t}, {h}], the stage expects [{T}, {hidden}]")
    if fnv1a64(payload) != check:
        raise StagePlanError(f"refused-stage-handoff: {path} fails its checksum")
    return torch.frombuffer(bytearray(payload), dtype=torch.bfloat16).view(T, hidden)


def stage_walk_reference(model, seq, ids: torch.Tensor, plan: StagePlan, handoff_dir: Optional[str] = None,
                         cut: bool = False) -> torch.Tensor:
    """Oracle forward as a walk over the plan's stages.  With `handoff_dir` every boundary goes through its file;
    `cut` skips the writes (the negative control: the next stage then reads a stale file or fails)."""
    x = None
    for k, (a, b) in enumerate(plan.stages):
        x = model.forward(seq, ids, layers=(a, b), hidden_in=x)
        if k + 1 < plan.world:
            if handoff_dir is not None:
                if not cut:
                    write_handoff(handoff_dir, k, x)
                x = read_handoff(handoff_dir, k, ids.shape[0], model.cfg.hidden).float()
            else:
                x = x.to(torch.bfloat16).float()
    return x


# ---------------------------------------------------------------------------------------- one stage per GPU
class PipelineStage:
    """This rank's stage of a pipeline over `group` (rank r runs plan.stages[r]).

    step(batch): the first stage embeds, every stage runs its layers on the native kernels, the residual stream moves
    to the next rank by NCCL send / recv (bf16 [T, hidden]); the last stage computes logits and arg-max ids and
    broadcasts them, so every rank returns the same ids."""

    def __init__(self, model, ws, kv, states, plan: StagePlan, rank: int, group=None):
        import torch.distributed as dist
        self.dist = dist
        self.model, self.ws, self.kv, self.states = model, ws, kv, states
        self.plan, self.rank, self.group = plan, rank, group
        if plan.world != dist.get_world_size(group):
            raise StagePlanError(f"refused-stage-layers-axis: {plan.world} stages for {dist.get_world_size(group)} ranks")
        self.first, self.end = plan.stages[rank]
        self.is_first, self.is_last = rank == 0, rank == plan.world - 1

    def step(self, batch) -> torch.Tensor:
        dist, m, ws = self.dist, self.model, self.ws
        T = batch.n_tokens
        if not self.is_first:
            dist.recv(ws.x[:T], src=dist.get_global_rank(self.group, self.rank - 1) if self.group is not None else self.rank - 1,
                      group=self.group)
        out = m.forward_hidden(ws, batch, self.kv, self.states, layers=(self.first, self.end))
        R = batch.logit_rows.numel()
        ids = ws.next_ids[:R]
        if self.is_last:
            if R:
                logits = m.logits(ws, batch, out)
                m.ops.argmax_rows(logits, ids, m.pdl)
        else:
            dist.send(ws.x[:T], dst=dist.get_global_rank(self.group, self.rank + 1) if self.group is not None else self.rank + 1,
                      group=self.group)
        if R:
            last = self.plan.world - 1
            dist.broadcast(ids, src=dist.get_global_rank(self.group, last) if self.group is not None else last, group=self.group)
        return ids
