"""One step's batch as the kernels see it.

AIR runs prompt chunks and decoded tokens through different entry points and never in one
launch (src/runtime/serving.cpp:1821-1941; src/cuda/cuda_backend.cu:2890, 3072, 3249).  Here a
step is one flat list of tokens: any number of requests, each with one or more next tokens.
The context carries, per token, its id, its position and the index of its request in the
batch; per request, where its tokens start, its length after the step and its state slot.  All of
it is packed into one pinned int32 buffer and copied to the device once.  The block tables
stay on the device (one row per slot, kept by the cache manager); kernels find a token's
pages through its slot.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from types import SimpleNamespace
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import HostBatch


LAST_SAMPLED = -1   # as a token: "the token that the device sampled last for this request"


@dataclass
class Entry:
    request: Hashable
    tokens: Sequence[int]        # token ids; [LAST_SAMPLED] feeds back the device's last choice
    want: Sequence[int] = ()     # places among `tokens` whose logits are wanted


@dataclass
class StepContext:
    num_tokens: int
    num_seqs: int
    token_ids: torch.Tensor        # [T] int32
    positions: torch.Tensor        # [T] int32
    token_seq: torch.Tensor        # [T] int32: state slot of the token's request (-1: padding, skipped)
    q_start: torch.Tensor          # [S+1] int32
    kv_len: torch.Tensor           # [S] int32: length of the request after this step
    slots: torch.Tensor            # [S] int32: state slot of the request
    logit_rows: torch.Tensor       # [R] int32: flat indices of the tokens whose logits are wanted
    row_slots: torch.Tensor        # [R] int32: state slot of the request of each wanted row
    block_tables: List[torch.Tensor]   # per group: [slots, max_blocks] int32 (row = slot), -1 where no page
    status: Optional[torch.Tensor]     # [1] int32, set by kernels that meet an impossible index
    # host copies, for parts that plan on the host
    q_start_host: List[int] = field(default_factory=list)
    kv_len_host: List[int] = field(default_factory=list)
    slots_host: List[int] = field(default_factory=list)
    max_q_len: int = 0
    max_kv_len: int = 0
    all_decode: bool = False
    last_token: Optional[torch.Tensor] = None   # [slots] int32: the device's last choice per request
    plans: Dict[Hashable, SimpleNamespace] = field(default_factory=dict)
                                                # what the parts planned for this step (Part.plan), by plan key:
                                                # their int32 arrays as device tensors, their host values
    residual: Optional[torch.Tensor] = None     # [T, hidden] float32, set by the block that runs: a mixer or a
                                                # feed-forward may add its output into it (in 32-bit) and return
                                                # None instead of returning the output for the next norm to add


def build_context(entries: Sequence[Entry], cache, device, status=None, planners=()) -> StepContext:
    """Packs the batch.  `cache` is the CacheManager; every request is open and has its pages
    reserved for this step.  `planners`: the parts of the model that plan on the host, one per plan
    key (Model.planners()); their arrays travel in the same copy as the batch."""
    # (single next tokens, the many entries of a mixed step, are written as plain numbers: an array per entry
    # costs more than the whole rest of the packing)
    T = sum(len(e.tokens) for e in entries)
    S = len(entries)
    ids = np.empty(T, dtype=np.int32)
    pos = np.empty(T, dtype=np.int32)
    tseq = np.empty(T, dtype=np.int32)
    q_start = [0]
    kv_len: List[int] = []
    slots: List[int] = []
    lengths: List[int] = []
    rows: List[int] = []
    row_slots: List[int] = []
    at = 0
    for e in entries:
        seq = cache.sequences[e.request]
        n = len(e.tokens)
        if n == 1:
            t = int(e.tokens[0])
            ids[at] = t if t >= 0 else -(seq.slot + 1)
            pos[at] = seq.length
            tseq[at] = seq.slot
        elif n:
            t = np.asarray(e.tokens, dtype=np.int64)
            ids[at:at + n] = np.where(t >= 0, t, -(seq.slot + 1))
            pos[at:at + n] = np.arange(seq.length, seq.length + n, dtype=np.int32)
            tseq[at:at + n] = seq.slot
        for w in e.want:
            if not (0 <= w < n):
                raise ValueError(f"request {e.request!r}: wanted place {w} is not among its {n} tokens")
            rows.append(at + int(w))
            row_slots.append(seq.slot)
        at += n
        q_start.append(at)
        kv_len.append(seq.length + n)
        lengths.append(seq.length)
        slots.append(seq.slot)
    cache.flush_tables()
    sections = [ids, pos, tseq]
    sections += [np.asarray(x, dtype=np.int32) for x in (q_start, kv_len, slots, rows, row_slots)]
    planned = []      # (plan key, name, shape, section index), and the plans' host values
    values = {}
    if planners:
        batch = HostBatch(counts=[len(e.tokens) for e in entries], lengths=lengths, slots=slots, q_start=q_start)
        for part in planners:
            plan = part.plan(batch)
            if plan is None:
                continue
            key = part.plan_key()
            values[key] = dict(plan.values)
            for name, array in plan.arrays.items():
                array = np.ascontiguousarray(array, dtype=np.int32)
                planned.append((key, name, array.shape, len(sections)))
                sections.append(array.reshape(-1))
    total = sum(len(x) for x in sections)
    host = torch.empty(max(total, 1), dtype=torch.int32, pin_memory=(torch.device(device).type == "cuda"))
    view = host.numpy()
    offset = 0
    spans = []
    for x in sections:
        view[offset:offset + len(x)] = x
        spans.append((offset, len(x)))
        offset += len(x)
    dev = host.to(device, non_blocking=True)

    def cut(i):
        o, n = spans[i]
        return dev[o:o + n]

    plans = {key: SimpleNamespace(**v) for key, v in values.items()}
    for key, name, shape, i in planned:
        setattr(plans[key], name, cut(i).view(shape))
    return StepContext(
        num_tokens=T, num_seqs=S, token_ids=cut(0), positions=cut(1), token_seq=cut(2), q_start=cut(3),
        kv_len=cut(4), slots=cut(5), logit_rows=cut(6), row_slots=cut(7),
        block_tables=list(cache.tables), plans=plans,
        status=status, q_start_host=q_start, kv_len_host=kv_len, slots_host=slots,
        max_q_len=max((len(e.tokens) for e in entries), default=0), max_kv_len=max(kv_len, default=0),
        all_decode=all(len(e.tokens) == 1 for e in entries))
