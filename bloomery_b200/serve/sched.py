"""Slot board: resident sequences, the request queue, slot choice.

Rules of the reference (``crates/serve/src/sched.rs:5-23``): the oldest request goes first;
it takes the free slot that shares the longest prefix with its prompt, provided the shared
part is at least ``similarity`` (0.1) of the prompt; among equals an empty slot is
preferred; otherwise the least recently used free slot.  ``queue_depth`` bounds the queue.
"""
from __future__ import annotations

import collections
import dataclasses
import threading
import time
from typing import Deque, Dict, List, Optional, Sequence, Tuple

from .promptcache import common_prefix


@dataclasses.dataclass
class Slot:
    id: int
    ids: List[int] = dataclasses.field(default_factory=list)   # tokens whose KV the slot holds
    busy: bool = False
    last_used: float = 0.0
    request_id: Optional[int] = None
    n_decoded: int = 0
    t_start: float = 0.0

    def state(self) -> str:
        return "processing" if self.busy else "idle"


class QueueFull(Exception):
    pass


class Board:
    def __init__(self, n_slots: int, queue_depth: int = 64, similarity: float = 0.1):
        self.slots = [Slot(i) for i in range(n_slots)]
        self.queue: Deque = collections.deque()
        self.queue_depth = queue_depth
        self.similarity = similarity
        self.lock = threading.Lock()
        self.wake = threading.Condition(self.lock)
        self.deferred = 0

    def submit(self, req) -> None:
        with self.wake:
            if len(self.queue) >= self.queue_depth:
                raise QueueFull(f"queue of {self.queue_depth} is full")
            self.queue.append(req)
            self.wake.notify_all()

    def pick_slot(self, prompt: Sequence[int], want: Optional[int] = None) -> Optional[Tuple[Slot, int]]:
        """(slot, shared positions) for a prompt, or None when every slot is busy."""
        free = [s for s in self.slots if not s.busy]
        if want is not None:
            free = [s for s in free if s.id == want]
        if not free:
            return None
        best, best_key = None, None
        for s in free:
            n = common_prefix(s.ids, prompt)
            if n < self.similarity * max(1, len(prompt)):
                n = 0
            # longer shared prefix first; then empty slots; then least recently used
            key = (n, 1 if not s.ids else 0, -s.last_used)
            if best_key is None or key > best_key:
                best, best_key = s, key
        return best, best_key[0]

    def next_request(self):
        """Pop the oldest request for which a slot is free; returns (req, slot, shared) or None."""
        with self.lock:
            if not self.queue:
                return None
            req = self.queue[0]
            got = self.pick_slot(req.prompt_ids, getattr(req, "id_slot", None))
            if got is None:
                self.deferred += 1
                return None
            self.queue.popleft()
            slot, shared = got
            slot.busy = True
            slot.request_id = req.id
            slot.t_start = time.time()
            slot.n_decoded = 0
            return req, slot, shared

    def release(self, slot: Slot) -> None:
        with self.wake:
            slot.busy = False
            slot.request_id = None
            slot.last_used = time.time()
            self.wake.notify_all()

    def busy_count(self) -> int:
        return sum(1 for s in self.slots if s.busy)

    def snapshot(self) -> List[Dict[str, object]]:
        return [{"id": s.id, "is_processing": s.busy, "state": s.state(), "n_ctx_used": len(s.ids),
                 "n_decoded": s.n_decoded, "id_task": s.request_id} for s in self.slots]
