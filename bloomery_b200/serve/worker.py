"""Engine thread and generation loop.

One thread owns the engine (``worker.rs:521,723`` in the reference).  Each round it
(1) admits queued requests into free slots (prompt-cache lookup, prefix reuse by ``cut``,
``share_prefix`` or ``restore``), (2) feeds one planned prompt chunk per starting request
(cut on the prompt quantum while other slots decode, ``worker.rs:45-51``), and (3) runs **one
decode round for all busy slots** as rows of one engine pass (``worker.rs:1047-1210``).
Per request the loop samples (``sampler.py``), applies stop rules, the reasoning split and
constraints, and pushes events to the HTTP thread (``genloop.rs``).
"""
from __future__ import annotations

import collections
import dataclasses
import itertools
import math
import queue
import sys
import threading
import time
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np

from .engine import Engine, EngineError
from .promptcache import PromptCache, common_prefix
from .sampler import Sampler, SamplingParams
from .sched import Board, QueueFull, Slot
from .tokenizer import StreamDecoder

_ids = itertools.count(1)


@dataclasses.dataclass
class Request:
    prompt_ids: List[int]
    sampling: SamplingParams = dataclasses.field(default_factory=SamplingParams)
    n_predict: int = -1
    stop: List[str] = dataclasses.field(default_factory=list)
    stream: bool = False
    cache_prompt: bool = True
    n_probs: int = 0
    ignore_eos: bool = False
    id_slot: Optional[int] = None
    constraint: Any = None                  # object with allowed(text_so_far, piece) -> bool and done(text) -> bool
    logit_bias: Dict[int, float] = dataclasses.field(default_factory=dict)
    t_max_predict_ms: float = 0.0
    endpoint: str = ""                      # the route that made the request (the per-request log line names it)
    reasoning_budget: int = -1              # generated ids the think span may take (-1: no budget)
    reasoning_loop: bool = False            # end a think span that repeats itself
    think_started: bool = False             # the template already opened the think span
    pick_rows: Optional[List[Tuple[int, np.ndarray]]] = None   # when a list: (length of the text so far, logits row) of each
                                                               # pick the constraint's walk read a row for
    id: int = dataclasses.field(default_factory=lambda: next(_ids))
    events: "queue.Queue" = dataclasses.field(default_factory=queue.Queue)
    cancelled: threading.Event = dataclasses.field(default_factory=threading.Event)
    created: float = dataclasses.field(default_factory=time.time)


@dataclasses.dataclass
class Active:
    req: Request
    slot: Slot
    sampler: Sampler
    decoder: StreamDecoder
    n_past: int = 0                 # positions of the prompt already in the slot
    n_cached: int = 0
    generated: List[int] = dataclasses.field(default_factory=list)
    text: str = ""
    sent: int = 0                   # characters of `text` already streamed
    pending_token: Optional[int] = None
    t_prompt0: float = 0.0
    t_prompt1: float = 0.0
    t_first: float = 0.0
    probs: List[dict] = dataclasses.field(default_factory=list)
    stop_type: str = ""
    stop_word: str = ""
    cache_ms: float = 0.0
    draft_n: int = 0
    n_drawn: int = 0              # uniforms consumed by the card's sampler for this request
    draft_accepted: int = 0


class Metrics:
    def __init__(self):
        self.lock = threading.Lock()
        self.c: Dict[str, float] = collections_default()

    def add(self, name: str, v: float = 1.0):
        with self.lock:
            self.c[name] = self.c.get(name, 0.0) + v

    def get(self, name: str) -> float:
        return self.c.get(name, 0.0)


def collections_default() -> Dict[str, float]:
    return {"prompt_tokens_total": 0.0, "prompt_seconds_total": 0.0, "tokens_predicted_total": 0.0,
            "tokens_predicted_seconds_total": 0.0, "n_decode_total": 0.0, "n_busy_slots_per_decode": 0.0,
            "requests_total": 0.0, "requests_failed_total": 0.0, "round_seconds_total": 0.0,
            "prompt_cache_hits_total": 0.0, "prompt_cache_tokens_total": 0.0, "draft_tokens_total": 0.0,
            "draft_accepted_total": 0.0}


class Worker(threading.Thread):
    def __init__(self, engine: Engine, board: Board, cache: PromptCache, prompt_quantum: int = 2048,
                 on_fatal: Optional[Callable[[BaseException], None]] = None):
        super().__init__(name="serve-engine", daemon=True)
        self.engine, self.board, self.cache = engine, board, cache
        self.prompt_quantum = prompt_quantum
        self.active: Dict[int, Active] = {}
        self.stop_flag = threading.Event()
        self.metrics = Metrics()
        self.rounds_by_width: Dict[int, int] = {}
        self.round_seconds_by_width: Dict[int, float] = {}
        self.round_card_wait_by_width: Dict[int, float] = {}          # the part of a round the engine waited for the card
        self.draft_by_depth: Dict[int, int] = {}        # drafted ids by their place in the draft
        self.accepted_by_depth: Dict[int, int] = {}
        self.on_fatal = on_fatal
        self.failed: Optional[BaseException] = None
        self.draft = None                       # runtime.speculative.NgramDraft (or another source with .propose)
        self.width = None                       # runtime.speculative.WidthChooser
        self.actions: "queue.Queue" = queue.Queue()     # slot actions run on the engine thread
        self.log_requests = True
        self.generating_every = 30.0            # seconds between the short lines of a request that is still generating

    # ---------------------------------------------------------------- admission
    def _admit(self) -> None:
        while True:
            got = self.board.next_request()
            if got is None:
                return
            req, slot, shared = got
            if req.cancelled.is_set():
                self.board.release(slot)
                continue
            ids = req.prompt_ids
            if len(ids) >= self.engine.slot_ctx:
                req.events.put(("error", 400, f"the prompt of {len(ids)} tokens exceeds the slot context of {self.engine.slot_ctx}"))
                self.board.release(slot)
                continue
            a = Active(req, slot, Sampler(req.sampling), StreamDecoder(self.engine.tokenizer))
            a.t_prompt0 = time.time()
            a.forced_ids = collections.deque()
            a.span = None
            if req.reasoning_budget >= 0 or req.reasoning_loop:
                from .reasoning import ThinkSpan
                a.span = ThinkSpan(started=req.think_started, budget=req.reasoning_budget, watch_loop=req.reasoning_loop)
                if a.span.force_close(""):                        # a budget of 0 closes an opened span before its first id
                    a.forced_ids.extend(self.engine.tokenizer.encode(a.span.close_tag, parse_special=True, add_bos=False))
            keep = shared if req.cache_prompt else 0
            # a longer match in another slot (shared KV pages) or in the host cache beats the slot's own prefix
            if req.cache_prompt:
                donor, dn = None, keep
                for other in self.board.slots:
                    if other is not slot:
                        n = common_prefix(other.ids, ids)
                        if n > dn:
                            donor, dn = other, n
                if donor is not None:
                    got_n = self.engine.share_prefix(donor.id, slot.id, dn, keep)
                    if got_n > keep:
                        slot.ids = list(donor.ids[:got_n])
                        keep = got_n
                t0 = time.time()
                saved, sn = self.cache.lookup(ids, at_least=keep + 1)
                if saved is not None and sn > keep:
                    got_n = self.engine.restore(slot.id, saved, sn)
                    if got_n > keep:
                        slot.ids = list(saved.ids[:got_n])
                        keep = got_n
                        self.metrics.add("prompt_cache_hits_total")
                a.cache_ms = (time.time() - t0) * 1e3
                self.cache.seconds += time.time() - t0
            keep = min(keep, len(ids) - 1)         # at least one prompt token is always evaluated
            keep = max(keep, 0)
            self.engine.cut(slot.id, keep)
            slot.ids = list(ids[:keep])
            a.n_past = a.n_cached = keep
            self.metrics.add("prompt_cache_tokens_total", keep)
            self.active[slot.id] = a

    # ---------------------------------------------------------------- prompt
    def _feed_prompt(self, a: Active) -> None:
        ids = a.req.prompt_ids
        todo = len(ids) - 1 - a.n_past          # the last prompt token goes through the decode round
        if todo <= 0:
            a.pending_token = ids[-1]
            a.t_prompt1 = time.time()
            return
        others_decoding = any(o.pending_token is not None for o in self.active.values() if o is not a)
        n = min(todo, self.prompt_quantum) if others_decoding else todo
        self.engine.prefill(a.slot.id, ids[a.n_past:a.n_past + n], a.n_past)
        a.slot.ids += ids[a.n_past:a.n_past + n]
        a.n_past += n
        if a.n_past >= len(ids) - 1:
            a.pending_token = ids[-1]
            a.t_prompt1 = time.time()

    # ---------------------------------------------------------------- decode
    def _finish(self, a: Active, stop_type: str, word: str = "") -> None:
        a.stop_type, a.stop_word = stop_type, word
        tail = a.decoder.flush()
        if tail and stop_type != "word":
            a.text += tail
        self._flush_text(a, final=True)
        now = time.time()
        n_prompt = len(a.req.prompt_ids)
        prompt_ms = max(0.0, (a.t_prompt1 - a.t_prompt0) * 1e3)
        pred_ms = max(0.0, (now - (a.t_first or now)) * 1e3)
        timings = {"cache_n": a.n_cached, "prompt_n": n_prompt - a.n_cached, "prompt_ms": prompt_ms,
                   "prompt_per_second": (n_prompt - a.n_cached) / max(prompt_ms / 1e3, 1e-9),
                   "predicted_n": len(a.generated), "predicted_ms": pred_ms,
                   "predicted_per_second": len(a.generated) / max(pred_ms / 1e3, 1e-9), "cache_ms": a.cache_ms,
                   "draft_n": a.draft_n, "draft_n_accepted": a.draft_accepted}
        a.req.events.put(("done", {"stop_type": stop_type, "stopping_word": word, "tokens_predicted": len(a.generated),
                                   "tokens_evaluated": n_prompt, "tokens_cached": a.n_cached, "timings": timings,
                                   "text": a.text, "tokens": list(a.generated), "probs": a.probs,
                                   "truncated": False, "id_slot": a.slot.id}))
        self._log_request(a, stop_type, n_prompt, prompt_ms, pred_ms)
        m = self.metrics
        m.add("requests_total"); m.add("prompt_tokens_total", n_prompt - a.n_cached); m.add("prompt_seconds_total", prompt_ms / 1e3)
        m.add("tokens_predicted_total", len(a.generated)); m.add("tokens_predicted_seconds_total", pred_ms / 1e3)
        if a.req.cache_prompt and a.slot.ids:
            t0 = time.time()
            self.cache.put(self.engine.snapshot(a.slot.id, a.slot.ids))
            self.cache.seconds += time.time() - t0
        del self.active[a.slot.id]
        self.board.release(a.slot)

    REASONS = {"eos": "eos", "word": "stop", "limit": "length", "cancelled": "cancel", "reasoning_loop": "reasoning_loop"}

    def _log_request(self, a: Active, stop_type: str, n_prompt: int, prompt_ms: float, pred_ms: float) -> None:
        """One stderr line a request when its generation ends (``docs/serving.md:466-470`` of the reference): what was
        evaluated and reused, both rates, why it stopped, how full the slot's context is."""
        if not self.log_requests:
            return
        new = n_prompt - a.n_cached
        g = len(a.generated)
        line = (f"bloomery-serve: request {a.req.id} {a.req.endpoint or '-'}: prompt {n_prompt} ids ({a.n_cached} reused) in "
                f"{prompt_ms / 1e3:.3f} s, {new / max(prompt_ms / 1e3, 1e-9):.1f} ids/s; generated {g} ids in {pred_ms / 1e3:.3f} s, "
                f"{g / max(pred_ms / 1e3, 1e-9):.1f} ids/s; stop {self.REASONS.get(stop_type, 'error')}; "
                f"ctx {len(a.slot.ids)}/{self.engine.slot_ctx}")
        print(line, file=sys.stderr, flush=True)
        ring = getattr(self, "request_lines", None)
        if ring is not None:
            ring.push(line)                         # the live view's last requests

    def _log_generating(self) -> None:
        """A request that has generated for more than ``generating_every`` seconds says so, and again every such span."""
        if not self.log_requests or not self.active:
            return
        now = time.time()
        for a in self.active.values():
            since = getattr(a, "t_logged", None) or a.t_first
            if since and now - since >= self.generating_every:
                a.t_logged = now
                print(f"bloomery-serve: request {a.req.id} {a.req.endpoint or '-'}: generating, {len(a.generated)} ids in "
                      f"{now - a.t_first:.0f} s", file=sys.stderr, flush=True)

    def _flush_text(self, a: Active, final: bool = False) -> None:
        if not a.req.stream:
            return
        # hold back a tail that could still grow into a stop string
        hold = 0
        if not final:
            for s in a.req.stop:
                for k in range(min(len(s) - 1, len(a.text) - a.sent), 0, -1):
                    if a.text.endswith(s[:k]):
                        hold = max(hold, k)
                        break
        upto = len(a.text) - hold
        if upto > a.sent:
            a.req.events.put(("text", a.text[a.sent:upto]))
            a.sent = upto

    def _pick(self, a: Active, greedy: int, logits: Optional[np.ndarray]) -> int:
        if getattr(a, "forced_ids", None):
            return int(a.forced_ids.popleft())               # text written for the model (the think span's closing tag)
        return self._pick_free(a, greedy, logits)

    def _pick_free(self, a: Active, greedy: int, logits: Optional[np.ndarray]) -> int:
        req = a.req
        if logits is None:
            return greedy
        row = logits
        if req.logit_bias or (req.ignore_eos and self.engine.tokenizer.eos_id >= 0):
            row = row.copy()
            for t, b in req.logit_bias.items():
                if 0 <= t < row.size:
                    row[t] = row[t] + b
            if req.ignore_eos:
                for t in (self.engine.tokenizer.eos_id, self.engine.tokenizer.eot_id):
                    if t >= 0:
                        row[t] = -np.inf
        recent = a.slot.ids[-max(req.sampling.repeat_last_n, 0):] if req.sampling.repeat_last_n else []
        watch_free = getattr(req.constraint, "free", None)
        if req.constraint is not None and not (watch_free is not None and watch_free(a.text)):
            tok = self._constrained_pick(a, row, recent)
        else:
            tok = a.sampler.sample(row, recent)
        if req.n_probs > 0:
            row = logits                        # the probabilities reported are the model's own row, before any bias
            top = np.argpartition(-row, min(req.n_probs, row.size - 1))[:req.n_probs]
            top = top[np.argsort(-row[top], kind="stable")]
            mx = float(np.max(row))
            lse = mx + math.log(float(np.exp((row - mx).astype(np.float64)).sum()))
            tk = self.engine.tokenizer
            a.probs.append({"id": int(tok), "token": tk.decode([int(tok)], skip_special=False), "logprob": float(row[tok]) - lse,
                            "top_logprobs": [{"id": int(t), "token": tk.decode([int(t)], skip_special=False),
                                              "logprob": float(row[t]) - lse} for t in top]})
        return tok

    def _constrained_pick(self, a: Active, row: np.ndarray, recent) -> int:
        """Masked pick: best-first over candidates until one keeps the output a valid prefix.  A segment program
        (``serve/constrain.py``) that knows the literal text every continuation shares is not asked about candidates at
        all: the first canonical token of that text is taken without reading the row (the jump arm)."""
        tk = self.engine.tokenizer
        forced = getattr(a.req.constraint, "forced_text", None)
        if forced is not None:
            text = forced(a.text)
            if text:
                ids = tk.encode(text, parse_special=False, add_bos=False)
                if ids:
                    piece = tk.decode([int(ids[0])], skip_special=True)
                    if piece and text.startswith(piece):
                        self.jumped = getattr(self, "jumped", 0) + 1
                        return int(ids[0])
        if a.req.pick_rows is not None:
            a.req.pick_rows.append((len(a.text), np.array(row, dtype=np.float32, copy=True)))

        def fits(t: int) -> bool:
            if tk.is_eog(t):
                return a.req.constraint.done(a.text)
            piece = tk.decode([t], skip_special=True)
            return bool(piece) and a.req.constraint.allowed(a.text, piece)
        sp = a.req.sampling
        if sp.temperature > 0 or sp.penalizes:
            # a positive temperature or a penalty draws with the request's own sampler from the masked row: the ids the
            # constraint allows among the best 256 keep their logits, every other id is out
            n_head = min(256, row.size)
            head = np.argpartition(-row, n_head - 1)[:n_head] if row.size > n_head else np.arange(row.size)
            keep = [int(t) for t in head if fits(int(t))]
            if keep:
                masked = np.full(row.size, -np.inf, dtype=np.float32)
                masked[keep] = row[keep]
                return int(a.sampler.sample(masked, recent))
        # the best 256 first (a partial sort); the whole row is sorted only when none of them fits
        if row.size > 512:
            head = np.argpartition(-row, 255)[:256]
            head = head[np.lexsort((head, -row[head]))]               # by logit, the lower id first on a tie
        else:
            head = np.argsort(-row, kind="stable")
        for t in head:
            if fits(int(t)):
                return int(t)
        if row.size > 512:
            for t in np.argsort(-row, kind="stable")[head.size:]:
                if fits(int(t)):
                    return int(t)
        return int(head[0])

    def enable_drafting(self, draft, width) -> None:
        """Turn on speculative decoding for greedy requests (``BLOOMERY_DRAFT``)."""
        self.draft, self.width = draft, width

    def _can_draft(self, a: Active) -> bool:
        r = a.req
        # greedy, biased, masked and probability-reporting requests draft alike (the kept ids are the request's own picks),
        # and so do sampled ones on an engine that samples on the host; where the card runs the whole sampling chain a
        # plain sampled request keeps that path (no logits row crosses to the host).  A think-span budget writes ids
        # for the model, which a draft cannot foresee
        return self.draft is not None and getattr(a, "span", None) is None and not self._card_samples(a)

    def _card_samples(self, a: Active) -> bool:
        """The card runs the whole sampling chain when nothing needs the logits on the host."""
        r = a.req
        return (getattr(self.engine, "device_sampling", False) and (r.sampling.temperature > 0 or r.sampling.penalizes)
                and r.n_probs == 0 and r.constraint is None and not r.logit_bias and not r.ignore_eos
                and getattr(a, "span", None) is None)

    def _turn(self):
        """The slots that run this round when the engine's slots take it in turns (``serve/swap.py``), else None."""
        turn = getattr(self.engine, "turn", None)
        return turn([a.slot.id for a in self.active.values()]) if turn is not None else None

    def _decode_round(self, live=None) -> None:
        rows, spans = [], []                    # spans: (active, first row index, drafted ids)
        for a in self.active.values():
            if a.pending_token is None or (live is not None and a.slot.id not in live):
                continue
            drafted: List[int] = []
            if self._can_draft(a):
                room = self.engine.slot_ctx - len(a.slot.ids) - 2
                if a.req.n_predict >= 0:
                    room = min(room, a.req.n_predict - len(a.generated) - 1)
                k = self.width.choose(min(room, self.engine.max_rows - 1)) if room > 0 else 0
                if k > 0:
                    if getattr(self.draft, "wants_slot", False):
                        drafted = self.draft.propose(a.slot.ids + [a.pending_token], k, a.slot.id)
                    else:
                        drafted = self.draft.propose(a.slot.ids + [a.pending_token], k)
            base = len(a.slot.ids)
            spans.append((a, len(rows), drafted))
            rows.append((a.slot.id, a.pending_token, base))
            for i, d in enumerate(drafted):
                rows.append((a.slot.id, d, base + 1 + i))
        if not rows:
            return
        who = [sp[0] for sp in spans]

        on_card = self._card_samples

        sampling = None
        if any(on_card(a) for a in who):
            sampling = [None] * len(rows)
            for a, r0, drafted in spans:
                if on_card(a) and not drafted:
                    sp = a.req.sampling
                    recent = (a.slot.ids + [a.pending_token])[-sp.repeat_last_n:] if sp.repeat_last_n > 0 else []
                    sampling[r0] = [sp, a.n_drawn, recent]
        need_logits = any((w.req.sampling.temperature > 0 or w.req.sampling.penalizes or w.req.n_probs > 0
                           or w.req.constraint is not None or w.req.logit_bias or w.req.ignore_eos) and not on_card(w) for w in who)
        t0 = time.time()
        kw = {}
        if getattr(self.draft, "wants_slot", False):
            kw["draft_slots"] = {sp[0].slot.id for sp in spans if self._can_draft(sp[0])}
        if sampling is not None:
            kw["sampling"] = sampling
        wait_of = getattr(self.engine, "card_wait_seconds", None)
        w0 = wait_of() if wait_of is not None else 0.0
        res = self.engine.step(rows, want_logits=need_logits, **kw)
        if wait_of is not None:
            waited = max(0.0, wait_of() - w0)
            self.round_card_wait_by_width[len(rows)] = self.round_card_wait_by_width.get(len(rows), 0.0) + waited
            self.metrics.add("card_wait_seconds_total", waited)
        if sampling is not None:
            for a, r0, _ in spans:
                if sampling[r0] is not None:
                    a.n_drawn = sampling[r0][1]      # the engine wrote back how many uniforms the chain has used
                    res[r0] = (res[r0][0], None)        # the id is the sampled one: nothing left to do on the host
        dt = time.time() - t0
        self.metrics.add("round_seconds_total", dt)
        self.metrics.add("n_decode_total")
        self.metrics.add("n_busy_slots_per_decode", len(spans))
        self.rounds_by_width[len(rows)] = self.rounds_by_width.get(len(rows), 0) + 1
        self.round_seconds_by_width[len(rows)] = self.round_seconds_by_width.get(len(rows), 0.0) + dt
        if self.width is not None and len(spans) == 1:
            self.width.observe_pass(len(rows), dt)
        for a, r0, drafted in spans:
            # Row j evaluated the pending token (j = 0) or draft j - 1; the request's own pick from that row -- greedy,
            # sampled, biased or masked, whatever the request asks -- is the next token, and draft j is kept exactly when
            # it equals that pick.  So a request takes the same ids with a draft as without one, sampled requests with
            # their seed included: a draw is consumed only for a row whose pick is used.
            base = len(a.slot.ids)
            kept = 0
            alive = True
            a.draft_n += len(drafted)              # before the rows settle: a request that ends in this pass reports them
            for j in range(len(drafted) + 1):
                tok_in = a.pending_token if j == 0 else drafted[j - 1]
                if j > 0:
                    a.draft_accepted += 1          # row j exists because draft j - 1 was kept
                alive = self._settle(a, tok_in, res[r0 + j][0], res[r0 + j][1])
                if not alive or j == len(drafted) or a.pending_token != drafted[j]:
                    break
                kept += 1
            if drafted:
                self.metrics.add("draft_tokens_total", len(drafted))
                self.metrics.add("draft_accepted_total", kept)
                for depth in range(len(drafted)):
                    self.draft_by_depth[depth] = self.draft_by_depth.get(depth, 0) + 1
                    if depth < kept:
                        self.accepted_by_depth[depth] = self.accepted_by_depth.get(depth, 0) + 1
                self.width.observe_accept(len(drafted), kept)
                if alive and kept < len(drafted):
                    self.engine.cut(a.slot.id, base + 1 + kept)     # rows of rejected drafts leave the KV

    def _settle(self, a: Active, tok_in: int, greedy: int, logits: Optional[np.ndarray]) -> bool:
        """Account one evaluated token and the token picked after it; False when the request ended."""
        tk = self.engine.tokenizer
        a.slot.ids.append(tok_in)
        tok = self._pick(a, greedy, logits)
        now = time.time()
        if not a.t_first:
            a.t_first = now
        req = a.req
        if req.cancelled.is_set():
            self._finish(a, "cancelled")
            return False
        if tk.is_eog(tok) and not req.ignore_eos:
            self._finish(a, "eos")
            return False
        a.generated.append(tok)
        a.slot.n_decoded = len(a.generated)
        a.text += a.decoder.push(tok)
        hit = None
        for s in req.stop:
            i = a.text.find(s, max(0, a.sent - len(s)))
            if i >= 0 and (hit is None or i < hit[0]):
                hit = (i, s)
        if hit is not None:
            a.text = a.text[:hit[0]]
            self._finish(a, "word", hit[1])
            return False
        self._flush_text(a)
        span = getattr(a, "span", None)
        if span is not None:
            span.note(a.text, len(a.generated))
            if span.force_close(a.text):
                a.forced_ids.extend(tk.encode(span.close_tag, parse_special=True, add_bos=False))
            elif span.looping(a.text, a.generated):
                self._finish(a, "reasoning_loop")
                return False
        if req.constraint is not None and req.constraint.done(a.text) and req.constraint.closed(a.text):
            self._finish(a, "eos")
            return False
        if 0 <= req.n_predict <= len(a.generated):
            self._finish(a, "limit")
            return False
        if len(a.slot.ids) + 1 >= self.engine.slot_ctx:
            self._finish(a, "limit")
            return False
        if req.t_max_predict_ms and (now - a.t_first) * 1e3 > req.t_max_predict_ms:
            self._finish(a, "limit")
            return False
        a.pending_token = tok
        return True

    # ---------------------------------------------------------------- loop
    def run(self) -> None:
        try:
            while not self.stop_flag.is_set():
                while True:
                    try:
                        fn, done = self.actions.get_nowait()
                    except queue.Empty:
                        break
                    try:
                        done.put(("ok", fn()))
                    except Exception as exc:       # noqa: BLE001 - reported to the caller of the action
                        done.put(("error", exc))
                self._admit()
                live = self._turn()
                for a in list(self.active.values()):
                    if a.pending_token is None and (live is None or a.slot.id in live):
                        self._feed_prompt(a)
                self._decode_round(live)
                self._log_generating()
                if not self.active:
                    with self.board.wake:
                        if not self.board.queue and self.actions.empty() and not self.stop_flag.is_set():
                            self.board.wake.wait(timeout=0.05)
        except BaseException as exc:               # noqa: BLE001 - engine failure is fatal by contract
            self.failed = exc
            for a in list(self.active.values()):
                a.req.events.put(("error", 500, f"engine failure: {exc}"))
            self.metrics.add("requests_failed_total", len(self.active))
            while self.board.queue:
                self.board.queue.popleft().events.put(("error", 500, f"engine failure: {exc}"))
            if self.on_fatal:
                self.on_fatal(exc)

    def run_on_engine_thread(self, fn: Callable[[], Any], timeout: float = 60.0):
        """Run a slot action (save / restore / erase) between rounds, on the engine thread."""
        done: "queue.Queue" = queue.Queue()
        self.actions.put((fn, done))
        with self.board.wake:
            self.board.wake.notify_all()
        kind, val = done.get(timeout=timeout)
        if kind == "error":
            raise val
        return val

    def shutdown(self) -> None:
        self.stop_flag.set()
        with self.board.wake:
            self.board.wake.notify_all()
