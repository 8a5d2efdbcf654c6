"""The engine surface the server drives, its GPU implementation and a mock.

``Engine`` mirrors the reference's trait (``crates/serve/src/engine.rs:255-706``): prompt rows
in, one row of logits (or a greedy pick) out per active slot, plus the slot operations the
scheduler needs -- ``cut`` (keep a prefix), ``reset``, ``share_prefix`` (map another slot's KV
pages copy-on-write), ``snapshot`` / ``restore`` (host prompt cache, slot files).
``MockEngine`` is the byte-vocabulary engine of the serve tests (``crates/serve/src/mock.rs``):
it echoes the prompt back, so every HTTP contract is testable without a model or a card.
"""
from __future__ import annotations

import dataclasses
import threading
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from .tokenizer import ByteTokenizer, Tokenizer


@dataclasses.dataclass
class Saved:
    """A sequence state kept on the host: the ids it covers and the engine's bytes for them."""

    ids: Tuple[int, ...]
    payload: object
    n_bytes: int


class EngineError(RuntimeError):
    """The engine cannot continue; the server answers 500, /health turns 503, exit code 70."""


class Engine:
    tokenizer: Tokenizer
    model_name = "model"
    n_slots = 1
    slot_ctx = 4096
    n_vocab = 0
    max_rows = 8

    def prefill(self, slot: int, ids: Sequence[int], start: int) -> None: ...
    def step(self, rows: Sequence[Tuple[int, int, int]], want_logits: bool = True) -> List[Tuple[int, Optional[np.ndarray]]]:
        """rows = (slot, token, position).  Returns per row (greedy id, logits row or None)."""
        raise NotImplementedError
    def cut(self, slot: int, n: int) -> None: ...
    def reset(self, slot: int) -> None: ...
    def share_prefix(self, src: int, dst: int, n: int, have: int = 0) -> int:
        """Share ``src``'s first ``n`` positions with ``dst``; ``have`` = positions of the same prefix ``dst`` already
        holds.  Returns the positions ``dst`` now shares, or 0 with ``dst`` untouched when that would not beat ``have``."""
        return 0
    def snapshot(self, slot: int, ids: Sequence[int]) -> Optional[Saved]:
        return None
    def restore(self, slot: int, saved: Saved, n: int) -> int:
        return 0
    def props(self) -> Dict[str, object]:
        return {}
    def embed(self, ids: Sequence[int]) -> Optional[np.ndarray]:
        return None
    def close(self) -> None: ...


class MockEngine(Engine):
    """Echo engine over the byte tokenizer: after a prompt it generates the prompt's own bytes
    again (a bigram table of the prompt), then EOS.  ``fail_at`` makes the k-th step raise."""

    def __init__(self, n_slots: int = 4, slot_ctx: int = 2048, fail_at: int = -1, step_delay: float = 0.0):
        self.step_delay = step_delay
        self.tokenizer = ByteTokenizer()
        self.n_slots, self.slot_ctx, self.n_vocab = n_slots, slot_ctx, self.tokenizer.n_vocab
        self.model_name = "mock-echo"
        self.seq: List[List[int]] = [[] for _ in range(n_slots)]
        self.prompt_len = [0] * n_slots
        self.steps = 0
        self.fail_at = fail_at
        self.prefill_calls: List[Tuple[int, int, int]] = []
        self.fresh = [True] * n_slots          # the next step of the slot carries the prompt's last token
        self.waited_s = 0.0                    # what step_delay has slept: this engine's stand-in for waiting on a card

    def _logits(self, slot: int) -> np.ndarray:
        seq = self.seq[slot]
        row = np.full(self.n_vocab, -10.0, dtype=np.float32)
        n_prompt = self.prompt_len[slot]
        k = len(seq) - n_prompt
        nxt = seq[k] if k < n_prompt else self.tokenizer.eos_id
        if nxt >= 256 and k < n_prompt:
            nxt = self.tokenizer.eos_id
        row[nxt] = 10.0
        row[(nxt + 1) % 256] = 8.0           # a runner-up so samplers have something to choose from
        return row

    def card_wait_seconds(self) -> float:
        return self.waited_s

    def prefill(self, slot, ids, start):
        self.prefill_calls.append((slot, start, len(ids)))
        del self.seq[slot][start:]
        self.seq[slot] += list(ids)
        self.prompt_len[slot] = len(self.seq[slot])
        self.fresh[slot] = True

    def step(self, rows, want_logits=True):
        self.steps += 1
        if self.step_delay:
            import time
            time.sleep(self.step_delay)
            self.waited_s += self.step_delay
        if self.fail_at >= 0 and self.steps >= self.fail_at:
            raise EngineError("mock engine failure (--mock-fail-at)")
        out = []
        for slot, tok, pos in rows:
            del self.seq[slot][pos:]
            self.seq[slot].append(tok)
            if self.fresh[slot]:
                self.prompt_len[slot] = pos + 1      # the first step after a prompt carries its last token
                self.fresh[slot] = False
            lg = self._logits(slot)
            out.append((int(lg.argmax()), lg if want_logits else None))
        return out

    def cut(self, slot, n):
        del self.seq[slot][n:]
        if n < self.prompt_len[slot]:           # cutting into the prompt starts a new one; dropping drafts does not
            self.prompt_len[slot] = n
            self.fresh[slot] = True

    def reset(self, slot):
        self.seq[slot] = []
        self.prompt_len[slot] = 0
        self.fresh[slot] = True

    def share_prefix(self, src, dst, n, have=0):
        n = min(n, len(self.seq[src]))
        if n <= have:
            return 0
        self.seq[dst] = self.seq[src][:n]
        self.prompt_len[dst] = n
        self.fresh[dst] = True
        return n

    def snapshot(self, slot, ids):
        return Saved(tuple(ids), list(self.seq[slot][:len(ids)]), 8 * len(ids))

    def restore(self, slot, saved, n):
        n = min(n, len(saved.ids))
        self.seq[slot] = list(saved.payload[:n])
        self.prompt_len[slot] = n
        self.fresh[slot] = True
        return n

    def props(self):
        return {"engine": "mock", "devices": []}


class GpuEngine(Engine):
    """``Engine`` over :class:`bloomery_b200.runtime.engine.DecodeEngine`."""

    def __init__(self, dec, tokenizer: Tokenizer, model_name: str = "model"):
        self.dec = dec
        self.tokenizer = tokenizer
        self.model_name = model_name
        self.n_slots, self.slot_ctx, self.n_vocab = dec.n_slots, dec.slot_ctx, dec.spec.vocab
        self._lock = threading.Lock()
        self._last_logits: Dict[int, np.ndarray] = {}

    def prefill(self, slot, ids, start):
        from ..runtime.engine import EngineFault, EngineStalled
        try:
            if len(ids):
                self.dec.prefill(slot, list(ids), start)
        except (EngineFault, EngineStalled) as exc:
            raise EngineError(str(exc)) from exc

    device_sampling = True

    batch_rows = 64             # more than max_rows rows in one round go through the batched tensor-core pass

    def _batch(self):
        """The batched pass of this engine (``runtime/batch_decode.py``), or None when the model is not one it serves."""
        if not hasattr(self, "_bd"):
            try:
                from ..runtime.batch_decode import BatchDecode
                from ..runtime.engine import DecodeEngine
                if type(self.dec) is not DecodeEngine:
                    raise NotImplementedError("tiered / sharded engines keep their own passes")
                self._bd = BatchDecode(self.dec, max_rows=self.batch_rows)
            except (NotImplementedError, ValueError):
                self._bd = None
        return self._bd

    def _sample_on_device(self, n_rows: int, specs, logits=None) -> Dict[int, int]:
        """Run the sampling chain on the card for the rows of the last pass that carry a spec
        (``[SamplingParams, draws so far, recent ids]``; the draw count is updated in place); returns row -> sampled id.  Same bits as the host chain
        (``serve/sampler.py``) for the same seed and draw number."""
        import torch
        from ..ops import decode as K
        dec = self.dec
        dev = dec.device
        M = n_rows
        W = max([len(sp[2]) for sp in specs if sp is not None] + [1])
        par = torch.zeros(M, 8, dtype=torch.float32)
        par[:, 0] = 0.0                                    # rows without a spec: temperature 0 = the greedy pick
        seeds = torch.zeros(M, dtype=torch.int64)
        draws = torch.zeros(M, dtype=torch.int64)
        rec = torch.zeros(M, W, dtype=torch.int32)
        nrec = torch.zeros(M, dtype=torch.int32)
        for r, sp in enumerate(specs):
            if sp is None:
                continue
            p_, n_drawn, recent = sp
            par[r] = torch.tensor([p_.temperature, p_.top_k, p_.top_p, p_.min_p, p_.repeat_penalty, p_.frequency_penalty,
                                   p_.presence_penalty, p_.repeat_last_n])
            seeds[r] = p_.seed if p_.seed < (1 << 63) else p_.seed - (1 << 64)
            draws[r] = n_drawn
            if len(recent):
                rec[r, :len(recent)] = torch.tensor(list(recent), dtype=torch.int32)
                nrec[r] = len(recent)
        if getattr(self, "_samp_work", None) is None or self._samp_work.shape[0] < M:
            self._samp_work = torch.zeros(max(M, self.max_rows), self.n_vocab, device=dev)
            self._samp_out = torch.zeros(max(M, self.max_rows), dtype=torch.int32, device=dev)
        draws_dev = draws.to(dev)
        ks = [int(k) for k in par[:, 1].tolist()]
        cap = 1024 if any(k <= 0 or k > 1024 for k in ks) else max(ks)
        K.sample_rows((dec.logits if logits is None else logits)[:M], self.n_vocab, M, par.to(dev), seeds.to(dev), draws_dev, self._samp_out,
                      recent=rec.to(dev), n_recent=nrec.to(dev), work=self._samp_work, cap=cap)
        got = self._samp_out[:M].cpu().tolist()
        after = draws_dev.cpu().tolist()
        for r, sp in enumerate(specs):
            if sp is not None:
                sp[1] = int(after[r])          # the chain draws only when more than one candidate survives
        return {r: int(got[r]) for r, sp in enumerate(specs) if sp is not None}

    def step(self, rows, want_logits=True, draft_slots=None, sampling=None):
        from ..runtime.engine import EngineFault, EngineStalled
        out = []
        try:
            # (with the draft layer on, every pass must also feed that layer's KV rows: those rounds keep the 8-row chain)
            bd = self._batch() if len(rows) > self.max_rows and not getattr(self.dec, "mtp_on", False) else None
            if bd is not None:
                # many sequences in one round: one batched pass per 64 rows instead of a pass per 8
                for i in range(0, len(rows), self.batch_rows):
                    chunk = list(rows[i:i + self.batch_rows])
                    picks = bd.step(chunk)
                    specs = sampling[i:i + self.batch_rows] if sampling is not None else None
                    if specs is not None and any(sp is not None for sp in specs):
                        for r, tok in self._sample_on_device(len(chunk), specs, logits=bd.logits).items():
                            picks[r] = tok
                    lg = bd.logits[:len(chunk)].float().cpu().numpy() if want_logits else None
                    for j, pk in enumerate(picks):
                        out.append((int(pk), lg[j] if lg is not None else None))
                return out
            for i in range(0, len(rows), self.max_rows):
                chunk = list(rows[i:i + self.max_rows])
                picks = self.dec.step(chunk)
                if sampling is not None and any(sp is not None for sp in sampling[i:i + self.max_rows]):
                    for r, tok in self._sample_on_device(len(chunk), sampling[i:i + self.max_rows]).items():
                        picks[r] = tok
                lg = self.dec.logits[:len(chunk)].float().cpu().numpy() if want_logits else None
                if draft_slots and getattr(self.dec, "mtp_on", False):
                    self.dec.draft_after(chunk, picks, draft_slots)
                for j, pk in enumerate(picks):
                    out.append((int(pk), lg[j] if lg is not None else None))
        except (EngineFault, EngineStalled) as exc:
            raise EngineError(str(exc)) from exc
        return out

    def card_wait_seconds(self) -> float:
        """Seconds this engine's host thread has waited for the card so far (the decode engine's own wait counter)."""
        waits = getattr(self.dec, "waits", None)
        return float(waits.ns.get("card", 0)) / 1e9 if waits is not None else 0.0

    def cut(self, slot, n):
        self.dec.cut(slot, n)

    def reset(self, slot):
        self.dec.reset(slot)

    def embed(self, ids):
        """Mean of the final hidden rows of ``ids`` (before the output norm), L2-normalised.  Runs in the last
        slot, whose sequence is saved and put back, so it may be called between rounds of a busy server."""
        import torch
        dec = self.dec
        if not hasattr(dec, "x") or not len(ids):
            return None
        slot = self.n_slots - 1
        keep = dec.slot_len[slot]
        snap = dec.kv.snapshot(slot, keep) if keep else None
        try:
            dec.reset(slot)
            acc = torch.zeros(dec.spec.hidden, dtype=torch.float64, device=dec.device)
            for i in range(0, len(ids), self.max_rows):
                chunk = list(ids[i:i + self.max_rows])
                dec.step([(slot, int(t), i + j) for j, t in enumerate(chunk)], head=False)
                torch.cuda.current_stream(dec.device).synchronize()
                acc += dec.x[:len(chunk)].double().sum(0)
            v = (acc / len(ids)).float()
            v = v / v.norm().clamp(min=1e-12)
            return v.cpu().numpy()
        finally:
            dec.reset(slot)
            if snap is not None:
                dec.kv.restore(slot, snap, keep)
                dec.kv.sync_table()
                dec.slot_len[slot] = keep

    def draft(self, slot: int, n_ids: int) -> List[int]:
        """The draft layer's id for the position after ``n_ids`` known ids of ``slot`` ([] when there is none)."""
        d = getattr(self.dec, "mtp_draft", {}).get(slot)
        return [int(d[1])] if d is not None and d[0] == n_ids else []

    def share_prefix(self, src, dst, n, have=0):
        got = self.dec.kv.share_prefix(src, dst, n, have)
        if got > 0:
            self.dec.slot_len[dst] = got
            self.dec.kv.sync_table()
        return got

    def snapshot(self, slot, ids):
        n = len(ids)
        if n == 0:
            return None
        snap = self.dec.kv.snapshot(slot, n)
        nb = snap["k"].numel() * snap["k"].element_size() * 2
        return Saved(tuple(ids), snap, nb)

    def restore(self, slot, saved, n):
        n = min(n, len(saved.ids))
        self.dec.kv.restore(slot, saved.payload, n)
        self.dec.kv.sync_table()
        self.dec.slot_len[slot] = n
        return n

    def props(self):
        s = self.dec.spec
        return {"engine": "cuda", "arch": s.arch, "n_layer": s.n_layer, "n_expert": s.n_expert,
                "memory": self.dec.memory_report(), "devices": [str(self.dec.device)],
                "launches_per_step": self.dec.launches_per_step}


class CpuEngine(Engine):
    """The CPU-only engine (``-dev none``): the plain PyTorch model, one KV list per slot, weights shared.

    The reference keeps a host seat for models that fit RAM (``crates/model`` CPU engine;
    ``crates/gpu-gates/src/bin/bloomery_serve.rs:46``)."""

    max_rows = 8

    def __init__(self, weights, tokenizer: Tokenizer, n_slots: int = 1, slot_ctx: int = 4096, model_name: str = "model"):
        import copy
        from ..models.cpu_ref import CpuModel
        base = CpuModel(weights)
        self.models = [base] + [copy.copy(base) for _ in range(n_slots - 1)]
        for m in self.models:
            m.reset()
        self.tokenizer, self.model_name = tokenizer, model_name
        self.n_slots, self.slot_ctx, self.n_vocab = n_slots, slot_ctx, weights.spec.vocab
        self.spec = weights.spec

    def _cut(self, m, n: int) -> None:
        if n < m.n_past:
            m.k = [k[:n] for k in m.k]
            m.v = [v[:n] for v in m.v]
            m.n_past = n

    def prefill(self, slot, ids, start):
        import torch
        m = self.models[slot]
        self._cut(m, start)
        if m.n_past != start:
            raise EngineError(f"slot {slot}: prompt rows start at {start} but {m.n_past} positions are kept")
        if len(ids):
            m.forward(torch.tensor(list(ids)))

    def step(self, rows, want_logits=True):
        import torch
        from ..models.cpu_ref import greedy_pick
        out = []
        for slot, tok, pos in rows:
            m = self.models[slot]
            self._cut(m, pos)
            if m.n_past != pos:
                raise EngineError(f"slot {slot}: row at {pos} but {m.n_past} positions are kept")
            if pos + 1 > self.slot_ctx:
                raise EngineError(f"slot {slot}: position {pos} is beyond the slot context")
            lg = m.forward(torch.tensor([tok]))[0]
            if not bool(torch.isfinite(lg).all()):
                raise EngineError("non-finite logits")
            out.append((greedy_pick(lg), lg.numpy() if want_logits else None))
        return out

    def cut(self, slot, n):
        self._cut(self.models[slot], n)

    def reset(self, slot):
        self.models[slot].reset()

    def share_prefix(self, src, dst, n, have=0):
        a, b = self.models[src], self.models[dst]
        n = min(n, a.n_past)
        if n <= have:
            return 0
        b.k = [k[:n].clone() for k in a.k]
        b.v = [v[:n].clone() for v in a.v]
        b.n_past = n
        return n

    def snapshot(self, slot, ids):
        m = self.models[slot]
        n = min(len(ids), m.n_past)
        if n == 0:
            return None
        pay = {"k": [k[:n].clone() for k in m.k], "v": [v[:n].clone() for v in m.v]}
        nb = sum(t.numel() * 4 for t in pay["k"] + pay["v"])
        return Saved(tuple(ids[:n]), pay, nb)

    def restore(self, slot, saved, n):
        m = self.models[slot]
        n = min(n, len(saved.ids))
        m.k = [k[:n].clone() for k in saved.payload["k"]]
        m.v = [v[:n].clone() for v in saved.payload["v"]]
        m.n_past = n
        return n

    def embed(self, ids):
        import copy
        import torch
        if not len(ids):
            return None
        m = copy.copy(self.models[0])
        m.reset()
        m.forward(torch.tensor(list(ids)))
        v = m.hidden.double().mean(0).float()
        return (v / v.norm().clamp(min=1e-12)).numpy()

    def props(self):
        s = self.spec
        return {"engine": "cpu", "arch": s.arch, "n_layer": s.n_layer, "n_expert": s.n_expert, "devices": ["cpu"]}


class NativeCpuEngine(CpuEngine):
    """The CPU-only engine over the native host step (``runtime/host_model.py``): one decoder, and so one cache, per
    slot; the weights stay in their resident quantised rows and are shared.  Embeddings come from the plain model, made
    on first use."""

    def __init__(self, weights, tokenizer: Tokenizer, n_slots: int = 1, slot_ctx: int = 4096, model_name: str = "model"):
        from ..runtime.host_model import HostDecoder
        self.weights = weights
        self.models = [HostDecoder(weights, ctx=slot_ctx) for _ in range(n_slots)]
        self.tokenizer, self.model_name = tokenizer, model_name
        self.n_slots, self.slot_ctx, self.n_vocab = n_slots, slot_ctx, weights.spec.vocab
        self.spec = weights.spec
        self._oracle = None

    def _cut(self, m, n: int) -> None:
        m.cut(n)

    def prefill(self, slot, ids, start):
        m = self.models[slot]
        m.cut(start)
        if m.n_past != start:
            raise EngineError(f"slot {slot}: prompt rows start at {start} but {m.n_past} positions are kept")
        if start + len(ids) > self.slot_ctx:
            raise EngineError(f"slot {slot}: the prompt ends beyond the slot context")
        for t in ids:
            m.step(int(t), want_logits=False)

    def step(self, rows, want_logits=True):
        import torch
        from ..models.cpu_ref import greedy_pick
        out = []
        for slot, tok, pos in rows:
            m = self.models[slot]
            m.cut(pos)
            if m.n_past != pos:
                raise EngineError(f"slot {slot}: row at {pos} but {m.n_past} positions are kept")
            if pos + 1 > self.slot_ctx:
                raise EngineError(f"slot {slot}: position {pos} is beyond the slot context")
            lg = m.step(int(tok))
            if not bool(torch.isfinite(lg).all()):
                raise EngineError("non-finite logits")
            out.append((greedy_pick(lg), lg.numpy().copy() if want_logits else None))
        return out

    def reset(self, slot):
        self.models[slot].reset()

    def share_prefix(self, src, dst, n, have=0):
        a, b = self.models[src], self.models[dst]
        n = min(n, a.n_past)
        if n <= have:
            return 0
        b.load_kv(*a.kv(n))
        return n

    def snapshot(self, slot, ids):
        m = self.models[slot]
        n = min(len(ids), m.n_past)
        if n == 0:
            return None
        k, v = m.kv(n)
        return Saved(tuple(ids[:n]), {"k": k, "v": v}, k.numel() * 8)

    def restore(self, slot, saved, n):
        n = min(n, len(saved.ids))
        return self.models[slot].load_kv(saved.payload["k"], saved.payload["v"], n)

    def embed(self, ids):
        if self._oracle is None:
            self._oracle = CpuEngine(self.weights, self.tokenizer, 1, self.slot_ctx, self.model_name)
        return self._oracle.embed(ids)

    def props(self):
        out = dict(super().props())
        out["engine"] = "cpu-native"
        return out

    def close(self):
        for m in self.models:
            m.close()
