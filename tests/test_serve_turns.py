"""Slots that take the engine in turns (``serve/swap.py``): the turn rule, the parked-state table, and a server whose
three clients share an engine of one sequence and still get the text each would get alone."""
import threading

import numpy as np
import pytest

from bloomery_b200.serve.api import Server
from bloomery_b200.serve.chat import ChatTemplate
from bloomery_b200.serve.engine import Engine, Saved
from bloomery_b200.serve.swap import ParkTable, SwapEngine
from bloomery_b200.serve.tokenizer import ByteTokenizer
from bloomery_b200.utils import flags
from bloomery_b200.utils.exit_codes import Refusal

from test_serve import call


class TailEngine(Engine):
    """The next token is a function of the sequence's last three tokens and its length: any state that is moved aside and
    put back wrongly shows as different text.  Ends a sequence after ``stop_at`` positions."""

    def __init__(self, n_slots, slot_ctx=512, stop_at=120, snapshots=True):
        self.tokenizer = ByteTokenizer()
        self.n_slots, self.slot_ctx, self.n_vocab = n_slots, slot_ctx, self.tokenizer.n_vocab
        self.model_name, self.max_rows = "tail", 8
        self.seq = [[] for _ in range(n_slots)]
        self.stop_at, self.snapshots = stop_at, snapshots
        self.prefilled = 0

    def _row(self, seq):
        row = np.full(self.n_vocab, -10.0, dtype=np.float32)
        if len(seq) >= self.stop_at:
            row[self.tokenizer.eos_id] = 10.0
        else:
            h = (sum((i + 3) * t for i, t in enumerate(seq[-3:])) + 7 * len(seq)) % 26
            row[ord("a") + h] = 10.0
        return row

    def prefill(self, slot, ids, start):
        assert len(self.seq[slot]) >= start
        self.seq[slot] = self.seq[slot][:start] + list(ids)
        self.prefilled += len(ids)

    def step(self, rows, want_logits=True):
        out = []
        for slot, tok, pos in rows:
            assert len(self.seq[slot]) >= pos, (slot, pos, len(self.seq[slot]))
            self.seq[slot] = self.seq[slot][:pos] + [tok]
            row = self._row(self.seq[slot])
            out.append((int(row.argmax()), row if want_logits else None))
        return out

    def cut(self, slot, n):
        del self.seq[slot][n:]

    def reset(self, slot):
        self.seq[slot] = []

    def snapshot(self, slot, ids):
        if not self.snapshots:
            return None
        assert self.seq[slot][:len(ids)] == list(ids)
        return Saved(tuple(ids), list(ids), 8 * len(ids))

    def restore(self, slot, saved, n):
        n = min(n, len(saved.ids))
        self.seq[slot] = list(saved.payload[:n])
        return n


def test_turn_rule_quantum_and_longest_waiting_first():
    eng = SwapEngine(TailEngine(1), 3, quantum=4)
    assert eng.turn([0]) == {0}
    eng.used[0] = 10
    assert eng.turn([0]) == {0}                       # past its quantum, but nobody waits
    assert eng.turn([0, 1, 2]) == {1}                 # 0 yields; 1 and 2 arrived together, the lower id first
    eng.used[1] = 3
    assert eng.turn([0, 1, 2]) == {1}                 # inside its quantum
    eng.used[1] = 4
    assert eng.turn([0, 1, 2]) == {2}                 # 2 has waited longest (0 queued behind it when it yielded)
    eng.used[2] = 4
    assert eng.turn([0, 1, 2]) == {0}
    assert eng.turn([1, 2]) == {1}                    # 0 ended: the seat goes to the one that waited longest
    two = SwapEngine(TailEngine(2), 3, quantum=4)
    assert two.turn([0, 1]) == {0, 1}
    two.used[0], two.used[1] = 9, 5
    assert two.turn([0, 1, 2]) == {1, 2}              # one seat short: only the slot that ran longest yields


def test_park_table_budget_idle_states_leave_first():
    t = ParkTable(100)
    s = lambda n: Saved((1,), None, n)            # noqa: E731
    assert t.put(0, s(40), idle=True) and t.put(1, s(40), idle=False)
    assert t.put(2, s(40), idle=False)                # the idle state of slot 0 makes room
    assert 0 not in t.held and t.evicted == 1
    assert not t.put(3, s(40), idle=False)            # only live states left: none of them leaves
    assert not t.put(3, s(101), idle=False)
    assert t.take(1).n_bytes == 40 and t.bytes() == 40


@pytest.mark.parametrize("park,snapshots", [("states", True), ("ids", True), ("states", False)])
def test_three_sequences_over_one_engine_sequence_decode_as_alone(park, snapshots):
    alone = TailEngine(3)
    inner = TailEngine(1, snapshots=snapshots)
    eng = SwapEngine(inner, 3, park=park, quantum=5)
    prompts = [[10 + s, 20, 30 + s, 40] for s in range(3)]
    want, got = [], [[], [], []]
    for s, pr in enumerate(prompts):
        alone.prefill(s, pr[:-1], 0)
        tok, seq = pr[-1], []
        for i in range(30):
            tok = alone.step([(s, tok, len(pr) - 1 + i)])[0][0]
            seq.append(tok)
        want.append(seq)
    cur = [pr[-1] for pr in prompts]
    fed = [False] * 3
    while any(len(g) < 30 for g in got):
        live = [s for s in range(3) if len(got[s]) < 30]
        for s in eng.turn(live):
            if not fed[s]:
                eng.prefill(s, prompts[s][:-1], 0)
                fed[s] = True
            cur[s] = eng.step([(s, cur[s], len(prompts[s]) - 1 + len(got[s]))])[0][0]
            got[s].append(cur[s])
    assert got == want
    assert eng.parks >= 6
    if park == "states" and snapshots:
        assert eng.restores >= 4 and inner.prefilled == 9         # every prompt was computed once
    else:
        assert eng.refeeds >= 4 and inner.prefilled > 9           # a parked slot feeds its ids again
    with pytest.raises(RuntimeError):
        eng.step([(0, 1, 0), (1, 1, 0)])                          # two slots in one call over one sequence


def test_server_with_more_clients_than_engine_sequences():
    opts = flags.parse(["--port", "0", "--mock"])
    plain = Server(opts)
    plain.start()
    plain.ready(TailEngine(3), ChatTemplate(), 0)
    prompts = ["first client", "the second one", "and a third"]
    want = [call(plain, "/completion", {"prompt": p, "temperature": 0, "n_predict": 90})[1]["content"] for p in prompts]
    plain.state.stop_event.set()
    plain.stop()

    server = Server(flags.parse(["--port", "0", "--mock"]))
    server.start()
    eng = SwapEngine(TailEngine(1), 3, quantum=8)
    server.ready(eng, ChatTemplate(), 0)
    out = [None] * 3

    def go(i):
        out[i] = call(server, "/completion", {"prompt": prompts[i], "temperature": 0, "n_predict": 90})[1]["content"]
    ts = [threading.Thread(target=go, args=(i,)) for i in range(3)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert out == want
    assert eng.parks > 0
    turns = call(server, "/props")[1]["model"]["turns"]
    assert turns["slots"] == 3 and turns["engine_sequences"] == 1
    server.state.stop_event.set()
    server.stop()


def test_engine_slots_flag_is_checked():
    from bloomery_b200.serve import cli
    assert cli.main(["--mock", "--port", "0", "-np", "2", "--engine-slots", "2", "--dry-run"]) == 64
    assert cli.main(["--mock", "--port", "0", "--engine-slots", "1", "--dry-run"]) == 64       # -np auto
