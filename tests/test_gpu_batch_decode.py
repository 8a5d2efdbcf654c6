"""Batched decode on the tensor cores against the 8-row int8-dot chain of the same engine: logits in a band, the same
arg-max for rows whose lead is clear, and a graph-replayed chain that keeps every sequence's positions moving."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _engine(n_slots):
    from bloomery_b200.models.spec import tiny_qwen3moe
    from bloomery_b200.models.weights import Weights, synth_tensors
    from bloomery_b200.runtime.engine import DecodeEngine
    spec = tiny_qwen3moe()
    w = Weights.from_items(spec, synth_tensors(spec, DEV, seed=3), DEV)
    return spec, DecodeEngine(w, n_slots=n_slots, slot_ctx=512)


@pytest.mark.parametrize("n_rows", [11, 40])
def test_batched_pass_matches_row_chain_in_band(n_rows):
    from bloomery_b200.runtime.batch_decode import BatchDecode
    spec, eng = _engine(n_rows)
    g = torch.Generator().manual_seed(7)
    rows = []
    for slot in range(n_rows):
        n = 5 + 3 * (slot % 7)                                  # every sequence its own length
        prompt = torch.randint(0, spec.vocab, (n,), generator=g).tolist()
        first = eng.prefill(slot, prompt, gemm=False)
        rows.append((slot, first, n))
    ref = torch.zeros(n_rows, spec.vocab, device=DEV)
    ref_tok = []
    for i in range(0, n_rows, 8):
        part = rows[i:i + 8]
        ref_tok += eng.step(part)
        ref[i:i + len(part)] = eng.logits[:len(part)]
    bd = BatchDecode(eng, max_rows=64)
    got_tok = bd.step(rows)                                     # same cells again: the KV rows are rewritten in place
    got = bd.logits[:n_rows]
    err = ((got - ref).abs().amax(dim=1) / ref.abs().amax(dim=1)).max().item()
    assert err < 5e-2, err
    top2 = ref.topk(2, dim=1).values
    clear = ((top2[:, 0] - top2[:, 1]) > 0.1 * ref.abs().amax(dim=1)).cpu().tolist()
    assert sum(clear) >= 1
    assert all(a == b for a, b, c in zip(got_tok, ref_tok, clear) if c)
    again = bd.step(rows)
    assert again == got_tok                                     # replay of the captured pass is deterministic


def test_batched_chain_advances_every_sequence():
    from bloomery_b200.runtime.batch_decode import BatchDecode
    spec, eng = _engine(16)
    g = torch.Generator().manual_seed(9)
    rows = []
    for slot in range(16):
        prompt = torch.randint(0, spec.vocab, (6 + slot,), generator=g).tolist()
        rows.append((slot, eng.prefill(slot, prompt, gemm=False), 6 + slot))
    bd = BatchDecode(eng, max_rows=16)
    # step by step through the host ...
    cur, seqs = list(rows), [[] for _ in rows]
    for _ in range(4):
        toks = bd.step(cur)
        for i, t in enumerate(toks):
            seqs[i].append(t)
        cur = [(s, t, p + 1) for (s, _, p), t in zip(cur, toks)]
    # ... and as a replayed chain that advances tokens and positions on the card
    for slot in range(16):
        eng.cut(slot, rows[slot][2])
    for slot, _, pos in rows:
        eng.kv.ensure(slot, pos + 5)
    M = bd.set_rows(rows)
    bd.counters[2:3].zero_()
    for _ in range(4):
        bd.launch(M, advance=True)
    torch.cuda.synchronize()
    hist = bd.hist[:4 * M].view(4, M).cpu()
    assert hist[:, :16].T.tolist() == seqs
    assert int(bd.status.item()) == 0
