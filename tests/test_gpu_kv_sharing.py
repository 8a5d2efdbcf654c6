"""Paged KV on the card through the serving engine's calls: a shared prefix that is not page aligned, copy-on-write under
a shared page, and a slot file of more than 100 MB whose restored sequence decodes to the logits of the original."""
import dataclasses

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PAGE = 64


def _serving(spec, n_slots, slot_ctx):
    from bloomery_b200.models.weights import Weights, synth_tensors
    from bloomery_b200.runtime.engine import DecodeEngine
    from bloomery_b200.serve.engine import GpuEngine
    from bloomery_b200.serve.tokenizer import ByteTokenizer
    dec = DecodeEngine(Weights.from_items(spec, synth_tensors(spec, DEV, seed=3), DEV), n_slots=n_slots, slot_ctx=slot_ctx)
    return GpuEngine(dec, ByteTokenizer(spec.vocab), spec.name)


def _last_logits(eng, slot, ids, start):
    """Prefill ``ids[start:-1]`` from ``start`` and decode the last token: its logits row."""
    eng.prefill(slot, ids[start:-1], start)
    return eng.step([(slot, ids[-1], len(ids) - 1)], want_logits=True)[0][1]


def _close(a, b, tol=5e-2):
    return float(np.abs(a - b).max() / np.abs(a).max()) < tol


def test_prefix_that_ends_inside_a_page_is_shared_by_whole_pages_only():
    from bloomery_b200.models.spec import tiny_qwen3moe
    spec = tiny_qwen3moe()
    eng = _serving(spec, 4, 512)
    g = torch.Generator().manual_seed(9)
    common = torch.randint(0, spec.vocab, (120,), generator=g).tolist()
    a = common + torch.randint(0, spec.vocab, (30,), generator=g).tolist()
    b = common + torch.randint(0, spec.vocab, (41,), generator=g).tolist()
    eng.prefill(0, a, 0)                                    # the donor
    want = _last_logits(eng, 3, b, 0)                       # the second prompt alone, in a slot of its own

    # the receiver already keeps 100 positions of the prefix: 64 shared ones would be a loss, nothing may change
    eng.prefill(1, common[:100], 0)
    assert eng.share_prefix(0, 1, 120, have=100) == 0
    assert eng.dec.slot_len[1] == 100
    assert _close(_last_logits(eng, 1, b, 100), want)

    # the receiver keeps 10: one whole page of the donor is mapped, the rest of the prompt is computed
    eng.prefill(2, common[:10], 0)
    assert eng.share_prefix(0, 2, 120, have=10) == PAGE
    assert eng.dec.slot_len[2] == PAGE
    assert _close(_last_logits(eng, 2, b, PAGE), want)


def test_write_under_a_shared_page_copies_it_and_leaves_the_donor_whole():
    from bloomery_b200.models.spec import tiny_qwen3moe
    spec = tiny_qwen3moe()
    eng = _serving(spec, 3, 512)
    g = torch.Generator().manual_seed(10)
    a = torch.randint(0, spec.vocab, (150,), generator=g).tolist()
    nxt = int(torch.randint(0, spec.vocab, (1,), generator=g))
    eng.prefill(0, a, 0)
    before = eng.step([(0, nxt, 150)], want_logits=True)[0][1]
    eng.cut(0, 150)

    assert eng.share_prefix(0, 1, 150, have=0) == 2 * PAGE
    other = a[:100] + torch.randint(0, spec.vocab, (60,), generator=g).tolist()
    eng.cut(1, 100)                                         # back into the second shared page
    got = _last_logits(eng, 1, other, 100)                  # writes positions 100.. : the page must be copied first
    assert _close(got, _last_logits(eng, 2, other, 0))
    after = eng.step([(0, nxt, 150)], want_logits=True)[0][1]
    assert np.array_equal(before, after)                    # the donor's positions 100..127 were not overwritten


def test_slot_file_of_more_than_100_mb_restores_to_the_same_logits(tmp_path):
    from bloomery_b200.models.spec import tiny_qwen3moe
    from bloomery_b200.serve.slotfile import read_slot_file, write_slot_file
    spec = dataclasses.replace(tiny_qwen3moe(), name="tiny-wide-kv", hidden=1024, n_q=8, n_kv=8, head_dim=128)
    n = 6500                                                # 4 layers x 2 x 8 heads x 128 x 2 B = 16 KB a position
    eng = _serving(spec, 2, 8192)
    g = torch.Generator().manual_seed(11)
    ids = torch.randint(0, spec.vocab, (n,), generator=g).tolist()
    nxt = int(torch.randint(0, spec.vocab, (1,), generator=g))
    eng.prefill(0, ids, 0)
    want = eng.step([(0, nxt, n)], want_logits=True)[0][1]
    eng.cut(0, n)
    saved = eng.snapshot(0, ids)
    assert saved.n_bytes > 100e6
    path = str(tmp_path / "slot.bin")
    assert write_slot_file(path, spec.vocab, ids, saved) > 100e6
    ids2, back = read_slot_file(path, spec.vocab)
    assert ids2 == ids
    assert eng.restore(1, back, n) == n
    got = eng.step([(1, nxt, n)], want_logits=True)[0][1]
    assert np.array_equal(want, got)
