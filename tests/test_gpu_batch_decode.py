"""Batched decode on the tensor cores against the 8-row int8-dot chain of the same engine: logits in a band, the same
arg-max for rows whose lead is clear, and a graph-replayed chain that keeps every sequence's positions moving."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _spec(arch):
    from bloomery_b200.models.spec import tiny_deepseek, tiny_qwen3moe
    return tiny_deepseek() if arch == "deepseek" else tiny_qwen3moe()


def _engine(n_slots, mix="Q4_K_M", arch="qwen3moe"):
    from bloomery_b200.models.weights import Weights, synth_tensors
    from bloomery_b200.runtime.engine import DecodeEngine
    spec = _spec(arch)
    w = Weights.from_items(spec, synth_tensors(spec, DEV, seed=3, mix=mix), DEV)
    return spec, DecodeEngine(w, n_slots=n_slots, slot_ctx=512)


@pytest.mark.parametrize("n_rows,mix,arch,native", [
    (11, "Q4_K_M", "qwen3moe", True), (40, "Q4_K_M", "qwen3moe", True), (19, "FP8_B128", "qwen3moe", False),
    (19, "FP8_B128", "qwen3moe", True), (19, "NVFP4", "qwen3moe", True), (21, "Q4_K_M", "deepseek", True),
    (40, "FP8_B128", "deepseek", False), (40, "FP8_B128", "deepseek", True)])
def test_batched_pass_matches_row_chain_in_band(n_rows, mix, arch, native):
    """FP8 and NVFP4 checkpoints take the same pass, and so does the DeepSeek layer plan: latent attention, a leading
    dense layer, sigmoid routing in groups, a shared expert.  FP8 weights run either expanded to bf16 inside the GEMM
    (``native`` off) or against E4M3 activations on the tensor cores (on: the activations' 3 mantissa bits widen the
    band)."""
    from bloomery_b200.runtime.batch_decode import BatchDecode
    spec, eng = _engine(n_rows, mix, arch)
    fp8_acts = native and mix == "FP8_B128"
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
    bd.fp8_native = native
    got_tok = bd.step(rows)                                     # same cells again: the KV rows are rewritten in place
    got = bd.logits[:n_rows]
    err = ((got - ref).abs().amax(dim=1) / ref.abs().amax(dim=1)).max().item()
    assert err < (0.2 if fp8_acts else 5e-2), err
    top2 = ref.topk(2, dim=1).values
    clear = ((top2[:, 0] - top2[:, 1]) > (0.4 if fp8_acts else 0.1) * ref.abs().amax(dim=1)).cpu().tolist()
    assert fp8_acts or sum(clear) >= 1
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


@pytest.mark.parametrize("world,arch,mix", [(2, "qwen3moe", "Q4_K_M"), (4, "qwen3moe", "Q4_K_M"), (2, "deepseek", "Q8_0"),
                                            (4, "deepseek", "Q8_0")])
def test_batched_pass_over_emulated_ranks_matches_one_gpu(world, arch, mix):
    """Experts split over ranks, attention and rows replicated, partial rows met in the rank-ordered all-reduce: the
    ranks walk a pass in lockstep on one stream and give the tokens and logits of the one-GPU batched pass."""
    from bloomery_b200.models.weights import Weights, synth_tensors
    from bloomery_b200.parallel.batch_dist import ShardedBatchDecode, lockstep
    from bloomery_b200.parallel.sharded import shard_items
    from bloomery_b200.runtime.batch_decode import BatchDecode
    from bloomery_b200.runtime.engine import DecodeEngine
    spec = _spec(arch)
    # the toy DeepSeek widths split four ways leave 64 columns of the shared expert: blocks of 32 (Q8_0) still divide
    # them (``shard_items`` cuts file-type rows; FP8 planes are built per rank by ``synth_tensors(shard=...)`` instead)
    items = list(synth_tensors(spec, DEV, seed=3, mix=mix))
    n_rows = 19
    full = DecodeEngine(Weights.from_items(spec, iter(items), DEV), n_slots=n_rows, slot_ctx=256)
    engs = [DecodeEngine(Weights.from_items(spec, shard_items(iter(items), spec, r, world, attn=False), DEV), n_slots=n_rows,
                         slot_ctx=256) for r in range(world)]
    g = torch.Generator().manual_seed(7)
    rows = []
    for slot in range(n_rows):
        n = 4 + slot % 5
        prompt = torch.randint(0, spec.vocab, (n,), generator=g).tolist()
        first = full.prefill(slot, prompt, gemm=False)
        rows.append((slot, first, n))
        for e in engs:                               # the emulated ranks get the same KV history (their own engines cannot
            for il in range(spec.n_layer):           # run a prompt: their expert stacks are partial)
                e.kv.ensure(slot, n + 1)
            e.kv.sync_table()
    for e in engs:
        e.kv.k.copy_(full.kv.k); e.kv.v.copy_(full.kv.v)
        e.kv.table.copy_(full.kv.table); e.kv.table_host.copy_(full.kv.table_host)
        e.kv.pages = [list(p_) for p_ in full.kv.pages]; e.kv.free = list(full.kv.free); e.kv.refs = list(full.kv.refs)
        e.slot_len = list(full.slot_len)
    ref = BatchDecode(full, max_rows=32)
    want = ref.step(rows)
    want_logits = ref.logits[:n_rows].clone()
    ranks = [ShardedBatchDecode(e, r, world, max_rows=32, local_only=True) for r, e in enumerate(engs)]
    for bd in ranks:
        bd.sym.adopt_peers([b.sym for b in ranks])
    Ms = [bd.set_rows(rows) for bd in ranks]
    for bd in ranks:
        bd._stream.synchronize()
    lockstep(ranks, Ms[0])
    torch.cuda.synchronize()
    for bd in ranks:
        assert int(bd.status.item()) == 0
        assert torch.equal(bd.logits[:n_rows], ranks[0].logits[:n_rows])          # every rank holds the same bits
        err = ((bd.logits[:n_rows] - want_logits).abs().amax(1) / want_logits.abs().amax(1)).max().item()
        assert err < 2e-2, err
    got = ranks[0].tokens_out[:n_rows].tolist()
    assert sum(int(a == b) for a, b in zip(got, want)) >= n_rows - 2


def test_serving_engine_takes_the_batched_pass_for_many_rows():
    """GpuEngine.step with more rows than the 8-row chain holds: one batched pass serves them all, greedy picks and
    sampled picks (the card's chain over the batched pass's logits) included."""
    from bloomery_b200.models.spec import tiny_qwen3moe
    from bloomery_b200.models.weights import Weights, synth_tensors
    from bloomery_b200.runtime.engine import DecodeEngine
    from bloomery_b200.serve.engine import GpuEngine
    from bloomery_b200.serve.sampler import Sampler, SamplingParams
    from bloomery_b200.serve.tokenizer import ByteTokenizer
    spec = tiny_qwen3moe()
    n = 13
    dec = DecodeEngine(Weights.from_items(spec, synth_tensors(spec, DEV, seed=3), DEV), n_slots=n, slot_ctx=256)
    eng = GpuEngine(dec, ByteTokenizer(spec.vocab), "tiny")
    g = torch.Generator().manual_seed(21)
    rows = []
    for slot in range(n):
        ids = torch.randint(0, spec.vocab, (5 + slot,), generator=g).tolist()
        eng.prefill(slot, ids[:-1], 0)
        rows.append((slot, ids[-1], len(ids) - 1))
    few = []
    for i in range(0, n, 8):
        few += eng.step(rows[i:i + 8], want_logits=True)          # the 8-row chain, for reference
    for slot, _, pos in rows:
        eng.cut(slot, pos)
    sp = SamplingParams(temperature=0.9, top_k=40, top_p=0.95, seed=5)
    specs = [None] * n
    specs[4] = [sp, 0, []]
    many = eng.step(rows, want_logits=True, sampling=specs)      # one batched pass
    assert eng._batch() is not None and (64, False) in eng._batch().graphs or (16, False) in eng._batch().graphs
    agree = 0
    for i, ((t8, l8), (tb, lb)) in enumerate(zip(few, many)):
        err = float(abs(l8 - lb).max() / abs(l8).max())
        assert err < 8e-2, (i, err)              # bf16 rows against q8 rows on nearly flat random-init logits
        if i != 4:
            agree += int(t8 == tb)
    assert agree >= n - 3
    assert many[4][0] == Sampler(sp).sample(many[4][1], [])       # the sampled row follows the host chain on its logits


def test_bf16_expert_stacks_serve_through_the_batched_pass():
    """A bf16 checkpoint has no int8-dot expert kernel: every pass of its engine, prompts of a few rows included, is the
    batched tensor-core pass on the bf16 rows as they are.  Same seeded weights as Q8_0 rows give logits in a band."""
    from bloomery_b200.runtime.batch_decode import BatchDecode
    spec, e_bf = _engine(24, "BF16")
    _, e_q8 = _engine(24, "Q8_0")
    assert e_bf._float_expert_pass() is not None and e_q8._float_expert_pass() is None
    g = torch.Generator().manual_seed(17)
    rows = []
    for slot in range(24):
        n = (90 if slot == 0 else 4) + slot % 5                 # slot 0: the GEMM prompt path, the rest: passes of 8 rows
        prompt = torch.randint(0, spec.vocab, (n,), generator=g).tolist()
        a, b = e_q8.prefill(slot, prompt), e_bf.prefill(slot, prompt)
        rows.append((slot, a, n))
    ref_tok = e_q8.step(rows[:6])
    ref = e_q8.logits[:6].clone()
    got_tok = e_bf.step(rows[:6])                               # six rows: still the batched pass
    got = e_bf.logits[:6]
    err = ((got - ref).abs().amax(dim=1) / ref.abs().amax(dim=1)).max().item()
    assert err < 5e-2, err
    top2 = ref.topk(2, dim=1).values
    clear = ((top2[:, 0] - top2[:, 1]) > 0.1 * ref.abs().amax(dim=1)).cpu().tolist()
    assert all(x == y for x, y, c in zip(got_tok, ref_tok, clear) if c)
    for e in (e_q8, e_bf):
        for slot, _, n in rows[:6]:
            e.cut(slot, n)
    many = BatchDecode(e_bf, max_rows=32)                       # and a round of 24 sequences
    wide = BatchDecode(e_q8, max_rows=32)
    many.step(rows)
    wide.step(rows)
    err = ((many.logits[:24] - wide.logits[:24]).abs().amax(dim=1) / wide.logits[:24].abs().amax(dim=1)).max().item()
    assert err < 5e-2, err


def test_prompt_through_passes_of_one_sequence_matches_the_row_chain():
    """``BatchDecode.prefill``: up to 64 consecutive positions of one sequence per pass, each row attending to the rows
    before it in the same pass; the token after the prompt and the next decode step match the 8-row chain's."""
    from bloomery_b200.runtime.batch_decode import BatchDecode
    spec, eng = _engine(2)
    g = torch.Generator().manual_seed(23)
    prompt = torch.randint(0, spec.vocab, (150,), generator=g).tolist()
    want = eng.prefill(0, prompt, gemm=False)
    ref = eng.logits[(150 - 1) % 8][None].clone()               # the chain's last pass held 6 rows: its last row's logits
    bd = BatchDecode(eng, max_rows=64)
    got = bd.prefill(1, prompt)
    n_last = 150 - 128 - 1                                      # the last pass held 22 rows: its last row's logits
    err = float((bd.logits[n_last] - ref[0]).abs().max() / ref.abs().max())
    assert err < 5e-2, err
    top2 = ref[0].topk(2).values
    if float(top2[0] - top2[1]) > 0.1 * float(ref.abs().max()):
        assert got == want
    a = eng.step([(0, want, 150)])
    la = eng.logits[:1].clone()
    eng.step([(1, want, 150)])                                  # the chain decodes on top of the KV the passes wrote
    err = float((eng.logits[0] - la[0]).abs().max() / la.abs().max())
    assert err < 5e-2, err
