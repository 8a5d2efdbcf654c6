"""The CUDA sampler against the host chain (serve/sampler.py) on the same logits and seeds."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run(logits, plist, seeds, recent=None, n_calls=1, split=None, cap=1024):
    from bloomery_b200.ops import decode as K
    M, V = logits.shape
    params = torch.tensor([[p.temperature, p.top_k, p.top_p, p.min_p, p.repeat_penalty, p.frequency_penalty,
                            p.presence_penalty, p.repeat_last_n] for p in plist], dtype=torch.float32, device=DEV)
    sd = torch.tensor(seeds, dtype=torch.int64, device=DEV)
    draws = torch.zeros(M, dtype=torch.int64, device=DEV)
    out = torch.zeros(M, dtype=torch.int32, device=DEV)
    ncand = torch.zeros(M, dtype=torch.int32, device=DEV)
    work = torch.zeros(M, V, device=DEV)
    rec = nrec = None
    if recent is not None:
        W = max(len(r) for r in recent)
        rec = torch.zeros(M, W, dtype=torch.int32, device=DEV)
        for i, r in enumerate(recent):
            rec[i, :len(r)] = torch.tensor(r, dtype=torch.int32)
        nrec = torch.tensor([len(r) for r in recent], dtype=torch.int32, device=DEV)
    picks = []
    for _ in range(n_calls):
        K.sample_rows(logits, V, M, params, sd, draws, out, recent=rec, n_recent=nrec, work=work, out_n_cand=ncand, split=split, cap=cap)
        picks.append(out.cpu().tolist())
    return picks, ncand.cpu().tolist()


@pytest.mark.parametrize("split", [False, True])
@pytest.mark.parametrize("V", [32000, 151936])
def test_sampler_matches_host_chain(V, split):
    from bloomery_b200.serve.sampler import Sampler, SamplingParams
    g = torch.Generator().manual_seed(V)
    logits = (torch.randn(6, V, generator=g) * 3).to(DEV)
    logits[1, 5] = float("nan")
    plist = [SamplingParams(seed=1), SamplingParams(seed=2, top_k=5, top_p=1.0, min_p=0.0, temperature=1.3),
             SamplingParams(seed=3, top_k=200, top_p=0.7, min_p=0.0), SamplingParams(seed=4, top_k=1024, top_p=1.0, min_p=0.02, temperature=0.5),
             SamplingParams(seed=5, temperature=0.0), SamplingParams(seed=6, top_k=1)]
    picks, ncand = _run(logits, plist, [p.seed for p in plist], n_calls=4, split=split)
    host = logits.cpu().numpy()
    agree = total = 0
    for m, p in enumerate(plist):
        s = Sampler(p)
        for c in range(4):
            want = s.sample(host[m])
            total += 1
            agree += int(want == picks[c][m])
            if c == 3:
                assert ncand[m] == len(s.candidates), (m, ncand[m], len(s.candidates))
    assert agree >= total - 1, (agree, total)          # a double-rounding difference may move one draw across a bin edge


@pytest.mark.parametrize("split", [False, True])
def test_sampler_penalties_greedy_and_ties(split):
    from bloomery_b200.serve.sampler import Sampler, SamplingParams
    V = 5000
    logits = torch.zeros(3, V, device=DEV)
    logits[0, 10] = 5.0; logits[0, 20] = 4.9
    logits[1, :] = 1.0                                 # all equal: the lowest ids win the top-k
    logits[2, 7] = 3.0; logits[2, 9] = 3.0
    pen = SamplingParams(temperature=0.0, repeat_penalty=1.5, frequency_penalty=0.1, presence_penalty=0.2, repeat_last_n=8)
    plist = [pen, SamplingParams(seed=9, top_k=4, top_p=1.0, min_p=0.0, temperature=1.0), SamplingParams(temperature=0.0)]
    picks, ncand = _run(logits, plist, [0, 9, 0], recent=[[10, 10, 3], [], []], split=split)
    host = logits.cpu().numpy()
    assert picks[0][0] == Sampler(pen).sample(host[0], [10, 10, 3]) == 20      # the repeated best is penalised away
    assert picks[0][1] in (0, 1, 2, 3) and ncand[1] == 4
    assert picks[0][2] == 7                                                    # equal logits: the lower id


def test_split_form_picks_the_same_ids_as_one_block_per_row():
    """32 blocks per row + the chain on the candidate lists against one block per row: same ids, same candidate counts,
    over penalties, ties, NaNs and a top-k that equals the candidate capacity."""
    from bloomery_b200.serve.sampler import SamplingParams
    g = torch.Generator().manual_seed(77)
    V = 151936
    logits = (torch.randn(8, V, generator=g) * 2).to(DEV)
    logits[0, ::3] = 1.5                                 # a huge tie class straddling every slice
    logits[1, 100:200] = float("nan")
    logits[2, :] = -float("inf"); logits[2, 70000] = 0.0; logits[2, 5] = 0.0
    plist = [SamplingParams(seed=1, top_k=64, top_p=0.95), SamplingParams(seed=2, top_k=40, repeat_penalty=1.3, repeat_last_n=64),
             SamplingParams(seed=3, top_k=50), SamplingParams(seed=4, top_k=100, min_p=0.05, temperature=0.7),
             SamplingParams(seed=5, temperature=0.0), SamplingParams(seed=6, top_k=1),
             SamplingParams(seed=7, top_k=100, frequency_penalty=0.3, presence_penalty=0.2, repeat_last_n=16),
             SamplingParams(seed=8, top_k=7, top_p=0.5)]
    recent = [[], list(range(90, 150)), [], [], [], [], [5, 5, 9, 70000, 5], []]
    a, na = _run(logits, plist, [p.seed for p in plist], recent=recent, n_calls=3, split=False)
    b, nb = _run(logits, plist, [p.seed for p in plist], recent=recent, n_calls=3, split=True, cap=100)
    assert a == b and na == nb


def test_serving_engine_samples_on_the_card_like_the_host_chain():
    """GpuEngine.step with a sampling spec returns the id the host chain picks from the same logits, seed and draw
    number, with penalties over the recent window."""
    from bloomery_b200.models.spec import tiny_qwen3moe
    from bloomery_b200.models.weights import Weights, synth_tensors
    from bloomery_b200.runtime.engine import DecodeEngine
    from bloomery_b200.serve.engine import GpuEngine
    from bloomery_b200.serve.sampler import Sampler, SamplingParams
    from bloomery_b200.serve.tokenizer import ByteTokenizer
    spec = tiny_qwen3moe()
    dec = DecodeEngine(Weights.from_items(spec, synth_tensors(spec, "cpu", seed=7), DEV), n_slots=2, slot_ctx=256)
    eng = GpuEngine(dec, ByteTokenizer(spec.vocab), "tiny")
    prompt = [5, 9, 300, 77, 9, 1234]
    eng.prefill(0, prompt[:-1], 0)
    eng.prefill(1, prompt[:-1], 0)
    sp = SamplingParams(temperature=1.1, top_k=50, top_p=0.9, min_p=0.01, repeat_penalty=1.3, repeat_last_n=4, seed=99)
    host = Sampler(sp)
    tok_h, tok_d, ids = prompt[-1], prompt[-1], list(prompt[:-1])
    agree = n_drawn = 0
    for i in range(6):
        pos = len(ids)
        recent = (ids + [tok_h])[-4:]
        res_h = eng.step([(0, tok_h, pos)], want_logits=True)
        pick_h = host.sample(res_h[0][1], recent)
        spec_d = [sp, n_drawn, recent]
        res_d = eng.step([(1, tok_d, pos)], want_logits=False, sampling=[spec_d])
        n_drawn = spec_d[1]
        assert res_d[0][1] is None
        agree += int(res_d[0][0] == pick_h)
        ids.append(tok_h)
        tok_h = tok_d = pick_h                 # keep both slots on the host chain's text
    assert agree >= 5, agree                   # a probability that ties at fp32 rounding may order differently once
