"""The CUDA sampler against the host chain (serve/sampler.py) on the same logits and seeds."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run(logits, plist, seeds, recent=None, n_calls=1):
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
        K.sample_rows(logits, V, M, params, sd, draws, out, recent=rec, n_recent=nrec, work=work, out_n_cand=ncand)
        picks.append(out.cpu().tolist())
    return picks, ncand.cpu().tolist()


@pytest.mark.parametrize("V", [32000, 151936])
def test_sampler_matches_host_chain(V):
    from bloomery_b200.serve.sampler import Sampler, SamplingParams
    g = torch.Generator().manual_seed(V)
    logits = (torch.randn(6, V, generator=g) * 3).to(DEV)
    logits[1, 5] = float("nan")
    plist = [SamplingParams(seed=1), SamplingParams(seed=2, top_k=5, top_p=1.0, min_p=0.0, temperature=1.3),
             SamplingParams(seed=3, top_k=200, top_p=0.7, min_p=0.0), SamplingParams(seed=4, top_k=1024, top_p=1.0, min_p=0.02, temperature=0.5),
             SamplingParams(seed=5, temperature=0.0), SamplingParams(seed=6, top_k=1)]
    picks, ncand = _run(logits, plist, [p.seed for p in plist], n_calls=4)
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


def test_sampler_penalties_greedy_and_ties():
    from bloomery_b200.serve.sampler import Sampler, SamplingParams
    V = 5000
    logits = torch.zeros(3, V, device=DEV)
    logits[0, 10] = 5.0; logits[0, 20] = 4.9
    logits[1, :] = 1.0                                 # all equal: the lowest ids win the top-k
    logits[2, 7] = 3.0; logits[2, 9] = 3.0
    pen = SamplingParams(temperature=0.0, repeat_penalty=1.5, frequency_penalty=0.1, presence_penalty=0.2, repeat_last_n=8)
    plist = [pen, SamplingParams(seed=9, top_k=4, top_p=1.0, min_p=0.0, temperature=1.0), SamplingParams(temperature=0.0)]
    picks, ncand = _run(logits, plist, [0, 9, 0], recent=[[10, 10, 3], [], []])
    host = logits.cpu().numpy()
    assert picks[0][0] == Sampler(pen).sample(host[0], [10, 10, 3]) == 20      # the repeated best is penalised away
    assert picks[0][1] in (0, 1, 2, 3) and ncand[1] == 4
    assert picks[0][2] == 7                                                    # equal logits: the lower id
