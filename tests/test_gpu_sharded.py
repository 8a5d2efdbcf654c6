"""TP-attention + EP-experts engine with the fused reductions, two ranks emulated on one GPU.

Kernels that wait on one another must never run as separate launches that could both be
waiting, so the two ranks' launch lists are interleaved on one stream: launch i of rank 0,
then launch i of rank 1.  Every consumer then finds both producers' flags already set and
the bounded wait returns at once; what is checked is the data path (push into the peer's
slot, flags, rank-ordered sum, residual ping-pong), against the single-GPU engine."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _engines(world=2, slot_ctx=256, spec=None, attn_replicated=False):
    from bloomery_b200.models.spec import tiny_qwen3moe
    from bloomery_b200.models.weights import Weights, synth_tensors
    from bloomery_b200.parallel.sharded import ShardedEngine, local_spec, shard_items
    from bloomery_b200.parallel.symm import SymmetricArena
    from bloomery_b200.runtime.engine import DecodeEngine
    spec = spec or tiny_qwen3moe()
    items = list(synth_tensors(spec, "cpu", seed=9))
    ref = DecodeEngine(Weights.from_items(spec, iter(items), DEV), n_slots=1, slot_ctx=slot_ctx, use_graphs=False)
    arenas = [SymmetricArena(spec.hidden, r, world, DEV, local_only=True) for r in range(world)]
    for a in arenas:
        a.adopt_peers(arenas)
    engs = []
    for r in range(world):
        w = Weights.from_items(local_spec(spec, world, attn=not attn_replicated),
                               shard_items(iter(items), spec, r, world, attn=not attn_replicated), DEV)
        engs.append(ShardedEngine(w, spec, r, world, fused=True, arena=arenas[r], n_slots=1, slot_ctx=slot_ctx,
                                  use_graphs=False, attn_replicated=attn_replicated))
    return spec, ref, engs


def _lockstep(engs, rows):
    Ms = [e.set_rows(rows) for e in engs]
    lists = [e.build_ops(Ms[0], True, False) for e in engs]
    assert len(set(len(l) for l in lists)) == 1
    for step in zip(*lists):
        for op in step:
            op()
    torch.cuda.synchronize()


@pytest.mark.parametrize("world", [2])
def test_two_emulated_ranks_match_single_gpu(world):
    spec, ref, engs = _engines(world)
    g = torch.Generator().manual_seed(3)
    toks = torch.randint(0, spec.vocab, (11,), generator=g).tolist()
    pos = 0
    for chunk in (toks[:8], toks[8:]):
        rows = [(0, t, pos + i) for i, t in enumerate(chunk)]
        ref.step(rows)
        _lockstep(engs, rows)
        pos += len(chunk)
        n = len(chunk)
        for e in engs:
            assert (int(e.fault) & 0xFFFFFFFF) == 0xFFFFFFFF
            assert torch.equal(e.logits[:n], engs[0].logits[:n])            # ranks agree bit for bit
        err = ((engs[0].logits[:n] - ref.logits[:n]).abs().max() / ref.logits[:n].abs().max()).item()
        assert err < 2e-2, err      # sum order differs; a 1-ulp change can flip a q8 code downstream
        assert engs[0].tokens_out[:n].tolist() == engs[1].tokens_out[:n].tolist()


@pytest.mark.parametrize("world", [4, 8])
def test_four_and_eight_emulated_ranks_match_single_gpu(world):
    """The same lockstep check at 4 and 8 ranks, on a shape whose o_proj columns split into whole 256-value blocks
    (16 query heads of 128, 8 KV heads: one or two KV heads and 2 or 4 experts per rank)."""
    from bloomery_b200.models.spec import ModelSpec
    spec = ModelSpec(arch="qwen3moe", name="tp-test", n_layer=2, hidden=512, n_q=16, n_kv=8, head_dim=128, vocab=4096,
                     ctx_train=4096, rms_eps=1e-6, rope_theta=1e6, qk_norm=True, n_expert=16, n_used=4, moe_inter=256)
    spec, ref, engs = _engines(world, spec=spec)
    g = torch.Generator().manual_seed(5)
    toks = torch.randint(0, spec.vocab, (9,), generator=g).tolist()
    pos = 0
    for chunk in (toks[:8], toks[8:]):
        rows = [(0, t, pos + i) for i, t in enumerate(chunk)]
        ref.step(rows)
        _lockstep(engs, rows)
        pos += len(chunk)
        n = len(chunk)
        for e in engs:
            assert (int(e.fault) & 0xFFFFFFFF) == 0xFFFFFFFF
            assert torch.equal(e.logits[:n], engs[0].logits[:n])
        err = ((engs[0].logits[:n] - ref.logits[:n]).abs().max() / ref.logits[:n].abs().max()).item()
        assert err < 2e-2, err
        assert all(e.tokens_out[:n].tolist() == engs[0].tokens_out[:n].tolist() for e in engs)


@pytest.mark.parametrize("world", [2, 4])
def test_emulated_ranks_with_latent_attention_dense_layer_and_shared_expert(world):
    """The DeepSeek layer plan over ranks: latent attention with the per-head products split by head, the leading dense
    FFN and the shared expert split by width, sigmoid routing with groups over expert-parallel ranks."""
    import dataclasses
    from bloomery_b200.models.spec import tiny_deepseek
    spec = dataclasses.replace(tiny_deepseek(), shared_inter=256 * world, dense_inter=1024)
    spec, ref, engs = _engines(world, spec=spec)
    g = torch.Generator().manual_seed(6)
    toks = torch.randint(0, spec.vocab, (10,), generator=g).tolist()
    pos = 0
    for chunk in (toks[:8], toks[8:]):
        rows = [(0, t, pos + i) for i, t in enumerate(chunk)]
        ref.step(rows)
        _lockstep(engs, rows)
        pos += len(chunk)
        n = len(chunk)
        for e in engs:
            assert (int(e.fault) & 0xFFFFFFFF) == 0xFFFFFFFF
            assert torch.equal(e.logits[:n], engs[0].logits[:n])
        err = ((engs[0].logits[:n] - ref.logits[:n]).abs().max() / ref.logits[:n].abs().max()).item()
        assert err < 2e-2, err
        assert all(e.tokens_out[:n].tolist() == engs[0].tokens_out[:n].tolist() for e in engs)


@pytest.mark.parametrize("plan", ["qwen", "deepseek"])
@pytest.mark.parametrize("world", [2, 4])
def test_replicated_attention_one_reduction_per_layer(world, plan):
    """Attention whole on every rank, only the FFN half split: one reduction per layer over alternating buffers."""
    import dataclasses
    from bloomery_b200.models.spec import tiny_deepseek
    spec = dataclasses.replace(tiny_deepseek(), shared_inter=256 * world, dense_inter=1024) if plan == "deepseek" else None
    spec, ref, engs = _engines(world, spec=spec, attn_replicated=True)
    g = torch.Generator().manual_seed(8)
    toks = torch.randint(0, spec.vocab, (11,), generator=g).tolist()
    pos = 0
    for chunk in (toks[:8], toks[8:]):
        rows = [(0, t, pos + i) for i, t in enumerate(chunk)]
        ref.step(rows)
        _lockstep(engs, rows)
        pos += len(chunk)
        n = len(chunk)
        for e in engs:
            assert (int(e.fault) & 0xFFFFFFFF) == 0xFFFFFFFF
            assert torch.equal(e.logits[:n], engs[0].logits[:n])
        err = ((engs[0].logits[:n] - ref.logits[:n]).abs().max() / ref.logits[:n].abs().max()).item()
        assert err < 2e-2, err
        assert all(e.tokens_out[:n].tolist() == engs[0].tokens_out[:n].tolist() for e in engs)


def test_missing_peer_times_out_with_a_status_not_a_hang():
    """A consumer whose peer never pushed gives up after its bounded wait and raises the
    wait-timeout site in the fault word; the context stays usable."""
    import time
    spec, ref, engs = _engines(2)
    e0 = engs[0]
    rows = [(0, 5, 0)]
    M = e0.set_rows(rows)
    ops = e0.build_ops(M, True, False)
    t0 = time.time()
    from bloomery_b200.ops import decode as K
    for op in ops:                # embed .. router of layer 0: the router waits for rank 1, which never runs
        op()
        if getattr(op, "func", None) is K.router:
            break
    torch.cuda.synchronize()
    assert time.time() - t0 < 20
    assert (int(e0.fault) & 0xFF) == 7                                      # FS_WAIT_TIMEOUT
    x = torch.ones(4, device=DEV)
    assert float((x + 1).sum()) == 8.0                                      # the context still answers


def test_shard_items_partition_the_weights():
    from bloomery_b200.models.spec import tiny_qwen3moe
    from bloomery_b200.models.weights import synth_tensors
    from bloomery_b200.parallel.sharded import shard_items
    spec = tiny_qwen3moe()
    items = list(synth_tensors(spec, "cpu", seed=1))
    full = {n: r for n, _, _, r in items}
    parts = [{n: (sh, r) for n, sh, _, r in shard_items(iter(items), spec, rk, 2)} for rk in range(2)]
    q = torch.cat([parts[0]["blk.0.attn_q.weight"][1], parts[1]["blk.0.attn_q.weight"][1]], 0)
    assert torch.equal(q, full["blk.0.attn_q.weight"])
    e = torch.cat([parts[0]["blk.1.ffn_down_exps.weight"][1], parts[1]["blk.1.ffn_down_exps.weight"][1]], 0)
    assert torch.equal(e, full["blk.1.ffn_down_exps.weight"])
    o0, o1 = parts[0]["blk.0.attn_output.weight"], parts[1]["blk.0.attn_output.weight"]
    assert o0[0] == (spec.hidden, spec.q_rows // 2) and o0[1].shape[1] + o1[1].shape[1] == full["blk.0.attn_output.weight"].shape[1]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_server_on_two_gpus_in_lockstep(tmp_path):
    """The server process with ``--place tp -dev 0,1``: rank 0 serves HTTP, rank 1 follows the mirrored calls;
    the greedy text equals the one-GPU server's on the same file (first tokens) and the cache path works."""
    import json
    import os
    import socket
    import subprocess
    import sys
    import time
    import urllib.request
    from bloomery_b200.models import weights as W
    from bloomery_b200.models.spec import tiny_qwen3moe
    spec = tiny_qwen3moe()
    spec.vocab = 2048
    path = str(tmp_path / "tiny.gguf")
    W.write_gguf(spec, W.synth_tensors(spec, "cpu", seed=9), path)

    def run(extra):
        with socket.socket() as so:
            so.bind(("127.0.0.1", 0))
            port = so.getsockname()[1]
        env = dict(os.environ, NCCL_NVLS_ENABLE="0")
        proc = subprocess.Popen([sys.executable, "-m", "bloomery_b200.serve", "-m", path, "--port", str(port), "-c", "2048",
                                 "-np", "2"] + extra, env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE)
        url = f"http://127.0.0.1:{port}"

        def call(p, body=None):
            req = urllib.request.Request(url + p, data=json.dumps(body).encode() if body else None,
                                         headers={"Content-Type": "application/json"})
            return json.loads(urllib.request.urlopen(req, timeout=60).read())
        try:
            for _ in range(1200):
                if proc.poll() is not None:
                    raise AssertionError("server exited: " + proc.stderr.read().decode()[-3000:])
                try:
                    call("/health")
                    break
                except Exception:
                    time.sleep(0.1)
            else:
                raise AssertionError("server did not become ready")
            prompt = [3, 77, 200, 411, 9, 1500, 77, 200, 5, 6, 7]
            r1 = call("/completion", {"prompt": prompt, "n_predict": 8, "temperature": 0, "return_tokens": True})
            r2 = call("/completion", {"prompt": prompt + r1["tokens"][:3], "n_predict": 4, "temperature": 0, "return_tokens": True})
            return r1, r2, call("/props")
        finally:
            proc.terminate()
            try:
                proc.wait(timeout=30)
            except subprocess.TimeoutExpired:
                proc.kill()

    a1, a2, props = run(["--place", "tp", "-dev", "0,1"])
    b1, b2, _ = run(["-dev", "0"])
    assert len(a1["tokens"]) == 8 and a2["tokens_cached"] >= 11
    assert a1["tokens"][:2] == b1["tokens"][:2], (a1["tokens"], b1["tokens"])
    assert a2["tokens"] == a1["tokens"][3:7]


def test_sharded_gemm_prefill_two_emulated_ranks(monkeypatch):
    """The several-GPU prompt path (peer TMA loads for the all-gather, adds into the owner's rows for the
    reduce-scatter and the expert combine), two ranks emulated on one GPU phase by phase, against the
    one-GPU GEMM prompt path: hidden state of the last row, the KV rows written, and the next token."""
    import bloomery_b200.parallel.prefill_dist as PD
    import bloomery_b200.runtime.prefill as PF
    from bloomery_b200.parallel.prefill_dist import ShardedGemmPrefill
    monkeypatch.setattr(PD, "POISON", True)        # scratch starts as NaN: nothing may read what was never written
    monkeypatch.setattr(PF, "POISON", True)
    spec, ref, engs = _engines(2, slot_ctx=512)
    g = torch.Generator().manual_seed(5)
    toks = torch.randint(0, spec.vocab, (300,), generator=g).tolist()
    ref.prefill(0, toks, gemm=True)
    x_ref = ref.x[0].clone()
    pres = [ShardedGemmPrefill(e, ubatch=512, local_only=True) for e in engs]
    for p in pres:
        p.sym.adopt_peers([q.sym for q in pres])
    for e in engs:
        e.kv.ensure(0, len(toks))
        e.kv.sync_table()
    lists = [p.phases(0, toks, 0) for p in pres]
    assert len(set(len(l) for l in lists)) == 1 and len(lists[0]) == 4 * spec.n_layer + 1
    for phase in zip(*lists):
        for fns in phase:                     # rank 0's launches of the phase, then rank 1's: stream order is the barrier
            for fn in fns:
                fn()
    torch.cuda.synchronize()
    for p in pres:
        assert int(p.status) == 0
    for e in engs:
        assert (int(e.fault) & 0xFFFFFFFF) == 0xFFFFFFFF
        err = ((e.x[0] - x_ref).abs().max() / x_ref.abs().max()).item()
        assert err < 3e-2, err
    assert torch.allclose(engs[0].x[0], engs[1].x[0])
    # rank r holds KV head r of the two; compare with the one-GPU cache (bf16 operands: band, not bits)
    for r, e in enumerate(engs):
        pg_ref, pg = ref.kv.pages[0][0], e.kv.pages[0][0]
        a = ref.kv.k[1, pg_ref, r, :64].float()
        b = e.kv.k[1, pg, 0, :64].float()
        assert ((a - b).abs().mean() / a.abs().mean()).item() < 3e-2
