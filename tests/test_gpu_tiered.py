"""Experts split between HBM slots and pinned host RAM: cold hits go through the in-graph
hand-off to the CPU leg, hot experts get promoted by the residency rule; tokens stay the
ones the all-on-card engine gives (in band: the CPU leg runs the same unit dots)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _pair(resident, residency="mid", graphs=True):
    from bloomery_b200.models.spec import tiny_qwen3moe
    from bloomery_b200.models.weights import Weights, synth_tensors
    from bloomery_b200.runtime.engine import DecodeEngine
    from bloomery_b200.runtime.tiered import TieredEngine
    spec = tiny_qwen3moe()
    items = list(synth_tensors(spec, "cpu", seed=21))
    full = DecodeEngine(Weights.from_items(spec, iter(items), DEV), n_slots=1, slot_ctx=256, use_graphs=graphs)
    tier = TieredEngine(Weights.from_items(spec, iter(items), DEV), resident, residency=residency, n_slots=1, slot_ctx=256,
                        use_graphs=graphs)
    return spec, full, tier


@pytest.mark.parametrize("resident", [0, 5])
def test_cold_experts_served_by_cpu_leg(resident):
    spec, full, tier = _pair(resident, residency="off")
    try:
        g = torch.Generator().manual_seed(2)
        prompt = torch.randint(0, spec.vocab, (21,), generator=g).tolist()
        a = full.score(0, prompt)
        b = tier.score(0, prompt)
        n_last = len(prompt) % 8 or 8
        err = ((full.logits[:n_last] - tier.logits[:n_last]).abs().max() / full.logits[:n_last].abs().max()).item()
        assert err < 2e-2, err
        assert sum(int(x == y) for x, y in zip(a, b)) >= len(prompt) - 2
        st = tier.stats()
        assert st["cold_slots_routed"] > 0 and st["cold_slots_served"] == st["cold_slots_routed"]
        if resident == 0:
            assert st["cold_slots_routed"] >= len(prompt) * spec.n_used * spec.n_layer      # --cpu-moe: every slot (plus warm-up passes)
        assert (int(tier.fault) & 0xFFFFFFFF) == 0xFFFFFFFF
        assert tier.memory_report()["experts_host"] > 0
    finally:
        tier.close()


def test_promotion_lands_and_output_stays_in_band():
    spec, full, tier = _pair(4, residency="high")
    try:
        g = torch.Generator().manual_seed(4)
        prompt = torch.randint(0, spec.vocab, (40,), generator=g).tolist()
        a = full.score(0, prompt)
        b = tier.score(0, prompt)
        st = tier.stats()
        assert st["flips"] > 0 and st["bytes_promoted"] > 0
        for il in tier.tiered.layers:                       # the device map mirrors the host's view
            sm = tier.tiered.slot_map[il].cpu().tolist()
            on = {e: s for e, s in enumerate(sm) if s >= 0}
            assert on == tier.tiered.slot_of[il] and len(set(on.values())) == len(on) <= tier.tiered.n_slots
        assert sum(int(x == y) for x, y in zip(a, b)) >= len(prompt) - 3
        first = b[-1]
        out = tier.decode_chain(0, first, len(prompt), 6)
        assert len(out) == 6 and (int(tier.fault) & 0xFFFFFFFF) == 0xFFFFFFFF
    finally:
        tier.close()


def test_cold_experts_paged_from_a_side_file(tmp_path):
    """The drive-backed arena behind the in-graph hand-off: cold experts are read from the side file into RAM
    slots on demand; tokens and logits stay those of the RAM-resident host tier."""
    from bloomery_b200.models.spec import tiny_qwen3moe
    from bloomery_b200.models.weights import Weights, synth_tensors
    from bloomery_b200.runtime.nvtier import NvmeTier, write_sidecar
    from bloomery_b200.runtime.tiered import TieredEngine
    spec = tiny_qwen3moe()
    items = list(synth_tensors(spec, "cpu", seed=21))
    path = str(tmp_path / "experts.side")
    write_sidecar(Weights.from_items(spec, iter(items), "cpu"), path)
    nv = NvmeTier(path, n_slots=10)
    ram = TieredEngine(Weights.from_items(spec, iter(items), DEV), 4, residency="off", n_slots=1, slot_ctx=256)
    drv = TieredEngine(Weights.from_items(spec, iter(items), DEV), 4, residency="off", nvme=nv, n_slots=1, slot_ctx=256)
    try:
        g = torch.Generator().manual_seed(6)
        prompt = torch.randint(0, spec.vocab, (24,), generator=g).tolist()
        a, b = ram.score(0, prompt), drv.score(0, prompt)
        assert a == b and torch.equal(ram.logits[:8], drv.logits[:8])
        st = drv.stats()["nvme"]
        assert st["misses"] > 0 and st["hits"] > 0 and st["failed"] == 0 and st["evictions"] >= 0
        assert drv.memory_report()["experts_host"] == 0
    finally:
        ram.close()
        drv.close()
        nv.close()


def test_prompt_streams_host_experts_through_the_gemm_path():
    """A long prompt on the tiered engine: whole expert stacks stream from pinned host memory into a two-half card
    ring one layer ahead of the GEMMs; the result is the all-on-card GEMM prompt path's, bit for bit."""
    spec, full, tier = _pair(4, residency="off")
    try:
        g = torch.Generator().manual_seed(8)
        prompt = torch.randint(0, spec.vocab, (200,), generator=g).tolist()
        a = full.prefill(0, prompt, gemm=True)
        b = tier.prefill(0, prompt, gemm=True)
        assert a == b and torch.equal(full.logits[0], tier.logits[0])
        assert tier._gemm_prefill.expert_source.__self__.bytes > 0
        # decode continues on the split engine from the KV the prompt path wrote
        ta = full.step([(0, a, len(prompt))])[0]
        tb = tier.step([(0, b, len(prompt))])[0]
        err = ((full.logits[0] - tier.logits[0]).abs().max() / full.logits[0].abs().max()).item()
        assert err < 2e-2 and ta == tb
    finally:
        tier.close()


def test_elastic_give_back_and_fill_keep_the_output():
    """The experts give slots back (their experts fall to the host leg) and take them again; the slot map, the card's
    copies and the model's output stay right through both moves."""
    from bloomery_b200.runtime.elastic import ElasticStats, TieredBody, settle_to_margin, with_room
    spec, full, tier = _pair(8, residency="off")
    try:
        g = torch.Generator().manual_seed(6)
        prompt = torch.randint(0, spec.vocab, (17,), generator=g).tolist()
        want = full.score(0, prompt)
        ref = full.logits[0].clone()
        body, stats = TieredBody(tier), ElasticStats()
        unit = body.unit_bytes
        before = tier.tiered.card_bytes()

        def check(n_slots):
            assert tier.tiered.n_slots == n_slots
            for il in tier.tiered.layers:
                sm = tier.tiered.slot_map[il].cpu().tolist()
                on = {e: s_ for e, s_ in enumerate(sm) if s_ >= 0}
                assert on == tier.tiered.slot_of[il] and sorted(on.values()) == list(range(n_slots))
                for e, slot in on.items():
                    for part in ("ffn_gate_exps", "ffn_down_exps"):
                        assert torch.equal(tier.tiered.card[il][part].data[slot].cpu(), tier.tiered.host[il][part].data[e])
            tier.reset(0)
            got = tier.score(0, prompt)
            err = ((tier.logits[0] - ref).abs().max() / ref.abs().max()).item()
            assert err < 2e-2 and sum(int(x == y) for x, y in zip(want, got)) >= len(prompt) - 2

        calls = []

        def op():                                   # an allocation that is refused until three units came back
            calls.append(1)
            if tier.tiered.n_slots > 5:
                raise torch.cuda.OutOfMemoryError("CUDA out of memory (test)")
            return "ok"
        assert with_room(op, body, 3 * unit, stats) == "ok" and len(calls) == 2
        assert stats.give_backs == 1 and stats.bytes_given == before - tier.tiered.card_bytes() > 0
        check(5)
        assert settle_to_margin(body, free_bytes=10 * unit, margin_bytes=8 * unit, stats=stats) > 0      # two units free past the margin
        check(7)
        assert settle_to_margin(body, free_bytes=unit, margin_bytes=3 * unit, stats=stats) < 0           # two units short
        check(5)
        assert stats.fills == 1 and stats.give_backs == 2
    finally:
        tier.close()
