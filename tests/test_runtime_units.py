"""Host-side runtime parts: watchdog, waits, capture lock, cost store and race, route traces, census."""
import dataclasses
import threading
import time

import pytest

from bloomery_b200.runtime import autotune as AT
from bloomery_b200.runtime import route_trace as RT
from bloomery_b200.runtime.watchdog import CaptureLock, Waits, Watchdog


def test_watchdog_names_a_wedged_wait_once_and_never_kills():
    now = [0.0]
    seen = []
    wd = Watchdog("m", bound_s=60.0, report=lambda site, age: seen.append((site, round(age))), clock=lambda: now[0])
    a = wd.enter("step readback")
    with wd.guard("prompt unit"):
        now[0] = 30.0
        assert wd.poll() == [] and not wd.is_wedged()
    now[0] = 61.0
    assert [s for s, _ in wd.poll()] == ["step readback"] and wd.is_wedged()
    now[0] = 200.0
    assert wd.poll() == []                       # reported once
    wd.leave(a)
    assert not wd.is_wedged() and seen == [("step readback", 61)]


def test_watchdog_thread_runs_and_stops():
    seen = []
    wd = Watchdog("m", bound_s=0.05, period_s=0.02, report=lambda s, a: seen.append(s)).start()
    t = wd.enter("host tier round")
    time.sleep(0.3)
    wd.stop()
    assert seen == ["host tier round"]
    wd.leave(t)


def test_waits_totals():
    w = Waits()
    w.add("card", 0.5)
    with w.timed("host_tier"):
        time.sleep(0.01)
    m = w.metrics()
    assert m["wait_card_seconds_total"] == 0.5 and m["wait_card_total"] == 1 and m["wait_host_tier_seconds_total"] > 0.005


def test_capture_lock_sync_waits_for_captures_and_blocks_new_ones():
    lk = CaptureLock()
    order = []
    lk.acquire_shared()

    def syncer():
        with lk.sync():
            order.append("sync")

    def late_capture():
        with lk.capture():
            order.append("capture2")
    t1 = threading.Thread(target=syncer)
    t1.start()
    time.sleep(0.05)
    t2 = threading.Thread(target=late_capture)      # queued behind the waiting exclusive holder
    t2.start()
    time.sleep(0.05)
    assert order == []
    order.append("capture1 ends")
    lk.release_shared()
    t1.join(2)
    t2.join(2)
    assert order == ["capture1 ends", "sync", "capture2"]


def test_cost_store_and_race(tmp_path):
    p = str(tmp_path / "c" / "costs.json")
    st = AT.CostStore(p)
    k = AT.CostStore.key("B200", "12.9", "abc", {"hidden": 2048})
    assert k == AT.CostStore.key("B200", "12.9", "abc", {"hidden": 2048}) and k != AT.CostStore.key("B200", "12.9", "abd", {"hidden": 2048})
    assert st.get(k) is None
    clock = {"a": [3.0, 1.0, 2.0], "b": [1.5, 1.5, 9.0]}
    calls = []
    win, costs = AT.race({"a": lambda: calls.append("a"), "b": lambda: calls.append("b")},
                         time_one=lambda fn: (fn(), clock[calls[-1]].pop(0))[1], reps=3, flush=lambda: calls.append("flush"))
    assert win == "b" and costs == {"a": 2.0, "b": 1.5} and calls.count("flush") == 6
    st.put(k, costs)
    assert AT.CostStore(p).get(k) == costs and AT.best_of({"x": 1.0, "a": 1.0}) == "a"
    open(p, "w").write("{not json")
    assert AT.CostStore(p).get(k) is None


def test_route_trace_roundtrip_and_census(tmp_path):
    p = str(tmp_path / "t" / "trace.blrt")
    w = RT.RouteTraceWriter(p, n_layer=2, top_k=3)
    w.add(0, 0, [5, 1, 9], [0.5, 0.25, 0.25])
    w.add(0, 1, [2, 3, -1], [0.6, 0.3, 0.1])
    with pytest.raises(ValueError):
        w.add(1, 0, [1, 2], [0.5, 0.5])
    w.close()
    n_layer, k, it = RT.read_trace(p)
    recs = list(it)
    assert (n_layer, k) == (2, 3) and recs[0][:3] == (0, 0, [5, 1, 9]) and recs[1][2] == [2, 3, -1]
    assert abs(recs[1][3][0] - 0.6) < 1e-6
    open(p, "ab").write(b"xx")
    with pytest.raises(ValueError):
        list(RT.read_trace(p)[2])
    c = RT.Census(2)
    slot_map = [-1] * 10
    slot_map[5] = 0
    slot_map[2] = 1
    c.add_picks(0, [5, 1, 9], slot_map)
    c.add_picks(1, [2, 3, -1], slot_map)
    assert c.totals() == {"card": 2, "host": 3, "peer": 1, "spare": 0} and abs(c.share("host") - 0.5) < 1e-9


def _inv(n_layer=4, n_expert=8, trunk_mib=100, expert_mib=10):
    inv = [("token_embd.weight", trunk_mib << 20)]
    for il in range(n_layer):
        inv.append((f"blk.{il}.attn_q.weight", 8 << 20))
        inv.append((f"blk.{il}.attn_norm.weight", 4096))
        for part in ("gate", "up", "down"):
            inv.append((f"blk.{il}.ffn_{part}_exps.weight", n_expert * expert_mib << 20))
    return inv


def test_placement_planner_rules():
    from bloomery_b200.runtime import placement as P
    kw = dict(n_layer=4, n_expert=8, first_dense=0, kv_bytes_per_token=1 << 16, n_kv_heads=4, ctx_train=32768,
              margin=64 << 20, work_bytes=64 << 20)
    inv = _inv()
    everything = 100 + 4 * 8 + 4 * 3 * 8 * 10           # MiB: trunk + experts
    big = P.plan(inv, budget=4 << 30, **kw)
    assert big.resident_per_layer == 8 and big.host_bytes == 0 and big.word() == "a"
    assert big.slot_ctx == 32768 and big.need()["fits"]
    # an asked context is never cut: the refusal names the largest that fits
    with pytest.raises(P.NoFit) as e:
        P.plan(inv, budget=(everything + 128 + 600) << 20, ctx_ask=16384, **kw)
    assert e.value.largest_ctx == 9216
    # experts that do not fit: refused unless they may stay on the host
    with pytest.raises(P.NoFit):
        P.plan(inv, budget=700 << 20, **kw)
    fit = P.plan(inv, budget=1250 << 20, host_experts="fit", ctx_ask=4096, **kw)
    assert 0 < fit.resident_per_layer < 8 and fit.resident_per_layer % 4 == 0 and fit.spare_slots == 1
    assert fit.host_bytes == 4 * 3 * 8 * 10 << 20 and fit.card_bytes <= fit.budget and "host[4/8]" in fit.word()
    none = P.plan(inv, budget=700 << 20, host_experts="all", **kw)
    assert none.resident_per_layer == 0 and all(p.where == "host" for p in none.places if p.split == "experts")
    # a trunk that does not fit is a refusal even with every expert on the host
    with pytest.raises(P.NoFit):
        P.plan(inv, budget=200 << 20, host_experts="all", **kw)
    # two ranks: heads and experts divide, the rest is replicated; KV divides with the KV heads
    tp = P.plan(inv, budget=4 << 30, world=2, **kw)
    assert tp.trunk_bytes == (100 << 20) + 4 * (4 << 20) + 4 * 4096 and tp.resident_per_layer == 4 and tp.word() == "tp2"
    assert tp.kv_bytes == big.kv_bytes // 2
    r0 = dict(P.rank_inventory(inv, 2, 0))
    assert r0["blk.0.attn_q.weight"] == 4 << 20 and r0["token_embd.weight"] == 100 << 20


def test_nvme_expert_arena_matches_ram_stacks_and_evicts_lru(tmp_path):
    """Experts paged from a side file: the leg over the arena equals the leg over RAM-resident stacks bit for bit;
    the arena holds n_slots experts per layer, evicts the least recently used, never a pinned one."""
    import torch
    from bloomery_b200.formats import quant as Q
    from bloomery_b200.formats.resident import WT
    from bloomery_b200.models.spec import tiny_qwen3moe
    from bloomery_b200.models.weights import Weights, synth_tensors
    from bloomery_b200.ops._lib import host, p as vp
    from bloomery_b200.runtime.nvtier import NvmeTier, write_sidecar
    spec = tiny_qwen3moe()
    spec.vocab, spec.n_layer = 256, 2
    w = Weights.from_items(spec, synth_tensors(spec, "cpu", seed=4), "cpu")
    path = str(tmp_path / "experts.side")
    ix = write_sidecar(w, path)
    assert set(ix["layers"]) == {"0", "1"} and all(v["blob"] % 4096 == 0 for v in ix["layers"].values())
    nv = NvmeTier(path, n_slots=6)
    torch.manual_seed(1)
    M, k, H, E = 2, spec.n_used, spec.hidden, spec.n_expert

    def leg(layer, ids):
        x = torch.randn(M, H)
        xq, xds = Q.quantize_act_q8(x)
        wts = torch.rand(M, k)
        got = nv.moe(layer, ids, wts, xq, xds)
        g, u, d = (w.q[f"blk.{layer}.ffn_{n}_exps.weight"] for n in ("gate", "up", "down"))
        ref = torch.zeros(M, H)
        rc = host().blh_moe_experts(M, H, spec.moe_inter, E, k, vp(ids), vp(wts), vp(xq), vp(xds), vp(g.data), vp(u.data),
                                    vp(d.data), WT[g.qtype], WT[d.qtype], vp(ref))
        assert rc == 0 and torch.equal(got, ref)
    a = torch.tensor([[0, 1, 2, 3], [1, 2, 4, -1]], dtype=torch.int32)
    leg(0, a)
    assert nv.resident(0) == [0, 1, 2, 3, 4] and nv.stats()["misses"] == 5
    nv.pin(0, 0)
    leg(0, torch.tensor([[5, 6, 7, 8], [5, 6, 7, 8]], dtype=torch.int32))      # 4 new experts into 6 slots: 3 of the old ones go
    res = nv.resident(0)
    assert 0 in res and {5, 6, 7, 8} <= set(res) and len(res) == 6 and nv.stats()["evictions"] == 3
    leg(1, a)                                                                   # layers keep separate arenas
    assert nv.resident(1) == [0, 1, 2, 3, 4]
    st = nv.stats()
    assert st["failed"] == 0 and st["bytes_read"] >= st["misses"] * min(v["blob"] for v in ix["layers"].values()) and st["hits"] >= 1
    leg(0, torch.arange(8, dtype=torch.int32).reshape(2, 4) + 8)               # 8 distinct experts, 6 slots: served row by row
    for e in nv.resident(0)[:3]:
        nv.pin(0, e)
    pinned = set(nv.resident(0)[:3])
    fresh = [e for e in range(E) if e not in nv.resident(0)][:4]
    with pytest.raises(OSError):                                                # one row needs 4 slots, pins leave 3
        nv.moe(0, torch.tensor([fresh], dtype=torch.int32), torch.rand(1, 4), *Q.quantize_act_q8(torch.randn(1, H)))
    assert pinned <= set(nv.resident(0))
    nv.close()


def test_expert_tier_node_over_tcp():
    """A tier node on loopback: census with sha256-checked rows, the expert leg over the wire equals the local leg
    bit for bit, a wrong model is refused at open, a lost node and a bad frame surface as TierLost."""
    import socket
    import torch
    from bloomery_b200.formats import quant as Q
    from bloomery_b200.models.spec import tiny_qwen3moe
    from bloomery_b200.models.weights import Weights, synth_tensors
    from bloomery_b200.parallel import tier_node as TN
    spec = tiny_qwen3moe()
    spec.vocab, spec.n_layer = 256, 2
    w = Weights.from_items(spec, synth_tensors(spec, "cpu", seed=4), "cpu")
    other = Weights.from_items(spec, synth_tensors(spec, "cpu", seed=5), "cpu")
    srv = TN.TierServer(w, layers=[1]).start()
    try:
        cl = TN.RemoteExpertTier(srv.addr, io_timeout=10)
        census = cl.open(w)
        assert list(census["layers"]) == ["1"] and census["n_expert"] == 16
        torch.manual_seed(0)
        ids = torch.tensor([[0, 5, 9, -1], [3, 5, 1, 2], [15, 14, 13, 12]], dtype=torch.int32)
        wts = torch.rand(3, 4)
        xq, xds = Q.quantize_act_q8(torch.randn(3, spec.hidden))
        got = cl.moe(1, ids, wts, xq, xds)
        assert torch.equal(got, TN.local_leg(w, 1, ids, wts, xq, xds)) and srv.served == 1
        with pytest.raises(TN.TierLost):                     # a layer the node does not hold
            cl.moe(0, ids, wts, xq, xds)
        assert torch.equal(cl.moe(1, ids, wts, xq, xds), got)     # the channel survives an error answer
        bad = TN.RemoteExpertTier(srv.addr, io_timeout=10)
        with pytest.raises(TN.TierLost):                     # same shapes, other rows: the sha256 check refuses
            bad.open(other)
        bad.close()
        with pytest.raises(ValueError):
            TN.unpack_moe(TN.pack_moe(1, ids, wts, xq, xds)[:-3])
        srv.close()
        cl.sock.settimeout(1.0)
        with pytest.raises(TN.TierLost):
            for _ in range(50):                              # the node is gone: the next exchanges fail within their deadline
                cl.moe(1, ids, wts, xq, xds)
        with socket.socket() as so:
            so.bind(("127.0.0.1", 0))
            dead = so.getsockname()
        with pytest.raises(TN.TierLost):
            TN.RemoteExpertTier(dead, io_timeout=1).open()
    finally:
        srv.close()


def test_kv_pool_spills_idle_slots_to_the_host_and_brings_them_back():
    import torch
    from bloomery_b200.runtime.kv import PAGE, KvPool, OutOfPages
    kv = KvPool(n_layer=2, n_kv=1, head_dim=8, n_pages=4, n_slots=3, max_pages_per_slot=3, device="cpu")
    def fill(slot, n, val):
        kv.protect = {slot}
        kv.ensure(slot, n)
        for pg in kv.pages[slot]:
            kv.k[:, pg] = val
            kv.v[:, pg] = -val
    fill(0, 2 * PAGE, 1.0)
    fill(1, 2 * PAGE, 2.0)
    assert kv.free_pages() == 0
    fill(2, PAGE + 5, 3.0)                       # needs 2 pages: slot 0 (least recently used) goes to the host
    assert 0 in kv.spilled and kv.n_spills == 1 and not kv.pages[0] and len(kv.pages[2]) == 2
    kv.truncate(0, PAGE)                         # a cut reaches a spilled slot too
    kv.protect = {0}
    kv.ensure(0, PAGE)                           # comes back (slot 1 is now the oldest and leaves)
    assert 0 not in kv.spilled and 1 in kv.spilled and kv.n_unspills == 1 and len(kv.pages[0]) == 1
    assert float(kv.k[0, kv.pages[0][0]].mean()) == 1.0 and float(kv.v[1, kv.pages[0][0]].mean()) == -1.0
    kv.protect = {1}
    kv.ensure(1, 2 * PAGE)
    assert all(float(kv.k[1, pg].mean()) == 2.0 for pg in kv.pages[1])
    kv.protect = {0, 1, 2}
    with pytest.raises(OutOfPages):              # every slot with pages is in the pass: nothing may leave
        kv.ensure(0, 3 * PAGE)
    kv.release(2)
    kv.ensure(0, 2 * PAGE)


def test_host_profile_levels_and_heat_files(tmp_path):
    import torch
    from bloomery_b200.runtime.timing import HostProfile, PromptTiming, load_heat, save_heat
    off, one, two = HostProfile(0), HostProfile(1), HostProfile(2)
    for p in (off, one, two):
        with p.span("matmul"):
            pass
        with p.span("rows", detail=True):
            pass
    assert off.report() == {} and set(one.report()) == {"matmul"} and set(two.report()) == {"matmul", "rows"}
    assert one.report()["matmul"]["calls"] == 1
    t = PromptTiming()
    t.mark(0, "qkv")                              # not armed: nothing is kept, no CUDA needed
    assert t.marks == [] and t.report() == {}
    heat = torch.tensor([[1, 0, 5], [2, 2, 2]])
    path = str(tmp_path / "heat.json")
    save_heat(heat, path, model="m")
    assert load_heat(path, 2, 3, model="m") == [[1, 0, 5], [2, 2, 2]]
    assert load_heat(path, 2, 4) is None and load_heat(path, 2, 3, model="other") is None
    assert load_heat(str(tmp_path / "none.json"), 2, 3) is None


def test_kv_pool_never_spills_the_slot_that_is_asking():
    """A pool smaller than one slot's context: the requester must not become its own spill victim."""
    from bloomery_b200.runtime.kv import PAGE, KvPool, OutOfPages
    kv = KvPool(n_layer=1, n_kv=1, head_dim=8, n_pages=2, n_slots=2, max_pages_per_slot=4, device="cpu")
    kv.protect = set()                            # as after a pass over other slots
    kv.ensure(0, 2 * PAGE)
    with pytest.raises(OutOfPages):
        kv.ensure(0, 3 * PAGE)                    # only slot 0 holds pages and it is the one growing
    assert 0 not in kv.spilled and len(kv.pages[0]) == 2 and kv.n_spills == 0
    assert 0 not in kv.protect                    # the self-protection ends with the call


def test_share_prefix_leaves_a_slot_alone_when_whole_pages_do_not_beat_its_own_prefix():
    from bloomery_b200.runtime.kv import PAGE, KvPool
    kv = KvPool(n_layer=1, n_kv=1, head_dim=8, n_pages=8, n_slots=2, max_pages_per_slot=4, device="cpu")
    kv.ensure(0, 120)                             # donor: common prefix 120 -> one whole page (64) can be mapped
    kv.ensure(1, 100)                             # the slot's own prefix: 100 positions
    mine = list(kv.pages[1])
    assert kv.share_prefix(0, 1, 120, have=100) == 0
    assert kv.pages[1] == mine                    # untouched: its 100 positions are still there
    assert kv.share_prefix(0, 1, 120, have=10) == PAGE
    assert kv.pages[1] == kv.pages[0][:1] and kv.refs[kv.pages[0][0]] == 2
    # copy-on-write: the donor is cut inside the shared page and appends; the sharer's page keeps its bytes
    kv.k[:, kv.pages[0][0]] = 7.0
    kv.truncate(0, 30)
    kv.own(0, 30)
    assert kv.pages[0][0] != kv.pages[1][0] and float(kv.k[0, kv.pages[1][0]].mean()) == 7.0
    assert float(kv.k[0, kv.pages[0][0]].mean()) == 7.0      # the private copy starts from the shared bytes


def test_levers_registry_rows_are_all_read_somewhere():
    """Every registry row is read by the package (a declared lever that nothing reads is refused here)."""
    import os, re
    from bloomery_b200.utils import levers
    root = os.path.join(os.path.dirname(levers.__file__), "..")
    text = ""
    for d, _, files in os.walk(root):
        for f in files:
            if f.endswith((".py", ".cpp", ".h", ".cu", ".cuh")) and not d.endswith("utils") or f in ("flags.py",):
                text += open(os.path.join(d, f), errors="ignore").read()
    dead = [l.name for l in levers.REGISTRY if not re.search(r'["\']' + l.name + r'["\']', text)]
    assert dead == [], dead


def test_elastic_with_room_and_settle_on_a_fake_body():
    from bloomery_b200.runtime.elastic import ElasticStats, NoRoom, settle_to_margin, with_room

    class Body:
        unit_bytes = 100

        def __init__(self, have):
            self.have = have

        def give_back(self, n):
            steps = min(self.have, -(-n // 100))
            self.have -= steps
            return steps * 100

        def fill(self, n):
            steps = n // 100
            self.have += steps
            return steps * 100
    b, st = Body(3), ElasticStats()
    tries = []

    def op():
        tries.append(b.have)
        if b.have > 1:
            raise MemoryError("out of memory")
        return 7
    assert with_room(op, b, 150, st) == 7 and tries == [3, 1] and st.give_backs == 1 and st.bytes_given == 200 and st.retries == 1
    with pytest.raises(NoRoom):
        with_room(lambda: (_ for _ in ()).throw(MemoryError("out of memory")), Body(0), 50, st)
    with pytest.raises(NoRoom):
        with_room(lambda: (_ for _ in ()).throw(MemoryError("out of memory")), Body(5), 50, st)      # refused again after the give-back
    with pytest.raises(KeyError):
        with_room(lambda: {}["x"], b, 50, st)                                                       # not a memory refusal: untouched
    b2 = Body(4)
    assert settle_to_margin(b2, free_bytes=50, margin_bytes=260, stats=st) == -300 and b2.have == 1
    assert settle_to_margin(b2, free_bytes=600, margin_bytes=260, stats=st) == 300 and b2.have == 4
    assert settle_to_margin(b2, free_bytes=300, margin_bytes=260, stats=st) == 0                    # less than a unit to spare


def test_tiered_experts_resize_keeps_the_hottest_on_cpu_tensors():
    import torch
    from bloomery_b200.models.spec import tiny_qwen3moe
    from bloomery_b200.models.weights import Weights, synth_tensors
    from bloomery_b200.runtime.residency import TieredExperts
    spec = tiny_qwen3moe()
    w = Weights.from_items(spec, synth_tensors(spec, "cpu", seed=5), "cpu")
    t = TieredExperts(spec, w, 6, "cpu", rule="off")
    heat = torch.zeros(spec.n_layer, spec.n_expert)
    heat[:, 3] = 9; heat[:, 11] = 8; heat[:, 0] = 7; heat[:, 14] = 6
    t.resize(2, heat)
    for il in t.layers:
        assert t.slot_of[il] == {3: 0, 0: 1}                    # the hottest residents stay (11 and 14 were not on the card)
        assert t.slot_map[il].tolist().count(-1) == spec.n_expert - 2
    t.resize(4, heat)
    for il in t.layers:
        assert set(t.slot_of[il]) == {3, 0, 11, 14} and sorted(t.slot_of[il].values()) == [0, 1, 2, 3]
        for e, slot in t.slot_of[il].items():
            assert torch.equal(t.card[il]["ffn_up_exps"].data[slot], t.host[il]["ffn_up_exps"].data[e])
    assert t.n_slots == 4 and t.slot_bytes() * 5 == t.card_bytes()      # n_slots + 1 spare in every layer


def test_expert_split_rule_balances_card_and_host_sides():
    """The prompt-time split of a layer's host experts (``runtime/xsplit.py``): hottest first, an expert moves to the card
    while the card's side after it stays under the host's side without it."""
    from bloomery_b200.runtime.xsplit import Costs, burst_share, split, stream_gate
    c = Costs(lane_b_per_us=50e3, expert_bytes=10_000_000, host_us_fixed=400.0, host_us_per_row=30.0, card_us_fixed=5.0,
              card_us_per_row=0.5, n_expert=8, top_k=2)
    counts = [40, 0, 12, 3, 90, 0, 7, 1]
    host = [0, 2, 3, 4, 6, 7]
    sp = split(counts, host, c)
    # hottest first: 4 (90 rows), 0 (40), 2 (12) ...; every streamed one is hotter than every kept one
    assert sp.streamed[:2] == (4, 0) and set(sp.streamed) | set(sp.kept) == {0, 2, 3, 4, 6, 7}
    assert min(counts[e] for e in sp.streamed) >= max(counts[e] for e in sp.kept)
    assert sp.card_us <= sp.host_us                                  # the walk stops short of the crossing
    rate = c.lane_b_per_us * (1 - burst_share(c, sum(counts[e] for e in host), 6))
    assert abs(sp.beside_b_per_us - rate) < 1e-9 and rate < c.lane_b_per_us
    nxt = sp.kept[0]                                                 # one more move would cross
    more = sp.card_us + c.expert_bytes / rate + c.card_us_fixed + c.card_us_per_row * counts[nxt]
    assert more > sp.host_us - max(c.host_us_fixed, c.host_us_per_row * counts[nxt])
    assert split(counts, host, c) == sp                              # the same counts give the same split
    assert split([1, 0, 0, 0, 0, 0, 0, 0], [0], c).streamed == ()    # a lone cold expert is not worth its copy
    busy = split(counts, host, c, card_base_us=1e6)                  # a card already behind takes nothing
    assert busy.streamed == () and len(busy.kept) == 6
    with pytest.raises(ValueError):
        split(counts[:-1], host, c)
    with pytest.raises(ValueError):
        split(counts, [0, 0], c)
    # the gate: narrow prompts stream nothing, wide ones do, and a faster lane lowers the width
    gate = stream_gate(c, n_host=6)
    assert 1 < gate <= 1 << 16
    per = lambda rows: [rows * c.top_k // c.n_expert] * c.n_expert            # noqa: E731
    assert not split(per(gate - 1), list(range(6)), c).streamed and split(per(gate), list(range(6)), c).streamed
    fast = dataclasses.replace(c, lane_b_per_us=500e3)
    assert stream_gate(fast, n_host=6) < gate
    assert stream_gate(dataclasses.replace(c, lane_b_per_us=1.0), n_host=6, limit=4096) == 4097


def test_os_shim_calls(tmp_path):
    """The operating-system calls behind one module: masks, memory, free bytes, page-cache residency, advice, no-replace
    rename; refusals carry the call's name."""
    import mmap
    import os
    from bloomery_b200.utils import osshim as O
    cpus = O.mask_cpus()
    assert cpus and all(isinstance(c, int) for c in cpus)
    O.set_mask(cpus)                                              # the mask it already has
    with pytest.raises(O.OsError):
        O.set_mask([])
    hm = O.host_memory()
    assert 0 < hm.available <= hm.total and (hm.locked_limit == -1 or hm.locked_limit >= 0)
    fake = tmp_path / "meminfo"
    fake.write_text("MemTotal:       1000 kB\nMemFree: 1 kB\nMemAvailable:    400 kB\n")
    fm = O.host_memory(str(fake))
    assert (fm.total, fm.available) == (1000 << 10, 400 << 10)
    assert O.page_bytes() in (4096, 16384, 65536) and O.max_rss_bytes() > 0
    assert O.free_bytes(str(tmp_path)) > 0
    with pytest.raises(O.OsError) as err:
        O.free_bytes(str(tmp_path / "missing"))
    assert err.value.what == "statvfs"
    p = tmp_path / "blob"
    p.write_bytes(os.urandom(3 * O.page_bytes() + 100))
    with open(p, "rb") as fh:
        m = mmap.mmap(fh.fileno(), 0, access=mmap.ACCESS_READ)
        O.advise(m, "sequential")
        O.advise(m, "willneed")
        _ = m[0], m[O.page_bytes()], m[-1]                       # touch every page
        got = O.populated(m)
        assert got.pages == 4 and got.resident == 4 and got.fraction == 1.0
        assert O.populated(m, O.page_bytes(), O.page_bytes()).pages == 1
        with pytest.raises(O.OsError):
            O.populated(m, 1)                                     # not on a page boundary
        with pytest.raises(O.OsError):
            O.advise(m, "sideways")
        O.fadvise_dontneed(fh.fileno())
        m.close()
    a, b = tmp_path / "a", tmp_path / "b"
    a.write_text("first")
    b.write_text("second")
    with pytest.raises(O.OsError):
        O.rename_noreplace(str(a), str(b))
    assert b.read_text() == "second" and a.exists()
    O.rename_noreplace(str(a), str(tmp_path / "c"))
    assert (tmp_path / "c").read_text() == "first" and not a.exists()
    fd = None
    try:
        fd = O.open_direct(str(p))
    except O.OsError as exc:                                      # tmpfs and some overlays refuse O_DIRECT by name
        assert exc.what == "open O_DIRECT"
    if fd is not None:
        os.close(fd)


def test_interleaved_ab_harness(capsys):
    """Two arms run alternately; the answer is medians, ratio, per-round wins and a sign test."""
    import json
    import sys
    from bloomery_b200.ops import ab
    assert ab.figure("noise\nqgu staged us per layer: 123.5 fault word: 0x0\nus per layer: 99.25 tail") == 99.25
    assert ab.figure('{"metric": "m", "value": 4553.2, "unit": "tok/s"}') == 4553.2
    with pytest.raises(ab.AbError):
        ab.figure("nothing here")
    order = []
    vals = {"A": iter([10.0, 10.2, 9.9, 10.1, 10.0, 10.3]), "B": iter([8.0, 8.1, 8.2, 7.9, 8.0, 8.1])}

    def fake(cmd, pattern, timeout):
        order.append(cmd)
        return next(vals[cmd])
    series = ab.interleave("A", "B", 6, run=fake)
    assert order == ["A", "B", "B", "A", "A", "B", "B", "A", "A", "B", "B", "A"]      # the arms swap places every round
    got = ab.compare(series["a"], series["b"])
    assert got["wins_b"] == 6 and got["wins_a"] == 0 and got["winner"] == "b" and got["sign_test_p"] < 0.05
    assert abs(got["ratio_b_over_a"] - 8.05 / 10.05) < 1e-9
    assert ab.compare([1.0, 2.0, 1.0, 2.0], [2.0, 1.0, 2.0, 1.0])["winner"] == "same"
    assert ab.compare([5.0] * 6, [4.0] * 6, higher_is_better=True)["winner"] == "a"
    py = sys.executable
    arm = lambda text: py + " -c " + '"' + text + '"'            # noqa: E731
    rc = ab.main([arm("print('us per layer: 12.5')"), arm("print('us per layer: 25.0')"), "--rounds", "2"])
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rc == 0 and out["median_a"] == 12.5 and out["ratio_b_over_a"] == 2.0 and out["a"] == [12.5, 12.5]
    assert ab.main([arm("import sys; sys.exit(3)"), arm("print(1)"), "--rounds", "1"]) == 1


def test_native_host_step_follows_the_oracle():
    """``runtime/host_model.py``: the whole decode step in C++ on the resident quantised rows.  Where the router is not
    at a near tie the logits equal the plain PyTorch model's to fp32 rounding; everywhere they stay in a band; the cache
    can be cut, saved and put back."""
    import torch
    from bloomery_b200.models.cpu_ref import CpuModel
    from bloomery_b200.models.spec import tiny_deepseek, tiny_qwen3moe
    from bloomery_b200.models.weights import Weights, synth_tensors
    from bloomery_b200.runtime.host_model import HostDecoder, covers
    spec = tiny_qwen3moe()
    assert covers(spec) and covers(tiny_deepseek()) and not covers(dataclasses.replace(spec, hidden=320))
    w = Weights.from_items(spec, synth_tensors(spec, "cpu", seed=0, mix="Q4_K_M"), "cpu")
    oracle, hd = CpuModel(w), HostDecoder(w, ctx=64)
    exact = 0
    for seed in (1234, 4):
        g = torch.Generator().manual_seed(seed)
        prompt = torch.randint(0, spec.vocab, (20,), generator=g)
        oracle.reset(); hd.reset()
        ref, got = oracle.forward(prompt), hd.forward(prompt.tolist())
        err = (got - ref).abs().amax(1) / ref.abs().amax(1)
        assert float(err.max()) < 0.06, err
        exact += int((err < 1e-5).sum())
    assert exact >= 8                                            # positions before any routing near-tie: the same numbers
    # cut and continue: the same rows again give the same logits bit for bit
    hd.reset()
    ids = torch.randint(0, spec.vocab, (12,), generator=torch.Generator().manual_seed(5)).tolist()
    first = hd.forward(ids)
    hd.cut(7)
    again = torch.stack([hd.step(t).clone() for t in ids[7:]])
    assert torch.equal(again, first[7:])
    # save and put back into another decoder
    k, v = hd.kv(9)
    other = HostDecoder(w, ctx=64)
    assert other.load_kv(k, v) == 9 and torch.equal(other.step(ids[9]), first[9])
    with pytest.raises(ValueError):
        other.load_kv(torch.zeros(spec.n_layer, 100, spec.n_kv * spec.head_dim), torch.zeros(spec.n_layer, 100, spec.n_kv * spec.head_dim))
    hd.close(); other.close()
    # the DeepSeek layer plan (latent attention in its absorbed form, a leading dense layer, sigmoid routing in groups
    # with the selection bias, a shared expert) and dense-only models: every q8 site may round a value the other way
    # when fp32 sums differ in their last bit, so whole prompts are compared in a band, and single tokens under a
    # decisive router (no routing near-ties) must mostly agree to fp32 rounding
    dspec = tiny_deepseek()
    wx = Weights.from_items(dspec, synth_tensors(dspec, "cpu", seed=0, mix="Q8_0"), "cpu")
    for n_, qw in wx.q.items():
        if n_.endswith("ffn_gate_inp.weight"):
            qw.data.view(torch.float32).mul_(60.0)
    ox, nx = CpuModel(wx), HostDecoder(wx, ctx=4)
    close = 0
    for tok in (5, 77, 1234, 4000, 9, 300):
        ox.reset(); nx.reset()
        r_, g_ = ox.forward(torch.tensor([tok]))[0], nx.step(tok)
        e_ = float((g_ - r_).abs().max() / r_.abs().max())
        assert e_ < 0.03, (tok, e_)
        close += int(e_ < 1e-5)
    assert close >= 3
    nx.close()
    plans = [(dspec, "Q8_0"), (dspec, "Q4_K_M"),
             (dataclasses.replace(spec, name="dense-gqa", n_expert=0, n_used=0, moe_inter=0, dense_inter=1024), "Q8_0"),
             (dataclasses.replace(dspec, name="dense-mla", n_expert=0, n_used=0, moe_inter=0, n_shared=0, shared_inter=0,
                                  first_dense=0, n_group=1, topk_group=1), "Q8_0")]
    for sp, mix in plans:
        wd = Weights.from_items(sp, synth_tensors(sp, "cpu", seed=0, mix=mix), "cpu")
        om, nd = CpuModel(wd), HostDecoder(wd, ctx=32)
        prompt = torch.randint(0, sp.vocab, (12,), generator=torch.Generator().manual_seed(3))
        ref, got = om.forward(prompt), nd.forward(prompt.tolist())
        err = (got - ref).abs().amax(1) / ref.abs().amax(1)
        assert float(err.max()) < 0.06, (sp.name, mix, err)
        kk, vv = nd.kv()
        assert kk.shape == (sp.n_layer, 12, (sp.kv_lora + sp.rope_dim) if sp.mla else sp.n_kv * sp.head_dim)
        assert vv.shape[-1] == (0 if sp.mla else sp.n_kv * sp.head_dim)
        nd.cut(5)
        assert torch.equal(torch.stack([nd.step(int(t)).clone() for t in prompt[5:]]), got[5:])
        nd.close()


def test_native_cpu_engine_slots_share_save_and_restore():
    import numpy as np
    import torch
    from bloomery_b200.models.spec import tiny_qwen3moe
    from bloomery_b200.models.weights import Weights, synth_tensors
    from bloomery_b200.serve.engine import EngineError, NativeCpuEngine
    from bloomery_b200.serve.tokenizer import ByteTokenizer
    spec = tiny_qwen3moe()
    w = Weights.from_items(spec, synth_tensors(spec, "cpu", seed=0, mix="Q4_K_M"), "cpu")
    eng = NativeCpuEngine(w, ByteTokenizer(spec.vocab), n_slots=3, slot_ctx=48)
    ids = torch.randint(0, spec.vocab, (14,), generator=torch.Generator().manual_seed(6)).tolist()
    eng.prefill(0, ids[:-1], 0)
    t0, l0 = eng.step([(0, ids[-1], 13)])[0]
    assert eng.share_prefix(0, 1, 10, have=0) == 10 and eng.share_prefix(0, 1, 10, have=10) == 0
    eng.prefill(1, ids[10:-1], 10)
    t1, l1 = eng.step([(1, ids[-1], 13)])[0]
    assert t1 == t0 and np.array_equal(l0, l1)                 # the shared prefix is the donor's own rows
    saved = eng.snapshot(0, ids)
    assert saved.n_bytes > 0 and eng.restore(2, saved, 13) == 13
    t2, l2 = eng.step([(2, ids[-1], 13)])[0]
    assert np.array_equal(l0, l2)
    eng.cut(2, 5)
    with pytest.raises(EngineError):
        eng.step([(2, ids[-1], 9)])                            # a row past what the slot keeps
    with pytest.raises(EngineError):
        eng.prefill(2, list(range(60)), 0)                     # beyond the slot context
    v = eng.embed(ids)
    assert v is not None and abs(float(np.linalg.norm(v)) - 1.0) < 1e-4
    assert eng.props()["engine"] == "cpu-native"
    eng.close()
