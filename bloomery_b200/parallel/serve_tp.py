"""Serving on several GPUs: rank 0 owns the HTTP server and the engine thread; every engine call
it makes is mirrored, in order, to the other ranks over a CPU control group, so that all ranks
enqueue the same passes and their fused reductions meet.

The reference runs its tensor-parallel ranks the same way: one process per rank, the leader's
greedy loop sends each step over a TCP control channel and the ranks exchange partial sums on
the data path (``crates/app/src/tp.rs:1-68``, ``crates/gpu/src/host/rank.rs``).  Here the control
channel is a gloo group on 127.0.0.1 and the data path is the in-kernel all-reduce over NVLink.

    python -m bloomery_b200.parallel.serve_tp --follower --rank R --world N --model FILE ...

is what the server's launcher starts for ranks 1..N-1.
"""
from __future__ import annotations

import argparse
import datetime
import itertools
import os
import subprocess
import sys
import weakref
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


class Lockstep:
    """Ordered command channel from rank 0 to all ranks of ``group`` (engine-agnostic)."""

    def __init__(self, group=None):
        self.group = group
        self.sent = 0

    def send(self, op: str, *args) -> None:
        dist.broadcast_object_list([(op, args)], src=0, group=self.group)
        self.sent += 1

    def recv(self) -> Tuple[str, tuple]:
        box: List[Any] = [None]
        dist.broadcast_object_list(box, src=0, group=self.group)
        return box[0]


def follow(target, chan: Lockstep, on_error=None) -> int:
    """Follower loop: apply every mirrored call to ``target`` until ``stop``.  A call that raises is
    reported and the loop goes on (the leader raised too: both engines were fed the same rows)."""
    n = 0
    while True:
        op, args = chan.recv()
        if op == "stop":
            return n
        try:
            getattr(target, op)(*args)
        except Exception as exc:  # noqa: BLE001
            if on_error is not None:
                on_error(op, exc)
        n += 1


class _RankOps:
    """What a follower does for each mirrored call (the engine-level twin of ``GpuEngine``)."""

    def __init__(self, dec):
        self.dec = dec
        self.saved: Dict[int, dict] = {}

    def prefill(self, slot, ids, start):
        if ids:
            self.dec.prefill(slot, list(ids), start)

    def step(self, rows):
        self.dec.step(list(rows))

    def cut(self, slot, n):
        self.dec.cut(slot, n)

    def reset(self, slot):
        self.dec.reset(slot)

    def share_prefix(self, src, dst, n, have=0):
        got = self.dec.kv.share_prefix(src, dst, n, have)
        if got > 0:
            self.dec.slot_len[dst] = got
            self.dec.kv.sync_table()

    def snapshot(self, slot, n, sid):
        self.saved[sid] = self.dec.kv.snapshot(slot, n)

    def restore(self, slot, sid, n):
        self.dec.kv.restore(slot, self.saved[sid], n)
        self.dec.kv.sync_table()
        self.dec.slot_len[slot] = n

    def drop(self, sids):
        for s in sids:
            self.saved.pop(s, None)


def leader_engine(dec, tokenizer, model_name: str, chan: Lockstep):
    """``GpuEngine`` whose every state-changing call is mirrored to the followers first."""
    from ..serve.engine import GpuEngine, Saved

    class TpGpuEngine(GpuEngine):
        device_sampling = False          # the followers do not mirror sampler state; the leader samples on the host

        def __init__(self):
            super().__init__(dec, tokenizer, model_name)
            self._sid = itertools.count(1)
            self._dropped: List[int] = []

        def _send(self, op, *args):
            if self._dropped:
                gone, self._dropped = self._dropped, []
                chan.send("drop", gone)
            chan.send(op, *args)

        def prefill(self, slot, ids, start):
            self._send("prefill", slot, list(ids), start)
            return super().prefill(slot, ids, start)

        def step(self, rows, want_logits=True):
            out = []
            for i in range(0, len(rows), self.max_rows):
                chunk = [tuple(int(v) for v in r) for r in rows[i:i + self.max_rows]]
                self._send("step", chunk)
                out.extend(super().step(chunk, want_logits))
            return out

        def cut(self, slot, n):
            self._send("cut", slot, n)
            super().cut(slot, n)

        def reset(self, slot):
            self._send("reset", slot)
            super().reset(slot)

        def share_prefix(self, src, dst, n, have=0):
            self._send("share_prefix", src, dst, n, have)
            return super().share_prefix(src, dst, n, have)

        def snapshot(self, slot, ids):
            if not len(ids):
                return None
            sid = next(self._sid)
            self._send("snapshot", slot, len(ids), sid)
            saved = super().snapshot(slot, ids)
            saved = Saved(saved.ids, {"sid": sid, "local": saved.payload}, saved.n_bytes)
            weakref.finalize(saved, self._dropped.append, sid)
            return saved

        def restore(self, slot, saved, n):
            n = min(n, len(saved.ids))
            self._send("restore", slot, saved.payload["sid"], n)
            return super().restore(slot, Saved(saved.ids, saved.payload["local"], saved.n_bytes), n)

        def props(self):
            p = super().props()
            p["devices"] = [f"cuda:{r}" for r in range(dist.get_world_size())]
            p["parallel"] = f"tp{dist.get_world_size()} (attention heads and routed experts sharded; reductions in-kernel over NVLink)"
            return p

        def close(self):
            chan.send("stop")

    return TpGpuEngine()


def gguf_items(g):
    """The tensors of an open GGUF file as a ``TensorItem`` stream (host memory)."""
    for name, info in g.tensors.items():
        yield name, tuple(info.shape), info.qtype.name, g.tensor_rows(name)


def open_rank(model: str, rank: int, world: int, device: int, n_slots: int, slot_ctx: int, fused: bool = True,
              use_graphs: bool = True):
    """Load this rank's shard of a GGUF model and build its engine; returns (engine, spec, gguf)."""
    from ..formats.gguf import Gguf
    from ..models.spec import ModelSpec
    from ..models.weights import Weights
    from .sharded import ShardedEngine, local_spec, shard_items
    g = Gguf.open(model)
    spec = ModelSpec.from_gguf(g)
    dev = f"cuda:{device}"
    torch.cuda.set_device(device)
    w = Weights.from_items(local_spec(spec, world), shard_items(gguf_items(g), spec, rank, world), dev)
    torch.cuda.synchronize()
    eng = ShardedEngine(w, spec, rank, world, fused=fused, n_slots=n_slots, slot_ctx=slot_ctx, use_graphs=use_graphs and fused)
    eng.gemm_threshold = 64 if fused else 0     # long prompts take the several-GPU GEMM path
    return eng, spec, g


def init_groups(rank: int, world: int, device: int, port: int, timeout_s: float = 600.0):
    """NCCL world group (bootstrap of the symmetric arena) + a gloo group for the command channel."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(device)
    to = datetime.timedelta(seconds=timeout_s)
    dist.init_process_group("nccl", rank=rank, world_size=world, timeout=to, device_id=torch.device(f"cuda:{device}"))
    return dist.new_group(backend="gloo", timeout=to)


def spawn_followers(model: str, devices: Sequence[int], port: int, n_slots: int, slot_ctx: int,
                    extra_env: Optional[Dict[str, str]] = None) -> List[subprocess.Popen]:
    procs = []
    for r in range(1, len(devices)):
        env = dict(os.environ, **(extra_env or {}))
        cmd = [sys.executable, "-m", "bloomery_b200.parallel.serve_tp", "--follower", "--rank", str(r), "--world",
               str(len(devices)), "--device", str(devices[r]), "--port", str(port), "--model", model, "--slots",
               str(n_slots), "--slot-ctx", str(slot_ctx)]
        procs.append(subprocess.Popen(cmd, env=env))
    return procs


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--follower", action="store_true")
    ap.add_argument("--rank", type=int, required=True)
    ap.add_argument("--world", type=int, required=True)
    ap.add_argument("--device", type=int, required=True)
    ap.add_argument("--port", type=int, required=True)
    ap.add_argument("--model", required=True)
    ap.add_argument("--slots", type=int, default=4)
    ap.add_argument("--slot-ctx", type=int, default=4096)
    a = ap.parse_args(argv)
    ctl = init_groups(a.rank, a.world, a.device, a.port)
    from ..utils import levers
    eng, _, _ = open_rank(a.model, a.rank, a.world, a.device, a.slots, a.slot_ctx,
                          fused=bool(levers.get("BLOOMERY_FUSED_COMM")), use_graphs=bool(levers.get("BLOOMERY_GRAPHS")))
    dist.barrier()
    n = follow(_RankOps(eng), Lockstep(ctl), on_error=lambda op, exc: print(f"rank {a.rank}: {op}: {exc}", file=sys.stderr))
    print(f"rank {a.rank}: {n} mirrored calls", file=sys.stderr)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
