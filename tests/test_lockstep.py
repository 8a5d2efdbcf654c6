"""The command channel of multi-GPU serving, on CPU: two gloo ranks, rank 0 mirrors its engine calls,
rank 1 applies them in order; a call that raises on the follower does not end the loop."""
import os
import socket
import subprocess
import sys

SCRIPT = r'''
import datetime, json, os, sys
import torch.distributed as dist
from bloomery_b200.parallel.serve_tp import Lockstep, follow
rank = int(sys.argv[1]); port = sys.argv[2]; out = sys.argv[3]
os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = port
dist.init_process_group("gloo", rank=rank, world_size=2, timeout=datetime.timedelta(seconds=60))
chan = Lockstep()
class Rec:
    def __init__(self): self.log = []
    def prefill(self, slot, ids, start): self.log.append(["prefill", slot, list(ids), start])
    def step(self, rows): self.log.append(["step", [list(r) for r in rows]])
    def cut(self, slot, n):
        if n < 0: raise ValueError("bad cut")
        self.log.append(["cut", slot, n])
rec = Rec()
errors = []
if rank == 0:
    for op, args in [("prefill", (0, [1, 2, 3], 0)), ("step", ([(0, 7, 3), (1, 8, 0)],)), ("cut", (0, -1)), ("cut", (0, 2))]:
        chan.send(op, *args)
        try: getattr(rec, op)(*args)
        except ValueError as e: errors.append(str(e))
    chan.send("stop")
else:
    n = follow(rec, chan, on_error=lambda op, e: errors.append(str(e)))
    assert n == 4, n
json.dump({"log": rec.log, "errors": errors}, open(out, "w"))
dist.destroy_process_group()
'''


def test_follower_applies_the_leaders_calls_in_order(tmp_path):
    with socket.socket() as so:
        so.bind(("127.0.0.1", 0))
        port = so.getsockname()[1]
    procs = [subprocess.Popen([sys.executable, "-c", SCRIPT, str(r), str(port), str(tmp_path / f"r{r}.json")],
                              env=dict(os.environ, PYTHONPATH=os.getcwd())) for r in range(2)]
    for p in procs:
        assert p.wait(timeout=120) == 0
    import json
    a, b = (json.load(open(tmp_path / f"r{r}.json")) for r in range(2))
    assert a == b and a["errors"] == ["bad cut"]
    assert [e[0] for e in a["log"]] == ["prefill", "step", "cut"]
