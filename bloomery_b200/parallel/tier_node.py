"""Expert tier node: another process (or machine) that holds routed experts in RAM and answers the expert
leg of a layer over a framed TCP channel.

    python -m bloomery_b200.parallel.tier_node --model FILE --listen 127.0.0.1:7071 [--layers 10:20]

Wire: every frame is ``u32 length | u8 tag | payload`` (little endian); every read and write has a deadline;
there is no authentication -- bind to loopback or a private link.  ``HELLO`` answers a census (shapes, types,
per-layer SHA-256 of the first expert's gate rows) that the client checks against its own file before it sends
work; ``MOE`` carries one layer's rows (ids, weights, q8 activations) and answers the fp32 sums.  A lost node
raises :class:`TierLost` on the client, which then serves the layer itself or gives up, its choice.

The reference's tier nodes: ``crates/gpu/src/host/node.rs`` and ``node/wire.rs`` (length + tag frames, every I/O
bounded, no auth, census, rows opened with a sha256 check), binary ``tier_server.rs``.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import socket
import struct
import sys
import threading
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

T_HELLO, T_CENSUS, T_MOE, T_SUMS, T_ERROR, T_BYE = 1, 2, 3, 4, 5, 6
MAX_FRAME = 256 << 20


class TierLost(ConnectionError):
    """The node did not answer within the deadline, closed the channel, or answered an error."""


def _recv_exact(sock: socket.socket, n: int) -> bytes:
    buf = bytearray()
    while len(buf) < n:
        chunk = sock.recv(n - len(buf))
        if not chunk:
            raise TierLost("channel closed")
        buf += chunk
    return bytes(buf)


def send_frame(sock: socket.socket, tag: int, payload: bytes = b"") -> None:
    sock.sendall(struct.pack("<IB", len(payload) + 1, tag) + payload)


def recv_frame(sock: socket.socket) -> Tuple[int, bytes]:
    try:
        (n,) = struct.unpack("<I", _recv_exact(sock, 4))
        if n < 1 or n > MAX_FRAME:
            raise TierLost(f"frame of {n} bytes")
        body = _recv_exact(sock, n)
    except socket.timeout:
        raise TierLost("deadline passed") from None
    except OSError as exc:
        raise TierLost(str(exc)) from None
    return body[0], body[1:]


def _digest(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().cpu().numpy().tobytes()).hexdigest()


def census_of(weights, layers: Optional[List[int]] = None) -> Dict[str, object]:
    s = weights.spec
    have = [il for il in range(s.n_layer + s.n_mtp) if f"blk.{il}.ffn_gate_exps.weight" in weights.q]
    layers = [il for il in have if layers is None or il in layers]
    out = {"n_expert": s.n_expert, "hidden": s.hidden, "inter": s.moe_inter, "n_used": s.n_used, "layers": {}}
    for il in layers:
        g, d = weights.q[f"blk.{il}.ffn_gate_exps.weight"], weights.q[f"blk.{il}.ffn_down_exps.weight"]
        out["layers"][str(il)] = {"gate_type": g.qtype, "down_type": d.qtype, "sha256": _digest(g.data[0])}
    return out


def pack_moe(layer: int, ids: torch.Tensor, wts: torch.Tensor, xq: torch.Tensor, xds: torch.Tensor) -> bytes:
    M, k = ids.shape
    K = xq.shape[1]
    head = struct.pack("<IIII", layer, M, k, K)
    return head + ids.to(torch.int32).contiguous().numpy().tobytes() + wts.float().contiguous().numpy().tobytes() + \
        xq.to(torch.int8).contiguous().numpy().tobytes() + xds.float().contiguous().numpy().tobytes()


def unpack_moe(p: bytes):
    layer, M, k, K = struct.unpack("<IIII", p[:16])
    if M < 1 or M > 4096 or k < 1 or k > 16 or K < 32 or K % 32:
        raise ValueError("bad shape in a MOE frame")
    o = 16
    need = M * k * 4 * 2 + M * K + M * (K // 32) * 8
    if len(p) - o != need:
        raise ValueError(f"MOE frame carries {len(p) - o} bytes, its header says {need}")
    ids = torch.from_numpy(np.frombuffer(p, np.int32, M * k, o).copy()).reshape(M, k); o += M * k * 4
    wts = torch.from_numpy(np.frombuffer(p, np.float32, M * k, o).copy()).reshape(M, k); o += M * k * 4
    xq = torch.from_numpy(np.frombuffer(p, np.int8, M * K, o).copy()).reshape(M, K); o += M * K
    xds = torch.from_numpy(np.frombuffer(p, np.float32, M * (K // 32) * 2, o).copy()).reshape(M, K // 32, 2)
    return layer, ids, wts, xq, xds


def local_leg(weights, layer: int, ids, wts, xq, xds) -> torch.Tensor:
    """The expert leg on this process's CPU (the C++ pool) over RAM-resident stacks."""
    from ..formats.resident import WT
    from ..ops._lib import host, p as vp
    s = weights.spec
    g, u, d = (weights.q[f"blk.{layer}.ffn_{n}_exps.weight"] for n in ("gate", "up", "down"))
    M, k = ids.shape
    out = torch.zeros(M, s.hidden)
    ids, wts, xq, xds = ids.contiguous(), wts.contiguous(), xq.contiguous(), xds.contiguous()
    rc = host().blh_moe_experts(M, s.hidden, s.moe_inter, g.data.shape[0], k, vp(ids), vp(wts), vp(xq), vp(xds), vp(g.data),
                                vp(u.data), vp(d.data), WT[g.qtype], WT[d.qtype], vp(out))
    if rc != 0:
        raise RuntimeError(f"expert leg refused layer {layer} (code {rc})")
    return out


class TierServer:
    def __init__(self, weights, host_: str = "127.0.0.1", port: int = 0, layers: Optional[List[int]] = None,
                 io_timeout: float = 30.0):
        self.w = weights
        self.census = census_of(weights, layers)
        self.io_timeout = io_timeout
        self.sock = socket.socket()
        self.sock.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        self.sock.bind((host_, port))
        self.sock.listen(8)
        self.addr = self.sock.getsockname()
        self.stop = threading.Event()
        self.served = 0
        self._thr: Optional[threading.Thread] = None

    def start(self) -> "TierServer":
        self._thr = threading.Thread(target=self._accept, name="tier-node", daemon=True)
        self._thr.start()
        return self

    def _accept(self) -> None:
        self.sock.settimeout(0.2)
        while not self.stop.is_set():
            try:
                c, _ = self.sock.accept()
            except socket.timeout:
                continue
            except OSError:
                return
            threading.Thread(target=self._serve, args=(c,), daemon=True).start()

    def _serve(self, c: socket.socket) -> None:
        c.settimeout(self.io_timeout)
        c.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        try:
            while not self.stop.is_set():
                tag, body = recv_frame(c)
                if tag == T_HELLO:
                    send_frame(c, T_CENSUS, json.dumps(self.census).encode())
                elif tag == T_MOE:
                    try:
                        layer, ids, wts, xq, xds = unpack_moe(body)
                        if str(layer) not in self.census["layers"]:
                            raise ValueError(f"layer {layer} is not held by this node")
                        out = local_leg(self.w, layer, ids, wts, xq, xds)
                        self.served += 1
                        send_frame(c, T_SUMS, out.numpy().tobytes())
                    except (ValueError, RuntimeError) as exc:
                        send_frame(c, T_ERROR, str(exc).encode())
                elif tag == T_BYE:
                    return
                else:
                    send_frame(c, T_ERROR, f"unknown tag {tag}".encode())
        except TierLost:
            pass
        finally:
            c.close()

    def close(self) -> None:
        self.stop.set()
        try:
            self.sock.close()
        except OSError:
            pass


class RemoteExpertTier:
    """Client side: one connection, census checked against the local file before any work is sent."""

    def __init__(self, addr: Tuple[str, int], io_timeout: float = 30.0):
        self.addr, self.io_timeout = addr, io_timeout
        self.sock: Optional[socket.socket] = None
        self.census: Dict[str, object] = {}

    def open(self, weights=None) -> Dict[str, object]:
        try:
            self.sock = socket.create_connection(self.addr, timeout=self.io_timeout)
        except OSError as exc:
            raise TierLost(f"cannot reach the tier node at {self.addr}: {exc}") from None
        self.sock.settimeout(self.io_timeout)
        self.sock.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        send_frame(self.sock, T_HELLO)
        tag, body = recv_frame(self.sock)
        if tag != T_CENSUS:
            raise TierLost("the node did not answer a census")
        self.census = json.loads(body)
        if weights is not None:
            mine = census_of(weights, [int(k) for k in self.census["layers"]])
            for key in ("n_expert", "hidden", "inter"):
                if mine[key] != self.census[key]:
                    raise TierLost(f"the node serves another model: {key} {self.census[key]} != {mine[key]}")
            for il, row in self.census["layers"].items():
                if mine["layers"].get(il) != row:
                    raise TierLost(f"the node's layer {il} differs from the local file (type or sha256 of its rows)")
        return self.census

    def moe(self, layer: int, ids, wts, xq, xds) -> torch.Tensor:
        if self.sock is None:
            raise TierLost("not connected")
        try:
            send_frame(self.sock, T_MOE, pack_moe(layer, ids, wts, xq, xds))
        except OSError as exc:
            self.close()
            raise TierLost(str(exc)) from None
        try:
            tag, body = recv_frame(self.sock)
        except TierLost:
            self.close()
            raise
        if tag == T_ERROR:
            raise TierLost(f"node error: {body.decode(errors='replace')}")
        M, K = ids.shape[0], xq.shape[1]
        if tag != T_SUMS or len(body) != M * K * 4:
            self.close()
            raise TierLost("malformed answer")
        return torch.from_numpy(np.frombuffer(body, np.float32).copy()).reshape(M, K)

    def close(self) -> None:
        if self.sock is not None:
            try:
                send_frame(self.sock, T_BYE)
            except OSError:
                pass
            self.sock.close()
            self.sock = None


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--listen", default="127.0.0.1:7071")
    ap.add_argument("--layers", default="", help="lo:hi (default: every layer with routed experts)")
    a = ap.parse_args(argv)
    from ..models.weights import open_model
    _, w, _ = open_model(a.model, "cpu")
    layers = None
    if a.layers:
        lo, hi = (int(x) for x in a.layers.split(":"))
        layers = list(range(lo, hi))
    host_, port = a.listen.rsplit(":", 1)
    srv = TierServer(w, host_, int(port), layers).start()
    print(json.dumps({"event": "tier_ready", "addr": f"{srv.addr[0]}:{srv.addr[1]}", "layers": sorted(int(k) for k in srv.census["layers"])}),
          flush=True)
    try:
        threading.Event().wait()
    except KeyboardInterrupt:
        srv.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
