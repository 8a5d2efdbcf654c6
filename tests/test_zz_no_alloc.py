"""The allocation-free attention entry point, called through its exported C symbol.

Some users of the library cannot call cudaMalloc when they need attention (their device
memory was handed out in full at start-up, or an allocation would stall a latency-critical
loop), so ``bl_flash_decode_static`` keeps its split-K partials in a device array inside the
library.  Its result must equal the ordinary entry point's, also on a second call, when
the shared array still holds the first call's partials.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(seed, lens, head=128, n_q=32, n_kv=4, n_seg=13):
    torch.manual_seed(seed)
    M = len(lens)
    n_pages, max_pages = 48, 16
    q = (torch.randn(M, n_q, head) / math.sqrt(head)).to(DEV)
    kc = torch.randn(n_pages, n_kv, 64, head).half().to(DEV)
    vc = torch.randn(n_pages, n_kv, 64, head).half().to(DEV)
    table = torch.stack([torch.randperm(n_pages)[:max_pages] for _ in range(M)]).to(torch.int32).to(DEV)
    pos = torch.tensor([L - 1 for L in lens], dtype=torch.int32, device=DEV)
    seq = torch.arange(M, dtype=torch.int32, device=DEV)
    return dict(q=q, kc=kc, vc=vc, table=table, pos=pos, seq=seq, M=M, head=head, n_q=n_q, n_kv=n_kv, n_seg=n_seg,
                n_pages=n_pages, max_pages=max_pages, ctx=max_pages * 64)


def _outputs(c):
    w = c["n_q"] * c["head"]
    return (torch.zeros(c["M"], w, device=DEV), torch.zeros(c["M"], w, dtype=torch.int8, device=DEV),
            torch.zeros(c["M"], w // 32, 2, device=DEV))


def _run_static(lib, c):
    out, outq, outds = _outputs(c)
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.bl_flash_decode_static(vp(c["q"]), vp(c["kc"]), vp(c["vc"]), vp(c["pos"]), vp(c["seq"]), vp(c["table"]),
                                    ctypes.c_int(c["max_pages"]), ctypes.c_int(c["n_pages"]), ctypes.c_int(c["head"]),
                                    ctypes.c_int(c["n_q"]), ctypes.c_int(c["n_kv"]), ctypes.c_int(c["M"]),
                                    ctypes.c_int(c["n_seg"]), ctypes.c_int(c["ctx"]), vp(out), vp(outq), vp(outds),
                                    ctypes.c_void_p(0), ctypes.c_int(0), st)
    return rc, out, outq, outds


def _run_ordinary(c):
    from bloomery_b200.ops import decode as K
    out, outq, outds = _outputs(c)
    cells = c["M"] * c["n_q"] * c["n_seg"]
    part_ml = torch.zeros(cells * 2, device=DEV)
    part_acc = torch.zeros(cells * c["head"], device=DEV)
    K.flash_decode(c["q"], c["kc"], c["vc"], c["pos"], c["seq"], c["table"], c["n_pages"], c["head"], c["n_q"],
                   c["n_kv"], c["M"], c["n_seg"], c["ctx"], part_ml, part_acc, out, outq, outds, None, 0)
    return out, outq, outds


def test_static_scratch_entry_matches_ordinary_entry_twice():
    from bloomery_b200.ops._lib import cuda
    lib = cuda()
    assert hasattr(lib, "bl_flash_decode_static")
    # two different problems back to back: the second one runs over the first one's leftovers
    # ... and a head size of 64 with 12 query heads per key/value head (the two-pass form of the segment kernel)
    for case in (_case(1, [700, 65, 1]), _case(2, [3, 1000, 512, 129], n_seg=7),
                 _case(4, [900, 64, 17], head=64, n_q=24, n_kv=2, n_seg=9)):
        rc, out, outq, outds = _run_static(lib, case)
        assert rc == 0
        ref_out, ref_q, ref_ds = _run_ordinary(case)
        torch.cuda.synchronize()
        assert torch.allclose(out, ref_out, rtol=2e-3, atol=2e-3)
        assert torch.equal(out, ref_out)          # same kernels, same order: in fact bit-equal
        assert torch.equal(outq, ref_q) and torch.equal(outds, ref_ds)


def test_static_scratch_entry_refuses_oversize():
    from bloomery_b200.ops._lib import cuda
    lib = cuda()
    big = _case(3, [10] * 8, n_q=64, n_seg=40)          # 8 * 64 * 40 cells > 8192
    rc, out, _, _ = _run_static(lib, big)
    assert rc == -5
    torch.cuda.synchronize()
    assert float(out.abs().sum()) == 0.0                 # nothing was launched
